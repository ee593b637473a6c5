"""Optional-dependency probes (counterpart of trl/import_utils.py:29-152)."""
from __future__ import annotations

import importlib.util
from functools import lru_cache

LIGER_KERNEL_MIN_VERSION = "0.8.0"


class TRLExperimentalWarning(UserWarning):
    """Raised (as a warning) when something under ``trl_b200.experimental`` is imported."""


@lru_cache(maxsize=None)
def _is_package_available(name: str) -> bool:
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError, AttributeError):
        return False


def _probe(name):
    def f() -> bool:
        return _is_package_available(name)
    f.__name__ = f"is_{name}_available"
    return f


is_deepspeed_available = _probe("deepspeed")
is_fastapi_available = _probe("fastapi")
is_harbor_available = _probe("harbor")
is_jmespath_available = _probe("jmespath")
is_joblib_available = _probe("joblib")
is_liger_kernel_available = _probe("liger_kernel")
is_math_verify_available = _probe("math_verify")
is_mergekit_available = _probe("mergekit")
is_openreward_available = _probe("openreward")
is_pydantic_available = _probe("pydantic")
is_requests_available = _probe("requests")
is_unsloth_available = _probe("unsloth")
is_uvicorn_available = _probe("uvicorn")
is_vllm_available = _probe("vllm")
is_vllm_ascend_available = _probe("vllm_ascend")
is_weave_available = _probe("weave")
is_wandb_available = _probe("wandb")
is_rich_available = _probe("rich")


def is_native_kernels_available() -> bool:
    """True when the in-tree sm_100a kernel library has been built."""
    import os

    from ._native import lib_path

    return os.path.exists(lib_path("libtrl_b200_kernels.so"))
