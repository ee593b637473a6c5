"""``trl env``: platform and library versions (trl/scripts/env.py:25-81)."""
from __future__ import annotations

import platform
import sys
from importlib.metadata import PackageNotFoundError, version


def _v(pkg):
    try:
        return version(pkg)
    except PackageNotFoundError:
        return "not installed"


def print_env():
    import torch

    from trl_b200 import __version__
    from trl_b200._native import lib_path
    import os

    devs = [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())] if torch.cuda.is_available() else []
    info = {
        "Platform": platform.platform(), "Python version": platform.python_version(),
        "trl_b200 version": __version__, "PyTorch version": torch.__version__,
        "accelerator(s)": ", ".join(devs) or "cpu", "Transformers version": _v("transformers"),
        "Datasets version": _v("datasets"), "Tokenizers version": _v("tokenizers"), "Safetensors version": _v("safetensors"),
        "sm_100a kernel library": "built" if os.path.exists(lib_path("libtrl_b200_kernels.so")) else "not built",
        "host runtime library": "built" if os.path.exists(lib_path("libtrl_b200_host.so")) else "not built",
        "NCCL": ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else "n/a",
    }
    print("\nCopy-paste the following information when reporting an issue:\n\n" + "\n".join(f"- {k}: {v}" for k, v in info.items()))


if __name__ == "__main__":
    print_env()
