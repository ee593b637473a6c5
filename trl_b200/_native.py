"""Loader for the in-tree native libraries (built by ``trl_b200/csrc/build.py``).

``libtrl_b200_kernels.so``  sm_100a CUDA kernels behind a C ABI (called through ctypes on the
                            caller's CUDA stream).
``libtrl_b200_host.so``     host runtime in C++: rollout scheduler / block allocator, packing.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_DIR = os.path.join(_HERE, "_lib")
_lock = threading.Lock()
_kernels = None
_host = None


def lib_path(name: str) -> str:
    return os.path.join(_LIB_DIR, name)


def kernels(required: bool = True):
    """ctypes handle of the CUDA kernel library; raises if it is missing and ``required``."""
    global _kernels
    with _lock:
        if _kernels is None:
            p = lib_path("libtrl_b200_kernels.so")
            if not os.path.exists(p):
                if required:
                    raise RuntimeError(
                        f"{p} not found: build the sm_100a kernels first (python -m trl_b200.csrc.build). "
                        "CUDA tensors never fall back to eager PyTorch for the ops this library owns.")
                return None
            _kernels = ctypes.CDLL(p, mode=ctypes.RTLD_GLOBAL)
        return _kernels


def host_runtime():
    """Python facade of the C++ host runtime, or None if the library has not been built."""
    global _host
    with _lock:
        if _host is None:
            p = lib_path("libtrl_b200_host.so")
            if not os.path.exists(p):
                return None
            from .utils.host_runtime import HostRuntime

            _host = HostRuntime(ctypes.CDLL(p))
        return _host
