"""Builds the in-tree native libraries.

    python -m trl_b200.csrc.build [--force] [--verbose]

* ``trl_b200/_lib/libtrl_b200_kernels.so``  every ``*.cu`` here, compiled by nvcc for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``); works without a GPU (cross-compile).
* ``trl_b200/_lib/libtrl_b200_host.so``     ``*.cpp`` host runtime (scheduler, packing), g++ -O3.

Objects are cached next to the sources' hashes, so unchanged files are not recompiled.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(os.path.dirname(HERE), "_lib")
OBJ = os.path.join(LIB, "obj")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v", "--expt-relaxed-constexpr"]
# every source here builds into the one library used at any GPU count (no loads shared across a thread-block cluster)


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _digest(path: str, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    with open(path, "rb") as f:
        h.update(f.read())
    for hdr in sorted(os.listdir(HERE)):
        if hdr.endswith((".cuh", ".h", ".hpp")):
            with open(os.path.join(HERE, hdr), "rb") as f:
                h.update(f.read())
    return h.hexdigest()[:16]


def _compile(src: str, force: bool, verbose: bool) -> str:
    is_cu = src.endswith(".cu")
    flags = NVCC_FLAGS if is_cu else ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread"]
    tag = _digest(src, " ".join(flags))
    obj = os.path.join(OBJ, f"{os.path.basename(src)}.{tag}.o")
    if os.path.exists(obj) and not force:
        return obj
    for old in os.listdir(OBJ):
        if old.startswith(os.path.basename(src) + "."):
            os.remove(os.path.join(OBJ, old))
    cmd = ([_nvcc()] + flags if is_cu else ["g++"] + flags) + ["-I", HERE, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = os.path.join(OBJ, os.path.basename(src) + ".log")
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"compilation of {src} failed (see {log})")
    return obj


def build(force: bool = False, verbose: bool = False) -> dict[str, str]:
    os.makedirs(OBJ, exist_ok=True)
    cus = sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".cu"))
    cpps = sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".cpp"))
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        cu_objs = list(ex.map(lambda s: _compile(s, force, verbose), cus))
        cpp_objs = list(ex.map(lambda s: _compile(s, force, verbose), cpps))
    out = {}
    if cu_objs:
        so = os.path.join(LIB, "libtrl_b200_kernels.so")
        if force or not os.path.exists(so) or any(os.path.getmtime(o) > os.path.getmtime(so) for o in cu_objs):
            cmd = [_nvcc(), "-shared", "-o", so] + cu_objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                              "-Xcompiler", "-fPIC", "-cudart", "shared"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        out["kernels"] = so
    if cpp_objs:
        so = os.path.join(LIB, "libtrl_b200_host.so")
        if force or not os.path.exists(so) or any(os.path.getmtime(o) > os.path.getmtime(so) for o in cpp_objs):
            r = subprocess.run(["g++", "-shared", "-o", so] + cpp_objs + ["-pthread"], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        out["host"] = so
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    for k, v in build(a.force, a.verbose).items():
        print(f"{k}: {v}")


if __name__ == "__main__":
    main()
