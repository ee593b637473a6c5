"""Phase timers.  Same metric names as trl/extras/profiling.py:35-226
(``profiling/Time taken: <Trainer>.<name>``); on GPUs the interval is measured with CUDA
events on the current stream (resolved lazily at log time, so timing adds no host sync).

Every phase is also an NVTX range on GPUs (visible in any CUDA timeline tool), and with
``TRL_B200_TRACE=<file>`` the phases of the run are written as a Chrome trace (``chrome://tracing`` /
Perfetto JSON: one row per rank, wall-clock start, device-measured duration) when training ends."""
from __future__ import annotations

import contextlib
import functools
import json
import os
import time

import torch


class ProfilingContext:
    def __init__(self, trainer, name: str):
        self.trainer, self.name = trainer, name
        self._ev = None

    def __enter__(self):
        self._t0 = time.perf_counter()
        if torch.cuda.is_available() and getattr(self.trainer.args, "device", torch.device("cpu")).type == "cuda":
            self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._ev[0].record()
            torch.cuda.nvtx.range_push(f"{type(self.trainer).__name__}.{self.name}")
        return self

    def __exit__(self, *exc):
        key = f"profiling/Time taken: {type(self.trainer).__name__}.{self.name}"
        mode = "train" if self.trainer.model is None or self.trainer.model.training else "eval"
        if self._ev is not None:
            self._ev[1].record()
            torch.cuda.nvtx.range_pop()
            dur = _LazyElapsed(*self._ev)
        else:
            dur = time.perf_counter() - self._t0
        self.trainer._metrics[mode][key].append(dur)
        if TRACE_PATH:
            _TRACE.append((f"{type(self.trainer).__name__}.{self.name}", self._t0, dur))
        return False


TRACE_PATH = os.environ.get("TRL_B200_TRACE", "")
_TRACE: list = []  # (name, wall-clock start in seconds, duration: float or _LazyElapsed)


def dump_trace(path: str | None = None, rank: int = 0) -> str | None:
    """Writes the phases recorded so far as Chrome-trace JSON (complete events, microseconds) and clears the buffer.
    Ranks other than 0 write ``<path>.rank<r>``."""
    path = path or TRACE_PATH
    if not path:
        return None
    if rank:
        path = f"{path}.rank{rank}"
    events = [{"name": n, "ph": "X", "ts": t0 * 1e6, "dur": float(d) * 1e6, "pid": rank, "tid": 0, "cat": "phase"}
              for n, t0, d in _TRACE]
    _TRACE.clear()
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
    return path


class _LazyElapsed:
    """Seconds between two CUDA events, read when the value is finally converted to float."""

    def __init__(self, a, b):
        self.a, self.b = a, b

    def __float__(self):
        self.b.synchronize()
        return self.a.elapsed_time(self.b) / 1e3

    def __radd__(self, o):
        return o + float(self)

    def __add__(self, o):
        return float(self) + o


def profiling_context(trainer, name: str):
    return ProfilingContext(trainer, name)


def profiling_decorator(func):
    @functools.wraps(func)
    def wrapper(self, *a, **k):
        with profiling_context(self, func.__name__):
            return func(self, *a, **k)
    return wrapper
