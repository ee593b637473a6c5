"""Phase timers.  Same metric names as trl/extras/profiling.py:35-226
(``profiling/Time taken: <Trainer>.<name>``); on GPUs the interval is measured with CUDA
events on the current stream (resolved lazily at log time, so timing adds no host sync)."""
from __future__ import annotations

import contextlib
import functools
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
        return self

    def __exit__(self, *exc):
        key = f"profiling/Time taken: {type(self.trainer).__name__}.{self.name}"
        mode = "train" if self.trainer.model is None or self.trainer.model.training else "eval"
        if self._ev is not None:
            self._ev[1].record()
            self.trainer._metrics[mode][key].append(_LazyElapsed(*self._ev))
        else:
            self.trainer._metrics[mode][key].append(time.perf_counter() - self._t0)
        return False


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
