"""Activation offloading to pinned host memory (semantics of trl/models/activation_offloading.py:83-781).

``OffloadActivations`` is a ``saved_tensors_hooks`` context: every tensor saved for backward that is at
least ``min_offload_size`` bytes, is not a parameter/buffer (or a view of one) and lives on the GPU is
copied to a pinned host buffer on a side stream at pack time and copied back on that stream at unpack
time, with the compute stream waiting only at the point of use.  Storage pointers de-duplicate views of
one buffer; up to ``max_fwd_stash_size`` device tensors stay alive until their copy event has completed.
Pinned buffers come from a size-keyed free list, so steady-state steps allocate nothing on the host.
The full-shard engine offloads its per-layer checkpoints through the same pool.
"""
from __future__ import annotations

import contextlib
import warnings
from collections import defaultdict, deque

import torch
from torch.autograd.graph import saved_tensors_hooks


class PinnedPool:
    """Free lists of pinned host buffers keyed by (numel, dtype)."""

    def __init__(self):
        self.free = defaultdict(list)
        self.bytes = 0

    def get(self, like: torch.Tensor) -> torch.Tensor:
        key = (like.numel(), like.dtype)
        if self.free[key]:
            return self.free[key].pop()
        self.bytes += like.numel() * like.element_size()
        return torch.empty(like.numel(), dtype=like.dtype, pin_memory=True)

    def put(self, t: torch.Tensor):
        self.free[(t.numel(), t.dtype)].append(t)


_POOL = PinnedPool()


class OffloadActivations(saved_tensors_hooks):
    def __init__(self, use_pin_memory: bool = True, use_streams: bool = True, min_offload_size: int = 1024,
                 max_fwd_stash_size: int = 5, model: torch.nn.Module | None = None):
        self.use_streams = use_streams and torch.cuda.is_available()
        self.min_offload_size, self.max_fwd_stash_size = min_offload_size, max_fwd_stash_size
        self.use_pin = use_pin_memory and torch.cuda.is_available()
        self.s1 = torch.cuda.Stream() if self.use_streams else None
        self.param_ptrs = set()
        if model is not None:
            for t in list(model.parameters()) + list(model.buffers()):
                self.param_ptrs.add(t.untyped_storage().data_ptr())
        self.tracker = {}       # id -> (host tensor | original, was_offloaded, meta)
        self.by_storage = {}    # storage ptr -> id (views of one buffer are copied once)
        self.fwd_stash = deque()
        self.next_id = 0
        self._warned = False
        super().__init__(self._pack, self._unpack)

    def __enter__(self):
        self.tracker.clear()
        self.by_storage.clear()
        self.fwd_stash.clear()
        return super().__enter__()

    def _eligible(self, t: torch.Tensor) -> bool:
        if not t.is_cuda or t.numel() * t.element_size() < self.min_offload_size:
            return False
        if isinstance(t, torch.nn.Parameter) or "float8" in str(t.dtype):
            return False
        return t.untyped_storage().data_ptr() not in self.param_ptrs

    def _pack(self, t: torch.Tensor):
        tid = self.next_id
        self.next_id += 1
        if not self._eligible(t):
            self.tracker[tid] = (t, False, None)
            return tid
        sp = (t.untyped_storage().data_ptr(), t.untyped_storage().nbytes())
        base_id = self.by_storage.get(sp)
        meta = (t.shape, t.stride(), t.storage_offset(), t.dtype, t.device)
        if base_id is not None and base_id in self.tracker and self.tracker[base_id][1]:
            self.tracker[tid] = (base_id, "view", meta)
            return tid
        # copy the whole storage once; views are rebuilt with as_strided at unpack time
        flat = torch.empty(0, dtype=t.dtype, device=t.device).set_(t.untyped_storage())
        host = _POOL.get(flat) if self.use_pin else torch.empty(flat.numel(), dtype=flat.dtype)
        if self.use_streams:
            self.s1.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.s1):
                host.copy_(flat, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.s1)
            self.fwd_stash.append((flat, ev))
            while len(self.fwd_stash) > self.max_fwd_stash_size:
                old, oev = self.fwd_stash.popleft()
                oev.synchronize()
        else:
            host.copy_(flat)
        self.by_storage[sp] = tid
        self.tracker[tid] = (host, True, meta)
        if not self._warned and _POOL.bytes > 0:
            try:
                import psutil

                if _POOL.bytes > 0.6 * psutil.virtual_memory().total:
                    warnings.warn("activation offloading is using more than 60% of host memory")
                    self._warned = True
            except Exception:
                pass
        return tid

    def _unpack(self, tid):
        entry = self.tracker[tid]
        if entry[1] is False:
            return entry[0]
        if entry[1] == "view":
            base = self._materialise(entry[0])
            shape, stride, off, dtype, dev = entry[2]
            return base.as_strided(shape, stride, off)
        base = self._materialise(tid)
        shape, stride, off, dtype, dev = entry[2]
        return base.as_strided(shape, stride, off)

    def _materialise(self, tid):
        host, flag, meta = self.tracker[tid]
        if isinstance(host, torch.Tensor) and host.is_cuda:
            return host
        dev = meta[4]
        if self.use_streams:
            with torch.cuda.stream(self.s1):
                gpu = torch.empty(host.numel(), dtype=host.dtype, device=dev)
                gpu.copy_(host, non_blocking=True)
            torch.cuda.current_stream().wait_stream(self.s1)
            gpu.record_stream(torch.cuda.current_stream())
        else:
            gpu = host.to(dev)
        if self.use_pin:
            _POOL.put(host)
        self.tracker[tid] = (gpu, True, meta)  # later views reuse the device copy
        return gpu


class NoOpManager(saved_tensors_hooks):
    """Inside this context saved tensors are left alone (used around the output head so the last,
    immediately re-used activation is not bounced through host memory)."""

    def __init__(self):
        super().__init__(lambda t: t, lambda t: t)


def get_act_offloading_ctx_manager(model, use_pin_memory=True, use_streams=True, min_offload_size=1024,
                                   max_fwd_stash_size=5, warn_if_no_head=True):
    if not torch.cuda.is_available():
        return contextlib.nullcontext()
    return OffloadActivations(use_pin_memory, use_streams, min_offload_size, max_fwd_stash_size, model)
