"""Activation offloading to pinned host memory (semantics of trl/models/activation_offloading.py:83-781).

``OffloadActivations`` is a ``saved_tensors_hooks`` context.  A tensor saved for backward that is at least
``min_offload_size`` bytes, lives on the GPU and is not a parameter, a buffer or a view of parameter storage is
copied to a pinned host buffer on a side stream when autograd packs it, and copied back when autograd unpacks it.

How the pieces are laid out for a GPU with 180 GB of HBM and a PCIe/C2C link that is three orders of magnitude
slower than HBM:

* **Forward.**  The device tensor stays alive in a small stash (at most ``max_fwd_stash_size`` tensors) until its
  copy has finished; when it leaves the stash the compute stream waits for the copy event, so the caching
  allocator can hand the block to the next layer at once.  While a storage is in the stash, further saves of the
  same storage (views, a tensor saved by two nodes) are kept on the device instead of being copied again.
* **Backward.**  The device buffer of a restored tensor is allocated on the compute stream, filled on the side
  stream, and the compute stream waits for that copy only.  The context keeps no reference to a tensor it has handed
  back: autograd drops it when the node that asked for it has run, and because the block belongs to the compute
  stream the allocator can reuse it for the next node without ``record_stream`` or a stash.  At any time only the
  tensors of the executing node and the prefetched ones are resident, which is what lowers the peak (the reference
  reaches the same end with a stash, node post-hooks and ``record_stream``, :456-544).
* **Prefetch.**  Tensors are unpacked roughly in reverse packing order, so unpacking id ``n`` starts the copies of
  the ``prefetch`` offloaded ids below ``n`` that are still on the host; their own unpack then finds the data on the
  device (or under way) and the link works one layer ahead of the compute stream.
* **Host memory.**  Pinned buffers come from a size-keyed free list and go back to it when the copy that read them
  has finished; steady-state steps pin nothing.  Crossing 60 % of host RAM warns once.

``NoOpManager`` disables the hooks around the output head, whose input is used again immediately.
``offload_checkpoint`` is an activation-checkpoint wrapper whose saved layer input goes through the hooks (the
library checkpoint keeps its inputs in a closure, out of reach of ``saved_tensors_hooks``).
"""
from __future__ import annotations

import contextlib
import warnings
from collections import OrderedDict, defaultdict

import torch
from torch.autograd.graph import saved_tensors_hooks


class PinnedPool:
    """Free lists of (pinned) host buffers keyed by (numel, dtype).  A buffer handed back with an event is reused
    only after the event (the copy that read it) has completed."""

    def __init__(self):
        self.free = defaultdict(list)
        self.busy = []  # (event, tensor)
        self.bytes = 0

    def get(self, numel: int, dtype: torch.dtype, pin: bool) -> torch.Tensor:
        self._reap()
        key = (numel, dtype, pin)
        if self.free[key]:
            return self.free[key].pop()
        self.bytes += numel * torch.empty(0, dtype=dtype).element_size()
        return torch.empty(numel, dtype=dtype, pin_memory=pin)

    def put(self, t: torch.Tensor, event=None):
        if event is None:
            self.free[(t.numel(), t.dtype, t.is_pinned() if torch.cuda.is_available() else False)].append(t)
        else:
            self.busy.append((event, t))

    def _reap(self):
        if not self.busy:
            return
        still = []
        for ev, t in self.busy:
            if ev.query():
                self.free[(t.numel(), t.dtype, t.is_pinned())].append(t)
            else:
                still.append((ev, t))
        self.busy = still


_POOL = PinnedPool()
_ACTIVE: list = []  # stack of OffloadActivations contexts entered on this thread


def offloading_active() -> bool:
    return bool(_ACTIVE)


class _Entry:
    """One packed tensor.  ``kind``: "keep" (left on the device), "host" (offloaded)."""

    __slots__ = ("kind", "tensor", "host", "meta", "device", "gpu", "gpu_event", "storage_key")

    def __init__(self, kind, tensor=None, host=None, meta=None, device=None, storage_key=None):
        self.kind, self.tensor, self.host, self.meta, self.device = kind, tensor, host, meta, device
        self.gpu, self.gpu_event, self.storage_key = None, None, storage_key


class OffloadActivations(saved_tensors_hooks):
    def __init__(self, use_pin_memory: bool = True, use_streams: bool = True, min_offload_size: int = 1024,
                 max_fwd_stash_size: int = 5, model: torch.nn.Module | None = None, prefetch: int = 2,
                 _offload_cpu_tensors: bool = False):
        if max_fwd_stash_size < 1:
            raise ValueError(f"max_fwd_stash_size should be at least 1 but is {max_fwd_stash_size}")
        cuda = torch.cuda.is_available()
        self.use_streams = bool(use_streams and cuda)
        self.use_pin = bool(use_pin_memory and cuda)
        self.min_offload_size, self.max_fwd_stash_size, self.prefetch = min_offload_size, max_fwd_stash_size, max(0, prefetch)
        # bookkeeping tests run the same pack / unpack path on CPU tensors (the "host copy" is then a plain copy)
        self._cpu_ok = _offload_cpu_tensors
        self.s1 = torch.cuda.Stream() if self.use_streams else None
        self.param_storages: set[int] = set()
        if model is not None:
            self.update_model_params(model)
        self.tracker: dict[int, _Entry] = {}
        self.live_storage: dict[tuple, int] = {}       # storage key -> id whose device tensor is still in the stash
        self.fwd_stash: "OrderedDict[int, tuple]" = OrderedDict()  # id -> (device tensor, copy event)
        self.next_id = 0
        self.stats = {"offloaded": 0, "offloaded_bytes": 0, "kept": 0, "restored": 0, "prefetched": 0}
        self._warned = False
        super().__init__(self._pack, self._unpack)

    # ---- set-up ----------------------------------------------------------------------------------------------------
    def update_model_params(self, model: torch.nn.Module):
        """Records the storages of ``model``'s parameters and buffers; tensors that alias them are never offloaded
        (flat parameter buckets of the sharded engines hand out views of one storage)."""
        for t in list(model.parameters()) + list(model.buffers()):
            try:
                self.param_storages.add(t.untyped_storage().data_ptr())
            except RuntimeError:
                pass

    def __enter__(self):
        # a backward that never ran (an exception, an evaluation forward) leaves entries behind: drop them
        self._drop_all()
        _ACTIVE.append(self)
        return super().__enter__()

    def __exit__(self, *exc):
        if _ACTIVE and _ACTIVE[-1] is self:
            _ACTIVE.pop()
        return super().__exit__(*exc)

    def _drop_all(self):
        for e in self.tracker.values():
            if e.kind == "host" and e.host is not None:
                _POOL.put(e.host, e.gpu_event)
        self.tracker.clear()
        self.live_storage.clear()
        self._drain_stash(0)

    # ---- pack ---------------------------------------------------------------------------------------------------------
    def _eligible(self, t: torch.Tensor) -> bool:
        if not (t.is_cuda or (self._cpu_ok and t.device.type == "cpu")):
            return False
        if t.numel() * t.element_size() < self.min_offload_size:
            return False
        if isinstance(t, torch.nn.Parameter) or (hasattr(torch.nn, "Buffer") and isinstance(t, torch.nn.Buffer)):
            return False
        if "float8" in str(t.dtype) or type(t).__name__ in ("Float8TrainingTensor", "ScaledMMConfig", "LinearMMConfig"):
            return False
        try:
            return t.untyped_storage().data_ptr() not in self.param_storages
        except RuntimeError:
            return False

    def _drain_stash(self, keep: int):
        """Lets the oldest stashed device tensors go until ``keep`` remain; the compute stream is made to wait for
        their copies first, so the blocks can be reused right away."""
        while len(self.fwd_stash) > keep:
            tid, (_, ev) = self.fwd_stash.popitem(last=False)
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)
            e = self.tracker.get(tid)
            if e is not None and e.storage_key is not None and self.live_storage.get(e.storage_key) == tid:
                del self.live_storage[e.storage_key]

    def _pack(self, t: torch.Tensor):
        tid = self.next_id
        self.next_id += 1
        if not self._eligible(t):
            self.tracker[tid] = _Entry("keep", tensor=t)
            self.stats["kept"] += 1
            return tid
        skey = (t.untyped_storage().data_ptr(), t.untyped_storage().nbytes())
        if skey in self.live_storage:  # this storage is already on its way to the host and still alive on the device
            self.tracker[tid] = _Entry("keep", tensor=t)
            self.stats["kept"] += 1
            return tid
        # what travels: the whole storage for dense tensors that cover it and for broadcast views (stride 0), so
        # that as_strided restores the exact view; otherwise a contiguous copy of just the viewed elements
        elems_in_storage = t.untyped_storage().nbytes() // t.element_size()
        if 0 in t.stride() or (t.is_contiguous() and t.storage_offset() == 0 and t.numel() == elems_in_storage):
            src = torch.as_strided(t, (elems_in_storage,), (1,), 0)
            meta = (tuple(t.shape), tuple(t.stride()), t.storage_offset())
        else:
            src = t.contiguous().view(-1) if t.is_contiguous() else t.reshape(-1)
            meta = (tuple(t.shape), None, 0)
        host = _POOL.get(src.numel(), src.dtype, self.use_pin)
        ev = None
        if self.use_streams:
            self.s1.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.s1):
                host.copy_(src, non_blocking=True)
                ev = self.s1.record_event()
        else:
            host.copy_(src)
        e = _Entry("host", host=host, meta=meta, device=t.device, storage_key=skey)
        self.tracker[tid] = e
        self.fwd_stash[tid] = (src, ev)       # keeps the device memory alive until the copy is done
        self.live_storage[skey] = tid
        self._drain_stash(self.max_fwd_stash_size if self.use_streams else 0)
        self.stats["offloaded"] += 1
        self.stats["offloaded_bytes"] += src.numel() * src.element_size()
        if not self._warned and self.use_pin:
            self._check_host_memory()
        return tid

    def _check_host_memory(self):
        try:
            import psutil

            if psutil.virtual_memory().percent > 60:
                warnings.warn("activation offloading: more than 60% of host memory is in use")
                self._warned = True
        except Exception:
            pass

    # ---- unpack -----------------------------------------------------------------------------------------------------
    def _start_restore(self, e: _Entry):
        """Allocates the device buffer on the compute stream and starts the host -> device copy on the side stream."""
        if e.gpu is not None:
            return
        if self.use_streams:
            cur = torch.cuda.current_stream()
            gpu = torch.empty(e.host.numel(), dtype=e.host.dtype, device=e.device)  # owned by the compute stream
            self.s1.wait_stream(cur)  # earlier users of this block are ordered before the copy
            with torch.cuda.stream(self.s1):
                gpu.copy_(e.host, non_blocking=True)
                e.gpu_event = self.s1.record_event()
        else:
            gpu = e.host.to(e.device, copy=True)
        e.gpu = gpu

    def _unpack(self, tid: int):
        if tid not in self.tracker:
            raise ValueError(f"untracked saved tensor with id {tid}")
        e = self.tracker.pop(tid)
        if e.kind == "keep":
            return e.tensor
        if e.storage_key is not None and self.live_storage.get(e.storage_key) == tid:
            del self.live_storage[e.storage_key]
        stashed = self.fwd_stash.pop(tid, None)
        shape, stride, offset = e.meta
        if stashed is not None:  # backward reached it while the forward copy still kept it on the device
            flat = stashed[0]
            _POOL.put(e.host, stashed[1])
        else:
            self._start_restore(e)
            if e.gpu_event is not None:
                torch.cuda.current_stream().wait_event(e.gpu_event)
            flat = e.gpu
            _POOL.put(e.host, e.gpu_event)
            self.stats["restored"] += 1
        # the forward is over once backward unpacks: nothing needs the remaining stash entries on the device
        if self.fwd_stash:
            self._drain_stash(0)
        self._prefetch_below(tid)
        if stride is None:
            return flat.view(shape)
        return torch.as_strided(flat, shape, stride, offset)

    def _prefetch_below(self, tid: int):
        if not self.prefetch:
            return
        started, probe = 0, tid - 1
        floor = tid - 8 * (self.prefetch + 1)  # saved tensors that stayed on the device lie between offloaded ones
        while started < self.prefetch and probe >= 0 and probe > floor:
            e = self.tracker.get(probe)
            if e is not None and e.kind == "host" and probe not in self.fwd_stash:
                if e.gpu is None:
                    self._start_restore(e)
                    self.stats["prefetched"] += 1
                started += 1
            probe -= 1


class NoOpManager(saved_tensors_hooks):
    """Inside this context saved tensors are left alone (used around the output head so the last, immediately
    re-used activation is not bounced through host memory; trl/models/activation_offloading.py:659-781)."""

    def __init__(self):
        super().__init__(lambda t: t, lambda t: t)


def no_offload():
    """Context for code whose saved tensors must stay on the device while an offloading context is active."""
    return NoOpManager() if offloading_active() else contextlib.nullcontext()


class _OffloadCheckpoint(torch.autograd.Function):
    """Recompute-in-backward for one layer with the layer input saved through ``save_for_backward``, so that an
    enclosing :class:`OffloadActivations` moves it to the host.  Parameters are reached through the closure: their
    gradients are accumulated by the inner backward (the engines' post-accumulate hooks fire as usual)."""

    @staticmethod
    def forward(ctx, run, anchor, x):
        ctx.run = run
        ctx.save_for_backward(x)
        with torch.no_grad():
            return run(x)

    @staticmethod
    def backward(ctx, gy):
        (x,) = ctx.saved_tensors
        xin = x.detach().requires_grad_(True)
        with torch.enable_grad():
            y = ctx.run(xin)
        torch.autograd.backward(y, gy)
        return None, None, xin.grad


def offload_checkpoint(run, x: torch.Tensor) -> torch.Tensor:
    """``run(x)`` without keeping its intermediate activations; ``x`` is saved through the saved-tensor hooks."""
    anchor = x if x.requires_grad else torch.zeros((), device=x.device, requires_grad=True)
    return _OffloadCheckpoint.apply(run, anchor, x)


def get_act_offloading_ctx_manager(model, use_pin_memory=True, use_streams=True, min_offload_size=1024,
                                   max_fwd_stash_size=5, warn_if_no_head=True, prefetch=2):
    """Offloading context for ``model`` (trl/models/activation_offloading.py:659-781).  The native decoders call their
    output head through fused functions that open :func:`no_offload` themselves, so no module hooks are installed;
    for other ``nn.Module`` models the output head (``lm_head`` / ``score`` / ``output``) gets NoOp pre/post hooks.
    On a machine without a GPU the context still runs (nothing qualifies for offloading there)."""
    ctx = OffloadActivations(use_pin_memory, use_streams, min_offload_size, max_fwd_stash_size, model, prefetch)
    if model is not None and getattr(model, "_is_native", False):
        model.offload_checkpoint_inputs = True
        return ctx
    head = None
    if model is not None:
        for name in ("lm_head", "score", "output", "classifier"):
            mod = getattr(model, name, None)
            if isinstance(mod, torch.nn.Module):
                head = mod
                break
    if head is None:
        if warn_if_no_head and model is not None:
            warnings.warn("activation offloading: no output head found on the model; its input will be offloaded too")
        return ctx
    if not getattr(head, "_trlb_noop_hooks", False):
        noop = NoOpManager()
        head.register_forward_pre_hook(lambda m, a: noop.__enter__())
        head.register_forward_hook(lambda m, a, o: noop.__exit__(None, None, None))
        head._trlb_noop_hooks = True
    return ctx
