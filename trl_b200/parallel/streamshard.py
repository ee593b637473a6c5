"""Full shard with streamed layers: parameter memory per rank really is 1 / world of the model.

``FullShardEngine`` keeps a full-size bf16 buffer for every layer and gathers into it once per optimizer step: fast,
but the parameters never shrink with the group, so a model must fit one GPU in bf16.  This engine is the other end
of the trade-off (ZeRO-3 / FSDP proper, what the reference reaches through accelerate's FSDP2 / DeepSpeed stage-3
profiles, trl/accelerate_configs/fsdp2.yaml and zero3.yaml):

* every decoder layer owns only its 1 / world slice of the layer's flat parameter buffer, plus fp32 master / AdamW
  moments / accumulated gradient for that slice;
* two full-size *slots* are shared by all layers (even layers use slot 0, odd layers slot 1, so a layer's weights
  survive while its neighbour is gathered).  A forward pre-hook all-gathers the layer's slices into its slot just
  before the layer runs - in the forward pass, and again when activation checkpointing recomputes the layer in the
  backward pass.  The parameters are permanent views into the slot, nothing is rebound;
* gradients of a layer are collected in one flat buffer as autograd produces them; when the last one has arrived the
  buffer is reduce-scattered and the owned slice is added to the fp32 accumulator, so no full-size gradient outlives
  its layer;
* embeddings, final norm and lm_head stay whole on every rank (gradient + optimizer state sharded, zero-2 style).

Activation checkpointing is required: with it autograd keeps no references to a layer's weights between forward and
backward, which is what makes overwriting the slot legal.  While a layer computes, the gather of the layer expected
next already fills the other slot (2 L - 2 gathers per forward + backward of L layers, none wasted).

On GPUs of one NVLink domain (bf16, symmetric memory available) the data movement is the framework's own kernels
over peer memory, not the backend's collectives:

* every rank keeps its bf16 slices in one symmetric arena.  A gather is ``shard_pull``: one kernel on a side stream
  that reads each owner's slice through its peer mapping straight into the local slot.  It needs no flag and no
  barrier, because slices change only inside the optimizer step, which is fenced by the gradient-norm all-reduce
  before it (every rank's gathers are joined first) and by the collective that republishes the replicated
  parameters after it;
* a layer's gradients are collected in one of three symmetric gradient buffers, and ``rs_reduce`` (accumulating
  form) runs on a second side stream as soon as the layer's last gradient has arrived: each rank reads its slice of
  every peer's buffer in place, averages in fp32 and adds to its accumulator, while the main stream goes on with the
  backward pass of the next layer.  The kernel's entry barrier is what makes reuse safe: a buffer is written again
  three layers later, after this rank's reduction of the layer in between has passed its barrier, which no rank
  passes before every rank has finished reading the earlier buffer.

Elsewhere (CPU / gloo, fp32, a single rank, ``TRL_B200_STREAM_FUSED=0``) the backend's all-gather / reduce-scatter are
used, issued asynchronously in the same order.  Gathering *inside* the consuming GEMM is the job of the fused
kernels in ``fullshard.py`` and is not repeated here.

Per rank and per parameter of a streamed layer: 4 + 8 (fp32 master, moments; the bf16 copy exists only inside the
slots) + 4 (gradient accumulator; 2 with ``grad_dtype=torch.bfloat16``) = 16 (14) bytes / world, plus 2 slots + 1
gradient buffer of one layer.  Llama-3-70B on 8 ranks: about 141 (124) GB of sharded state + 5 GB of slots per GPU,
against 140 GB for the bf16 weights alone under ``FullShardEngine``.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as td
import torch.nn as nn

from .engine import _ALIGN, adamw_flat


class _EventWork:
    """Stands where an async collective's work handle would: ``wait()`` orders the current stream after the event."""

    def __init__(self, event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


class _LayerShard:
    """Bookkeeping of one streamed layer."""

    def __init__(self, idx, module, names, params, offsets, numel, slot):
        self.idx, self.module, self.names, self.params, self.offsets, self.numel, self.slot = (
            idx, module, names, params, offsets, numel, slot)
        self.master = self.exp_avg = self.exp_avg_sq = self.grad_acc = None
        self.arrived = 0
        self.no_decay = []  # (lo, hi) ranges of 1-D parameters inside the flat layout


def _rebind(root: nn.Module, dotted: str, value: torch.Tensor, requires_grad: bool = True) -> nn.Parameter:
    """Replaces the (meta) parameter ``root.<dotted>`` by a parameter over ``value``."""
    *path, leaf = dotted.split(".")
    mod = root
    for part in path:
        mod = getattr(mod, part)
    p = nn.Parameter(value, requires_grad=requires_grad)
    mod._parameters[leaf] = p
    return p


@torch.no_grad()
def _init_param(name: str, v: torch.Tensor, std: float, gen: torch.Generator):
    """Same rule as ``CausalLM.reset_parameters``: norm weights one, other vectors zero, matrices N(0, std)."""
    leaf = name.rsplit(".", 1)[-1]
    if v.ndim == 1 and ("layernorm" in leaf or leaf == "norm" or leaf.endswith("_norm")):
        v.fill_(1.0)
    elif v.ndim == 1:
        v.zero_()
    else:
        v.normal_(0.0, std, generator=gen)


class StreamShardEngine:
    sharded = True
    mode = "full_shard_stream"

    def __init__(self, model: nn.Module, *, betas=(0.9, 0.999), eps=1e-8, weight_decay: float = 0.0, group=None,
                 device=None, init_seed: int = 0, init_std: float = 0.02, grad_dtype: torch.dtype | None = None, prefetch: bool = True,
                 frozen: bool = False):
        """``model`` may live on the meta device (``CausalLM(cfg, device="meta")``): then ``device`` names where the
        slices go and every layer is initialised inside its slot with a generator seeded by (``init_seed``, layer), so
        that all ranks draw the same weights and the whole model never exists anywhere (load real weights afterwards
        with ``load_weights``).  ``frozen=True`` shards a model that is only evaluated (a reference model): every
        parameter is streamed, a slice is kept in the model's own dtype (2 bytes / parameter / world for bf16) and there
        is no optimizer state, no gradient buffer and no gradient hook."""
        self.model, self.group, self.frozen = model, group, frozen
        self.world = td.get_world_size(group) if td.is_initialized() else 1
        self.rank = td.get_rank(group) if td.is_initialized() else 0
        self.betas, self.eps, self.weight_decay = betas, eps, weight_decay
        self.step_count = 0
        # accumulator of the reduced layer gradients.  fp32 by default; the compute dtype loses nothing when every
        # optimizer step has one micro-batch (the reduce-scatter already delivers that dtype) and saves 2 bytes / param
        self.grad_dtype = grad_dtype or torch.float32
        layers = getattr(model, "layers", None)
        if layers is None or len(layers) == 0:
            raise ValueError("the streamed full-shard engine needs a model with a `layers` list")
        first = next(model.parameters())
        meta = first.is_meta
        if meta and device is None:
            raise ValueError("a model on the meta device needs `device`")
        self.dev, self.dtype = (torch.device(device) if meta else first.device), first.dtype
        unit = self.world * _ALIGN
        self.layers: list[_LayerShard] = []
        in_layers = set()
        for i, mod in enumerate(layers):
            items = [(n, p) for n, p in mod.named_parameters() if p.requires_grad or frozen]
            if any(p.dtype != self.dtype for _, p in items):
                raise ValueError("all parameters of a streamed layer must share one dtype")
            offs, cur = [], 0
            for _, p in items:
                offs.append(cur)
                cur += (p.numel() + 15) // 16 * 16
            numel = (cur + unit - 1) // unit * unit
            ls = _LayerShard(i, mod, [n for n, _ in items], [p for _, p in items], offs, numel, i % 2)
            ls.no_decay = [(o, o + p.numel()) for (_, p), o in zip(items, offs) if p.ndim <= 1]
            self.layers.append(ls)
            in_layers.update(id(p) for _, p in items)
        slot_numel = max(l.numel for l in self.layers)
        # separate allocations: autograd tracks in-place writes per base tensor
        self.slots = [torch.zeros(slot_numel, dtype=self.dtype, device=self.dev) for _ in range(2)]
        self.fused = False
        if (self.dev.type == "cuda" and self.world > 1 and self.dtype == torch.bfloat16
                and os.environ.get("TRL_B200_STREAM_FUSED", "1") != "0"):
            from .symm import SymmArena, SyncWords, symmetric_available

            if symmetric_available():
                nbytes = sum(l.numel // self.world * 2 + 256 for l in self.layers) + 4096
                nbytes += 0 if frozen else 3 * (slot_numel * 2 + 256)
                self.arena = SymmArena(nbytes, self.dev, group)
                self.fused = True
                self._gstream, self._rstream = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
                self._pull_ctas = int(os.environ.get("TRL_B200_STREAM_PULL_CTAS", "32"))
                self._reduce_ctas = int(os.environ.get("TRL_B200_STREAM_REDUCE_CTAS", "32"))
                for l in self.layers:
                    l.shard16, l.shard16_off = self.arena.carve(l.numel // self.world, torch.bfloat16)
                if not frozen:
                    self._gbufs = [self.arena.carve(slot_numel, torch.bfloat16) for _ in range(3)]
                    self._gbuf_done = [None, None, None]
                    self._n_flush, self._cur = 0, 0
                    self._rs_sync = SyncWords(self.dev, channel=2)
                    self._sq_scratch = torch.zeros(1, dtype=torch.float32, device=self.dev)
                    self._tick = torch.zeros(1, dtype=torch.float32, device=self.dev)
        if frozen:
            self.gbuf = None
        elif self.fused:
            self.gbuf = self._gbufs[0][0]
        else:
            self.gbuf = torch.zeros(slot_numel, dtype=self.dtype, device=self.dev)
        self._resident = [None, None]  # layer index whose gathered weights a slot holds (or is receiving), or None
        self._inflight = [None, None]  # per slot: (layer, async work handle, send buffer) of a gather not yet waited for
        self._last_idx = None
        self.prefetch = prefetch
        for ls in self.layers:
            per = ls.numel // self.world
            lo = self.rank * per
            slot = self.slots[ls.slot]
            views = [slot[o:o + p.numel()].view(p.shape) for p, o in zip(ls.params, ls.offsets)]
            if meta:
                gen = torch.Generator(device=self.dev).manual_seed(init_seed * 1000003 + ls.idx + 1)
                ls.params = [_rebind(ls.module, n, v, not frozen) for n, v in zip(ls.names, views)]
                for n, v in zip(ls.names, views):
                    _init_param(n, v, init_std, gen)
            else:
                for p, v in zip(ls.params, views):
                    v.copy_(p.data)   # layers two apart share the slot: the slice is taken right below
                    p.data = v        # the original storage is released here
            if self.fused:
                ls.shard16.copy_(slot[lo:lo + per])
            if frozen:
                # the slice in the model's dtype is all a frozen model needs
                ls.master = ls.shard16 if self.fused else slot[lo:lo + per].clone()
                continue
            ls.master = slot[lo:lo + per].to(torch.float32, copy=True)  # fp32 owned slice; the compute-dtype copy is made when gathering
            ls.exp_avg = torch.zeros(per, dtype=torch.float32, device=self.dev)
            ls.exp_avg_sq = torch.zeros(per, dtype=torch.float32, device=self.dev)
            ls.grad_acc = torch.zeros(per, dtype=self.grad_dtype, device=self.dev)
        if self.fused:  # every owner's slices are in place before anybody pulls
            torch.cuda.synchronize(self.dev)
            td.barrier(group=self.group)
        # ---- everything outside the layers: whole on every rank, zero-2 style state ----
        if frozen:  # embeddings / norm / lm_head of a frozen model stay as they are (whole, own storage)
            if meta:  # same generator and order as the trainable path below: a frozen copy starts equal to the policy
                gen = torch.Generator(device=self.dev).manual_seed(init_seed * 1000003)
                layer_params = {id(q) for l in self.layers for q in l.params}
                seen = set()
                for n, p in list(model.named_parameters()):
                    if id(p) in layer_params or id(p) in seen or not p.is_meta:
                        continue
                    seen.add(id(p))
                    v = torch.empty(p.shape, dtype=p.dtype, device=self.dev)
                    _init_param(n, v, init_std, gen)
                    _rebind(model, n, v, False)
            self.rest_names, self.rest_params, self.rest_offsets, self.rest_numel = [], [], [], 0
            self._hooks = [l.module.register_forward_pre_hook(lambda mod, args, i=l.idx: self.materialize(i))
                           for l in self.layers]
            self._pending = None
            return
        rest = [(n, p) for n, p in model.named_parameters() if p.requires_grad and id(p) not in in_layers
                and not any(p is q for l in self.layers for q in l.params)]
        seen, uniq = set(), []
        for n, p in rest:
            if id(p) not in seen:
                seen.add(id(p))
                uniq.append((n, p))
        self.rest_names, self.rest_params, self.rest_offsets = [n for n, _ in uniq], [p for _, p in uniq], []
        cur = 0
        for _, p in uniq:
            self.rest_offsets.append(cur)
            cur += (p.numel() + 15) // 16 * 16
        self.rest_numel = (cur + unit - 1) // unit * unit if uniq else 0
        self.rest_flat = torch.zeros(self.rest_numel, dtype=self.dtype, device=self.dev)
        self.rest_grad = torch.zeros(self.rest_numel, dtype=torch.float32, device=self.dev)
        gen = torch.Generator(device=self.dev).manual_seed(init_seed * 1000003) if meta else None
        for j, (n, p, o) in enumerate(zip(self.rest_names, list(self.rest_params), self.rest_offsets)):
            v = self.rest_flat[o:o + p.numel()].view(p.shape)
            if meta:
                self.rest_params[j] = _rebind(model, n, v)
                _init_param(n, v, init_std, gen)
            else:
                v.copy_(p.data)
                p.data = v
        per = self.rest_numel // self.world
        self.rest_lo, self.rest_hi = self.rank * per, (self.rank + 1) * per
        sh = self.rest_flat[self.rest_lo:self.rest_hi]
        self.rest_master = sh if self.dtype == torch.float32 else sh.float()
        self.rest_exp_avg = torch.zeros(per, dtype=torch.float32, device=self.dev)
        self.rest_exp_avg_sq = torch.zeros(per, dtype=torch.float32, device=self.dev)
        self.rest_no_decay = [(o, o + p.numel()) for p, o in zip(self.rest_params, self.rest_offsets) if p.ndim <= 1]
        self._hooks = []
        self._pending = None
        self._install_hooks()

    # ---- gather / gradient collection ------------------------------------------------------------------------------
    def _gather_into(self, out: torch.Tensor, shard: torch.Tensor):
        if self.world == 1:
            out.copy_(shard)
        else:
            td.all_gather_into_tensor(out, shard.contiguous(), group=self.group)

    def _wait_slot(self, slot: int):
        fl = self._inflight[slot]
        if fl is not None:
            fl[1].wait()  # stream-ordered on GPUs: later kernels of the current stream see the gathered weights
            self._inflight[slot] = None

    def _invalidate(self):
        """The owned slices changed (optimizer step, checkpoint load): whatever the slots hold is stale."""
        for slot in (0, 1):
            self._wait_slot(slot)
        self._resident = [None, None]
        self._last_idx = None

    def _start_gather(self, idx: int):
        ls = self.layers[idx]
        self._wait_slot(ls.slot)
        if self.fused:
            from ..ops import cuda as K

            # the slot is free once everything queued so far on this stream (its previous tenant's kernels) has run
            self._gstream.wait_event(torch.cuda.current_stream().record_event())
            with torch.cuda.stream(self._gstream):
                K.shard_pull(self.arena, ls.shard16_off, ls.numel // self.world, self.slots[ls.slot], ctas=self._pull_ctas)
                done = self._gstream.record_event()
            self._inflight[ls.slot] = (idx, _EventWork(done), None)
            self._resident[ls.slot] = idx
            return
        src = ls.master.to(self.dtype)
        work = td.all_gather_into_tensor(self.slots[ls.slot][:ls.numel], src, group=self.group, async_op=True)
        self._inflight[ls.slot] = (idx, work, src)  # src must outlive the collective
        self._resident[ls.slot] = idx

    @torch.no_grad()
    def materialize(self, idx: int):
        """Makes layer ``idx``'s weights valid in its slot (collective: every rank calls it for the same layer), then
        starts the gather of the layer expected next into the OTHER slot, so that it travels while this layer
        computes: ``idx + 1`` when the layers are visited upwards (forward), ``idx - 1`` downwards or on a repeat
        (the recompute order of the backward pass).  A wrong guess only costs one unused gather."""
        ls = self.layers[idx]
        if self._resident[ls.slot] != idx:
            if self.world == 1:
                self.slots[ls.slot][:ls.numel].copy_(ls.master)
                self._resident[ls.slot] = idx
            else:
                self._start_gather(idx)
        self._wait_slot(ls.slot)
        last, self._last_idx = self._last_idx, idx
        if self.prefetch and self.world > 1:
            nxt = idx + 1 if (last is None or idx > last) else idx - 1
            if 0 <= nxt < len(self.layers) and self._resident[self.layers[nxt].slot] != nxt:
                self._start_gather(nxt)

    def _reduce_to_shard(self, flat: torch.Tensor, numel: int) -> torch.Tensor:
        """Average of ``flat[:numel]`` over the ranks, this rank's slice, fp32."""
        per = numel // self.world
        if self.world == 1:
            return flat[:numel].float()
        if flat.is_cuda:
            out = torch.empty(per, dtype=flat.dtype, device=flat.device)
            td.reduce_scatter_tensor(out, flat[:numel], op=td.ReduceOp.AVG, group=self.group)
            return out.float()
        buf = flat[:numel].float()  # gloo: no reduce-scatter, and sums in fp32 rather than bf16
        td.all_reduce(buf, group=self.group)
        return buf[self.rank * per:(self.rank + 1) * per] / self.world

    def _flush_layer(self, ls: _LayerShard):
        if self.fused and ls.grad_acc.dtype == torch.float32:
            from ..ops import cuda as K

            k, per = self._cur, ls.numel // self.world
            self._rstream.wait_event(torch.cuda.current_stream().record_event())  # the layer's gradients are in the buffer
            with torch.cuda.stream(self._rstream):
                K.rs_reduce_accum(self.arena, self._gbufs[k][1], True, self.rank * per, per, ls.grad_acc, self._sq_scratch,
                                  self._rs_sync, max_ctas=self._reduce_ctas)
                self._gbuf_done[k] = self._rstream.record_event()
            self._n_flush += 1
        else:
            ls.grad_acc.add_(self._reduce_to_shard(self.gbuf, ls.numel).to(ls.grad_acc.dtype))
        ls.arrived = 0
        self._pending = None

    def _next_gbuf(self):
        """Fused path: the gradient buffer of the layer whose first gradient has just arrived.  Its previous contents
        (three reductions ago) may be overwritten once this rank's reduction of two layers ago has run: that kernel's
        entry barrier is passed only after every rank has finished the reduction before it."""
        k = self._n_flush % 3
        ev = self._gbuf_done[(k + 1) % 3]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        self._cur, self.gbuf = k, self._gbufs[k][0]

    def _install_hooks(self):
        for ls in self.layers:
            self._hooks.append(ls.module.register_forward_pre_hook(lambda mod, args, i=ls.idx: self.materialize(i)))
            n_params = len(ls.params)
            for p, o in zip(ls.params, ls.offsets):
                def hook(param, ls=ls, o=o, n_params=n_params):
                    pend = getattr(self, "_pending", None)
                    if pend is not None and pend is not ls:
                        self._flush_layer(pend)  # the previous layer had parameters without a gradient
                    if ls.arrived == 0:
                        if self.fused:
                            self._next_gbuf()
                        self.gbuf[:ls.numel].zero_()  # padding and parameters without a gradient contribute zero
                        self._pending = ls
                    self.gbuf[o:o + param.numel()].copy_(param.grad.reshape(-1))
                    param.grad = None
                    ls.arrived += 1
                    if ls.arrived == n_params:
                        self._flush_layer(ls)

                self._hooks.append(p.register_post_accumulate_grad_hook(hook))
        for p, o in zip(self.rest_params, self.rest_offsets):
            def rhook(param, o=o):
                self.rest_grad[o:o + param.numel()].add_(param.grad.reshape(-1))
                param.grad = None

            self._hooks.append(p.register_post_accumulate_grad_hook(rhook))

    # ---- step API (same surface as TrainEngine) ----------------------------------------------------------------------
    def zero_grad(self):
        for ls in self.layers:
            ls.grad_acc.zero_()
            ls.arrived = 0
        self.rest_grad.zero_()

    def backward(self, loss: torch.Tensor):
        if not getattr(self.model, "gradient_checkpointing", False) or getattr(self.model, "checkpoint_num_layers", None):
            raise RuntimeError("the streamed full-shard engine overwrites layer weights between forward and backward: "
                               "enable activation checkpointing for all layers (gradient_checkpointing=True)")
        self.align_ranks()
        loss.backward()
        for ls in self.layers:  # a layer some of whose parameters got no gradient never reached its count
            if ls.arrived:
                self._flush_layer(ls)

    def _adamw(self, master, grad, m, v, shadow, lr, scale, no_decay, lo):
        b1, b2 = self.betas
        if self.weight_decay and no_decay:
            mask = torch.ones_like(master)
            for a, b in no_decay:
                a2, b2_ = max(a, lo) - lo, min(b, lo + master.numel()) - lo
                if b2_ > a2:
                    mask[a2:b2_] = 0
            g = grad * scale
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
            master.mul_(1 - lr * self.weight_decay * mask)
            master.addcdiv_(m / bc1, (v / bc2).sqrt().add_(self.eps), value=-lr)
            if shadow is not None:
                shadow.copy_(master)
        else:
            adamw_flat(master, grad, m, v, self.step_count, lr, b1, b2, self.eps,
                       self.weight_decay if not no_decay else 0.0, scale, shadow)

    def align_ranks(self):
        """Fused path: the per-layer reductions wait at most a second for a peer; ranks that start a step seconds apart
        (an online trainer whose completions differ in length) meet here first, through the backend."""
        if self.fused and not self.frozen:
            td.all_reduce(self._tick, group=self.group)

    def _join_side_streams(self):
        for slot in (0, 1):
            self._wait_slot(slot)
        if self.fused and not self.frozen:
            torch.cuda.current_stream().wait_stream(self._rstream)

    def step(self, lr: float, max_grad_norm: float | None = None) -> torch.Tensor:
        self.step_count += 1
        # fused path: nothing of this rank still reads a peer's slices or adds into an accumulator when the norm
        # all-reduce below runs, and no rank updates its slices before every rank has passed that all-reduce
        self._join_side_streams()
        rest_g = self._reduce_to_shard(self.rest_grad, self.rest_numel) if self.rest_numel else None
        sq = torch.zeros((), dtype=torch.float32, device=self.dev)
        from .engine import _sumsq

        for ls in self.layers:
            sq += _sumsq(ls.grad_acc)
        if rest_g is not None:
            sq += _sumsq(rest_g)
        if self.world > 1:
            td.all_reduce(sq, group=self.group)
        norm = sq.sqrt()
        scale = 1.0
        if max_grad_norm is not None and max_grad_norm > 0:
            scale = torch.clamp(max_grad_norm / (norm + 1e-6), max=1.0)
        for ls in self.layers:
            per = ls.numel // self.world
            g = ls.grad_acc if ls.grad_acc.dtype == torch.float32 else ls.grad_acc.float()
            self._adamw(ls.master, g, ls.exp_avg, ls.exp_avg_sq, ls.shard16 if self.fused else None, lr, scale,
                        ls.no_decay, self.rank * per)
        if rest_g is not None:
            sh = self.rest_flat[self.rest_lo:self.rest_hi]
            shadow = None if self.dtype == torch.float32 else sh
            self._adamw(self.rest_master, rest_g, self.rest_exp_avg, self.rest_exp_avg_sq, shadow, lr, scale,
                        self.rest_no_decay, self.rest_lo)
            self._gather_into(self.rest_flat, sh.clone())
        elif self.fused:
            td.all_reduce(sq, group=self.group)  # closing fence: every rank's new slices are written before anyone pulls
        self._invalidate()
        return norm

    # ---- checkpoints ---------------------------------------------------------------------------------------------
    def optimizer_state_dict(self) -> dict:
        return {"step": self.step_count, "mode": self.mode, "world": self.world, "rank": self.rank,
                "layers": [{"master": l.master.cpu(), "exp_avg": l.exp_avg.cpu(), "exp_avg_sq": l.exp_avg_sq.cpu()}
                           for l in self.layers],
                "rest": {"master": self.rest_master.cpu(), "exp_avg": self.rest_exp_avg.cpu(),
                         "exp_avg_sq": self.rest_exp_avg_sq.cpu()}}

    def load_optimizer_state_dict(self, sd: dict):
        if sd.get("world") != self.world or sd.get("mode") != self.mode:
            raise ValueError("optimizer state was saved by a different engine mode or world size")
        self.step_count = sd["step"]
        for l, s in zip(self.layers, sd["layers"]):
            l.master.copy_(s["master"])
            l.exp_avg.copy_(s["exp_avg"])
            l.exp_avg_sq.copy_(s["exp_avg_sq"])
        self.rest_master.copy_(sd["rest"]["master"])
        self.rest_exp_avg.copy_(sd["rest"]["exp_avg"])
        self.rest_exp_avg_sq.copy_(sd["rest"]["exp_avg_sq"])
        self._publish_rest()
        self._publish_shards()
        self._invalidate()

    @torch.no_grad()
    def load_optimizer_state_resharded(self, shards: list[dict]):
        """Elastic resume from the per-rank files of a streamed run with another world size: slices are concatenated
        in rank order and cut again (layer lengths differ only in their zero padding)."""
        shards = sorted(shards, key=lambda s: s.get("rank", 0))
        if any(s.get("mode") != self.mode for s in shards) or len(shards) != shards[0].get("world"):
            raise ValueError("need the optimizer files of every rank of a streamed full-shard run")
        self.step_count = shards[0]["step"]

        def recut(parts, numel, lo, hi, dst):
            full = torch.cat([p.reshape(-1).float() for p in parts])
            buf = torch.zeros(numel, dtype=torch.float32)
            n = min(full.numel(), numel)
            buf[:n] = full[:n]
            dst.copy_(buf[lo:hi].to(dst.dtype))

        for i, l in enumerate(self.layers):
            per = l.numel // self.world
            for k, dst in (("master", l.master), ("exp_avg", l.exp_avg), ("exp_avg_sq", l.exp_avg_sq)):
                recut([s["layers"][i][k] for s in shards], l.numel, self.rank * per, (self.rank + 1) * per, dst)
        for k, dst in (("master", self.rest_master), ("exp_avg", self.rest_exp_avg), ("exp_avg_sq", self.rest_exp_avg_sq)):
            recut([s["rest"][k] for s in shards], self.rest_numel, self.rest_lo, self.rest_hi, dst)
        self._publish_rest()
        self._publish_shards()
        self._invalidate()

    def _publish_shards(self):
        """Fused path: the fp32 slices were replaced outside the optimizer step (checkpoint load): refresh the bf16
        slices the peers pull from, and make sure nobody pulls before every rank has done so."""
        if not self.fused:
            return
        self._join_side_streams()
        if not self.frozen:
            for ls in self.layers:
                ls.shard16.copy_(ls.master)
        torch.cuda.synchronize(self.dev)
        td.barrier(group=self.group)

    def _publish_rest(self):
        sh = self.rest_flat[self.rest_lo:self.rest_hi]
        if self.rest_master is not sh and self.rest_master.data_ptr() != sh.data_ptr():
            sh.copy_(self.rest_master)
        if self.rest_numel:
            self._gather_into(self.rest_flat, sh.clone())

    def refresh_master_from_params(self):
        """The parameters outside the layers were overwritten in place: take them as the new master values.  Layer
        weights cannot be refreshed this way (their parameters alias the shared slots): use ``load_weights``."""
        self.rest_master.copy_(self.rest_flat[self.rest_lo:self.rest_hi])

    @torch.no_grad()
    def load_weights(self, hf_state: dict, strict: bool = True):
        """Loads a complete checkpoint (HF names): every layer is written into its slot and sliced at once."""
        from ..models.hf_io import load_hf_state_dict

        self._invalidate()  # no gather may still be writing into a slot

        def reslice(i):
            ls = self.layers[i]
            per = ls.numel // self.world
            self._wait_slot(ls.slot)
            ls.master.copy_(self.slots[ls.slot][self.rank * per:(self.rank + 1) * per])
            self._resident[ls.slot] = None

        lm = getattr(self.model, "language_model", self.model)
        load_hf_state_dict(lm, hf_state, strict=strict, after_layer=reslice)
        if not self.frozen:
            self.refresh_master_from_params()
        self._publish_shards()

    @torch.no_grad()
    def export_weights(self, target: nn.Module):
        """Writes the current weights into ``target``, a whole copy of the same architecture (the generation replica
        of the online trainers): layer by layer through the slots (collective), the parameters outside the layers
        directly.  What the reference does with ``ds3_gather_for_generation`` (trl/models/utils.py
        ``unwrap_model_for_generation``), without ever holding a second full copy on the training side."""
        t_layers = getattr(target, "layers")
        for ls in self.layers:
            self.materialize(ls.idx)
            tgt = dict(t_layers[ls.idx].named_parameters())
            for n, p in zip(ls.names, ls.params):
                tgt[n].data.copy_(p.data)
        named = dict(target.named_parameters())
        for n, p in zip(self.rest_names, self.rest_params):
            if n in named and named[n].data_ptr() != p.data_ptr():
                named[n].data.copy_(p.data)

    @torch.no_grad()
    def streamed_hf_state_dict(self, to_cpu: bool = True) -> dict:
        """Complete checkpoint tensors, built one layer at a time (collective).  With ``to_cpu`` every layer is copied
        to host memory before its slot is reused; ranks that do not save pass False and get an empty dict."""
        from ..models.hf_io import to_hf_state_dict

        lm = getattr(self.model, "language_model", self.model)
        return to_hf_state_dict(lm, before_layer=self.materialize, copy_to="cpu" if to_cpu else None)

    def grad_tensors(self):
        return [l.grad_acc for l in self.layers] + [self.rest_grad]
