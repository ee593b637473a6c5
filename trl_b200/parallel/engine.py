"""Flat-bucket training engine: gradient reduction + sharded AdamW.

One bucket per decoder layer (plus embeddings / head).  A bucket owns

* ``flat_param``  - the compute copy (bf16 on GPUs, fp32 on CPU); every
  ``nn.Parameter`` of the bucket is a view into it,
* ``flat_grad``   - the accumulation buffer (fp32 "main grads" by default),
* an fp32 ``master / exp_avg / exp_avg_sq`` triple for the slice this rank owns.

Modes (they replace the reference's accelerate profiles, trl/accelerate_configs/*.yaml):

``ddp``        gradients all-reduced, optimizer state replicated.
``zero1/2``    gradients reduce-scattered, optimizer state sharded, updated
               parameters all-gathered (ZeRO-1/2; the two differ only in when
               the full gradient buffer is released, which flat buckets make moot).
``full_shard`` parameters live as 1/world shards between uses; see
               :mod:`trl_b200.parallel.fullshard`, which reuses the buckets below.

Expert-parallel parameters (flagged ``_ep_local`` by ``parallel.expert_parallel.shard_experts``) differ between the
ranks by construction: they go to *local* buckets whose gradients are not reduced (the dispatch already brought every
rank's tokens to the expert; the gradient is scaled by 1 / world like the averaged ones), whose optimizer state is
whole on the owner, and whose squared norm enters the global gradient norm once.

On GPUs the reduce-scatter, the fp32 cast/scale, the norm partials and the
AdamW update are the ``rs_adamw`` kernels over symmetric memory
(:mod:`trl_b200.parallel.symm`); the NCCL calls below are the measured baseline
and the gloo/CPU path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as td
import torch.nn as nn

from . import dist as D


def adamw_flat(*a, **k):  # imported on use: loop/ imports this module
    from ..loop.optim import adamw_flat as f

    return f(*a, **k)

_ALIGN = 256  # elements; keeps every shard 16-byte aligned for TMA / vector access


def _sumsq(g: torch.Tensor) -> torch.Tensor:
    """Sum of squares of a flat gradient as a 0-dim fp32 tensor: one read of the buffer on GPUs (the eager
    ``float().pow(2).sum()`` writes and re-reads an fp32 temporary of the same size)."""
    if g.is_cuda and g.dtype in (torch.float32, torch.bfloat16) and g.is_contiguous():
        from ..ops.cuda import sumsq

        return sumsq(g)[0]
    return g.float().pow(2).sum()


@dataclass
class Bucket:
    name: str
    names: list[str]
    params: list[nn.Parameter]
    offsets: list[int]
    numel: int  # padded to world * _ALIGN
    flat_param: torch.Tensor = None
    flat_grad: torch.Tensor = None
    decay_mask: torch.Tensor | None = None  # None => uniform decay
    lo: int = 0
    hi: int = 0
    master: torch.Tensor = None
    exp_avg: torch.Tensor = None
    exp_avg_sq: torch.Tensor = None
    no_decay_ranges: list = field(default_factory=list)
    local: bool = False  # expert-parallel parameters: owned whole by this rank, never reduced or gathered

    def shard(self, t: torch.Tensor) -> torch.Tensor:
        return t[self.lo:self.hi]


def _merge_ranges(ranges, limit: int = 16):
    """Adjacent exempt ranges (a layer's norm weights and biases often touch) merged; the fused kernel takes up to
    ``limit``."""
    out = []
    for lo, hi in sorted(ranges):
        if out and lo <= out[-1][1]:
            out[-1] = (out[-1][0], max(out[-1][1], hi))
        else:
            out.append((lo, hi))
    if len(out) > limit:
        raise ValueError(f"{len(out)} separate no-decay ranges in one bucket; the fused optimizer kernel takes {limit}")
    return out


def default_bucket_of(name: str) -> str:
    parts = name.split(".")
    if parts[0] == "layers":
        return f"layers.{parts[1]}"
    return parts[0]


class TrainEngine:
    def __init__(self, model: nn.Module, *, mode: str = "ddp", betas=(0.9, 0.999), eps=1e-8,
                 weight_decay: float = 0.0, grad_dtype: torch.dtype | None = None, bucket_of=default_bucket_of,
                 use_symm_kernels: bool | None = None, group=None, optimizer_factory=None):
        """``optimizer_factory(param_groups) -> torch.optim.Optimizer``: another update rule than the built-in AdamW.
        It is given two groups of fp32 tensors (decayed / exempt from decay: slices of this rank's master copy) and
        runs on the backend path (no fused comm kernels); the engine still does reduction, clipping, the bf16 refresh
        and the gathers."""
        self.model = model
        self.optimizer_factory = optimizer_factory
        self.custom_opt = None
        self.world, self.rank = D.world_size(), D.rank()
        self.group = group
        self.mode = "ddp" if (mode in ("auto", None) or self.world == 1 and mode != "full_shard") else mode
        if mode == "auto" and self.world > 1:
            self.mode = "zero2"
        self.betas, self.eps, self.weight_decay = betas, eps, weight_decay
        self.step_count = 0
        self.sharded = self.mode in ("zero1", "zero2", "full_shard") and self.world > 1
        first = next((p for p in model.parameters() if p.requires_grad), None)
        on_gpu = first is not None and first.is_cuda
        if use_symm_kernels is None:
            from .symm import symmetric_available
            import os

            use_symm_kernels = (self.sharded and on_gpu and first.dtype == torch.bfloat16 and symmetric_available()
                                and os.environ.get("TRL_B200_NCCL_OPTIMIZER", "0") != "1")
        if optimizer_factory is not None:
            use_symm_kernels = False
        self.use_symm = bool(use_symm_kernels)
        self.use_multimem = False
        self._arenas = {}
        self._build_buckets(bucket_of, grad_dtype)
        if self.use_symm:
            from .symm import SyncWords

            dev = self.buckets[0].flat_param.device
            self._sync = SyncWords(dev, channel=0)
            self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
            self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
            self._clip = torch.ones(1, dtype=torch.float32, device=dev)
            self._reduced = [torch.empty(b.hi - b.lo, dtype=torch.float32, device=dev) for b in self.buckets]
            import os

            self.use_multimem = bool(self._arenas["param"].multicast_ptr) and os.environ.get("TRL_B200_MULTIMEM", "1") == "1"
        self._hooks = []
        # a model that an earlier engine has wrapped (one trainer after another on the same object): that engine's
        # gradient hooks would fire next to this one's and hand it an already consumed gradient
        prev = getattr(model, "_trlb_engine_ref", None)
        prev = prev() if prev is not None else None
        if prev is not None and prev is not self and hasattr(prev, "release_hooks"):
            prev.release_hooks()
        import weakref

        try:
            model._trlb_engine_ref = weakref.ref(self)
        except Exception:  # noqa: BLE001  (objects without attribute storage)
            pass
        self._install_grad_views()

    @torch.no_grad()
    def sync_master_from_params(self):
        """After weights were written into the parameters from outside (a checkpoint loaded in place): refresh this
        rank's fp32 master slices so that the next optimizer step starts from them."""
        for b in self.buckets:
            if b.master.data_ptr() != b.flat_param[b.lo:b.hi].data_ptr():
                b.master.copy_(b.flat_param[b.lo:b.hi])

    def release_hooks(self):
        """Detaches this engine's gradient hooks from the parameters (the buffers stay valid)."""
        for h in self._hooks:
            h.remove()
        self._hooks = []

    # ---- construction ---------------------------------------------------------
    def _build_buckets(self, bucket_of, grad_dtype):
        groups: dict[str, list] = {}
        seen = set()
        for n, p in self.model.named_parameters():
            if not p.requires_grad or id(p) in seen:
                continue
            seen.add(id(p))
            bname = bucket_of(n) + (".ep" if getattr(p, "_ep_local", False) else "")
            groups.setdefault((bname, p.dtype), []).append((n, p))
        is_local = {key: all(getattr(p, "_ep_local", False) for _, p in items) for key, items in groups.items()}
        self.buckets: list[Bucket] = []
        unit = self.world * _ALIGN
        if self.use_symm:
            # one symmetric arena for all parameter buckets and one for all gradient buckets:
            # a single rendezvous each, peer address = peer base + the bucket's byte offset
            from .symm import SymmArena

            gd0 = grad_dtype or torch.float32
            tot_p = tot_g = 0
            for (bn, dtype), items in groups.items():
                if is_local[(bn, dtype)]:
                    continue
                cur = sum((p.numel() + 15) // 16 * 16 for _, p in items)
                numel = (cur + unit - 1) // unit * unit
                tot_p += numel * torch.empty(0, dtype=dtype).element_size() + 256
                tot_g += numel * torch.empty(0, dtype=gd0).element_size() + 256
            dev0 = next(iter(groups.values()))[0][1].device
            self._arenas["param"] = SymmArena(tot_p, dev0, self.group)
            self._arenas["grad"] = SymmArena(tot_g + 4096, dev0, self.group)
            self._norm_slots, self._norm_off = self._arenas["grad"].carve(64, torch.float32)
        self._offsets = {}
        for (bname, dtype), items in groups.items():
            offs, cur = [], 0
            for _, p in items:
                offs.append(cur)
                cur += (p.numel() + 15) // 16 * 16
            numel = (cur + unit - 1) // unit * unit
            dev = items[0][1].device
            b = Bucket(bname, [n for n, _ in items], [p for _, p in items], offs, numel, local=is_local[(bname, dtype)])
            b.flat_param = self._alloc("param", b, numel, dtype, dev)
            for (n, p), o in zip(items, offs):
                b.flat_param[o:o + p.numel()].view_as(p).copy_(p.data)
                p.data = b.flat_param[o:o + p.numel()].view_as(p)
                if p.ndim <= 1:  # biases and norm weights: no weight decay (HF convention)
                    b.no_decay_ranges.append((o, o + p.numel()))
            gd = grad_dtype or torch.float32
            b.flat_grad = self._alloc("grad", b, numel, gd, dev)
            if self.sharded and not b.local:
                per = numel // self.world
                b.lo, b.hi = self.rank * per, (self.rank + 1) * per
            else:
                b.lo, b.hi = 0, numel
            n_sh = b.hi - b.lo
            if dtype == torch.float32:
                b.master = b.flat_param[b.lo:b.hi]  # alias: fp32 params are their own master
            else:
                b.master = b.flat_param[b.lo:b.hi].float()
            b.exp_avg = torch.zeros(n_sh, dtype=torch.float32, device=dev)
            b.exp_avg_sq = torch.zeros(n_sh, dtype=torch.float32, device=dev)
            if self.weight_decay and b.no_decay_ranges:
                mask = torch.ones(numel, dtype=torch.float32, device=dev)
                for lo, hi in b.no_decay_ranges:
                    mask[lo:hi] = 0
                b.decay_mask = mask[b.lo:b.hi].contiguous()
            self.buckets.append(b)

    def _alloc(self, kind, bucket, numel, dtype, dev):
        if not self.use_symm or bucket.local:
            return torch.zeros(numel, dtype=dtype, device=dev)
        t, off = self._arenas[kind].carve(numel, dtype)
        self._offsets[(kind, bucket.name, str(bucket.params[0].dtype))] = off
        return t

    def _install_grad_views(self):
        for b in self.buckets:
            same = b.flat_grad.dtype == b.flat_param.dtype
            for p, o in zip(b.params, b.offsets):
                gview = b.flat_grad[o:o + p.numel()].view_as(p)
                if same:
                    p.grad = gview
                else:
                    p.grad = None

                    def hook(param, gview=gview):
                        g = param.grad
                        if (g.is_cuda and g.dtype == torch.bfloat16 and gview.dtype == torch.float32 and g.is_contiguous()
                                and g.data_ptr() % 16 == 0 and gview.data_ptr() % 16 == 0):
                            from ..ops.cuda import accum_grad  # one vectorised pass instead of a mixed-dtype add

                            accum_grad(gview, g)
                        else:
                            gview.add_(g)
                        param.grad = None

                    self._hooks.append(p.register_post_accumulate_grad_hook(hook))

    # ---- step API ---------------------------------------------------------------
    def zero_grad(self):
        for b in self.buckets:
            b.flat_grad.zero_()
            if b.flat_grad.dtype == b.flat_param.dtype:
                for p, o in zip(b.params, b.offsets):
                    if p.grad is None or p.grad.data_ptr() != b.flat_grad[o:o + 1].data_ptr():
                        p.grad = b.flat_grad[o:o + p.numel()].view_as(p)

    def backward(self, loss: torch.Tensor):
        loss.backward()

    def _reduce(self, b: Bucket) -> torch.Tensor:
        """Average gradients over ranks; returns this rank's (shard of the) reduced gradient."""
        if self.world == 1:
            return b.flat_grad
        if b.local:  # every rank's tokens already reached the expert: only the 1 / world of the averaged objective
            b.flat_grad /= self.world
            return b.flat_grad
        if self.sharded:
            out = torch.empty(b.hi - b.lo, dtype=b.flat_grad.dtype, device=b.flat_grad.device)
            if b.flat_grad.is_cuda:
                td.reduce_scatter_tensor(out, b.flat_grad, op=td.ReduceOp.AVG, group=self.group)
            else:  # gloo has no reduce_scatter: all-reduce then slice
                td.all_reduce(b.flat_grad, group=self.group)
                out = b.flat_grad[b.lo:b.hi] / self.world
            return out
        td.all_reduce(b.flat_grad, group=self.group)
        b.flat_grad /= self.world
        return b.flat_grad

    def step(self, lr: float, max_grad_norm: float | None = None) -> torch.Tensor:
        """Reduce, clip by global norm, AdamW, refresh the compute copy.  Returns the pre-clip norm."""
        self.step_count += 1
        if self.use_symm:
            return self._step_fused(lr, max_grad_norm)
        reduced = [self._reduce(b) for b in self.buckets]
        sq = torch.zeros((), dtype=torch.float32, device=reduced[0].device)
        sq_local = torch.zeros_like(sq)  # parts every rank holds a different piece of: shards, expert-parallel buckets
        for b, g in zip(self.buckets, reduced):
            part = _sumsq(g)
            if self.sharded or (b.local and self.world > 1):
                sq_local += part
            else:
                sq += part
        if self.sharded or any(b.local for b in self.buckets) and self.world > 1:
            D.all_reduce(sq_local, "sum", group=self.group)
        sq = sq + sq_local
        norm = sq.sqrt()
        scale = 1.0
        if max_grad_norm is not None and max_grad_norm > 0:
            scale = torch.clamp(max_grad_norm / (norm + 1e-6), max=1.0)
        if self.optimizer_factory is not None:
            self._custom_step(reduced, lr, scale)
            return norm
        b1, b2 = self.betas
        for b, g in zip(self.buckets, reduced):
            shadow = None if b.flat_param.dtype == torch.float32 else b.flat_param[b.lo:b.hi]
            gs = scale  # python float or 0-dim tensor (stays on device: no host sync)
            if b.decay_mask is None:  # uniform decay over the bucket (or none at all)
                adamw_flat(b.master, g, b.exp_avg, b.exp_avg_sq, self.step_count, lr, b1, b2, self.eps,
                           self.weight_decay, gs, shadow)
            else:  # biases / norm weights inside the bucket are exempt from decay
                self._masked_adamw(b, g, lr, gs, shadow)
            if self.sharded and not b.local:
                td.all_gather_into_tensor(b.flat_param, b.flat_param[b.lo:b.hi].clone(), group=self.group)
        return norm

    # ---- an update rule of the caller's ----------------------------------------------------------------------------
    def _custom_params(self):
        """Leaf tensors over this rank's master slices, one per (parameter, slice) piece, split by decay exemption."""
        decay, exempt, self._custom_views = [], [], []
        for b in self.buckets:
            cuts = sorted({b.lo, b.hi, *[x for r in b.no_decay_ranges for x in r if b.lo < x < b.hi]})
            for lo, hi in zip(cuts[:-1], cuts[1:]):
                is_exempt = any(r0 <= lo and hi <= r1 for r0, r1 in b.no_decay_ranges)
                t = torch.nn.Parameter(b.master[lo - b.lo:hi - b.lo], requires_grad=False)
                (exempt if is_exempt else decay).append(t)
                self._custom_views.append((b, lo - b.lo, hi - b.lo, t))
        return [{"params": decay, "weight_decay": self.weight_decay}, {"params": exempt, "weight_decay": 0.0}]

    @torch.no_grad()
    def _custom_step(self, reduced, lr, scale):
        if self.custom_opt is None:
            self.custom_opt = self.optimizer_factory(self._custom_params())
        for g in self.custom_opt.param_groups:
            g["lr"] = lr
        by_bucket = {id(b): g for b, g in zip(self.buckets, reduced)}
        for b, lo, hi, t in self._custom_views:
            t.grad = by_bucket[id(b)][lo:hi] * scale
        self.custom_opt.step()
        for _, _, _, t in self._custom_views:
            t.grad = None
        for b in self.buckets:
            if b.master.data_ptr() != b.flat_param[b.lo:b.hi].data_ptr():
                b.flat_param[b.lo:b.hi].copy_(b.master)
            if self.sharded and not b.local:
                td.all_gather_into_tensor(b.flat_param, b.flat_param[b.lo:b.hi].clone(), group=self.group)

    def align_ranks(self):
        """Stream-ordered meeting of the ranks through the backend (one element).  The cross-rank waits inside the comm
        kernels give up after a second, which is right for a peer that is gone but not for one that is merely late:
        ranks reach an optimizer step seconds apart when their micro-batches differ in length.  After this call they
        are within a launch of each other."""
        if self.world > 1 and self.use_symm:
            if not hasattr(self, "_tick"):
                self._tick = torch.zeros(1, dtype=torch.float32, device=self.buckets[0].flat_param.device)
            td.all_reduce(self._tick, group=self.group)

    def _step_fused(self, lr: float, max_grad_norm: float | None) -> torch.Tensor:
        """Optimizer step on the comm kernels: per bucket a reduce-scatter that reads the peers' gradient
        buffers in place (fp32 cast, 1/world, norm partial), one exchange of the norm partials, then AdamW
        whose bf16 output is stored into every rank's parameter replica.  No host sync; the only library
        collective is the one-element meeting in front (see ``align_ranks``)."""
        from ..ops import cuda as K

        self.align_ranks()
        ga, pa = self._arenas["grad"], self._arenas["param"]
        self._sumsq.zero_()
        for b, red in zip(self.buckets, self._reduced):
            if b.local:  # expert-parallel bucket: scale, add its squared norm to this rank's partial
                red.copy_(b.flat_grad).div_(self.world)
                self._sumsq += _sumsq(red)
                continue
            key = (b.name, str(b.params[0].dtype))
            K.rs_reduce(ga, self._offsets[("grad",) + key], b.flat_grad.dtype == torch.bfloat16, b.lo, b.hi - b.lo, red,
                        self._sumsq, self._sync, use_multimem=self.use_multimem)
        K.norm_allreduce(ga, self._norm_off, self._sumsq, max_grad_norm or 0.0, self._norm, self._clip, self._sync)
        b1, b2 = self.betas
        for b, red in zip(self.buckets, self._reduced):
            if b.local:
                shadow = None if b.flat_param.dtype == torch.float32 else b.flat_param
                if b.decay_mask is None:
                    adamw_flat(b.master, red, b.exp_avg, b.exp_avg_sq, self.step_count, lr, b1, b2, self.eps,
                               self.weight_decay, self._clip[0], shadow)
                else:
                    self._masked_adamw(b, red, lr, self._clip[0], shadow)
                continue
            key = (b.name, str(b.params[0].dtype))
            K.adamw_bcast(pa, self._offsets[("param",) + key], b.lo, b.hi - b.lo, b.master, red, b.exp_avg, b.exp_avg_sq,
                          self.step_count, lr, b1, b2, self.eps, self.weight_decay, self._clip, self._sync,
                          use_multimem=self.use_multimem,
                          no_decay_ranges=_merge_ranges(b.no_decay_ranges) if self.weight_decay else ())
        return self._norm[0].clone()

    @torch.no_grad()
    def comm_selfcheck(self) -> str:
        """Checks the fused collectives against the library ones on live buffers; returns "ok" or what differed.

        (1) the gradient reduce-scatter kernel (peer loads, or multimem.ld_reduce) of the first bucket against an
        NCCL all-reduce of the same rank-dependent values; (2) after the last optimizer step every rank's bf16
        parameter replica must be the same (the AdamW kernel stores its shard into all replicas): compared through
        min / max reductions of per-bucket checksums.  Gradients are zeroed afterwards; call it between steps."""
        if not self.use_symm:
            return "skipped: fused collectives not in use"
        from ..ops import cuda as K

        b = next(bk for bk in self.buckets if not bk.local)
        key = (b.name, str(b.params[0].dtype))
        n = b.flat_grad.numel()
        idx = torch.arange(n, device=b.flat_grad.device, dtype=torch.float32)
        b.flat_grad.copy_((torch.sin(idx * 0.37 + self.rank) * (1.0 + 0.1 * self.rank)).to(b.flat_grad.dtype))
        want = b.flat_grad.float().clone()
        torch.cuda.synchronize()
        td.barrier(group=self.group)
        td.all_reduce(want, group=self.group)
        want = want[b.lo:b.hi] / self.world
        got = torch.empty(b.hi - b.lo, dtype=torch.float32, device=want.device)
        self._sumsq.zero_()
        K.rs_reduce(self._arenas["grad"], self._offsets[("grad",) + key], b.flat_grad.dtype == torch.bfloat16, b.lo,
                    b.hi - b.lo, got, self._sumsq, self._sync, use_multimem=self.use_multimem)
        torch.cuda.synchronize()
        err = (got - want).abs().max()
        sums = torch.stack([bk.flat_param.float().sum() for bk in self.buckets if not bk.local])
        hi_, lo_ = sums.clone(), sums.clone()
        td.all_reduce(hi_, op=td.ReduceOp.MAX, group=self.group)
        td.all_reduce(lo_, op=td.ReduceOp.MIN, group=self.group)
        bad = torch.stack([err > 1e-5, (hi_ != lo_).any()]).float()
        td.all_reduce(bad, op=td.ReduceOp.MAX, group=self.group)
        td.barrier(group=self.group)
        self.zero_grad()
        if bad[0] > 0:
            return f"reduce-scatter differs from the library all-reduce (max abs error {float(err):.3e} on this rank)"
        if bad[1] > 0:
            return "parameter replicas differ between ranks after the fused AdamW"
        return "ok"

    def _masked_adamw(self, b: Bucket, g, lr, gs, shadow):
        b1, b2 = self.betas
        before = b.master.clone()
        adamw_flat(b.master, g, b.exp_avg, b.exp_avg_sq, self.step_count, lr, b1, b2, self.eps, 0.0, gs, None)
        b.master.sub_(before * b.decay_mask * (lr * self.weight_decay))
        if shadow is not None:
            shadow.copy_(b.master)

    @property
    def per_rank_state(self) -> bool:
        """Whether every rank has optimizer state of its own to save (shards, or expert-parallel buckets)."""
        return self.sharded or (self.world > 1 and any(b.local for b in self.buckets))

    # ---- (de)serialisation of optimizer state -------------------------------------
    def optimizer_state_dict(self) -> dict:
        if self.custom_opt is not None:  # the caller's rule: its own state, keyed by the order of the master pieces
            return {"step": self.step_count, "mode": self.mode, "world": self.world, "rank": self.rank,
                    "custom": self.custom_opt.state_dict(),
                    "masters": {b.name + "|" + str(b.flat_param.dtype): b.master.detach().cpu().clone() for b in self.buckets}}
        return {
            "step": self.step_count, "mode": self.mode, "world": self.world, "rank": self.rank,
            "buckets": {b.name + "|" + str(b.flat_param.dtype): {
                "names": b.names, "lo": b.lo, "hi": b.hi, "local": b.local,
                "master": b.master.detach().cpu().clone(), "exp_avg": b.exp_avg.cpu(), "exp_avg_sq": b.exp_avg_sq.cpu()}
                for b in self.buckets},
        }

    def load_optimizer_state_dict(self, sd: dict):
        self.step_count = sd["step"]
        if "custom" in sd:
            if self.optimizer_factory is None:
                raise ValueError("the checkpoint holds the state of a custom optimizer; pass the same optimizer again")
            for b in self.buckets:
                b.master.copy_(sd["masters"][b.name + "|" + str(b.flat_param.dtype)])
            if self.custom_opt is None:
                self.custom_opt = self.optimizer_factory(self._custom_params())
            self.custom_opt.load_state_dict(sd["custom"])
            return
        for b in self.buckets:
            s = sd["buckets"][b.name + "|" + str(b.flat_param.dtype)]
            if (s["lo"], s["hi"]) != (b.lo, b.hi):
                raise ValueError("optimizer shard layout changed (world size differs from the checkpoint)")
            b.master.copy_(s["master"])
            b.exp_avg.copy_(s["exp_avg"])
            b.exp_avg_sq.copy_(s["exp_avg_sq"])

    @torch.no_grad()
    def load_optimizer_state_resharded(self, shards: list[dict]):
        """Elastic resume: ``shards`` are the optimizer files of ALL ranks of the run that saved (one file for a
        replicated run).  Every bucket is put back together in slice order and cut again for this run's world size
        and mode; bucket lengths differ only in their zero padding (a multiple of world * 256 elements)."""
        self.step_count = shards[0]["step"]
        for b in self.buckets:
            key = b.name + "|" + str(b.flat_param.dtype)
            if any(key not in s["buckets"] for s in shards):
                raise ValueError(f"the checkpoint's optimizer state has no bucket {key!r}: it was written by an engine with "
                                 f"another bucket layout (mode {shards[0].get('mode')!r}, this run {self.mode!r})")
            if b.local:
                # expert-parallel buckets are whole on their owner: they survive a change of shard mode, not of world size
                mine = [s for s in shards if s.get("rank") == self.rank and s.get("world") == self.world]
                if len(mine) != 1:
                    raise ValueError("expert-parallel optimizer state can only be resumed with the same number of ranks")
                for k, dst in (("master", b.master), ("exp_avg", b.exp_avg), ("exp_avg_sq", b.exp_avg_sq)):
                    dst.copy_(mine[0]["buckets"][key][k].to(dst.dtype))
                if b.master.data_ptr() != b.flat_param.data_ptr():
                    b.flat_param.copy_(b.master.to(b.flat_param.dtype))
                continue
            parts = sorted((s["buckets"][key] for s in shards), key=lambda x: x["lo"])
            if parts[0]["names"] != b.names:
                raise ValueError(f"bucket {b.name}: the checkpoint holds other parameters ({parts[0]['names'][:3]}...)")
            for k, dst in (("master", b.master), ("exp_avg", b.exp_avg), ("exp_avg_sq", b.exp_avg_sq)):
                full = torch.cat([p[k].reshape(-1).float() for p in parts])
                buf = torch.zeros(b.numel, dtype=torch.float32)
                n = min(full.numel(), b.numel)
                buf[:n] = full[:n]
                dst.copy_(buf[b.lo:b.hi].to(dst.dtype))
            if b.master.data_ptr() != b.flat_param[b.lo:b.hi].data_ptr():
                b.flat_param[b.lo:b.hi].copy_(b.master.to(b.flat_param.dtype))

    @torch.no_grad()
    def refresh_master_from_params(self):
        """Re-derive the fp32 master shard after weights were loaded into the compute copy."""
        for b in self.buckets:
            if b.master.data_ptr() != b.flat_param[b.lo:b.hi].data_ptr():
                b.master.copy_(b.flat_param[b.lo:b.hi])

    def grad_tensors(self):
        return [b.flat_grad for b in self.buckets]
