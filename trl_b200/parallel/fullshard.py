"""Full-shard (ZeRO-3 / FSDP) engine on the flat buckets.

Between uses a bucket is only valid in the slice its rank owns.  The missing parts arrive

* for decoder layers: inside the layer's QKV GEMM (``trlb_ag_gemm_bf16_tn``): copier CTAs of that kernel pull the
  whole layer bucket from the peers while the tensor-core CTAs start on locally owned weight tiles, so when the
  GEMM returns the O / gate-up / down weights of the layer are in place too (forward and the recompute in backward);
* for the embedding, final norm and lm_head buckets: ``shard_allgather`` right after the optimizer step.

Gradients accumulate locally over the micro-batches and are reduce-scattered by ``rs_reduce`` at the step; AdamW then
updates only the owned slice (no parameter broadcast: the next use gathers).  The reference gets this behaviour from
DeepSpeed ZeRO-3 / torch FSDP with per-layer NCCL all-gather + reduce-scatter (trl/accelerate_configs/zero3.yaml,
fsdp2.yaml).

Memory note: every bucket keeps a full-size symmetric buffer here (what is sharded is validity and optimizer state,
as well as all communication volume); rotating two layer-sized buffers instead is a local change in ``_alloc``.
"""
from __future__ import annotations

import os

import torch

from .engine import TrainEngine, default_bucket_of

_VECTOR_PARAMS = ("input_layernorm", "post_attention_layernorm", "qkv_bias", "q_norm", "k_norm")


def fullshard_bucket_of(name: str) -> str:
    """Per-layer buckets hold the matrices; the layers' norm weights and biases share one small bucket that is
    completed right after the optimizer step, because the input norm and the QKV bias are read before (or while)
    the layer's gather runs."""
    parts = name.split(".")
    if parts[0] == "layers" and parts[-1] in _VECTOR_PARAMS:
        return "layer_vectors"
    return default_bucket_of(name)


class _AgLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, gather):
        from ..ops.cuda_comm import ag_gemm

        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if gather.fresh:  # later micro-batches and the recompute in backward: the buffer is still complete
            y = x2 @ weight.t()
        else:
            if gather.align is not None:  # ranks may come out of a generation phase seconds apart
                gather.align()
            y = ag_gemm(x2, gather.arena, gather.byte_offset, gather.per, gather.total, gather.w_off, weight.shape[0],
                        gather.state, bias=None)
            gather.fresh = True
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.shape = x.shape
        return y.view(x.shape[:-1] + (weight.shape[0],))

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = (dy2 @ weight).view(ctx.shape) if ctx.needs_input_grad[0] else None
        dw = dy2.t() @ x2 if ctx.needs_input_grad[1] else None
        db = dy2.sum(0) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, None


class LayerGather:
    """What a decoder layer needs to run its QKV GEMM as an all-gather-fused GEMM."""

    def __init__(self, arena, byte_offset, per, total, w_off, device, copiers, align=None):
        from ..ops.cuda_comm import AgGemmState

        self.align = align  # called before the first gather after an optimizer step (only layer 0 has one)
        self.arena, self.byte_offset, self.per, self.total, self.w_off = arena, byte_offset, per, total, w_off
        self.state = AgGemmState(device, copiers=copiers)
        self.fresh = False  # True from the first gather after an optimizer step until the next step

    def qkv(self, x, weight, bias):
        # one autograd node on both paths (gathering or not), so activation checkpointing sees the same graph
        y = _AgLinearFn.apply(x, weight, None, self)
        return y if bias is None else y + bias  # the bias lives in the vector bucket, complete since the last step


class FullShardEngine(TrainEngine):
    def __init__(self, model, *, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, grad_dtype=None,
                 copiers: int | None = None, group=None):
        super().__init__(model, mode="full_shard", betas=betas, eps=eps, weight_decay=weight_decay,
                         grad_dtype=grad_dtype, use_symm_kernels=True, group=group, bucket_of=fullshard_bucket_of)
        self.poison = os.environ.get("TRL_B200_FULLSHARD_POISON", "0") == "1"
        if copiers is None:
            # CTAs of the QKV GEMM that only pull peers' shards: enough of them to keep NVLink busy, growing with the
            # remote fraction of the bucket (7/8 at 8 ranks)
            copiers = int(os.environ.get("TRL_B200_AG_COPIERS", "0")) or min(64, max(32, 6 * self.world))
        self._layer_buckets, self._other_buckets = [], []
        by_name = {b.name: b for b in self.buckets}
        for i, layer in enumerate(getattr(model, "layers", [])):
            b = by_name.get(f"layers.{i}")
            if b is None or b.flat_param.dtype != torch.bfloat16:
                continue
            qname = f"layers.{i}.qkv_proj"
            if qname not in b.names:
                continue
            w_off = b.offsets[b.names.index(qname)]
            key = ("param", b.name, str(b.params[0].dtype))
            layer._shard_gather = LayerGather(self._arenas["param"], self._offsets[key], b.hi - b.lo, b.numel, w_off,
                                              b.flat_param.device, copiers, align=self.align_ranks if i == 0 else None)
            self._layer_buckets.append(b)
        self._other_buckets = [b for b in self.buckets if b not in self._layer_buckets]
        model._trl_b200_engine = self
        self._after_update()

    def _after_update(self):
        """Non-layer buckets are completed right away; layer buckets stay sharded until their QKV GEMM."""
        from ..ops import cuda as K

        pa = self._arenas["param"]
        for b in self._other_buckets:
            key = ("param", b.name, str(b.params[0].dtype))
            if b.flat_param.dtype == torch.bfloat16:
                K.shard_allgather(pa, self._offsets[key], b.hi - b.lo, self._sync, use_multimem=False)
            else:
                torch.distributed.all_gather_into_tensor(b.flat_param, b.flat_param[b.lo:b.hi].clone(), group=self.group)
        for layer in getattr(self.model, "layers", []):
            if getattr(layer, "_shard_gather", None) is not None:
                layer._shard_gather.fresh = False
        if self.poison:  # prove that nothing reads a stale remote slice
            for b in self._layer_buckets:
                b.flat_param[:b.lo].fill_(float("nan"))  # the owned slice is never touched: peers may be reading it
                b.flat_param[b.hi:].fill_(float("nan"))

    def gather_full_params(self):
        """Complete every bucket (checkpoint save, rollout engines that read the weights directly)."""
        from ..ops import cuda as K

        pa = self._arenas["param"]
        for b in self._layer_buckets:
            key = ("param", b.name, str(b.params[0].dtype))
            K.shard_allgather(pa, self._offsets[key], b.hi - b.lo, self._sync, use_multimem=False)
        for layer in getattr(self.model, "layers", []):
            if getattr(layer, "_shard_gather", None) is not None:
                layer._shard_gather.fresh = True

    def _step_fused(self, lr, max_grad_norm):
        from ..ops import cuda as K

        self.align_ranks()
        ga = self._arenas["grad"]
        self._sumsq.zero_()
        for b, red in zip(self.buckets, self._reduced):
            key = (b.name, str(b.params[0].dtype))
            K.rs_reduce(ga, self._offsets[("grad",) + key], b.flat_grad.dtype == torch.bfloat16, b.lo, b.hi - b.lo, red,
                        self._sumsq, self._sync, use_multimem=self.use_multimem)
        K.norm_allreduce(ga, self._norm_off, self._sumsq, max_grad_norm or 0.0, self._norm, self._clip, self._sync)
        b1, b2 = self.betas
        for b, red in zip(self.buckets, self._reduced):
            shadow = b.flat_param[b.lo:b.hi] if b.flat_param.dtype != torch.float32 else None
            wd = 0.0 if all(p.ndim <= 1 for p in b.params) else self.weight_decay  # vectors: no decay
            K.adamw_flat(b.master, red, b.exp_avg, b.exp_avg_sq, self.step_count, lr, b1, b2, self.eps, wd,
                         self._clip, shadow)
        # every rank's owned slices are final before anybody gathers them
        K.norm_allreduce(ga, self._norm_off, self._sumsq, 0.0, self._norm_scratch(), self._clip_scratch(), self._sync)
        self._after_update()
        return self._norm[0].clone()

    def _norm_scratch(self):
        if not hasattr(self, "_ns"):
            self._ns = torch.zeros(1, dtype=torch.float32, device=self._norm.device)
            self._cs = torch.zeros(1, dtype=torch.float32, device=self._norm.device)
        return self._ns

    def _clip_scratch(self):
        self._norm_scratch()
        return self._cs
