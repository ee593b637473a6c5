"""Context parallelism for long packed sequences: local queries against gathered keys / values.

The ranks of a context-parallel group hold consecutive equal chunks of the packed token stream (the same sharding as
the Ulysses path, ``ulysses.shard_sequence``).  Token-local work runs on the chunk.  For attention every rank
all-gathers K and V of the group (with grouped-query models these are the small tensors: 2 * Hk * D per token against
Hq * D for the queries) and attends with its own queries over the part of the gathered stream it needs: the packed
documents that overlap its chunk, from the start of the first one to the end of the chunk.  The causal mask is aligned
to the end of each key segment, so a query chunk that is the tail of a document sees the whole prefix.  Unlike
Ulysses there is no limit from the head count, and the query / output tensors never move.

The all-gather is one differentiable collective (backward: reduce-scatter of dK / dV), so the same code serves
forward, backward and checkpoint recompute.  Work per rank grows with the rank's position inside a long document
(contiguous chunks, no zig-zag reordering); with many packed documents per stream the imbalance stays small.

The reference reaches context parallelism through accelerate's ``ParallelismConfig(cp_size=...)`` and torch's ring
attention for SDPA (docs/source/distributing_training.md:160-232); the trainer side there only shards the batch
along the sequence (trl/trainer/sft_trainer.py:139-142 consumes pre-shifted labels).
"""
from __future__ import annotations

import torch
import torch.distributed as td


class _GatherTokens(torch.autograd.Function):
    """[Tl, ...] on every rank -> [size * Tl, ...] in rank order; backward sums the ranks' gradients per chunk."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.contiguous()
        n = td.get_world_size(group)
        out = x.new_empty((n * x.shape[0],) + tuple(x.shape[1:]))
        td.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        group = ctx.group
        n, r = td.get_world_size(group), td.get_rank(group)
        g = g.contiguous()
        tl = g.shape[0] // n
        if td.get_backend(group) == "nccl":
            out = g.new_empty((tl,) + tuple(g.shape[1:]))
            td.reduce_scatter_tensor(out, g, group=group)
            return out, None
        td.all_reduce(g, group=group)  # backends without reduce-scatter
        return g[r * tl:(r + 1) * tl].clone(), None


def plan(ctx):
    """Host-side geometry of this rank's chunk, computed once per forward and kept on ``ctx`` (one device-to-host
    read of the document boundaries): the slice of the gathered stream to attend over and the query / key segment
    boundaries inside it."""
    cached = getattr(ctx, "_cp_plan", None)
    if cached is not None:
        return cached
    sp = ctx.sp
    cu = [int(c) for c in ctx.cu_seqlens.tolist()]
    total = cu[-1]
    tl = total // sp.size
    a, b = sp.rank * tl, (sp.rank + 1) * tl
    cuts = [a] + [c for c in cu if a < c < b] + [b]
    s0 = max(c for c in cu if c <= a)  # start of the document the chunk begins in
    cu_q = [c - a for c in cuts]
    cu_k = [0] + [c - s0 for c in cuts[1:]]
    dev = ctx.cu_seqlens.device
    out = {
        "k_start": s0, "k_end": b,
        "cu_q": torch.tensor(cu_q, dtype=torch.int32, device=dev),
        "cu_k": torch.tensor(cu_k, dtype=torch.int32, device=dev),
        "max_q": max(y - x for x, y in zip(cu_q, cu_q[1:])),
        "max_k": max(y - x for x, y in zip(cu_k, cu_k[1:])),
    }
    ctx._cp_plan = out
    return out


def attention(q, k, v, ctx, attend):
    """q [T/cp, Hq, D], k / v [T/cp, Hk, D] of the local chunk.  ``attend(q, k, v, cu_q, cu_k, max_q, max_k)`` runs
    causal varlen attention whose mask is aligned to the end of every key segment.  Returns [T/cp, Hq, D]."""
    p = plan(ctx)
    kv = _GatherTokens.apply(torch.stack([k, v], dim=1), ctx.sp.group)  # [T, 2, Hk, D]
    kv = kv[p["k_start"]:p["k_end"]]
    return attend(q, kv[:, 0], kv[:, 1], p["cu_q"], p["cu_k"], p["max_q"], p["max_k"])
