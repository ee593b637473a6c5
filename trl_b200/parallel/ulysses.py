"""Ulysses sequence parallelism for long packed sequences.

The ranks of a sequence-parallel group hold consecutive chunks of the packed token stream.  Everything that is
token-local (embeddings, norms, projections, MLP, lm_head, loss) runs on the local chunk.  Attention needs whole
sequences, so around it the layout is transposed with one all-to-all each way:

    [T/sp tokens, H heads, D]  --all-to-all-->  [T tokens, H/sp heads, D]  --attention-->  ... back

(heads are independent, so each rank attends over the full sequences for its share of the heads).  KV heads are
repeated first when there are fewer of them than ranks.  The collectives are differentiable
(``torch.distributed.nn.functional``), so the same code serves forward and backward.

The reference reaches this through DeepSpeed ALST behind accelerate's ``ParallelismConfig(sp_backend="deepspeed")``
(docs/source/distributing_training.md:236-330, examples/accelerate_configs/alst_ulysses_4gpu.yaml); its trainer only
consumes pre-shifted ``shift_labels`` (trl/trainer/sft_trainer.py:139-142)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as td


@dataclass
class SpInfo:
    group: Any
    size: int
    rank: int
    mode: str = "ulysses"  # "ulysses": heads are exchanged; "allgather_kv": context parallel (context_parallel.py)


def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(x)
    if torch.is_grad_enabled() and x.requires_grad:
        import torch.distributed.nn.functional as dfn

        return dfn.all_to_all_single(out, x, group=group)
    td.all_to_all_single(out, x, group=group)
    return out


def seq_to_head(x: torch.Tensor, sp: SpInfo) -> torch.Tensor:
    """[T/sp, H, D] (my tokens, all heads) -> [T, H/sp, D] (all tokens, my heads)."""
    Tl, H, D = x.shape
    hs = H // sp.size
    x = x.reshape(Tl, sp.size, hs, D).permute(1, 0, 2, 3).contiguous()  # [dest rank, Tl, hs, D]
    y = _a2a(x, sp.group)                                               # [source rank, Tl, hs, D]
    return y.reshape(sp.size * Tl, hs, D)


def head_to_seq(x: torch.Tensor, sp: SpInfo) -> torch.Tensor:
    """[T, H/sp, D] -> [T/sp, H, D]."""
    T, hs, D = x.shape
    Tl = T // sp.size
    y = _a2a(x.reshape(sp.size, Tl, hs, D).contiguous(), sp.group)      # [source head group, Tl, hs, D]
    return y.permute(1, 0, 2, 3).reshape(Tl, sp.size * hs, D)


def attention(q, k, v, ctx, attend):
    """q [T/sp, Hq, D], k / v [T/sp, Hk, D] of the local chunk; ``attend(q, k, v)`` runs varlen attention on full
    sequences (global ``cu_seqlens``).  Returns [T/sp, Hq, D]."""
    sp = ctx.sp
    Hq, Hk = q.shape[1], k.shape[1]
    if Hq % sp.size:
        raise ValueError(f"sequence parallel size {sp.size} must divide the number of attention heads ({Hq})")
    if Hk % sp.size:  # fewer KV heads than ranks (or not divisible): repeat them up to the query heads' grouping
        rep = sp.size // Hk if sp.size % Hk == 0 else Hq // Hk
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    o = attend(seq_to_head(q, sp), seq_to_head(k, sp), seq_to_head(v, sp))
    return head_to_seq(o, sp)


def shard_sequence(flat: torch.Tensor, targets: torch.Tensor, ctx, sp: SpInfo, pad_id: int = 0):
    """Pads the packed stream to a multiple of sp (the pad tokens form one extra document without labels) and returns
    this rank's chunk: (ids, targets, ctx with local positions and global sequence geometry)."""
    from ..models.decoder import SeqCtx

    T = flat.numel()
    pad = (-T) % sp.size
    pos, cu, mx = ctx.positions, ctx.cu_seqlens, ctx.max_seqlen
    if pad:
        flat = torch.cat([flat, flat.new_full((pad,), pad_id)])
        targets = torch.cat([targets, targets.new_full((pad,), -100)])
        pos = torch.cat([pos, torch.arange(pad, device=pos.device, dtype=pos.dtype)])
        cu = torch.cat([cu, cu.new_tensor([T + pad])])
        mx = max(mx, pad)
    Tl = (T + pad) // sp.size
    sl = slice(sp.rank * Tl, (sp.rank + 1) * Tl)
    local = SeqCtx(pos[sl].contiguous(), cu, mx)
    local.sp = sp
    return flat[sl].contiguous(), targets[sl].contiguous(), local
