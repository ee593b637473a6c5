"""Trainer -> generator weight sync straight from parameter shards.

With the full-shard engine a rank holds valid data only for its slice of every layer bucket, and a tensor-parallel
rollout rank needs other slices: rows of the QKV and gate/up matrices, columns of the O and down matrices.  Instead
of completing every bucket first (an all-gather of the whole model) and then slicing locally, the resharder builds,
once, the list of contiguous ranges each TP weight buffer is made of, resolves every range to the rank that owns it
and its address in that rank's mapping of the symmetric parameter arena, and a single kernel (``trlb_copy_list``)
pulls exactly the bytes this rank needs: 1/tp of the model instead of all of it.

When the rollout engine keeps its slices tile-major (the fused tensor-parallel decode path) the pull goes layer by
layer into one layer-sized row-major staging set, and each matrix is re-tiled from there into the engine's buffer:
a 128-byte tile row is too small a unit for a copy list (60 M entries for a 7 B model).

The reference moves weights to its generator with per-parameter ``full_tensor()`` gathers and NCCL broadcasts
(trl/generation/vllm_generation.py:400-470, trl/generation/vllm_client.py:481-512)."""
from __future__ import annotations

import numpy as np
import torch


class WeightResharder:
    def __init__(self, engine, tp_engine):
        """engine: FullShardEngine of the policy; tp_engine: TPRolloutEngine built on the same model."""
        from ..ops.cuda import lib  # noqa: F401  (fails early when the kernel library is missing)

        self.engine, self.tp = engine, tp_engine
        arena = engine._arenas["param"]
        cfg, r, tp = tp_engine.cfg, tp_engine.tp_rank, tp_engine.tp
        if cfg.is_moe:
            raise NotImplementedError("full shard -> tensor-parallel copy lists for expert weights (gather the "
                                      "parameters and call the engine's sync_weights instead)")
        D, I, H = cfg.head_dim, cfg.intermediate_size, cfg.hidden_size
        qs, ks = cfg.q_size, cfg.kv_size
        ql, kl, il = tp_engine.hq_local * D, tp_engine.hk_local * D, I // tp
        by_name = {b.name: b for b in engine.buckets}
        entries: list[tuple[int, int, int]] = []
        self.tiled = bool(getattr(tp_engine, "fused", False))
        dt, dev = torch.bfloat16, tp_engine.dev
        self.stage = ({"qkv": torch.empty(ql + 2 * kl, H, dtype=dt, device=dev), "o": torch.empty(H, ql, dtype=dt, device=dev),
                       "gu": torch.empty(2 * il, H, dtype=dt, device=dev), "down": torch.empty(H, il, dtype=dt, device=dev)}
                      if self.tiled else None)
        self.layer_ranges: list[tuple[int, int]] = []

        def add(bucket, elem_off, n_elems, dst_ptr):
            """[elem_off, elem_off + n) of the bucket -> dst; split at ownership boundaries."""
            key = ("param", bucket.name, str(bucket.params[0].dtype))
            base = engine._offsets[key]
            per = bucket.numel // engine.world
            while n_elems > 0:
                owner = elem_off // per
                n = min(n_elems, (owner + 1) * per - elem_off)
                src = arena.peer_ptrs[owner] + base + elem_off * 2
                if src % 16 or dst_ptr % 16 or (n * 2) % 16:
                    raise ValueError("weight slices must be 16-byte aligned for the reshard copy")
                entries.append((src, dst_ptr, n * 2))
                elem_off, n_elems, dst_ptr = elem_off + n, n_elems - n, dst_ptr + n * 2

        for i, w in enumerate(tp_engine.w):
            first = len(entries)
            if self.tiled:
                w = self.stage
            b = by_name[f"layers.{i}"]
            off = {n.split(".")[-1]: o for n, o in zip(b.names, b.offsets)}
            # row slices: contiguous
            o = 0
            for start, n in ((r * ql, ql), (qs + r * kl, kl), (qs + ks + r * kl, kl)):
                add(b, off["qkv_proj"] + start * H, n * H, w["qkv"].data_ptr() + o * H * 2)
                o += n
            add(b, off["gate_up_proj"] + r * il * H, il * H, w["gu"].data_ptr())
            add(b, off["gate_up_proj"] + (I + r * il) * H, il * H, w["gu"].data_ptr() + il * H * 2)
            # column slices: one range per row
            for row in range(H):
                add(b, off["o_proj"] + row * qs + r * ql, ql, w["o"].data_ptr() + row * ql * 2)
                add(b, off["down_proj"] + row * I + r * il, il, w["down"].data_ptr() + row * il * 2)
            self.layer_ranges.append((first, len(entries)))
        self.n = len(entries)
        self.bytes = sum(e[2] for e in entries)
        self.table = torch.from_numpy(np.asarray(entries, dtype=np.uint64).reshape(-1, 3).view(np.int64).copy()).to(tp_engine.dev)
        self._bias = cfg.attention_bias

    @torch.no_grad()
    def run(self):
        """Pull this rank's TP slices from their owners.  Call after the optimizer step (the engine's step ends with a
        cross-rank barrier, so every owner's slice is final)."""
        from ctypes import c_int

        from ..ops.cuda import _chk, _p, _s, lib

        if self.tiled:
            from ..ops import cuda as K

            ql, kl, il = self.tp._dims
            H = self.tp.cfg.hidden_size
            kb_h = -(-H // 64)
            for (a, b), w in zip(self.layer_ranges, self.tp.w):
                _chk(lib().trlb_copy_list(_p(self.table[a:]), c_int(b - a), _s()), "copy_list")
                # pieces are whole 128-row slabs (the fused path requires it), so they tile independently
                o = 0
                for n in (ql, kl, kl):
                    K.tile_weights(self.stage["qkv"][o:o + n], out=w["qkv"][o * kb_h * 64:(o + n) * kb_h * 64])
                    o += n
                K.tile_weights(self.stage["o"], out=w["o"])
                K.tile_weights(self.stage["gu"][:il], out=w["gu"][: il * kb_h * 64])
                K.tile_weights(self.stage["gu"][il:], out=w["gu"][il * kb_h * 64:])
                K.tile_weights(self.stage["down"], out=w["down"])
        else:
            _chk(lib().trlb_copy_list(_p(self.table), c_int(self.n), _s()), "copy_list")
        if self._bias:  # biases live in the replicated vector bucket: slice locally
            tp = self.tp
            D = tp.cfg.head_dim
            qs, ks = tp.cfg.q_size, tp.cfg.kv_size
            ql, kl = tp.hq_local * D, tp.hk_local * D
            for l, w in zip(tp.model.layers, tp.w):
                o = 0
                for start, n in ((tp.tp_rank * ql, ql), (qs + tp.tp_rank * kl, kl), (qs + ks + tp.tp_rank * kl, kl)):
                    w["qkv_b"][o:o + n].copy_(l.qkv_bias[start:start + n])
                    o += n
