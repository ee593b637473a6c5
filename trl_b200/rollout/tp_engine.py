"""Tensor-parallel rollout engine (decode split over the ranks of a TP group).

Layout per rank r of tp: attention heads [r*Hq/tp, (r+1)*Hq/tp) with their KV heads (the paged cache holds
local heads only), MLP columns [r*I/tp, (r+1)*I/tp); embeddings, norms and the lm_head are replicated.

Fused path (``TRL_B200_TP_FUSED=1``; batches of at most 128 rows, 128-row-aligned slices): every decode linear is the
weight-streaming tcgen05 GEMM on tile-major weight slices (the repack that tensor parallelism needs anyway writes
them tile-major, so each 16 KB weight tile is one sequential DRAM burst).  The two row-parallel GEMMs of a layer
(O-proj, down-proj) are fused with their all-reduce: the stream-K partial sums meet in a local staging buffer and
the warp that completes a 32-feature quarter of a slab adds it once into the accumulator of EVERY rank over NVLink
(16-byte vector red.global on peer pointers) and bumps an arrival counter on every rank; the consumer
(residual add + RMSNorm) waits on its own counter, reads one local buffer and clears it.  No rank reads a peer's
memory, no separate all-reduce kernel runs and no barrier has two directions: a rank only ever waits for "all
partial sums have landed here".  Accumulator reuse needs no extra handshake: a peer can reach the next GEMM on the
same accumulator only after it has consumed this rank's partial sums of the GEMM in between, which this rank
launched after clearing the accumulator.  Partial sums arrive in no fixed order, so the ranks' logits may differ
in the last bit; rank 0's sampled tokens are therefore copied to the other ranks (one small message per step).

Default path (also for shapes outside the fused kernels): library GEMMs write bf16 partials into symmetric memory
and ONE kernel, ``allreduce_add_rmsnorm``, sums them over peer loads behind a two-sided barrier, adds the residual
and normalises.  It is the default because it is the faster one at the batch a tensor-parallel group decodes (the
rows of all its ranks, 128 at the benchmark's 64 per GPU): timed on one B200 with the per-rank shapes of TP=2 and 128
rows, the four GEMMs of the 28 layers take 1.58 ms through the library against 4.70 ms through the fused path (row-
parallel O-proj 56 us against 11 us, down-proj 73 us against 27 us: at this batch the fp32 partial sums of the stream-K
split are as many bytes as the weights, and the staging, counting and hand-over of each quarter is a serial tail;
the SwiGLU GEMM cannot split K and fills only 74 of 148 SMs).  At 64 rows and TP=1, where the stream-K kernels
equal the library, they are the default (``rollout/engine.py``).

Weight "sync": under the zero modes every rank already holds the full bf16 parameters, so the TP layout is a
local repack (``sync_weights``); under full-shard the buckets are first completed with the ``shard_allgather``
kernel.  Prompts of the group's ranks are gathered so all ranks run the same batch; each rank keeps its own
completions (vllm_generation.py:636-699 does the same around vLLM's TP workers).
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as td

from ..parallel.symm import SymmArena, SyncWords
from .engine import Completion, RolloutEngine
from .sampling import SamplingParams


class TPRolloutEngine(RolloutEngine):
    def __init__(self, model, tp_group, max_num_seqs: int = 64, max_model_len: int = 2048, **kw):
        self.group = tp_group
        tp, tp_rank = td.get_world_size(tp_group), td.get_rank(tp_group)
        super().__init__(model, max_num_seqs=max_num_seqs * tp, max_model_len=max_model_len, tp=tp, tp_rank=tp_rank, **kw)
        cfg, dev, dt = self.cfg, self.dev, torch.bfloat16
        if self.max_seqs > 148:
            raise ValueError("TP decode batch (max_num_seqs * tp) is limited to 148 rows per step")
        # mixture-of-experts layers: every rank keeps 1 / tp of every expert's intermediate dimension (router replicated),
        # so the block's output is a partial sum like a dense MLP's and rides on the same all-reduce
        H, D, I = cfg.hidden_size, cfg.head_dim, (cfg.moe_intermediate_size if cfg.is_moe else cfg.intermediate_size)
        if I % tp or (cfg.is_moe and (I // tp) % 8):
            raise ValueError(f"tensor parallel size {tp} must divide the MLP width {I} (in multiples of 8 for experts)")
        ql, kl, il = self.hq_local * D, self.hk_local * D, I // tp
        self._dims = (ql, kl, il)
        self.fused = (os.environ.get("TRL_B200_TP_FUSED", "0") == "1" and not cfg.is_moe and self.max_seqs <= 128 and H <= 8192 and H % 8 == 0
                      and D <= 128 and ql % 128 == 0 and kl % 128 == 0 and il % 128 == 0 and tp <= 8)
        self._pdl = os.environ.get("TRL_B200_PDL", "1") == "1"
        self.w = []
        if self.fused:
            from ..ops import cuda as K

            L_ = K.lib()
            L_.trlb_tiled_elems.restype = __import__("ctypes").c_longlong
            n_el = lambda rows, k: int(L_.trlb_tiled_elems(rows, k))
            for _ in cfg_layers(cfg):
                self.w.append({
                    "qkv": torch.empty(n_el(ql + 2 * kl, H), dtype=dt, device=dev),
                    "qkv_b": torch.empty(ql + 2 * kl, dtype=dt, device=dev) if cfg.attention_bias else None,
                    "o": torch.empty(n_el(H, ql), dtype=dt, device=dev),
                    "gu": torch.empty(n_el(2 * il, H), dtype=dt, device=dev),
                    "down": torch.empty(n_el(H, il), dtype=dt, device=dev),
                })
            B = self.max_seqs
            # symmetric: two fp32 accumulators [B, H], two arrival counters, a token mailbox and its flag
            acc_bytes = B * H * 4
            self.arena = SymmArena(2 * acc_bytes + 4096 + 2 * B * 4 + 1024, dev, tp_group)
            self._acc_o, self._acc_o_off = self.arena.carve(B * H, torch.float32)
            self._acc_d, self._acc_d_off = self.arena.carve(B * H, torch.float32)
            self._acc_o, self._acc_d = self._acc_o.view(B, H), self._acc_d.view(B, H)
            self._ctr, self._ctr_off = self.arena.carve(64, torch.int32)   # [0] O-proj arrivals, [16] down-proj arrivals
            self._mail, self._mail_off = self.arena.carve(2 * B, torch.int32)
            self._flag, self._flag_off = self.arena.carve(64, torch.int32)
            peers = [p for p in range(tp) if p != tp_rank]
            base = self.arena.peer_ptrs
            self._peer_acc_o = [base[p] + self._acc_o_off for p in peers]
            self._peer_acc_d = [base[p] + self._acc_d_off for p in peers]
            self._arrive_o = [base[tp_rank] + self._ctr_off] + [base[p] + self._ctr_off for p in peers]
            self._arrive_d = [base[tp_rank] + self._ctr_off + 64] + [base[p] + self._ctr_off + 64 for p in peers]
            self._mail_ptrs = [base[p] + self._mail_off for p in range(tp)]
            self._flag_ptrs = [base[p] + self._flag_off for p in range(tp)]
            self._local = torch.zeros(16, dtype=torch.int32, device=dev)  # [0] done word O, [4] done word down, [8] epoch
            self._acc_qkv = torch.zeros(B, ql + 2 * kl, dtype=torch.float32, device=dev)
            self._act_buf = torch.empty(B, il, dtype=dt, device=dev)
            self._logits_buf = torch.empty(B, cfg.vocab_size, dtype=dt, device=dev)
            self._stage = torch.zeros(B, H, dtype=torch.float32, device=dev)  # both GEMMs: they never overlap
            self._slab_ctr = torch.zeros(4 * (-(-H // 128)), dtype=torch.int32, device=dev)
            self._target_o = self._target_d = tp * K.decode_gemm_arrivals(H)
        else:
            for _ in cfg_layers(cfg):
                self.w.append({
                    "qkv": torch.empty(ql + 2 * kl, H, dtype=dt, device=dev),
                    "qkv_b": torch.empty(ql + 2 * kl, dtype=dt, device=dev) if cfg.attention_bias else None,
                    "o": torch.empty(H, ql, dtype=dt, device=dev),
                    "gu": torch.empty(*((cfg.num_experts,) if cfg.is_moe else ()), 2 * il, H, dtype=dt, device=dev),
                    "down": torch.empty(*((cfg.num_experts,) if cfg.is_moe else ()), H, il, dtype=dt, device=dev),
                })
            self.n_sites = 2 * cfg.num_hidden_layers
            self.site_elems = self.max_seqs * H
            self.arena = SymmArena(self.n_sites * self.site_elems * 2 + 4096, dev, tp_group)
            self.partials, self.partials_off = self.arena.carve(self.n_sites * self.site_elems, dt)
            self.sync = SyncWords(dev, channel=1)
        self.sync_weights()

    @torch.no_grad()
    def sync_weights(self, model=None):
        cfg, r, tp = self.cfg, self.tp_rank, self.tp
        D, I, H = cfg.head_dim, cfg.intermediate_size, cfg.hidden_size
        qs, ks = cfg.q_size, cfg.kv_size
        ql, kl, il = self._dims
        if self.fused:
            from ..ops import cuda as K

            kb_h = -(-H // 64)
            tile = 128 * 64
            for l, w in zip(self.model.layers, self.w):
                # every piece is a whole number of 128-row slabs, so it lands at a slab boundary of the tiled buffer
                o = 0
                for start, n in ((r * ql, ql), (qs + r * kl, kl), (qs + ks + r * kl, kl)):
                    K.tile_weights(l.qkv_proj[start:start + n], out=w["qkv"][o * kb_h * 64:(o + n) * kb_h * 64])
                    if w["qkv_b"] is not None:
                        w["qkv_b"][o:o + n].copy_(l.qkv_bias[start:start + n])
                    o += n
                K.tile_weights(l.o_proj[:, r * ql:(r + 1) * ql], out=w["o"])
                K.tile_weights(l.gate_up_proj[r * il:(r + 1) * il], out=w["gu"][: il * kb_h * 64])
                K.tile_weights(l.gate_up_proj[I + r * il:I + (r + 1) * il], out=w["gu"][il * kb_h * 64:])
                K.tile_weights(l.down_proj[:, r * il:(r + 1) * il], out=w["down"])
            return
        for l, w in zip(self.model.layers, self.w):
            rows = [(0 + r * ql, ql), (qs + r * kl, kl), (qs + ks + r * kl, kl)]
            o = 0
            for start, n in rows:
                w["qkv"][o:o + n].copy_(l.qkv_proj[start:start + n])
                if w["qkv_b"] is not None:
                    w["qkv_b"][o:o + n].copy_(l.qkv_bias[start:start + n])
                o += n
            w["o"].copy_(l.o_proj[:, r * ql:(r + 1) * ql])
            if cfg.is_moe:
                Im = cfg.moe_intermediate_size
                w["gu"][:, :il].copy_(l.experts_gate_up[:, r * il:(r + 1) * il])
                w["gu"][:, il:].copy_(l.experts_gate_up[:, Im + r * il:Im + (r + 1) * il])
                w["down"].copy_(l.experts_down[:, :, r * il:(r + 1) * il])
                continue
            w["gu"][:il].copy_(l.gate_up_proj[r * il:(r + 1) * il])
            w["gu"][il:].copy_(l.gate_up_proj[I + r * il:I + (r + 1) * il])
            w["down"].copy_(l.down_proj[:, r * il:(r + 1) * il])

    def _site(self, i: int) -> torch.Tensor:
        return self.partials[i * self.site_elems:(i + 1) * self.site_elems].view(self.max_seqs, self.cfg.hidden_size)

    def _decode_step(self, sp: SamplingParams, max_total_len: int):
        from ..ops import cuda as K

        if self.fused:
            was = K.set_pdl(self._pdl)
            try:
                logits = self._decode_layers_fused()
            finally:
                K.set_pdl(was)
            self._sample(logits, sp)
            # the ranks' logits can differ in the last bit (partial sums arrive in no fixed order): rank 0 decides
            K.tp_token_sync(self._mail_ptrs, self._flag_ptrs, self.tp_rank, self.tp, self.tok, self.logp, self._local[8:9])
        else:
            self._sample(self._decode_layers_legacy(), sp)
        K.advance(self.tok, self.logp, None, self.seq_lens, self.n_gen, self.finished, self.out_tokens, self.out_logps,
                  sp.eos_token_id, max_total_len, self.next_input, self.step_counter, 1)
        if self.seen is not None:
            self.seen.scatter_(1, self.next_input[:, None], 1)

    def _decode_layers_fused(self):
        from ..ops import cuda as K

        cfg, m = self.cfg, self.model
        eps, scale = cfg.rms_norm_eps, 1.0 / math.sqrt(cfg.head_dim)
        H = cfg.hidden_size
        ql, kl, il = self._dims
        x = torch.nn.functional.embedding(self.next_input, m.embed_tokens)
        loc = self._local.data_ptr()
        for li, (l, w) in enumerate(zip(m.layers, self.w)):
            if li == 0:
                h = K.rmsnorm_infer(x, l.input_layernorm, eps)
            else:
                h = K.add_rmsnorm_f32_wait(x, self._acc_d, l.input_layernorm, eps, self._arrive_d[0], self._target_d, loc + 16)
            K.decode_gemm(h, w["qkv"], y32=self._acc_qkv, tiled_shape=(ql + 2 * kl, H))
            K.rope_kv_write_f32(self._acc_qkv, w["qkv_b"], l.q_norm if cfg.qk_norm else None,
                                l.k_norm if cfg.qk_norm else None, eps, self.seq_lens, None, self.block_table,
                                self.block_size, self.q_buf, self.k_cache[li], self.v_cache[li], self.hq_local,
                                self.hk_local, cfg.head_dim, cfg.rope_theta, v_transposed=self.attn_tc, pos_delta=self.rope_delta)
            self._decode_attention(li, scale)
            K.decode_gemm(self.attn_buf.view(self.max_seqs, -1), w["o"], y32=self._acc_o, tiled_shape=(H, ql),
                          peers=(self._peer_acc_o, self._arrive_o, self._stage, self._slab_ctr))
            h = K.add_rmsnorm_f32_wait(x, self._acc_o, l.post_attention_layernorm, eps, self._arrive_o[0], self._target_o, loc)
            act = K.decode_gemm(h, w["gu"], out=self._act_buf, swiglu=True, tiled_shape=(2 * il, H))
            K.decode_gemm(act, w["down"], y32=self._acc_d, tiled_shape=(H, il), peers=(self._peer_acc_d, self._arrive_d, self._stage, self._slab_ctr))
        hN = K.add_rmsnorm_f32_wait(x, self._acc_d, m.norm, eps, self._arrive_d[0], self._target_d, loc + 16)
        return K.decode_gemm(hN, m.lm_head_weight, out=self._logits_buf)

    def _decode_layers_legacy(self):
        from ..ops import cuda as K

        cfg, m, F = self.cfg, self.model, torch.nn.functional
        eps, scale = cfg.rms_norm_eps, 1.0 / math.sqrt(cfg.head_dim)
        x = F.embedding(self.next_input, m.embed_tokens)
        site = 0
        h = None
        for li, (l, w) in enumerate(zip(m.layers, self.w)):
            if li == 0:
                h = K.rmsnorm_infer(x, l.input_layernorm, eps)
            else:
                h = K.allreduce_add_rmsnorm(self.arena, self.partials_off + (site - 1) * self.site_elems * 2, 0, x,
                                            l.input_layernorm, eps, self.sync)
            qkv = F.linear(h, w["qkv"], w["qkv_b"])
            if cfg.qk_norm:  # per-head RMSNorm of this rank's q and k heads (Qwen3 families)
                ql, kl, _ = self._dims
                qn = K.rmsnorm_infer(qkv[:, :ql].reshape(-1, cfg.head_dim).contiguous(), l.q_norm, eps)
                kn = K.rmsnorm_infer(qkv[:, ql:ql + kl].reshape(-1, cfg.head_dim).contiguous(), l.k_norm, eps)
                qkv = torch.cat([qn.view(-1, ql), kn.view(-1, kl), qkv[:, ql + kl:]], dim=1)
            K.rope_kv_write(qkv, self.seq_lens, None, self.block_table, self.block_size, self.q_buf, self.k_cache[li],
                            self.v_cache[li], self.hq_local, self.hk_local, cfg.head_dim, cfg.rope_theta,
                            v_transposed=self.attn_tc, pos_delta=self.rope_delta)
            self._decode_attention(li, scale)
            torch.matmul(self.attn_buf.view(self.max_seqs, -1), w["o"].t(), out=self._site(site))
            h = K.allreduce_add_rmsnorm(self.arena, self.partials_off + site * self.site_elems * 2, 0, x,
                                        l.post_attention_layernorm, eps, self.sync)
            site += 1
            if cfg.is_moe:
                from ..ops import functional as F_

                y, _, _ = F_.moe_mlp(h, l.router, w["gu"], w["down"], cfg.num_experts_per_tok, cfg.norm_topk_prob)
                self._site(site).copy_(y)
            else:
                gu = F.linear(h, w["gu"])
                torch.matmul(K.swiglu_infer(gu), w["down"].t(), out=self._site(site))
            site += 1
        hN = K.allreduce_add_rmsnorm(self.arena, self.partials_off + (site - 1) * self.site_elems * 2, 0, x, m.norm, eps,
                                     self.sync)
        return F.linear(hN, m.lm_head_weight)

    @torch.no_grad()
    def generate(self, prompts, sp: SamplingParams, images=None) -> list[Completion]:
        """Every rank passes its own prompts; the group runs the union; each rank gets its own completions."""
        if images is not None:
            raise NotImplementedError("tensor-parallel generation with image prompts")
        gathered = [None] * self.tp
        td.all_gather_object(gathered, [list(p) for p in prompts], group=self.group)
        counts = [len(g) for g in gathered]
        allp = [p for g in gathered for p in g]
        sp_group = SamplingParams(**{**sp.__dict__, "seed": sp.seed - self.tp_rank * 0})
        seed = [sp.seed]
        td.broadcast_object_list(seed, src=td.get_global_rank(self.group, 0), group=self.group)
        sp_group.seed = seed[0]
        outs = super().generate(allp, sp_group)
        start = sum(counts[:self.tp_rank]) * sp.n
        return outs[start:start + counts[self.tp_rank] * sp.n]


def cfg_layers(cfg):
    return range(cfg.num_hidden_layers)
