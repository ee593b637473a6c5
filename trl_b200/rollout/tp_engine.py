"""Tensor-parallel rollout engine (decode split over the ranks of a TP group).

Layout per rank r of tp: attention heads [r*Hq/tp, (r+1)*Hq/tp) with their KV heads (the paged cache holds
local heads only), MLP columns [r*I/tp, (r+1)*I/tp); embeddings, norms and the lm_head are replicated so that
every rank samples from bit-identical logits with the same counter-based RNG and no token exchange is needed.

Per layer the two row-parallel GEMMs (O-proj, down-proj) write their partial [T, H] outputs into symmetric
memory; the following norm is ``allreduce_add_rmsnorm``: it sums the ranks' partials over NVLink in rank order,
adds the residual and normalises in one kernel.  There are 2L+1 such call sites per step, each with its own
buffer: a buffer is rewritten one full step later, after 2L other cross-rank barriers, so no reader can still
be on it.  The whole step is one CUDA graph per rank.

Weight "sync": under the zero modes every rank already holds the full bf16 parameters, so the TP layout is a
local repack (row/column slices copied into contiguous TP buffers, ``sync_weights``); under full-shard the
buckets are first completed with the ``shard_allgather`` kernel.  Prompts of the group's ranks are gathered so
all ranks run the same batch; each rank keeps its own completions (vllm_generation.py:636-699 does the same
around vLLM's TP workers).
"""
from __future__ import annotations

import math

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
        if cfg.is_moe:
            raise NotImplementedError("TP decode of MoE layers")
        if self.max_seqs > 148:
            raise ValueError("TP decode batch (max_num_seqs * tp) is limited to 148 rows per step")
        H, D, I = cfg.hidden_size, cfg.head_dim, cfg.intermediate_size
        ql, kl, il = self.hq_local * D, self.hk_local * D, I // tp
        self.w = []
        for _ in cfg_layers(cfg):
            self.w.append({
                "qkv": torch.empty(ql + 2 * kl, H, dtype=dt, device=dev),
                "qkv_b": torch.empty(ql + 2 * kl, dtype=dt, device=dev) if cfg.attention_bias else None,
                "o": torch.empty(H, ql, dtype=dt, device=dev),
                "gu": torch.empty(2 * il, H, dtype=dt, device=dev),
                "down": torch.empty(H, il, dtype=dt, device=dev),
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
        D, I = cfg.head_dim, cfg.intermediate_size
        qs, ks = cfg.q_size, cfg.kv_size
        ql, kl, il = self.hq_local * D, self.hk_local * D, I // tp
        for l, w in zip(self.model.layers, self.w):
            rows = [(0 + r * ql, ql), (qs + r * kl, kl), (qs + ks + r * kl, kl)]
            o = 0
            for start, n in rows:
                w["qkv"][o:o + n].copy_(l.qkv_proj[start:start + n])
                if w["qkv_b"] is not None:
                    w["qkv_b"][o:o + n].copy_(l.qkv_bias[start:start + n])
                o += n
            w["o"].copy_(l.o_proj[:, r * ql:(r + 1) * ql])
            w["gu"][:il].copy_(l.gate_up_proj[r * il:(r + 1) * il])
            w["gu"][il:].copy_(l.gate_up_proj[I + r * il:I + (r + 1) * il])
            w["down"].copy_(l.down_proj[:, r * il:(r + 1) * il])

    def _site(self, i: int) -> torch.Tensor:
        return self.partials[i * self.site_elems:(i + 1) * self.site_elems].view(self.max_seqs, self.cfg.hidden_size)

    def _decode_step(self, sp: SamplingParams, max_total_len: int):
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
            K.rope_kv_write(qkv, self.seq_lens, None, self.block_table, self.block_size, self.q_buf, self.k_cache[li],
                            self.v_cache[li], self.hq_local, self.hk_local, cfg.head_dim, cfg.rope_theta,
                            v_transposed=self.attn_tc)
            self._decode_attention(li, scale)
            torch.matmul(self.attn_buf.view(self.max_seqs, -1), w["o"].t(), out=self._site(site))
            h = K.allreduce_add_rmsnorm(self.arena, self.partials_off + site * self.site_elems * 2, 0, x,
                                        l.post_attention_layernorm, eps, self.sync)
            site += 1
            gu = F.linear(h, w["gu"])
            torch.matmul(K.swiglu_infer(gu), w["down"].t(), out=self._site(site))
            site += 1
        hN = K.allreduce_add_rmsnorm(self.arena, self.partials_off + (site - 1) * self.site_elems * 2, 0, x, m.norm, eps,
                                     self.sync)
        logits = F.linear(hN, m.lm_head_weight)
        self._sample(logits, sp)
        K.advance(self.tok, self.logp, None, self.seq_lens, self.n_gen, self.finished, self.out_tokens, self.out_logps,
                  sp.eos_token_id, max_total_len, self.next_input, self.step_counter, 1)
        if self.seen is not None:
            self.seen.scatter_(1, self.next_input[:, None], 1)

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
