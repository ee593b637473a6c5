"""In-box rollout engine: paged KV cache, continuous batching, CUDA-graph decode.

This replaces the reference's vLLM colocate/server modes
(trl/generation/vllm_generation.py:111-704).  One engine lives in each training
process and reads the policy's bf16 weights in place (TP=1: zero-copy "weight
sync"; TP>1: :mod:`trl_b200.rollout.tp` holds resharded copies that the
weight-sync kernel refreshes).

GPU path
    prefill   packed varlen forward of the admitted prompts; K/V written straight into the
              paged cache; completions sampled from one prompt share its full prompt blocks.
    decode    one CUDA graph per engine: embed -> L x (RMSNorm, QKV GEMM, RoPE+KV-append,
              split-KV paged attention, O GEMM, RMSNorm, gate/up GEMM, SwiGLU, down GEMM)
              -> RMSNorm -> lm_head GEMM -> fused sampler -> advance.  No per-step host work:
              the host polls the ``finished`` flags every ``poll_every`` steps.
    scheduler C++ (``csrc/host_runtime.cpp``): waiting queue, slots, ref-counted block pool.

CPU path (tests, tiny models): :class:`EagerGenerator`, same sampling semantics.
"""
from __future__ import annotations

import os
import time

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..models.decoder import CausalLM, SeqCtx
from ..models.vision import merge_vision_entries, vision_entry_numel
from .sampling import SamplingParams, apply_repetition_penalty, filter_top_k_top_p, sample_reference


@dataclass
class Completion:
    prompt_ids: list
    token_ids: list
    logprobs: list
    finish_reason: str = "length"


_KERNEL_SEED = 0x5EED1234


class EagerGenerator:
    """Reference generator: recomputes the full forward every step (fine for tiny CPU models)."""

    def __init__(self, model: CausalLM):
        self.model = model

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sp: SamplingParams, images=None) -> list[Completion]:
        """``images``: per prompt the pixel tensor [n_images, C, S, S] of a vision-language model (or None)."""
        dev = self.model.device
        g = torch.Generator(device="cpu").manual_seed(sp.seed)
        seqs = [list(p) for p in prompts for _ in range(sp.n)]
        pix = None if images is None else [x for x in images for _ in range(sp.n)]
        outs = [Completion(list(s), [], []) for s in seqs]
        alive = list(range(len(seqs)))
        was_training = self.model.training
        self.model.eval()
        seen = None
        if sp.repetition_penalty != 1.0:
            seen = torch.zeros(len(seqs), self.model.config.vocab_size, dtype=torch.bool)
            for i, s in enumerate(seqs):
                seen[i, torch.tensor(s, dtype=torch.long)] = True
        for _ in range(sp.max_tokens):
            if not alive:
                break
            lens = [len(seqs[i]) for i in alive]
            flat = torch.tensor([t for i in alive for t in seqs[i]], dtype=torch.long, device=dev)
            ctx = SeqCtx.from_lengths(lens, dev)
            kw = {}
            if pix is not None:
                kw = merge_vision_entries([pix[i] for i in alive], dev)
            hidden = self.model.forward_hidden(flat, ctx, **kw)
            last = (ctx.cu_seqlens[1:] - 1).long()
            logits = (hidden[last].float() @ self.model.lm_head_weight.float().t()).cpu()
            tok, lp = sample_reference(logits, sp, g, None if seen is None else seen[alive])
            nxt = []
            for j, i in enumerate(alive):
                t = int(tok[j])
                seqs[i].append(t)
                outs[i].token_ids.append(t)
                outs[i].logprobs.append(float(lp[j]))
                if seen is not None:
                    seen[i, t] = True
                if sp.eos_token_id is not None and (t == sp.eos_token_id or t in sp.stop_token_ids):
                    outs[i].finish_reason = "stop"
                else:
                    nxt.append(i)
            alive = nxt
        if was_training:
            self.model.train()
        return outs


class _PrefillKV:
    """Attention hook used during prefill: append K/V to the paged cache, then varlen attention."""

    def __init__(self, engine: "RolloutEngine", tok_slot, tok_pos):
        self.e, self.tok_slot, self.tok_pos = engine, tok_slot, tok_pos

    def attend(self, layer_idx, q, k, v, ctx):
        from ..ops import cuda as K

        e = self.e
        if e.tp > 1:  # this rank caches only its own KV heads
            sl = slice(e.tp_rank * e.hk_local, (e.tp_rank + 1) * e.hk_local)
            kw, vw = k[:, sl].contiguous(), v[:, sl].contiguous()
        else:
            kw, vw = k.contiguous(), v.contiguous()
        K.kv_write_prefill(kw, vw, self.tok_slot, self.tok_pos, e.block_table, e.block_size,
                           e.k_cache[layer_idx], e.v_cache[layer_idx], v_transposed=e.attn_tc)
        return K.attention_varlen(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, True)


class RolloutEngine:
    def _decode_attention(self, li: int, scale: float):
        """q_buf x paged KV of layer ``li`` -> attn_buf (tcgen05 kernel when the cache layout allows it)."""
        from ..ops import cuda as K

        if self.attn_tc:
            K.paged_decode_attn_tc(self.q_buf, self.k_cache[li], self.v_cache[li], self.seq_lens, None, self.block_table,
                                   scale, self.kv_splits, self.part_o, self.part_ml, self.attn_buf,
                                   groups=self.attn_groups)
        else:
            K.paged_decode_attn(self.q_buf, self.k_cache[li], self.v_cache[li], self.seq_lens, None, self.block_table,
                                self.block_size, scale, self.kv_splits, self.part_o, self.part_ml, self.attn_buf)

    def __init__(self, model: CausalLM, max_num_seqs: int = 64, max_model_len: int = 2048, block_size: int | None = None,
                 num_blocks: int | None = None, poll_every: int = 16, use_cuda_graph: bool = True, kv_splits: int = 0,
                 tp: int = 1, tp_rank: int = 0):
        # vision-language model: the decoder runs here; image features are spliced into the prefill embeddings
        self.vlm = model if getattr(model, "is_vlm", False) else None
        if self.vlm is not None:
            model = model.language_model
        cfg = model.config
        if cfg.num_attention_heads % tp or cfg.num_key_value_heads % tp:
            raise ValueError(f"tensor parallel size {tp} must divide the head counts")
        self.tp, self.tp_rank = tp, tp_rank
        self.hq_local, self.hk_local = cfg.num_attention_heads // tp, cfg.num_key_value_heads // tp
        self.model, self.cfg = model, cfg
        self.dev = model.device
        if self.dev.type != "cuda":
            raise RuntimeError("RolloutEngine needs a CUDA device; use EagerGenerator on CPU")
        if cfg.hidden_act != "silu" or cfg.norm_plus_one or cfg.embed_scale != 1.0 or cfg.head_dim not in (64, 128):
            raise NotImplementedError("the decode kernels cover SwiGLU models with head_dim 64 or 128; use EagerGenerator "
                                      f"for model_type={cfg.model_type!r}")
        if cfg.sliding_window and max_model_len > cfg.sliding_window:
            raise NotImplementedError(f"the paged decode attention attends over the whole context: sliding_window="
                                      f"{cfg.sliding_window} < max_model_len={max_model_len}; use EagerGenerator")
        from .._native import host_runtime

        rt = host_runtime()
        if rt is None:
            raise RuntimeError("libtrl_b200_host.so missing: run python -m trl_b200.csrc.build")
        # head_dim 128 with at most 8 query heads per KV head: tensor-core decode attention, which wants 64-token
        # pages and V transposed inside a page; anything else keeps 16-token pages and the CUDA-core kernel
        tc_ok = cfg.head_dim == 128 and self.hq_local // self.hk_local <= 8
        if not block_size:
            block_size = 64 if tc_ok else 16
        self.attn_tc = tc_ok and block_size == 64
        self.attn_groups = int(os.environ.get("TRL_B200_DECODE_ATTN_GROUPS", "1"))  # 2: two softmax groups per CTA
        self.max_seqs, self.max_len, self.block_size = max_num_seqs, max_model_len, block_size
        self.max_blocks = (max_model_len + block_size - 1) // block_size
        self.num_blocks = num_blocks or max_num_seqs * self.max_blocks
        self.sched = rt.scheduler(max_num_seqs, self.num_blocks, block_size, self.max_blocks)
        L, Hk, D = cfg.num_hidden_layers, self.hk_local, cfg.head_dim
        dt = torch.bfloat16
        self.k_cache = [torch.zeros(self.num_blocks, block_size, Hk, D, dtype=dt, device=self.dev) for _ in range(L)]
        v_shape = (self.num_blocks, Hk, D, block_size) if self.attn_tc else (self.num_blocks, block_size, Hk, D)
        self.v_cache = [torch.zeros(*v_shape, dtype=dt, device=self.dev) for _ in range(L)]
        i32 = dict(dtype=torch.int32, device=self.dev)
        self.block_table = torch.zeros(max_num_seqs, self.max_blocks, **i32)
        self.block_table_host = torch.zeros(max_num_seqs, self.max_blocks, dtype=torch.int32).pin_memory()
        self.seq_lens = torch.full((max_num_seqs,), -1, **i32)
        # multimodal RoPE: rotary position of a slot's next token = its length + rope_delta[slot]
        self.rope_delta = (torch.zeros(max_num_seqs, dtype=torch.int32, device=self.dev)
                           if self.vlm is not None and cfg.extra.get("mrope_section") else None)
        self.n_gen = torch.zeros(max_num_seqs, **i32)
        self.finished = torch.zeros(max_num_seqs, **i32)
        self.next_input = torch.zeros(max_num_seqs, dtype=torch.int64, device=self.dev)
        self.step_counter = torch.zeros(1, **i32)
        self.tok = torch.zeros(max_num_seqs, **i32)
        self.logp = torch.zeros(max_num_seqs, dtype=torch.float32, device=self.dev)
        self.poll_every, self.use_graph = poll_every, use_cuda_graph
        # enough CTAs for ~4 per SM: the kernel is latency-bound on KV loads, occupancy hides it
        self.kv_splits = kv_splits or max(1, min(8, -(-(4 * 148) // max(1, max_num_seqs * Hk))))
        if self.attn_tc and not kv_splits:  # persistent CTAs, one per SM: split only to give every SM an item
            self.kv_splits = max(1, min(8, 148 // max(1, max_num_seqs * Hk)))
        self.part_o = torch.empty(max_num_seqs * self.hq_local * self.kv_splits * D, dtype=torch.float32, device=self.dev)
        self.part_ml = torch.empty(max_num_seqs * self.hq_local * self.kv_splits * 2, dtype=torch.float32, device=self.dev)
        self.q_buf = torch.empty(max_num_seqs, self.hq_local, D, dtype=dt, device=self.dev)
        self._fused_gate_up = (os.environ.get("TRL_B200_DECODE_FUSED_GATE_UP", "1") == "1" and not cfg.is_moe and tp == 1
                               and cfg.hidden_size % 8 == 0 and cfg.intermediate_size % 8 == 0)
        # decode linears on the weight-streaming tcgen05 kernel (stream-K over every SM, fp32 sums consumed and cleared
        # by the next kernel, programmatic dependent launch); TRL_B200_DECODE_GEMM=cublas keeps the library GEMMs
        self._own_gemm = (os.environ.get("TRL_B200_DECODE_GEMM", "own") != "cublas" and tp == 1 and max_num_seqs <= 128
                          and cfg.hidden_size <= 8192 and cfg.hidden_size % 8 == 0 and cfg.head_dim <= 128
                          and (cfg.is_moe or cfg.intermediate_size % 8 == 0))
        self._pdl = os.environ.get("TRL_B200_PDL", "1") == "1"
        if self._own_gemm:  # fp32 accumulators; their consumers clear them after reading
            f32 = dict(dtype=torch.float32, device=self.dev)
            qkv_out = (self.hq_local + 2 * self.hk_local) * cfg.head_dim
            self._acc_qkv = torch.zeros(max_num_seqs, qkv_out, **f32)
            self._acc_o = torch.zeros(max_num_seqs, cfg.hidden_size, **f32)
            self._acc_d = torch.zeros(max_num_seqs, cfg.hidden_size, **f32)
            self._logits_buf = torch.empty(max_num_seqs, cfg.vocab_size, dtype=dt, device=self.dev)
            if not cfg.is_moe:
                self._act_buf = torch.empty(max_num_seqs, cfg.intermediate_size // tp, dtype=dt, device=self.dev)
        if self._fused_gate_up and not self._own_gemm:
            self._one_group = torch.tensor([0, max_num_seqs], dtype=torch.int32, device=self.dev)
            self._act_buf = torch.empty(max_num_seqs, cfg.intermediate_size, dtype=dt, device=self.dev)
        self.attn_buf = torch.empty(max_num_seqs, self.hq_local, D, dtype=dt, device=self.dev)
        self.seen = None
        self.out_tokens = self.out_logps = None
        self._graph = None
        self._graph_key = None
        self.stats = {"decode_steps": 0, "prefill_tokens": 0, "generated_tokens": 0}

    # ---- weights ------------------------------------------------------------------------------
    def sync_weights(self, model: CausalLM | None = None):
        """TP=1 shares storage with the policy, so there is nothing to copy; the captured graph
        reads the live parameter storage, hence optimizer updates are visible immediately."""
        if model is not None and model is not self.model:
            with torch.no_grad():
                for (n, p), (_, q) in zip(self.model.named_parameters(), model.named_parameters()):
                    p.copy_(q)

    def reset_prefix_cache(self):
        pass  # prefix blocks live only for the duration of one generate() call

    # ---- one decode step (graph body) --------------------------------------------------------------
    def _decode_step(self, sp: SamplingParams, max_total_len: int):
        from ..ops import cuda as K

        if self._own_gemm:
            was = K.set_pdl(self._pdl)
            try:
                logits = self._decode_layers_own()
            finally:
                K.set_pdl(was)
        else:
            logits = self._decode_layers_lib()
        self._sample(logits, sp)
        K.advance(self.tok, self.logp, None, self.seq_lens, self.n_gen, self.finished, self.out_tokens, self.out_logps,
                  sp.eos_token_id, max_total_len, self.next_input, self.step_counter, 1)
        if self.seen is not None:
            self.seen.scatter_(1, self.next_input[:, None], 1)

    def _decode_layers_own(self):
        """Decoder stack of one decode step on this library's kernels only: every linear is the weight-streaming
        tcgen05 GEMM; q/k/v, attention output and MLP output travel as fp32 sums that the next kernel consumes."""
        from ..ops import cuda as K

        cfg, m = self.cfg, self.model
        eps = cfg.rms_norm_eps
        x = torch.nn.functional.embedding(self.next_input, m.embed_tokens)
        scale = 1.0 / math.sqrt(cfg.head_dim)
        pending = False  # the MLP output of the previous layer still sits in _acc_d
        for li, l in enumerate(m.layers):
            if pending:
                h = K.add_rmsnorm_f32_infer(x, self._acc_d, l.input_layernorm, eps)
            else:
                h = K.rmsnorm_infer(x, l.input_layernorm, eps)
            K.decode_gemm(h, l.qkv_proj, y32=self._acc_qkv)
            K.rope_kv_write_f32(self._acc_qkv, l.qkv_bias, l.q_norm if cfg.qk_norm else None,
                                l.k_norm if cfg.qk_norm else None, eps, self.seq_lens, None, self.block_table,
                                self.block_size, self.q_buf, self.k_cache[li], self.v_cache[li], cfg.num_attention_heads,
                                cfg.num_key_value_heads, cfg.head_dim, cfg.rope_theta, v_transposed=self.attn_tc, pos_delta=self.rope_delta)
            self._decode_attention(li, scale)
            K.decode_gemm(self.attn_buf.view(self.max_seqs, -1), l.o_proj, y32=self._acc_o)
            h = K.add_rmsnorm_f32_infer(x, self._acc_o, l.post_attention_layernorm, eps)
            if cfg.is_moe:
                from ..ops import functional as F_

                y, _, _ = F_.moe_mlp(h, l.router, l.experts_gate_up, l.experts_down, cfg.num_experts_per_tok,
                                     cfg.norm_topk_prob)
                x.add_(y)
                pending = False
            else:
                act = K.decode_gemm(h, l.gate_up_proj, out=self._act_buf, swiglu=True)
                K.decode_gemm(act, l.down_proj, y32=self._acc_d)
                pending = True
        if pending:
            hN = K.add_rmsnorm_f32_infer(x, self._acc_d, m.norm, eps)
        else:
            hN = K.rmsnorm_infer(x, m.norm, eps)
        return K.decode_gemm(hN, m.lm_head_weight, out=self._logits_buf)

    def _decode_layers_lib(self):
        """The same stack with library GEMMs for the plain linears (comparison path, and the path of shapes the
        weight-streaming kernel does not cover)."""
        from ..ops import cuda as K

        cfg, m = self.cfg, self.model
        eps = cfg.rms_norm_eps
        x = torch.nn.functional.embedding(self.next_input, m.embed_tokens)
        scale = 1.0 / math.sqrt(cfg.head_dim)
        fuse = cfg.hidden_size <= 8192  # residual add folded into the following RMSNorm
        pending = None  # block output not yet added to the residual stream
        for li, l in enumerate(m.layers):
            if pending is None:
                h = K.rmsnorm_infer(x, l.input_layernorm, eps)
            else:
                h = K.add_rmsnorm_infer(x, pending, l.input_layernorm, eps)
                pending = None
            qkv = torch.nn.functional.linear(h, l.qkv_proj, l.qkv_bias)
            if cfg.qk_norm:
                qs, ks = cfg.q_size, cfg.kv_size
                qn = K.rmsnorm_infer(qkv[:, :qs].reshape(-1, cfg.head_dim).contiguous(), l.q_norm, eps)
                kn = K.rmsnorm_infer(qkv[:, qs:qs + ks].reshape(-1, cfg.head_dim).contiguous(), l.k_norm, eps)
                qkv = torch.cat([qn.view(-1, qs), kn.view(-1, ks), qkv[:, qs + ks:]], dim=1)
            K.rope_kv_write(qkv, self.seq_lens, None, self.block_table, self.block_size, self.q_buf, self.k_cache[li],
                            self.v_cache[li], cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                            cfg.rope_theta, v_transposed=self.attn_tc, pos_delta=self.rope_delta)
            self._decode_attention(li, scale)
            if fuse:
                attn_out = torch.nn.functional.linear(self.attn_buf.view(self.max_seqs, -1), l.o_proj)
                h = K.add_rmsnorm_infer(x, attn_out, l.post_attention_layernorm, eps)
            else:
                x = x + torch.nn.functional.linear(self.attn_buf.view(self.max_seqs, -1), l.o_proj)
                h = K.rmsnorm_infer(x, l.post_attention_layernorm, eps)
            if cfg.is_moe:
                from ..ops import functional as F_

                y, _, _ = F_.moe_mlp(h, l.router, l.experts_gate_up, l.experts_down, cfg.num_experts_per_tok,
                                     cfg.norm_topk_prob)
            elif self._fused_gate_up:
                # gate/up GEMM with the SwiGLU epilogue (the grouped kernel with one group): the [B, 2I] intermediate
                # and one launch per layer disappear
                act = K.grouped_gemm(h, l.gate_up_proj.unsqueeze(0), self._one_group, cfg.intermediate_size, swiglu=True,
                                     out=self._act_buf)
                y = torch.nn.functional.linear(act, l.down_proj)
            else:
                gu = torch.nn.functional.linear(h, l.gate_up_proj)
                y = torch.nn.functional.linear(K.swiglu_infer(gu), l.down_proj)
            if fuse:
                pending = y
            else:
                x = x + y
        if pending is None:
            hN = K.rmsnorm_infer(x, m.norm, eps)
        else:
            hN = K.add_rmsnorm_infer(x, pending, m.norm, eps)
        return torch.nn.functional.linear(hN, m.lm_head_weight)

    def _sample(self, logits, sp: SamplingParams, rows: Optional[torch.Tensor] = None, tok=None, logp=None):
        from ..ops import cuda as K

        tok = self.tok if tok is None else tok
        logp = self.logp if logp is None else logp
        z = logits
        if self.seen is not None and sp.repetition_penalty != 1.0:
            seen = self.seen if rows is None else self.seen[rows]
            z = apply_repetition_penalty(z.float(), seen, sp.repetition_penalty)
        if sp.needs_filter_pass:
            z = filter_top_k_top_p(z.float() / max(sp.temperature, 1e-6), sp.top_k, sp.top_p).contiguous()
            inv_t = 1.0
        else:
            inv_t = 1.0 / max(sp.temperature, 1e-6)
        # the seed argument is a constant (it is baked into the captured graph); the call's seed enters through the
        # start value of the device-side step counter, so a new seed needs no new capture
        K.sample_tokens(z, inv_t, sp.min_p, sp.eos_token_id, sp.eos_prob_floor, _KERNEL_SEED, self.step_counter,
                        sp.greedy or sp.temperature == 0, tok, logp)

    # ---- prefill -------------------------------------------------------------------------------------
    @torch.no_grad()
    def _prefill(self, owners: list[tuple[int, list]], pixels: list | None = None) -> torch.Tensor:
        """owners: [(slot, prompt_ids)]; pixels: per owner the pixel tensor of its images (vision-language models).
        Returns last-token hidden states [len(owners), H]."""
        lens = [len(p) for _, p in owners]
        flat = torch.tensor([t for _, p in owners for t in p], dtype=torch.long).pin_memory().to(self.dev, non_blocking=True)
        tok_slot = torch.tensor([s for (s, p) in owners for _ in p], dtype=torch.int32).to(self.dev, non_blocking=True)
        ctx = SeqCtx.from_lengths(lens, self.dev)
        ctx.kv = _PrefillKV(self, tok_slot, ctx.positions.to(torch.int32))
        self.stats["prefill_tokens"] += int(flat.numel())
        was = self.model.training
        self.model.eval()
        embeds = self._vision_prefill(flat, ctx, pixels)
        hidden = self.model.forward_hidden(flat, ctx, inputs_embeds=embeds)
        if was:
            self.model.train()
        return hidden[(ctx.cu_seqlens[1:] - 1).long()]

    # ---- public API -----------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sp: SamplingParams, images=None) -> list[Completion]:
        """``images``: per prompt the pixel tensor [n_images, C, S, S] (vision-language models), or None."""
        from ..ops import cuda as K

        if images is not None and self.vlm is None:
            raise ValueError("images were passed to a text-only rollout engine")
        n_req = len(prompts) * sp.n
        max_new = sp.max_tokens
        max_prompt = max(len(p) for p in prompts)
        max_total = min(self.max_len, max_prompt + max_new)
        if max_prompt + 1 > self.max_len:
            raise ValueError(f"prompt of {max_prompt} tokens does not fit max_model_len={self.max_len}")
        dev = self.dev
        if self.out_tokens is None or self.out_tokens.shape[1] != max_new:
            self.out_tokens = torch.zeros(self.max_seqs, max_new, dtype=torch.int32, device=dev)
            self.out_logps = torch.zeros(self.max_seqs, max_new, dtype=torch.float32, device=dev)
            self._graph = None
        if sp.repetition_penalty != 1.0 and self.seen is None:
            self.seen = torch.zeros(self.max_seqs, self.cfg.vocab_size, dtype=torch.uint8, device=dev)
            self._graph = None
        reqs = []
        for pi, p in enumerate(prompts):
            for j in range(sp.n):
                rid = len(reqs)
                reqs.append((list(p), pi))
                self.sched.add(rid, len(p), min(max_new, self.max_len - len(p)), pi)
        results: list[Optional[Completion]] = [None] * n_req
        slot_req = [-1] * self.max_seqs
        delta_of_prompt: dict[int, int] = {}  # multimodal RoPE: rotary lead of every prefilled prompt
        self.seq_lens.fill_(-1)
        self.finished.zero_()
        self.n_gen.zero_()
        if self._own_gemm:  # a step that raised half-way may have left partial sums behind
            self._acc_qkv.zero_()
            self._acc_o.zero_()
            self._acc_d.zero_()
        bt_np = self.block_table_host.numpy()
        timing = os.environ.get("TRL_B200_ROLLOUT_TIMING", "0") == "1"  # wall-clock sections in self.stats (adds syncs)
        graph_key = (sp.temperature, sp.top_p, sp.top_k, sp.min_p, sp.repetition_penalty, sp.eos_token_id,
                     sp.eos_prob_floor, sp.greedy, max_total, max_new)
        # random stream of this call: the sampler hashes (step counter, row); the counter starts at a mix of the seed
        self.step_counter.fill_((int(sp.seed) * 0x9E3779B1 + 0x7F4A7C15) & 0x3FFFFFFF)
        # every request retires after at most max_new decode steps; a generous bound on the number of
        # polls turns a scheduling or kernel fault into an error instead of an endless host loop
        max_polls = (n_req // max(1, self.max_seqs) + 2) * (max_new // self.poll_every + 2) + 8
        polls = 0
        while True:
            polls += 1
            if polls > max_polls:
                K.check_status(dev)
                raise RuntimeError(f"rollout did not finish within {max_polls} polls "
                                   f"(running={self.sched.num_running}, waiting={self.sched.num_waiting})")
            admitted = self.sched.admit(bt_np)
            t_sec = time.perf_counter() if timing else 0.0
            if admitted:
                self.block_table.copy_(self.block_table_host, non_blocking=True)
                owners = [(slot, reqs[rid][0]) for rid, slot, pre, _ in admitted if pre]
                group_row = {reqs[rid][1]: i for i, (rid, slot, pre, _) in enumerate([a for a in admitted if a[2]])}
                own_px = None if images is None else [images[reqs[rid][1]] for rid, slot, pre, _ in admitted if pre]
                last_h = self._prefill(owners, own_px) if owners else None
                if self.rope_delta is not None:
                    if owners:
                        for (rid, _, _, _), d in zip([a for a in admitted if a[2]], self._prefill_delta):
                            delta_of_prompt[reqs[rid][1]] = d
                    self.rope_delta[torch.tensor([a[1] for a in admitted], device=dev)] = torch.tensor(
                        [delta_of_prompt[reqs[a[0]][1]] for a in admitted], dtype=torch.int32, device=dev)
                # sharers: copy the partial tail block of the prompt from the group's owner
                # (all sharers of the batch at once: two gathers + scatters per layer instead of two copies per sharer)
                pairs = [(int(bt_np[slot, len(reqs[rid][0]) // self.block_size]), copy_blk)
                         for rid, slot, pre, copy_blk in admitted if not pre and copy_blk >= 0]
                if pairs:
                    dst_t = torch.tensor([p[0] for p in pairs], dtype=torch.long, device=dev)
                    src_t = torch.tensor([p[1] for p in pairs], dtype=torch.long, device=dev)
                    for li in range(self.cfg.num_hidden_layers):
                        self.k_cache[li].index_copy_(0, dst_t, self.k_cache[li].index_select(0, src_t))
                        self.v_cache[li].index_copy_(0, dst_t, self.v_cache[li].index_select(0, src_t))
                slots = torch.tensor([a[1] for a in admitted], dtype=torch.int32, device=dev)
                plen_t = torch.tensor([len(reqs[a[0]][0]) for a in admitted], dtype=torch.int32, device=dev)
                self.seq_lens[slots.long()] = plen_t
                self.finished[slots.long()] = 0
                self.n_gen[slots.long()] = 0
                if self.seen is not None:
                    self.seen[slots.long()] = 0
                    for a in admitted:
                        self.seen[a[1], torch.tensor(reqs[a[0]][0], device=dev)] = 1
                # first token of every admitted request from its group's last-prompt-token logits
                if last_h is not None and len(group_row) == len(set(reqs[a[0]][1] for a in admitted)):
                    rows = torch.tensor([group_row[reqs[a[0]][1]] for a in admitted], device=dev)
                    h_rows = last_h[rows]
                else:  # a sharer admitted after its owner's batch: recompute the prompt's last hidden state
                    need = {}
                    for a in admitted:
                        need.setdefault(reqs[a[0]][1], a)
                    tmp = self._prefill_hidden_only([reqs[a[0]][0] for a in need.values()],
                                                    None if images is None else [images[g] for g in need])
                    gi = {g: i for i, g in enumerate(need)}
                    h_rows = tmp[torch.tensor([gi[reqs[a[0]][1]] for a in admitted], device=dev)]
                logits = torch.nn.functional.linear(h_rows, self.model.lm_head_weight)
                tok = torch.empty(len(admitted), dtype=torch.int32, device=dev)
                lp = torch.empty(len(admitted), dtype=torch.float32, device=dev)
                self._sample(logits, sp, rows=slots.long(), tok=tok, logp=lp)
                K.advance(tok, lp, slots, self.seq_lens, self.n_gen, self.finished, self.out_tokens, self.out_logps,
                          sp.eos_token_id, max_total, self._scatter_next(slots), self.step_counter, 0)
                self.next_input[slots.long()] = self._tmp_next[: len(admitted)]
                if self.seen is not None:
                    self.seen.scatter_(1, self.next_input[:, None], 1)
                for rid, slot, _, _ in admitted:
                    slot_req[slot] = rid
            if timing and admitted:
                torch.cuda.synchronize()
                self.stats["t_admit_prefill"] = self.stats.get("t_admit_prefill", 0.0) + time.perf_counter() - t_sec
            if self.sched.num_running == 0:
                break
            t_sec = time.perf_counter() if timing else 0.0
            # ---- decode until the next poll ----
            if self.use_graph:
                if self._graph is None or self._graph_key != graph_key:
                    self._capture(sp, max_total, graph_key)
                for _ in range(self.poll_every):
                    self._graph.replay()
                K.LAUNCHES[0] += self.poll_every * self._graph_kernels
            else:
                for _ in range(self.poll_every):
                    self._decode_step(sp, max_total)
            self.stats["decode_steps"] += self.poll_every
            fin = self.finished.cpu().numpy()  # host sync: the only one per poll
            if timing:
                self.stats["t_decode"] = self.stats.get("t_decode", 0.0) + time.perf_counter() - t_sec
                t_sec = time.perf_counter()
            done_slots = [s for s in range(self.max_seqs) if slot_req[s] >= 0 and fin[s]]
            if done_slots:
                ds = torch.tensor(done_slots, device=dev)
                ng = self.n_gen[ds].cpu().numpy()
                toks = self.out_tokens[ds].cpu().numpy()
                lps = self.out_logps[ds].cpu().numpy()
                for j, s in enumerate(done_slots):
                    rid = slot_req[s]
                    n = int(min(ng[j], max_new))
                    t = toks[j, :n].tolist()
                    reason = "stop" if (sp.eos_token_id is not None and n and t[-1] == sp.eos_token_id) else "length"
                    results[rid] = Completion(reqs[rid][0], t, lps[j, :n].tolist(), reason)
                    self.stats["generated_tokens"] += n
                    self.sched.retire(s, reqs[rid][1])
                    slot_req[s] = -1
                self.seq_lens[ds] = -1
                self.finished[ds] = 0
            if timing:
                self.stats["t_collect"] = self.stats.get("t_collect", 0.0) + time.perf_counter() - t_sec
        K.check_status(dev)
        return results  # type: ignore[return-value]

    def _scatter_next(self, slots):
        self._tmp_next = torch.zeros(self.max_seqs, dtype=torch.int64, device=self.dev)
        return self._tmp_next

    def _prefill_hidden_only(self, prompts, pixels: list | None = None):
        lens = [len(p) for p in prompts]
        flat = torch.tensor([t for p in prompts for t in p], dtype=torch.long, device=self.dev)
        ctx = SeqCtx.from_lengths(lens, self.dev)
        hidden = self.model.forward_hidden(flat, ctx, inputs_embeds=self._vision_prefill(flat, ctx, pixels))
        return hidden[(ctx.cu_seqlens[1:] - 1).long()]

    def _vision_prefill(self, flat, ctx, pixels):
        """Vision-language models: input embeddings with the image features spliced in (None for text-only batches).
        With multimodal RoPE the three position rows go into ``ctx`` and ``self._prefill_delta`` gets, per sequence,
        how far the next rotary position leads (or trails) the sequence length."""
        self._prefill_delta = None
        if self.vlm is None:
            return None
        embeds, kw = None, {}
        if pixels is not None and any(vision_entry_numel(x) for x in pixels):
            embeds = self.model.embed(flat)
            kw = merge_vision_entries(pixels, self.dev, embeds.dtype)
            feats = self.vlm.image_features(**kw).to(embeds.dtype)
            tid = getattr(self.vlm.config, "image_token_index", None)
            slots = (flat == tid).nonzero().flatten()
            if slots.numel() != feats.shape[0]:
                raise ValueError(f"{slots.numel()} image placeholder tokens for {feats.shape[0]} image features")
            embeds.index_copy_(0, slots, feats)
        if self.rope_delta is not None:
            from ..models.vision_qwen import rope_index

            pos3 = rope_index(flat, ctx.cu_seqlens, kw.get("image_grid_thw"), self.vlm.config)
            ctx.mrope_positions = pos3
            cu = ctx.cu_seqlens.tolist()
            top = pos3.max(0).values
            self._prefill_delta = [int(top[a:b].max()) + 1 - (b - a) for a, b in zip(cu[:-1], cu[1:])]
        return embeds

    def _capture(self, sp, max_total, key):
        # one eager step on a side stream warms every allocation and scratch buffer, but it also
        # advances the state: snapshot and restore the mutable tensors around warm-up and capture.
        state = [t.clone() for t in (self.seq_lens, self.n_gen, self.finished, self.next_input, self.step_counter,
                                     self.out_tokens, self.out_logps)]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._decode_step(sp, max_total)
        torch.cuda.current_stream().wait_stream(s)
        from ..ops import cuda as K

        g = torch.cuda.CUDAGraph()
        n0 = K.LAUNCHES[0]
        with torch.cuda.graph(g):
            self._decode_step(sp, max_total)
        self._graph_kernels = K.LAUNCHES[0] - n0  # library kernels replayed by every graph launch
        for t, o in zip((self.seq_lens, self.n_gen, self.finished, self.next_input, self.step_counter, self.out_tokens,
                         self.out_logps), state):
            t.copy_(o)
        self._graph, self._graph_key = g, key
