"""Native decoder-only transformer (Llama / Qwen2 / Qwen3 / Qwen3-MoE).

The model is padding-free at its core: it consumes a flat token stream ``[T]``
plus a :class:`SeqCtx` (positions, ``cu_seqlens``).  Padded ``[B, S]`` batches
are un-padded on entry and re-padded on exit, so a padded call and a packed
call execute the same kernels.

In memory QKV and gate/up are fused (one GEMM each); on disk the checkpoint
uses the Hugging Face names (``model.layers.N.self_attn.q_proj.weight`` ...),
see :mod:`trl_b200.models.hf_io`.  The reference relies on transformers model
code for this layer (trl/trainer/utils.py:1123-1170 ``create_model_from_path``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Optional

import torch
import torch.nn as nn

from ..ops import functional as ops
from .configuration import ModelArch


@dataclass
class SeqCtx:
    """Sequence geometry of one packed micro-batch."""

    positions: torch.Tensor  # [T] int32/int64
    cu_seqlens: torch.Tensor  # [n_docs+1] int32
    max_seqlen: int
    # rollout-only: paged KV cache handles (see trl_b200.rollout.kv_cache)
    kv: Any = None
    router_records: list = field(default_factory=list)
    # sequence parallelism (parallel/ulysses.py): positions are this rank's chunk, cu_seqlens / max_seqlen are global
    sp: Any = None
    # multimodal rotary positions [3, T] (temporal, height, width; models/vision_qwen.py); None = ordinary RoPE
    mrope_positions: Any = None

    @staticmethod
    def from_lengths(lengths, device) -> "SeqCtx":
        lengths = torch.as_tensor(lengths, dtype=torch.int32)
        cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
        cu[1:] = lengths.cumsum(0)
        pos = torch.cat([torch.arange(int(n), dtype=torch.int32) for n in lengths.tolist()]) if len(lengths) else torch.zeros(0, dtype=torch.int32)
        return SeqCtx(pos.to(device), cu.to(device), int(lengths.max()) if len(lengths) else 0)

    @staticmethod
    def from_position_ids(position_ids: torch.Tensor) -> "SeqCtx":
        """Documents start wherever ``position_ids == 0`` (padding-free collator output)."""
        pos = position_ids.reshape(-1)
        starts = (pos == 0).nonzero().flatten()
        if starts.numel() == 0 or starts[0] != 0:
            starts = torch.cat([starts.new_zeros(1), starts])
        cu = torch.cat([starts, starts.new_tensor([pos.numel()])]).to(torch.int32)
        max_len = int((cu[1:] - cu[:-1]).max())
        return SeqCtx(pos.to(torch.int32), cu, max_len)


class LoraSlot(nn.Module):
    """One low-rank adapter ``B @ A`` attached to a (slice of a) fused projection."""

    def __init__(self, in_f, out_f, r, alpha, dropout, rslora=False, dtype=torch.float32, device=None):
        super().__init__()
        self.lora_A = nn.Parameter(torch.empty(r, in_f, dtype=dtype, device=device))
        self.lora_B = nn.Parameter(torch.zeros(out_f, r, dtype=dtype, device=device))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.scaling = alpha / math.sqrt(r) if rslora else alpha / r
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        self.r = r

    def delta(self, x):
        return (self.dropout(x) @ self.lora_A.to(x.dtype).t()) @ self.lora_B.to(x.dtype).t() * self.scaling

    def delta_weight(self):
        return (self.lora_B.float() @ self.lora_A.float()) * self.scaling


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelArch, layer_idx: int, dtype, device):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        h = cfg.hidden_size
        kw = dict(dtype=dtype, device=device)
        self.input_layernorm = nn.Parameter(torch.ones(h, **kw))
        self.qkv_proj = nn.Parameter(torch.empty(cfg.q_size + 2 * cfg.kv_size, h, **kw))
        self.qkv_bias = nn.Parameter(torch.zeros(cfg.q_size + 2 * cfg.kv_size, **kw)) if cfg.attention_bias else None
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(cfg.head_dim, **kw))
            self.k_norm = nn.Parameter(torch.ones(cfg.head_dim, **kw))
        self.o_proj = nn.Parameter(torch.empty(h, cfg.q_size, **kw))
        self.post_attention_layernorm = nn.Parameter(torch.ones(h, **kw))
        if cfg.is_moe:
            I = cfg.moe_intermediate_size
            self.router = nn.Parameter(torch.empty(cfg.num_experts, h, **kw))
            self.experts_gate_up = nn.Parameter(torch.empty(cfg.num_experts, 2 * I, h, **kw))
            self.experts_down = nn.Parameter(torch.empty(cfg.num_experts, h, I, **kw))
        else:
            I = cfg.intermediate_size
            self.gate_up_proj = nn.Parameter(torch.empty(2 * I, h, **kw))
            self.down_proj = nn.Parameter(torch.empty(h, I, **kw))
        self.lora = nn.ModuleDict()  # hf module name ("q_proj", ...) -> LoraSlot
        self.lora_enabled = True
        self.attn_dropout = nn.Dropout(0.0)

    # ---- slices of the fused projections, keyed by HF module name ----------
    def proj_slices(self) -> dict[str, tuple[str, slice]]:
        c = self.cfg
        out = {
            "q_proj": ("qkv_proj", slice(0, c.q_size)),
            "k_proj": ("qkv_proj", slice(c.q_size, c.q_size + c.kv_size)),
            "v_proj": ("qkv_proj", slice(c.q_size + c.kv_size, c.q_size + 2 * c.kv_size)),
            "o_proj": ("o_proj", slice(None)),
        }
        if not c.is_moe:
            I = c.intermediate_size
            out.update(gate_proj=("gate_up_proj", slice(0, I)), up_proj=("gate_up_proj", slice(I, 2 * I)),
                       down_proj=("down_proj", slice(None)))
        return out

    def _lora_add(self, y, x, names):
        if not self.lora_enabled or len(self.lora) == 0:
            return y
        sl = self.proj_slices()
        pieces = None
        for n in names:
            if n in self.lora:
                s = sl[n][1]
                d = self.lora[n].delta(x)
                if s == slice(None):
                    y = y + d
                else:
                    if pieces is None:
                        pieces = []
                    pieces.append((s, d))
        if pieces:
            # out-of-place so autograd sees it
            full = torch.zeros_like(y)
            for s, d in pieces:
                full[..., s] = d
            y = y + full
        return y

    def attn_block(self, x, ctx: SeqCtx):
        c = self.cfg
        T = x.shape[0]
        gather = getattr(self, "_shard_gather", None)
        if gather is not None and x.is_cuda:
            # full-shard engine: this GEMM also pulls the layer's missing parameter shards over NVLink
            qkv = gather.qkv(x, self.qkv_proj, self.qkv_bias)
        else:
            qkv = ops.linear(x, self.qkv_proj, self.qkv_bias)
        qkv = self._lora_add(qkv, x, ("q_proj", "k_proj", "v_proj"))
        q = qkv[:, : c.q_size].reshape(T, c.num_attention_heads, c.head_dim)
        k = qkv[:, c.q_size: c.q_size + c.kv_size].reshape(T, c.num_key_value_heads, c.head_dim)
        v = qkv[:, c.q_size + c.kv_size:].reshape(T, c.num_key_value_heads, c.head_dim)
        if c.qk_norm:
            q = ops.rms_norm(q.contiguous(), self.q_norm, c.rms_norm_eps)
            k = ops.rms_norm(k.contiguous(), self.k_norm, c.rms_norm_eps)
        if ctx.mrope_positions is not None and c.extra.get("mrope_section"):
            q, k = ops.apply_mrope_qk(q, k, ctx.mrope_positions, c.rope_theta, c.extra["mrope_section"])
        else:
            q, k = ops.apply_rope_qk(q, k, ctx.positions, c.rope_theta)
        if ctx.kv is not None:
            o = ctx.kv.attend(self.layer_idx, q, k, v, ctx)
        elif ctx.sp is not None and ctx.sp.mode == "allgather_kv":
            from ..parallel import context_parallel

            if c.sliding_window:
                raise NotImplementedError("context parallelism with sliding-window attention")
            o = context_parallel.attention(q, k, v, ctx, ops.attention_varlen_qk)
        elif ctx.sp is not None:
            from ..parallel import ulysses

            o = ulysses.attention(q, k, v, ctx, lambda a, b, d: ops.attention_varlen(a, b, d, ctx.cu_seqlens, ctx.max_seqlen,
                                                                                   causal=True, window=c.sliding_window))
        else:
            o = ops.attention_varlen(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, causal=True, window=c.sliding_window)
        o = o.reshape(T, c.q_size)
        out = ops.linear(o, self.o_proj)
        return self._lora_add(out, o, ("o_proj",))

    def mlp_block(self, x, ctx: SeqCtx):
        c = self.cfg
        if c.is_moe:
            ep = getattr(self, "ep", None)
            if ep is not None:  # expert parallel (parallel/expert_parallel.py:shard_experts): this rank holds a slice
                w, idx, probs = ops.moe_router(x, self.router, c.num_experts_per_tok, c.norm_topk_prob)
                out = ep(x, self.experts_gate_up, self.experts_down, w, idx)
            else:
                out, probs, idx = ops.moe_mlp(x, self.router, self.experts_gate_up, self.experts_down,
                                              c.num_experts_per_tok, c.norm_topk_prob)
            ctx.router_records.append((probs, idx))
            return out
        gu = ops.linear(x, self.gate_up_proj)
        gu = self._lora_add(gu, x, ("gate_proj", "up_proj"))
        if c.hidden_act == "silu":
            a = ops.swiglu(gu)
        else:  # GeGLU (Gemma): gelu(gate) * up
            g, u = gu.chunk(2, dim=-1)
            a = torch.nn.functional.gelu(g, approximate="tanh" if "tanh" in c.hidden_act else "none") * u
        out = ops.linear(a, self.down_proj)
        return self._lora_add(out, a, ("down_proj",))

    def forward(self, x, ctx: SeqCtx):
        c = self.cfg
        w1, w2 = self.input_layernorm, self.post_attention_layernorm
        if c.norm_plus_one:  # Gemma stores w - 1
            w1, w2 = w1 + 1.0, w2 + 1.0
        x = x + self.attn_block(ops.rms_norm(x, w1, c.rms_norm_eps), ctx)
        x = x + self.mlp_block(ops.rms_norm(x, w2, c.rms_norm_eps), ctx)
        return x


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None
    aux_loss: Optional[torch.Tensor] = None
    router_logits: Any = None

    def __getitem__(self, k):
        if isinstance(k, str):
            return getattr(self, k)
        return tuple(v for v in (self.loss, self.logits) if v is not None)[k]


class CausalLM(nn.Module):
    """Decoder with an LM head (``num_labels == 0``) or a scalar/score head."""

    supports_gradient_checkpointing = True
    _is_native = True

    def __init__(self, cfg: ModelArch, dtype=torch.float32, device=None, init: bool = True):
        super().__init__()
        self.config = cfg
        kw = dict(dtype=dtype, device=device)
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self.layers = nn.ModuleList([DecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, **kw))
        if cfg.num_labels:
            self.score = nn.Parameter(torch.empty(cfg.num_labels, cfg.hidden_size, **kw))
            self.lm_head = None
        elif cfg.tie_word_embeddings:
            self.lm_head = None
        else:
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self.gradient_checkpointing = False
        self.name_or_path = ""
        self.generation_config = None
        self.warnings_issued = {}
        if init and (device is None or str(device) != "meta"):
            self.reset_parameters()

    # ---- init -----------------------------------------------------------
    @torch.no_grad()
    def reset_parameters(self, std: float = 0.02, generator: torch.Generator | None = None):
        for name, p in self.named_parameters():
            if "lora" in name:
                continue
            if p.ndim == 1 and ("layernorm" in name or name == "norm" or name.endswith("_norm")):
                p.fill_(1.0)
            elif p.ndim == 1:
                p.zero_()
            else:
                # normal_ in fp32 chunks keeps init cheap and device-agnostic
                p.normal_(0.0, std, generator=generator)

    # ---- accessors --------------------------------------------------------
    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.embed_tokens if self.lm_head is None else self.lm_head

    @property
    def device(self):
        return self.embed_tokens.device

    @property
    def dtype(self):
        return self.embed_tokens.dtype

    def get_input_embeddings(self):
        return self.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head_weight

    def num_parameters(self, only_trainable=False):
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not only_trainable)

    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs=None):
        """``gradient_checkpointing_kwargs={"num_layers": n}`` recomputes only the first n layers and keeps the
        activations of the rest (a memory/time dial between "off" and "all layers")."""
        self.gradient_checkpointing = True
        n = (gradient_checkpointing_kwargs or {}).get("num_layers")
        self.checkpoint_num_layers = None if n is None else int(n)

    def gradient_checkpointing_disable(self):
        self.gradient_checkpointing = False

    @property
    def is_gradient_checkpointing(self):
        return self.gradient_checkpointing

    def enable_input_require_grads(self):
        pass

    def resize_token_embeddings(self, new_size: int, pad_to_multiple_of: int | None = None):
        if pad_to_multiple_of:
            new_size = (new_size + pad_to_multiple_of - 1) // pad_to_multiple_of * pad_to_multiple_of
        old = self.config.vocab_size
        if new_size == old:
            return
        for attr in ("embed_tokens", "lm_head"):
            w = getattr(self, attr)
            if w is None:
                continue
            nw = torch.empty(new_size, w.shape[1], dtype=w.dtype, device=w.device).normal_(0, 0.02)
            n = min(old, new_size)
            nw[:n] = w.data[:n]
            setattr(self, attr, nn.Parameter(nw))
        self.config.vocab_size = new_size

    # ---- stages (used directly by the sharded engine) -----------------------
    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        x = torch.nn.functional.embedding(input_ids, self.embed_tokens)
        if self.config.embed_scale != 1.0:
            x = x * torch.tensor(self.config.embed_scale, dtype=x.dtype)  # rounded to the model dtype like the reference model
        return x

    def final_norm(self, x):
        w = self.norm + 1.0 if self.config.norm_plus_one else self.norm
        return ops.rms_norm(x, w, self.config.rms_norm_eps)

    def forward_hidden(self, input_ids: torch.Tensor, ctx: SeqCtx, inputs_embeds: torch.Tensor | None = None) -> torch.Tensor:
        """Flat ids [T] -> final-norm hidden [T, H].  ``inputs_embeds`` [T, H] replaces the embedding lookup (vision-
        language models splice image features into it)."""
        x = self.embed(input_ids) if inputs_embeds is None else inputs_embeds
        alpha = getattr(self, "neftune_noise_alpha", None)
        if alpha and self.training:
            # NEFTune: uniform noise of magnitude alpha / sqrt(sequence length * hidden size) on the input embeddings
            # while training (the loop sets the attribute from `neftune_noise_alpha` and removes it afterwards)
            lens = (ctx.cu_seqlens[1:] - ctx.cu_seqlens[:-1]).to(x.device)
            per_tok = torch.repeat_interleave(lens, lens.long(), output_size=x.shape[0]).to(torch.float32)
            mag = float(alpha) / torch.sqrt(per_tok * x.shape[-1])
            x = x + ((torch.rand_like(x, dtype=torch.float32) * 2 - 1) * mag[:, None]).to(x.dtype)
        n_ckpt = getattr(self, "checkpoint_num_layers", None)
        keep = None
        for li, layer in enumerate(self.layers):
            if (self.gradient_checkpointing and self.training and torch.is_grad_enabled()
                    and (n_ckpt is None or li < n_ckpt)):
                from .activation_offloading import offload_checkpoint, offloading_active

                if keep is None and x.is_cuda:
                    from ..ops.cuda import AttnKeep as keep

                    fwd_id = keep.new_forward()

                def run(h, c=ctx, layer=layer, li=li):
                    # both the forward pass and its recompute go through here under the same name, so the attention
                    # output of the first is handed to the second (ops/cuda.py: AttnKeep)
                    if keep is None:
                        return layer(h, c)
                    with keep.scope((fwd_id, li)):
                        return layer(h, c)

                if getattr(self, "offload_checkpoint_inputs", False) and offloading_active():
                    # the layer input is saved through the saved-tensor hooks, i.e. it goes to pinned host memory
                    x = offload_checkpoint(run, x)
                else:
                    from torch.utils.checkpoint import checkpoint

                    x = checkpoint(run, x, use_reentrant=False)
            else:
                x = layer(x, ctx)
        return self.final_norm(x)

    def aux_loss(self, ctx: SeqCtx, token_mask=None):
        if not self.config.is_moe or not ctx.router_records:
            return None
        # checkpoint recompute appends duplicates: keep the first L records
        recs = ctx.router_records[: self.config.num_hidden_layers]
        probs = torch.cat([r[0] for r in recs], 0)
        idx = torch.cat([r[1] for r in recs], 0)
        m = None if token_mask is None else token_mask.reshape(-1).repeat(len(recs))
        return ops.load_balancing_loss(probs, idx, self.config.num_experts, self.config.num_experts_per_tok, m)

    # ---- HF-style call ------------------------------------------------------
    def pack_inputs(self, input_ids, attention_mask=None, position_ids=None):
        """Returns (flat_ids, ctx, scatter) where ``scatter(flat)`` re-pads to [B, S, ...]."""
        if input_ids.ndim == 1:
            input_ids = input_ids[None]
        B, S = input_ids.shape
        dev = input_ids.device
        if attention_mask is not None and not bool(attention_mask.all()):
            mask = attention_mask.bool()
            lengths = mask.sum(1)
            idx = mask.reshape(-1).nonzero().flatten()
            flat = input_ids.reshape(-1)[idx]
            pos = (mask.long().cumsum(1) - 1).reshape(-1)[idx].to(torch.int32)
            keep = lengths > 0
            cu = torch.zeros(int(keep.sum()) + 1, dtype=torch.int32, device=dev)
            cu[1:] = lengths[keep].cumsum(0)
            ctx = SeqCtx(pos, cu, int(lengths.max()))

            def scatter(t):
                out = t.new_zeros((B * S,) + t.shape[1:])
                out[idx] = t
                return out.reshape((B, S) + t.shape[1:])

            return flat, ctx, scatter
        if position_ids is not None and B == 1:
            ctx = SeqCtx.from_position_ids(position_ids.to(dev))
        else:
            ctx = SeqCtx.from_lengths([S] * B, dev)
        return input_ids.reshape(-1), ctx, (lambda t: t.reshape((B, S) + t.shape[1:]))

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, labels=None,
                output_hidden_states=False, use_cache=False, output_router_logits=None,
                logits_to_keep: int | None = None, return_hidden_only=False, **unused):
        flat, ctx, scatter = self.pack_inputs(input_ids, attention_mask, position_ids)
        hidden = self.forward_hidden(flat, ctx)
        out = CausalLMOutput()
        if self.config.is_moe:
            tm = None
            if attention_mask is not None and not bool(attention_mask.all()):
                tm = None  # packed stream already excludes pad tokens
            out.aux_loss = self.aux_loss(ctx, tm)
        if return_hidden_only:
            out.hidden_states = scatter(hidden)
            return out
        if self.config.num_labels:
            # score at the last real token of every sequence
            last = (ctx.cu_seqlens[1:] - 1).long()
            logits = ops.linear(hidden[last], self.score)
            if attention_mask is not None and logits.shape[0] != input_ids.shape[0]:
                full = logits.new_zeros(input_ids.shape[0], logits.shape[1])
                full[attention_mask.sum(1) > 0] = logits
                logits = full
            out.logits = logits
            return out
        hp = scatter(hidden)
        if logits_to_keep:
            hp = hp[:, -logits_to_keep:]
        logits = ops.linear(hp, self.lm_head_weight)
        if self.config.final_logit_softcapping:
            cap = self.config.final_logit_softcapping
            logits = torch.tanh(logits / cap) * cap
        out.logits = logits
        if output_hidden_states:
            out.hidden_states = hp
        if labels is not None:
            sl = logits[:, :-1].reshape(-1, logits.shape[-1]).float()
            out.loss = torch.nn.functional.cross_entropy(sl, labels[:, 1:].reshape(-1), ignore_index=-100)
            if out.aux_loss is not None:
                out.loss = out.loss + self.config.router_aux_loss_coef * out.aux_loss
        return out

    # ---- LoRA helpers -------------------------------------------------------
    def set_adapter_enabled(self, flag: bool):
        for l in self.layers:
            l.lora_enabled = flag

    @torch.no_grad()
    def merge_adapter(self, sign: float = 1.0):
        for l in self.layers:
            sl = l.proj_slices()
            for name, slot in l.lora.items():
                pname, s = sl[name]
                w = getattr(l, pname)
                w.data[s] += (sign * slot.delta_weight()).to(w.dtype)

    def unmerge_adapter(self):
        self.merge_adapter(-1.0)

    # ---- persistence (HF safetensors layout) ---------------------------------
    def save_pretrained(self, path: str, safe_serialization: bool = True, state_dict=None, **kw):
        from .hf_io import save_model

        save_model(self, path, state_dict=state_dict)

    @classmethod
    def from_pretrained(cls, path_or_name: str, dtype=None, torch_dtype=None, device=None, **kw):
        from .hf_io import load_model

        return load_model(path_or_name, dtype=dtype or torch_dtype, device=device, **kw)

    def state_dict_hf(self):
        from .hf_io import to_hf_state_dict

        return to_hf_state_dict(self)
