"""Architecture description for the native decoder families.

One flat dataclass covers Llama, Qwen2/2.5, Qwen3 and Qwen3-MoE. It round-trips
to and from a Hugging Face ``config.json`` so checkpoints written by
``save_pretrained`` load in ``transformers`` and vice versa.

Reference parity: the reference resolves the architecture from
``config.architectures[0]`` (trl/trainer/utils.py:1123-1170); here the same
``config.json`` keys select one of the native families.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any

_FAMILY_ARCH = {
    "llama": "LlamaForCausalLM",
    "qwen2": "Qwen2ForCausalLM",
    "qwen3": "Qwen3ForCausalLM",
    "qwen3_moe": "Qwen3MoeForCausalLM",
    "mistral": "MistralForCausalLM",
    "phi3": "Phi3ForCausalLM",
    "gemma": "GemmaForCausalLM",
}


@dataclass
class ModelArch:
    model_type: str = "qwen2"
    vocab_size: int = 1024
    hidden_size: int = 64
    intermediate_size: int = 256
    num_hidden_layers: int = 2
    num_attention_heads: int = 4
    num_key_value_heads: int = 2
    head_dim: int | None = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position_embeddings: int = 32768
    attention_bias: bool | None = None  # QKV bias (Qwen2: True)
    qk_norm: bool | None = None  # per-head RMSNorm on q,k (Qwen3)
    tie_word_embeddings: bool = False
    # MoE (Qwen3-MoE)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.001
    output_router_logits: bool = False
    # heads
    num_labels: int = 0  # >0 => sequence-classification / reward head
    pad_token_id: int | None = None
    bos_token_id: int | None = None
    eos_token_id: int | None = None
    final_logit_softcapping: float | None = None
    # every token attends to itself and the sliding_window - 1 tokens before it (Mistral v0.1, Phi-3-mini; None = full)
    sliding_window: int | None = None
    # Gemma: GeGLU instead of SwiGLU, RMSNorm scales by (1 + w), embeddings multiplied by sqrt(hidden)
    hidden_act: str = "silu"
    norm_plus_one: bool = False
    embed_scale: float = 1.0
    extra: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.attention_bias is None:
            self.attention_bias = self.model_type == "qwen2"
        if self.qk_norm is None:
            self.qk_norm = self.model_type in ("qwen3", "qwen3_moe")
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.model_type == "gemma":
            self.norm_plus_one, self.embed_scale = True, float(self.hidden_size) ** 0.5
            self.tie_word_embeddings = True
            if self.hidden_act == "silu":
                self.hidden_act = "gelu_pytorch_tanh"

    # ---- derived sizes -------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def num_parameters(self, exclude_embeddings: bool = False) -> int:
        h, L = self.hidden_size, self.num_hidden_layers
        attn = h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        if self.attention_bias:
            attn += self.q_size + 2 * self.kv_size
        if self.qk_norm:
            attn += 2 * self.head_dim
        if self.is_moe:
            mlp = self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
        else:
            mlp = 3 * h * self.intermediate_size
        n = L * (attn + mlp + 2 * h) + h
        if not exclude_embeddings:
            n += self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return n

    # ---- HF config.json round trip ------------------------------------
    def to_hf_dict(self) -> dict[str, Any]:
        d = {
            "architectures": [_FAMILY_ARCH.get(self.model_type, "LlamaForCausalLM")],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": self.hidden_act,
            **({"hidden_activation": self.hidden_act} if self.model_type == "gemma" else {}),
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_parameters": {"rope_type": "default", "rope_theta": self.rope_theta},
            "max_position_embeddings": self.max_position_embeddings,
            "attention_bias": self.attention_bias,
            "tie_word_embeddings": self.tie_word_embeddings,
            "pad_token_id": self.pad_token_id,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": self.eos_token_id,
            "torch_dtype": "bfloat16",
        }
        if self.is_moe:
            d.update(
                num_experts=self.num_experts,
                num_experts_per_tok=self.num_experts_per_tok,
                moe_intermediate_size=self.moe_intermediate_size,
                norm_topk_prob=self.norm_topk_prob,
                router_aux_loss_coef=self.router_aux_loss_coef,
                output_router_logits=self.output_router_logits,
                decoder_sparse_step=1,
                mlp_only_layers=[],
            )
        if self.num_labels:
            d["num_labels"] = self.num_labels
            d["architectures"] = [d["architectures"][0].replace("ForCausalLM", "ForSequenceClassification")]
        if self.final_logit_softcapping:
            d["final_logit_softcapping"] = self.final_logit_softcapping
        if self.model_type in ("mistral", "phi3") or self.sliding_window:
            d["sliding_window"] = self.sliding_window
            if self.model_type in ("qwen2", "qwen3", "qwen3_moe"):
                d["use_sliding_window"] = bool(self.sliding_window)
        d.update(self.extra)
        return d

    @classmethod
    def from_hf_dict(cls, d: dict[str, Any]) -> "ModelArch":
        if hasattr(d, "to_dict"):
            d = d.to_dict()
        mt = d.get("model_type", "llama")
        if mt not in _FAMILY_ARCH:
            raise ValueError(
                f"model_type={mt!r} has no native decoder; supported: {sorted(_FAMILY_ARCH)}"
            )
        theta = d.get("rope_theta")
        if theta is None:
            theta = (d.get("rope_parameters") or {}).get("rope_theta", 10000.0)
        nl = 0
        archs = d.get("architectures") or []
        if archs and "SequenceClassification" in archs[0]:
            nl = int(d.get("num_labels", len(d.get("id2label", {"0": 0})) or 1))
        return cls(
            model_type=mt,
            hidden_act=(d.get("hidden_activation") or d.get("hidden_act") or "silu") if mt == "gemma" else "silu",
            vocab_size=d["vocab_size"],
            hidden_size=d["hidden_size"],
            intermediate_size=d.get("intermediate_size", 4 * d["hidden_size"]),
            num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=d["num_attention_heads"],
            num_key_value_heads=d.get("num_key_value_heads") or d["num_attention_heads"],
            head_dim=d.get("head_dim"),
            rms_norm_eps=d.get("rms_norm_eps", 1e-6),
            rope_theta=float(theta),
            max_position_embeddings=d.get("max_position_embeddings", 32768),
            attention_bias=d.get("attention_bias", mt == "qwen2") if mt != "qwen2" else True,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            num_experts=d.get("num_experts", d.get("num_local_experts", 0)) if mt == "qwen3_moe" else 0,
            num_experts_per_tok=d.get("num_experts_per_tok", 0) if mt == "qwen3_moe" else 0,
            moe_intermediate_size=d.get("moe_intermediate_size", 0) if mt == "qwen3_moe" else 0,
            norm_topk_prob=d.get("norm_topk_prob", True),
            router_aux_loss_coef=d.get("router_aux_loss_coef", 0.001),
            output_router_logits=d.get("output_router_logits", False),
            num_labels=nl,
            pad_token_id=d.get("pad_token_id"),
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=d.get("eos_token_id") if not isinstance(d.get("eos_token_id"), list) else d["eos_token_id"][0],
            final_logit_softcapping=d.get("final_logit_softcapping"),
            # the Qwen families carry a sliding_window value that only applies when use_sliding_window is set
            sliding_window=(d.get("sliding_window") if (mt in ("mistral", "phi3") or d.get("use_sliding_window"))
                            else None) or None,
        )

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelArch":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_dict(json.load(f))

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.to_hf_dict(), f, indent=2)

    def to_dict(self) -> dict:
        return asdict(self)

    # attribute aliases so code written against PretrainedConfig keeps working
    @property
    def _name_or_path(self) -> str:
        return self.extra.get("_name_or_path", "")

    @property
    def architectures(self) -> list[str]:
        return self.to_hf_dict()["architectures"]


# ---- named presets (the architectures the benchmark configs quote) ------
PRESETS: dict[str, dict] = {
    "tiny-qwen2": dict(model_type="qwen2", vocab_size=1024, hidden_size=64, intermediate_size=256,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rope_theta=1e6),
    "tiny-llama": dict(model_type="llama", vocab_size=1024, hidden_size=64, intermediate_size=256,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rope_theta=5e5),
    "tiny-qwen3-moe": dict(model_type="qwen3_moe", vocab_size=1024, hidden_size=64, intermediate_size=256,
                           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                           num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64),
    "tiny-mistral": dict(model_type="mistral", vocab_size=1024, hidden_size=64, intermediate_size=256,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2),
    "tiny-phi3": dict(model_type="phi3", vocab_size=1024, hidden_size=64, intermediate_size=256,
                      num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2),
    "tiny-gemma": dict(model_type="gemma", vocab_size=1024, hidden_size=64, intermediate_size=256,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, head_dim=32, rope_theta=10000.0),
    "tiny-qwen3": dict(model_type="qwen3", vocab_size=1024, hidden_size=64, intermediate_size=256,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32),
    "llama-3-8b": dict(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                       num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                       rope_theta=5e5, rms_norm_eps=1e-5, max_position_embeddings=8192),
    "llama-3-70b": dict(model_type="llama", vocab_size=128256, hidden_size=8192, intermediate_size=28672,
                        num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
                        rope_theta=5e5, rms_norm_eps=1e-5, max_position_embeddings=8192),
    "qwen2.5-7b": dict(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                       num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
                       rope_theta=1e6, rms_norm_eps=1e-6),
    "qwen2.5-0.5b": dict(model_type="qwen2", vocab_size=151936, hidden_size=896, intermediate_size=4864,
                         num_hidden_layers=24, num_attention_heads=14, num_key_value_heads=2,
                         rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "qwen3-30b-a3b": dict(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                          num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                          num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                          rope_theta=1e6, rms_norm_eps=1e-6),
}


def preset(name: str, **overrides) -> ModelArch:
    cfg = dict(PRESETS[name])
    cfg.update(overrides)
    return ModelArch(**cfg)
