"""Vision-language model: CLIP-style vision tower + MLP projector in front of a native decoder (LLaVA layout).

An image becomes ``(image_size / patch_size)^2`` patch features; the features of a chosen tower layer (default: the
one before the last, class token dropped) go through a two-layer MLP into the decoder's hidden size and REPLACE the
embeddings of the image placeholder tokens, in order.  Everything after that is the ordinary packed decoder
(``CausalLM.forward_hidden`` with ``inputs_embeds``), so the trainers' loss kernels, packing and the sharded engines
see a text model whose forward takes one more tensor.

On disk this is the ``llava`` checkpoint format of transformers (config.json with ``vision_config`` / ``text_config``;
``model.vision_tower.vision_model.*``, ``model.multi_modal_projector.linear_{1,2}.*``, ``model.language_model.*``,
``lm_head.weight``), so checkpoints move both ways.  The reference handles vision-language models by passing
``pixel_values`` through to the transformers model (trl/trainer/sft_trainer.py:538-760 collates them,
trl/trainer/sft_trainer.py:1200-1260 forwards them); here the tower is native.

The tower's GEMMs and attention go through the same ``ops`` entry points as the decoder (library GEMM, varlen
attention with ``causal=False`` over one segment per image).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from .configuration import ModelArch
from .decoder import CausalLM, CausalLMOutput, SeqCtx


@dataclass
class VisionArch:
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    image_size: int = 336
    patch_size: int = 14
    num_channels: int = 3
    layer_norm_eps: float = 1e-5
    hidden_act: str = "quick_gelu"

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        d.update(model_type="clip_vision_model", projection_dim=self.hidden_size)
        return d

    @classmethod
    def from_hf_dict(cls, d: dict) -> "VisionArch":
        keys = cls.__dataclass_fields__.keys()
        return cls(**{k: d[k] for k in keys if k in d})


@dataclass
class VlmArch:
    """LLaVA-style composition.  ``text`` is any native decoder family."""
    text: ModelArch
    vision: VisionArch
    image_token_index: int = 32000
    vision_feature_layer: int = -2
    vision_feature_select_strategy: str = "default"  # "default" drops the class token, "full" keeps it
    projector_hidden_act: str = "gelu"
    multimodal_projector_bias: bool = True
    extra: dict = field(default_factory=dict)

    model_type = "llava"
    is_vlm = True

    def __getattr__(self, name):  # text attributes (vocab_size, hidden_size, eos_token_id, ...) read through
        if name in ("text", "vision", "extra") or name.startswith("__"):
            raise AttributeError(name)
        return getattr(self.text, name)

    @property
    def image_seq_length(self) -> int:
        return self.vision.num_patches + (1 if self.vision_feature_select_strategy == "full" else 0)

    def to_hf_dict(self) -> dict:
        return {
            "architectures": ["LlavaForConditionalGeneration"], "model_type": "llava",
            "image_token_index": self.image_token_index, "image_seq_length": self.image_seq_length,
            "vision_feature_layer": self.vision_feature_layer,
            "vision_feature_select_strategy": self.vision_feature_select_strategy,
            "projector_hidden_act": self.projector_hidden_act,
            "multimodal_projector_bias": self.multimodal_projector_bias,
            "tie_word_embeddings": bool(self.text.tie_word_embeddings),
            "text_config": self.text.to_hf_dict(), "vision_config": self.vision.to_hf_dict(),
        }

    def to_dict(self) -> dict:
        return self.to_hf_dict()

    @classmethod
    def from_hf_dict(cls, d: dict) -> "VlmArch":
        if hasattr(d, "to_dict"):
            d = d.to_dict()
        return cls(text=ModelArch.from_hf_dict(d["text_config"]), vision=VisionArch.from_hf_dict(d["vision_config"]),
                   image_token_index=d.get("image_token_index", d.get("image_token_id", 32000)),
                   vision_feature_layer=d.get("vision_feature_layer", -2),
                   vision_feature_select_strategy=d.get("vision_feature_select_strategy", "default"),
                   projector_hidden_act=d.get("projector_hidden_act", "gelu"),
                   multimodal_projector_bias=d.get("multimodal_projector_bias", True))

    @classmethod
    def from_pretrained(cls, path: str) -> "VlmArch":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_dict(json.load(f))

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.to_hf_dict(), f, indent=2)


def _act(name: str, x: torch.Tensor) -> torch.Tensor:
    if name == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if name in ("gelu_pytorch_tanh", "gelu_new", "gelu_fast"):
        return F.gelu(x, approximate="tanh")
    if name == "gelu":
        return F.gelu(x)
    if name in ("silu", "swish"):
        return F.silu(x)
    raise ValueError(f"unsupported activation {name!r}")


class VisionLayer(nn.Module):
    """Pre-LayerNorm transformer block with biased projections (fused QKV in memory, split on disk)."""

    def __init__(self, cfg: VisionArch, dtype, device):
        super().__init__()
        self.cfg = cfg
        H, I = cfg.hidden_size, cfg.intermediate_size
        kw = dict(dtype=dtype, device=device)
        self.ln1_w, self.ln1_b = nn.Parameter(torch.ones(H, **kw)), nn.Parameter(torch.zeros(H, **kw))
        self.ln2_w, self.ln2_b = nn.Parameter(torch.ones(H, **kw)), nn.Parameter(torch.zeros(H, **kw))
        self.qkv_w, self.qkv_b = nn.Parameter(torch.empty(3 * H, H, **kw)), nn.Parameter(torch.zeros(3 * H, **kw))
        self.out_w, self.out_b = nn.Parameter(torch.empty(H, H, **kw)), nn.Parameter(torch.zeros(H, **kw))
        self.fc1_w, self.fc1_b = nn.Parameter(torch.empty(I, H, **kw)), nn.Parameter(torch.zeros(I, **kw))
        self.fc2_w, self.fc2_b = nn.Parameter(torch.empty(H, I, **kw)), nn.Parameter(torch.zeros(H, **kw))

    def forward(self, x: torch.Tensor, cu: torch.Tensor, seg: int) -> torch.Tensor:
        c = self.cfg
        T, H = x.shape
        nh, hd = c.num_attention_heads, c.hidden_size // c.num_attention_heads
        h = F.layer_norm(x, (H,), self.ln1_w, self.ln1_b, c.layer_norm_eps)
        qkv = ops.linear(h, self.qkv_w, self.qkv_b).reshape(T, 3, nh, hd)
        o = ops.attention_varlen(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, seg, causal=False)
        x = x + ops.linear(o.reshape(T, H), self.out_w, self.out_b)
        h = F.layer_norm(x, (H,), self.ln2_w, self.ln2_b, c.layer_norm_eps)
        return x + ops.linear(_act(c.hidden_act, ops.linear(h, self.fc1_w, self.fc1_b)), self.fc2_w, self.fc2_b)


class ClipVisionTower(nn.Module):
    def __init__(self, cfg: VisionArch, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        H, P = cfg.hidden_size, cfg.patch_size
        kw = dict(dtype=dtype, device=device)
        self.class_embedding = nn.Parameter(torch.empty(H, **kw))
        self.patch_embedding = nn.Parameter(torch.empty(H, cfg.num_channels * P * P, **kw))  # conv kernel, flattened
        self.position_embedding = nn.Parameter(torch.empty(cfg.num_patches + 1, H, **kw))
        self.pre_ln_w, self.pre_ln_b = nn.Parameter(torch.ones(H, **kw)), nn.Parameter(torch.zeros(H, **kw))
        self.post_ln_w, self.post_ln_b = nn.Parameter(torch.ones(H, **kw)), nn.Parameter(torch.zeros(H, **kw))
        self.layers = nn.ModuleList([VisionLayer(cfg, dtype, device) for _ in range(cfg.num_hidden_layers)])

    def forward(self, pixel_values: torch.Tensor, feature_layer: int = -2) -> torch.Tensor:
        """[N, C, S, S] -> hidden states [N, 1 + patches, H] after ``feature_layer`` (index into the list
        [embeddings, layer 1, ..., layer L], negative from the end; the final LayerNorm is not applied, as in LLaVA)."""
        c = self.cfg
        N, C, S, _ = pixel_values.shape
        P, H = c.patch_size, c.hidden_size
        g = S // P
        # a stride-P convolution is a GEMM over unfolded patches
        patches = pixel_values.reshape(N, C, g, P, g, P).permute(0, 2, 4, 1, 3, 5).reshape(N * g * g, C * P * P)
        x = ops.linear(patches.to(self.patch_embedding.dtype), self.patch_embedding).reshape(N, g * g, H)
        x = torch.cat([self.class_embedding.expand(N, 1, H), x], dim=1) + self.position_embedding[None]
        L1 = g * g + 1
        x = F.layer_norm(x, (H,), self.pre_ln_w, self.pre_ln_b, c.layer_norm_eps).reshape(N * L1, H)
        n_run = feature_layer if feature_layer >= 0 else c.num_hidden_layers + 1 + feature_layer
        cu = torch.arange(0, (N + 1) * L1, L1, dtype=torch.int32, device=x.device)
        for layer in self.layers[:n_run]:
            x = layer(x, cu, L1)
        return x.reshape(N, L1, H)


class VisionLanguageModel(nn.Module):
    """``language_model`` (a ``CausalLM``) with image features spliced into its input embeddings."""

    supports_gradient_checkpointing = True
    _is_native = True
    is_vlm = True

    def __init__(self, cfg: VlmArch, dtype=torch.float32, device=None, init: bool = True):
        super().__init__()
        self.config = cfg
        self.language_model = CausalLM(cfg.text, dtype=dtype, device=device, init=init)
        self.vision_tower = ClipVisionTower(cfg.vision, dtype=dtype, device=device)
        kw = dict(dtype=dtype, device=device)
        Hv, Ht = cfg.vision.hidden_size, cfg.text.hidden_size
        self.proj1_w = nn.Parameter(torch.empty(Ht, Hv, **kw))
        self.proj2_w = nn.Parameter(torch.empty(Ht, Ht, **kw))
        if cfg.multimodal_projector_bias:
            self.proj1_b, self.proj2_b = nn.Parameter(torch.zeros(Ht, **kw)), nn.Parameter(torch.zeros(Ht, **kw))
        else:
            self.proj1_b = self.proj2_b = None
        self.name_or_path = ""
        self.generation_config = None
        self.warnings_issued = {}
        if init and (device is None or str(device) != "meta"):
            self.reset_vision_parameters()

    @torch.no_grad()
    def reset_vision_parameters(self, std: float = 0.02):
        for mod in (self.vision_tower, ):
            for name, p in mod.named_parameters():
                if p.ndim >= 2 or name in ("class_embedding",):
                    p.normal_(0.0, std)
        self.proj1_w.normal_(0.0, std)
        self.proj2_w.normal_(0.0, std)

    # ---- what the trainers read -------------------------------------------------------------------------------------
    @property
    def lm_head_weight(self):
        return self.language_model.lm_head_weight

    @property
    def layers(self):
        return self.language_model.layers

    @property
    def device(self):
        return self.language_model.device

    @property
    def dtype(self):
        return self.language_model.dtype

    @property
    def gradient_checkpointing(self):
        return self.language_model.gradient_checkpointing

    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs=None):
        self.language_model.gradient_checkpointing_enable(gradient_checkpointing_kwargs)

    def gradient_checkpointing_disable(self):
        self.language_model.gradient_checkpointing_disable()

    @property
    def is_gradient_checkpointing(self):
        return self.language_model.gradient_checkpointing

    def enable_input_require_grads(self):
        pass

    def get_input_embeddings(self):
        return self.language_model.embed_tokens

    def num_parameters(self, only_trainable=False):
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not only_trainable)

    def aux_loss(self, ctx, token_mask=None):
        return self.language_model.aux_loss(ctx, token_mask)

    def pack_inputs(self, input_ids, attention_mask=None, position_ids=None):
        return self.language_model.pack_inputs(input_ids, attention_mask, position_ids)

    # ---- forward ----------------------------------------------------------------------------------------------------
    def image_features(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """[N, C, S, S] -> [N * image_seq_length, H_text]."""
        c = self.config
        h = self.vision_tower(pixel_values, c.vision_feature_layer)
        if c.vision_feature_select_strategy == "default":
            h = h[:, 1:]
        h = h.reshape(-1, h.shape[-1])
        h = _act(c.projector_hidden_act, ops.linear(h, self.proj1_w, self.proj1_b))
        return ops.linear(h, self.proj2_w, self.proj2_b)

    def forward_hidden(self, input_ids: torch.Tensor, ctx: SeqCtx, pixel_values: Optional[torch.Tensor] = None):
        """Flat ids [T] (+ images of the packed batch, in reading order) -> final-norm hidden [T, H]."""
        lm = self.language_model
        x = lm.embed(input_ids)
        if pixel_values is not None and pixel_values.numel():
            feats = self.image_features(pixel_values).to(x.dtype)
            slots = (input_ids == self.config.image_token_index).nonzero().flatten()
            if slots.numel() != feats.shape[0]:
                raise ValueError(f"image placeholder tokens ({slots.numel()}) and image features ({feats.shape[0]}) "
                                 f"do not match: every image needs {self.config.image_seq_length} placeholder tokens")
            x = x.index_copy(0, slots, feats)
        return lm.forward_hidden(input_ids, ctx, inputs_embeds=x)

    def forward(self, input_ids=None, attention_mask=None, pixel_values=None, position_ids=None, labels=None,
                logits_to_keep: int | None = None, **unused):
        lm = self.language_model
        flat, ctx, scatter = lm.pack_inputs(input_ids, attention_mask, position_ids)
        hp = scatter(self.forward_hidden(flat, ctx, pixel_values))
        if logits_to_keep:
            hp = hp[:, -logits_to_keep:]
        out = CausalLMOutput()
        out.logits = ops.linear(hp, self.lm_head_weight)
        if labels is not None:
            labels = labels.masked_fill(labels == self.config.image_token_index, -100)  # placeholders carry no target
            sl = out.logits[:, :-1].reshape(-1, out.logits.shape[-1]).float()
            out.loss = F.cross_entropy(sl, labels[:, 1:].reshape(-1), ignore_index=-100)
        return out

    # ---- checkpoints (transformers "llava" layout) ------------------------------------------------------------------
    def hf_state_dict(self) -> dict[str, torch.Tensor]:
        from .hf_io import to_hf_state_dict

        sd = {}
        for k, v in to_hf_state_dict(self.language_model).items():
            if k.startswith("model."):
                sd["model.language_model." + k[len("model."):]] = v
            else:
                sd[k] = v  # lm_head.weight
        vt, pre = self.vision_tower, "model.vision_tower.vision_model."
        c = self.config.vision
        sd[pre + "embeddings.class_embedding"] = vt.class_embedding.detach()
        sd[pre + "embeddings.patch_embedding.weight"] = vt.patch_embedding.detach().reshape(
            c.hidden_size, c.num_channels, c.patch_size, c.patch_size)
        sd[pre + "embeddings.position_embedding.weight"] = vt.position_embedding.detach()
        sd[pre + "pre_layrnorm.weight"], sd[pre + "pre_layrnorm.bias"] = vt.pre_ln_w.detach(), vt.pre_ln_b.detach()
        sd[pre + "post_layernorm.weight"], sd[pre + "post_layernorm.bias"] = vt.post_ln_w.detach(), vt.post_ln_b.detach()
        H = c.hidden_size
        for i, l in enumerate(vt.layers):
            p = f"{pre}encoder.layers.{i}."
            for j, n in enumerate(("q_proj", "k_proj", "v_proj")):
                sd[p + f"self_attn.{n}.weight"] = l.qkv_w.detach()[j * H:(j + 1) * H]
                sd[p + f"self_attn.{n}.bias"] = l.qkv_b.detach()[j * H:(j + 1) * H]
            sd[p + "self_attn.out_proj.weight"], sd[p + "self_attn.out_proj.bias"] = l.out_w.detach(), l.out_b.detach()
            sd[p + "layer_norm1.weight"], sd[p + "layer_norm1.bias"] = l.ln1_w.detach(), l.ln1_b.detach()
            sd[p + "layer_norm2.weight"], sd[p + "layer_norm2.bias"] = l.ln2_w.detach(), l.ln2_b.detach()
            sd[p + "mlp.fc1.weight"], sd[p + "mlp.fc1.bias"] = l.fc1_w.detach(), l.fc1_b.detach()
            sd[p + "mlp.fc2.weight"], sd[p + "mlp.fc2.bias"] = l.fc2_w.detach(), l.fc2_b.detach()
        mp = "model.multi_modal_projector."
        sd[mp + "linear_1.weight"], sd[mp + "linear_2.weight"] = self.proj1_w.detach(), self.proj2_w.detach()
        if self.proj1_b is not None:
            sd[mp + "linear_1.bias"], sd[mp + "linear_2.bias"] = self.proj1_b.detach(), self.proj2_b.detach()
        return {k: v.contiguous() for k, v in sd.items()}

    @torch.no_grad()
    def load_hf_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        from .hf_io import load_hf_state_dict

        # key layouts seen in the wild: "model.language_model.*" (in memory, transformers >= 4.52),
        # "language_model.model.*" + "language_model.lm_head.weight" (older files) and the mix of both that
        # transformers 5 writes ("model.language_model.model.*")
        text = {}
        for k, v in sd.items():
            if k in ("lm_head.weight", "language_model.lm_head.weight", "model.language_model.lm_head.weight"):
                text["lm_head.weight"] = v
                continue
            for pre in ("model.language_model.model.", "language_model.model.", "model.language_model."):
                if k.startswith(pre):
                    text["model." + k[len(pre):]] = v
                    break
        load_hf_state_dict(self.language_model, text, strict=True)
        vt, c = self.vision_tower, self.config.vision
        pre = "model.vision_tower.vision_model." if any(k.startswith("model.vision_tower.") for k in sd) \
            else "vision_tower.vision_model."
        mp = "model.multi_modal_projector." if any(k.startswith("model.multi_modal_projector.") for k in sd) \
            else "multi_modal_projector."

        def put(param, t):
            param.copy_(t.reshape(param.shape).to(param.dtype))

        put(vt.class_embedding, sd[pre + "embeddings.class_embedding"])
        put(vt.patch_embedding, sd[pre + "embeddings.patch_embedding.weight"])
        put(vt.position_embedding, sd[pre + "embeddings.position_embedding.weight"])
        put(vt.pre_ln_w, sd[pre + "pre_layrnorm.weight"]), put(vt.pre_ln_b, sd[pre + "pre_layrnorm.bias"])
        put(vt.post_ln_w, sd[pre + "post_layernorm.weight"]), put(vt.post_ln_b, sd[pre + "post_layernorm.bias"])
        for i, l in enumerate(vt.layers):
            p = f"{pre}encoder.layers.{i}."
            put(l.qkv_w, torch.cat([sd[p + f"self_attn.{n}.weight"] for n in ("q_proj", "k_proj", "v_proj")]))
            put(l.qkv_b, torch.cat([sd[p + f"self_attn.{n}.bias"] for n in ("q_proj", "k_proj", "v_proj")]))
            put(l.out_w, sd[p + "self_attn.out_proj.weight"]), put(l.out_b, sd[p + "self_attn.out_proj.bias"])
            put(l.ln1_w, sd[p + "layer_norm1.weight"]), put(l.ln1_b, sd[p + "layer_norm1.bias"])
            put(l.ln2_w, sd[p + "layer_norm2.weight"]), put(l.ln2_b, sd[p + "layer_norm2.bias"])
            put(l.fc1_w, sd[p + "mlp.fc1.weight"]), put(l.fc1_b, sd[p + "mlp.fc1.bias"])
            put(l.fc2_w, sd[p + "mlp.fc2.weight"]), put(l.fc2_b, sd[p + "mlp.fc2.bias"])
        put(self.proj1_w, sd[mp + "linear_1.weight"]), put(self.proj2_w, sd[mp + "linear_2.weight"])
        if self.proj1_b is not None:
            put(self.proj1_b, sd[mp + "linear_1.bias"]), put(self.proj2_b, sd[mp + "linear_2.bias"])

    def state_dict_for_save(self):
        return self.hf_state_dict()

    def save_pretrained(self, path: str, state_dict=None, safe_serialization: bool = True, **unused):
        from .hf_io import save_state_dict_sharded

        os.makedirs(path, exist_ok=True)
        self.config.save_pretrained(path)
        save_state_dict_sharded(state_dict if state_dict is not None else self.hf_state_dict(), path)
        t = self.config.text
        with open(os.path.join(path, "generation_config.json"), "w") as f:
            json.dump({"_from_model_config": True, "bos_token_id": t.bos_token_id, "eos_token_id": t.eos_token_id,
                       "pad_token_id": t.pad_token_id}, f, indent=2)

    @classmethod
    def from_pretrained(cls, path: str, dtype=None, device=None, **unused) -> "VisionLanguageModel":
        from .hf_io import load_state_dict_dir, resolve_dtype

        cfg = VlmArch.from_pretrained(path)
        model = cls(cfg, dtype=resolve_dtype(dtype) or torch.float32, device=device)
        model.load_hf_state_dict(load_state_dict_dir(path))
        model.name_or_path = path
        return model


def tiny_vlm_arch(text_preset: str = "tiny-llama", image_token_index: int = 5) -> VlmArch:
    """A few-thousand-parameter LLaVA for tests: 28 x 28 images, 14 x 14 patches (4 image tokens per image)."""
    from .configuration import preset

    vis = VisionArch(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, image_size=28,
                     patch_size=14)
    return VlmArch(text=preset(text_preset), vision=vis, image_token_index=image_token_index)


# ---- per-sequence image inputs ------------------------------------------------------------------------------------------
# The online trainers and the rollout engines carry the images of every sequence as one "entry": a tensor
# [n_images, C, S, S] for fixed-resolution towers, or a pair (patches [N, D], grid [n_images, 3]) for towers that take
# images of any size as a flat list of patches.  These helpers are the only code that looks inside an entry.
def vision_entry_numel(e) -> int:
    if e is None:
        return 0
    return int((e[0] if isinstance(e, tuple) else e).numel())


def same_vision_entry(a, b) -> bool:
    if a is None or b is None:
        return a is None and b is None
    if isinstance(a, tuple) != isinstance(b, tuple):
        return False
    xs, ys = (a, b) if isinstance(a, tuple) else ((a,), (b,))
    return all(x.shape == y.shape and torch.equal(x, y) for x, y in zip(xs, ys))


def merge_vision_entries(entries, device, dtype=None) -> dict:
    """Entries of the sequences of one packed batch, in order -> keyword arguments of ``forward_hidden``."""
    live = [e for e in entries if vision_entry_numel(e)]
    if not live:
        return {"pixel_values": None}
    if isinstance(live[0], tuple):
        return {"pixel_values": torch.cat([e[0] for e in live]).to(device, dtype),
                "image_grid_thw": torch.cat([e[1] for e in live]).to(device)}
    return {"pixel_values": torch.cat(live).to(device, dtype)}


def split_vision_batch(enc: dict, counts: list[int]) -> list:
    """Output of a processor for a batch whose example i has ``counts[i]`` images -> one entry per example."""
    pv, grid = enc.get("pixel_values"), enc.get("image_grid_thw")
    if pv is None:
        return [None] * len(counts)
    pv = torch.as_tensor(pv)
    out, o = [], 0
    if grid is None:
        for n in counts:
            out.append(pv[o:o + n])
            o += n
        return out
    grid = torch.as_tensor(grid)
    per_image = grid.prod(-1).tolist()
    po = 0
    for n in counts:
        k = sum(per_image[o:o + n])
        out.append((pv[po:po + k], grid[o:o + n]) if n else None)
        o, po = o + n, po + k
    return out
