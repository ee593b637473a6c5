"""Qwen2-VL-style vision-language model: dynamic-resolution vision tower + native decoder with multimodal RoPE.

What differs from the LLaVA composition in ``vision.py``:

* images are not resized to one square: the processor cuts every image (or video frame pair) into 14 x 14 patches,
  ``pixel_values`` is the flat list of patches of all images ``[sum_i t_i h_i w_i, C * 2 * 14 * 14]`` and
  ``image_grid_thw`` ``[n_images, 3]`` says how many patches every image has along time, height and width;
* the tower runs full (non-causal) attention inside every image (``cu_seqlens`` from the grid) with a 2-D rotary
  embedding over (row, column), then merges every 2 x 2 block of patches into one token of the language model;
* the language model rotates with three position rows (temporal, height, width): text tokens carry the same value in
  all three, the tokens of an image carry their grid coordinates (``rope_index``), so an image of 1000 tokens advances
  the text position only by the larger side of its grid.

Checkpoints use the transformers layout (``model.visual.*``, ``model.language_model.*``, ``lm_head.weight``); the
logits are checked against ``transformers.Qwen2VLForConditionalGeneration`` in ``tests/test_vision_cpu.py``.
The reference trains these models through transformers (trl/trainer/sft_trainer.py:1144-1162 collates
``pixel_values`` + ``image_grid_thw``; trl/trainer/utils.py:995-1076 ``split_pixel_values_by_grid``)."""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from .configuration import ModelArch
from .decoder import CausalLM, CausalLMOutput, SeqCtx


@dataclass
class QwenVisionArch:
    depth: int = 2
    embed_dim: int = 32
    hidden_size: int = 64  # output width = hidden size of the language model
    num_heads: int = 2
    mlp_ratio: int = 4
    in_channels: int = 3
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    hidden_act: str = "quick_gelu"

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


@dataclass
class Qwen2VLArch:
    text: ModelArch = field(default_factory=ModelArch)
    vision: QwenVisionArch = field(default_factory=QwenVisionArch)
    image_token_id: int = 5
    video_token_id: int = 6
    vision_start_token_id: int = 3
    vision_end_token_id: int = 4
    model_type: str = "qwen2_vl"

    def __getattr__(self, name):  # text attributes (vocab_size, hidden_size, eos_token_id, ...) read through
        if name in ("text", "vision") or name.startswith("__"):
            raise AttributeError(name)
        return getattr(self.text, name)

    @property
    def image_token_index(self) -> int:
        return self.image_token_id

    def to_hf_dict(self) -> dict:
        t = self.text.to_hf_dict()
        t["rope_scaling"] = {"type": "mrope", "mrope_section": list(self.text.extra.get("mrope_section", []))}
        t["model_type"] = "qwen2_vl_text"
        v = asdict(self.vision)
        v["model_type"] = "qwen2_vl"
        return {"architectures": ["Qwen2VLForConditionalGeneration"], "model_type": "qwen2_vl", "text_config": t,
                "vision_config": v, "image_token_id": self.image_token_id, "video_token_id": self.video_token_id,
                "vision_start_token_id": self.vision_start_token_id, "vision_end_token_id": self.vision_end_token_id,
                "tie_word_embeddings": self.text.tie_word_embeddings}

    to_dict = to_hf_dict

    @classmethod
    def from_hf_dict(cls, d: dict) -> "Qwen2VLArch":
        t = dict(d.get("text_config") or {})
        rs = t.get("rope_scaling") or t.get("rope_parameters") or d.get("rope_scaling") or {}
        t["model_type"] = "qwen2"
        text = ModelArch.from_hf_dict(t)
        text.extra["mrope_section"] = list(rs.get("mrope_section", []))
        vkeys = {f for f in QwenVisionArch.__dataclass_fields__}
        vision = QwenVisionArch(**{k: v for k, v in (d.get("vision_config") or {}).items() if k in vkeys})
        return cls(text, vision, d.get("image_token_id", 5), d.get("video_token_id", 6),
                   d.get("vision_start_token_id", 3), d.get("vision_end_token_id", 4))

    @classmethod
    def from_pretrained(cls, path: str) -> "Qwen2VLArch":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_dict(json.load(f))

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.to_hf_dict(), f, indent=2)


def _vision_rope(x: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
    """x [N, heads, d]; ang [N, d/2] (row angles then column angles): rotate-half with the angles repeated over both
    halves, computed in fp32."""
    cos, sin = torch.cat([ang, ang], -1).cos()[:, None, :], torch.cat([ang, ang], -1).sin()[:, None, :]
    xf = x.float()
    half = x.shape[-1] // 2
    rot = torch.cat([-xf[..., half:], xf[..., :half]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


class QwenVisionBlock(nn.Module):
    def __init__(self, cfg: QwenVisionArch, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        D, M = cfg.embed_dim, int(cfg.embed_dim * cfg.mlp_ratio)
        self.heads = cfg.num_heads
        self.norm1_w, self.norm1_b = nn.Parameter(torch.ones(D, **kw)), nn.Parameter(torch.zeros(D, **kw))
        self.norm2_w, self.norm2_b = nn.Parameter(torch.ones(D, **kw)), nn.Parameter(torch.zeros(D, **kw))
        self.qkv_w, self.qkv_b = nn.Parameter(torch.empty(3 * D, D, **kw)), nn.Parameter(torch.zeros(3 * D, **kw))
        self.proj_w, self.proj_b = nn.Parameter(torch.empty(D, D, **kw)), nn.Parameter(torch.zeros(D, **kw))
        self.fc1_w, self.fc1_b = nn.Parameter(torch.empty(M, D, **kw)), nn.Parameter(torch.zeros(M, **kw))
        self.fc2_w, self.fc2_b = nn.Parameter(torch.empty(D, M, **kw)), nn.Parameter(torch.zeros(D, **kw))

    def forward(self, x, ang, cu, max_len):
        N, D = x.shape
        h = F.layer_norm(x, (D,), self.norm1_w, self.norm1_b, 1e-6)
        qkv = ops.linear(h, self.qkv_w, self.qkv_b).reshape(N, 3, self.heads, D // self.heads)
        q, k, v = _vision_rope(qkv[:, 0], ang), _vision_rope(qkv[:, 1], ang), qkv[:, 2]
        o = ops.attention_varlen(q.contiguous(), k.contiguous(), v.contiguous(), cu, max_len, causal=False)
        x = x + ops.linear(o.reshape(N, D), self.proj_w, self.proj_b)
        h = F.layer_norm(x, (D,), self.norm2_w, self.norm2_b, 1e-6)
        h = ops.linear(h, self.fc1_w, self.fc1_b)
        h = h * torch.sigmoid(1.702 * h)  # quick_gelu
        return x + ops.linear(h, self.fc2_w, self.fc2_b)


class QwenVisionTower(nn.Module):
    def __init__(self, cfg: QwenVisionArch, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        D, m2 = cfg.embed_dim, cfg.spatial_merge_size ** 2
        self.patch_w = nn.Parameter(torch.empty(D, cfg.patch_dim, **kw))  # the strided 3-D convolution as a matrix
        self.blocks = nn.ModuleList([QwenVisionBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        self.ln_q_w, self.ln_q_b = nn.Parameter(torch.ones(D, **kw)), nn.Parameter(torch.zeros(D, **kw))
        self.merge1_w, self.merge1_b = nn.Parameter(torch.empty(D * m2, D * m2, **kw)), nn.Parameter(torch.zeros(D * m2, **kw))
        self.merge2_w = nn.Parameter(torch.empty(cfg.hidden_size, D * m2, **kw))
        self.merge2_b = nn.Parameter(torch.zeros(cfg.hidden_size, **kw))

    def rot_angles(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """[N, head_dim / 2]: (row, column) of every patch, in the processor's order (2 x 2 merge windows are
        contiguous), times the inverse frequencies of a rotary embedding of width head_dim / 2 per axis."""
        c = self.cfg
        m = c.spatial_merge_size
        hd = c.embed_dim // c.num_heads
        pos = []
        for t, h, w in grid_thw.tolist():
            rows = torch.arange(h)[:, None].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            cols = torch.arange(w)[None, :].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            pos.append(torch.stack([rows, cols], -1).repeat(t, 1))
        pos = torch.cat(pos).to(grid_thw.device)
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32, device=pos.device) / (hd // 2)))
        ang = pos.float()[:, :, None] * inv[None, None, :]  # [N, 2, hd / 4]
        return ang.flatten(1)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """[N patches, C * T * P * P], [n_images, 3] -> [N / merge^2, hidden_size]."""
        c = self.cfg
        x = ops.linear(pixel_values.to(self.patch_w.dtype), self.patch_w)
        ang = self.rot_angles(grid_thw)
        per_frame = (grid_thw[:, 1] * grid_thw[:, 2]).repeat_interleave(grid_thw[:, 0])  # attention stays inside a frame
        cu = F.pad(per_frame.cumsum(0), (1, 0)).to(torch.int32).to(x.device)
        max_len = int(per_frame.max())
        for blk in self.blocks:
            x = blk(x, ang, cu, max_len)
        x = F.layer_norm(x, (c.embed_dim,), self.ln_q_w, self.ln_q_b, 1e-6).reshape(-1, c.embed_dim * c.spatial_merge_size ** 2)
        x = F.gelu(ops.linear(x, self.merge1_w, self.merge1_b))
        return ops.linear(x, self.merge2_w, self.merge2_b)


def rope_index(input_ids: torch.Tensor, cu_seqlens: torch.Tensor, grid_thw: Optional[torch.Tensor], cfg: Qwen2VLArch):
    """Multimodal rotary positions [3, T] of a packed stream.  Per sequence: text tokens count up with the same value
    in the three rows; the ``t * (h / m) * (w / m)`` placeholder tokens of an image take (frame, row, column) offsets
    from the position where the image starts; the text after it continues at the largest value used so far + 1.
    Tensor operations only (no loop over tokens): the stream may be a whole packed batch."""
    dev = input_ids.device
    T = input_ids.numel()
    cu = cu_seqlens.to(dev).long()
    lens = cu[1:] - cu[:-1]
    seq_of = torch.repeat_interleave(torch.arange(lens.numel(), device=dev), lens, output_size=T)
    adv = torch.ones(T, dtype=torch.long, device=dev)          # how far every token moves the text position
    img_pos = None
    if grid_thw is not None and grid_thw.numel():
        m = cfg.vision.spatial_merge_size
        g = grid_thw.to(dev).long()
        t, gh, gw = g[:, 0], g[:, 1] // m, g[:, 2] // m
        n = t * gh * gw                                         # placeholder tokens per image
        total = int(n.sum())
        slots = (input_ids == cfg.image_token_id).nonzero().flatten()
        if slots.numel() < total:
            raise ValueError("an image's placeholder tokens run past the end of their sequence")
        slots = slots[:total]                                   # placeholders beyond the images count as text
        first = torch.cumsum(n, 0) - n                          # index into `slots` of every image's first token
        start, last = slots[first], slots[first + n - 1]
        if bool(((last - start) != n - 1).any()) or bool((seq_of[start] != seq_of[last]).any()):
            raise ValueError("an image's placeholder tokens run past the end of their sequence")
        adv[slots] = 0
        adv[start] = torch.maximum(t, torch.maximum(gh, gw))
        img_of = torch.repeat_interleave(torch.arange(n.numel(), device=dev), n, output_size=total)
        r = torch.arange(total, device=dev) - first[img_of]     # index of the token inside its image
        hw = (gh * gw)[img_of]
        img_pos = (slots, img_of, torch.stack([r // hw, (r // gw[img_of]) % gh[img_of], r % gw[img_of]]))
    before = torch.cumsum(adv, 0) - adv                         # text position if the stream were one sequence
    pos = before - before[cu[:-1]][seq_of]                      # ... restarted at every sequence
    out = pos[None].repeat(3, 1)
    if img_pos is not None:
        slots, img_of, offs = img_pos
        base = pos[slots[(torch.cumsum(n, 0) - n)]]             # position at which every image starts
        out[:, slots] = base[img_of][None] + offs
    return out


class Qwen2VLModel(nn.Module):
    """``language_model`` (a ``CausalLM`` with multimodal RoPE) fed with merged patch features of ``visual``."""

    supports_gradient_checkpointing = True
    _is_native = True
    is_vlm = True

    def __init__(self, cfg: Qwen2VLArch, dtype=torch.float32, device=None, init: bool = True):
        super().__init__()
        self.config = cfg
        if not cfg.text.extra.get("mrope_section"):
            raise ValueError("the text configuration needs extra['mrope_section'] (sizes summing to head_dim / 2)")
        self.language_model = CausalLM(cfg.text, dtype=dtype, device=device, init=init)
        self.visual = QwenVisionTower(cfg.vision, dtype=dtype, device=device)
        self.name_or_path = ""
        self.generation_config = None
        self.warnings_issued = {}
        if init and (device is None or str(device) != "meta"):
            with torch.no_grad():
                for p in self.visual.parameters():
                    if p.ndim >= 2:
                        p.normal_(0.0, 0.02)

    lm_head_weight = property(lambda self: self.language_model.lm_head_weight)
    layers = property(lambda self: self.language_model.layers)
    device = property(lambda self: self.language_model.device)
    dtype = property(lambda self: self.language_model.dtype)
    gradient_checkpointing = property(lambda self: self.language_model.gradient_checkpointing)
    is_gradient_checkpointing = property(lambda self: self.language_model.gradient_checkpointing)

    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs=None):
        self.language_model.gradient_checkpointing_enable(gradient_checkpointing_kwargs)

    def gradient_checkpointing_disable(self):
        self.language_model.gradient_checkpointing_disable()

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

    def image_features(self, pixel_values: torch.Tensor, image_grid_thw: torch.Tensor) -> torch.Tensor:
        """Patches of all images [N, C * T * P * P] + their grids -> merged features [N / merge^2, H_text]."""
        if image_grid_thw is None:
            raise ValueError("this model takes images as flat patches: pass image_grid_thw with pixel_values")
        return self.visual(pixel_values, image_grid_thw)

    def forward_hidden(self, input_ids: torch.Tensor, ctx: SeqCtx, pixel_values: Optional[torch.Tensor] = None,
                       image_grid_thw: Optional[torch.Tensor] = None):
        """Flat ids [T] (+ the patches and grids of the batch's images, in reading order) -> final-norm hidden [T, H]."""
        lm = self.language_model
        x = lm.embed(input_ids)
        if pixel_values is not None and pixel_values.numel():
            feats = self.image_features(pixel_values, image_grid_thw).to(x.dtype)
            slots = (input_ids == self.config.image_token_id).nonzero().flatten()
            if slots.numel() != feats.shape[0]:
                raise ValueError(f"image placeholder tokens ({slots.numel()}) and merged patch features "
                                 f"({feats.shape[0]}) do not match")
            x = x.index_copy(0, slots, feats)
        ctx.mrope_positions = rope_index(input_ids, ctx.cu_seqlens, image_grid_thw, self.config)
        return lm.forward_hidden(input_ids, ctx, inputs_embeds=x)

    def forward(self, input_ids=None, attention_mask=None, pixel_values=None, image_grid_thw=None, position_ids=None,
                labels=None, logits_to_keep: int | None = None, **unused):
        lm = self.language_model
        flat, ctx, scatter = lm.pack_inputs(input_ids, attention_mask, position_ids)
        hp = scatter(self.forward_hidden(flat, ctx, pixel_values, image_grid_thw))
        if logits_to_keep:
            hp = hp[:, -logits_to_keep:]
        out = CausalLMOutput()
        out.logits = ops.linear(hp, self.lm_head_weight)
        if labels is not None:
            labels = labels.masked_fill(labels == self.config.image_token_id, -100)
            sl = out.logits[:, :-1].reshape(-1, out.logits.shape[-1]).float()
            out.loss = F.cross_entropy(sl, labels[:, 1:].reshape(-1), ignore_index=-100)
        return out

    # ---- checkpoints (transformers "qwen2_vl" layout) ---------------------------------------------------------------
    _BLOCK_KEYS = {"norm1.weight": "norm1_w", "norm1.bias": "norm1_b", "norm2.weight": "norm2_w", "norm2.bias": "norm2_b",
                   "attn.qkv.weight": "qkv_w", "attn.qkv.bias": "qkv_b", "attn.proj.weight": "proj_w",
                   "attn.proj.bias": "proj_b", "mlp.fc1.weight": "fc1_w", "mlp.fc1.bias": "fc1_b",
                   "mlp.fc2.weight": "fc2_w", "mlp.fc2.bias": "fc2_b"}
    _TOWER_KEYS = {"merger.ln_q.weight": "ln_q_w", "merger.ln_q.bias": "ln_q_b", "merger.mlp.0.weight": "merge1_w",
                   "merger.mlp.0.bias": "merge1_b", "merger.mlp.2.weight": "merge2_w", "merger.mlp.2.bias": "merge2_b"}

    def hf_state_dict(self) -> dict[str, torch.Tensor]:
        from .hf_io import to_hf_state_dict

        sd = {}
        for k, v in to_hf_state_dict(self.language_model).items():
            sd[k if k.startswith("lm_head") else "model.language_model." + k[len("model."):]] = v
        c = self.config.vision
        sd["model.visual.patch_embed.proj.weight"] = self.visual.patch_w.detach().reshape(
            c.embed_dim, c.in_channels, c.temporal_patch_size, c.patch_size, c.patch_size)
        for i, b in enumerate(self.visual.blocks):
            for hk, ok in self._BLOCK_KEYS.items():
                sd[f"model.visual.blocks.{i}.{hk}"] = getattr(b, ok).detach()
        for hk, ok in self._TOWER_KEYS.items():
            sd[f"model.visual.{hk}"] = getattr(self.visual, ok).detach()
        return sd

    @torch.no_grad()
    def load_hf_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        from .hf_io import load_hf_state_dict

        # layouts seen: "model.language_model.*" + "model.visual.*" (in memory), "model.*" + "visual.*" (files of the
        # original release) and the mix transformers 5 writes ("model.layers.*" beside "model.visual.*")
        text = {}
        for k, v in sd.items():
            if k.startswith("model.language_model."):
                text["model." + k[len("model.language_model."):]] = v
            elif k.startswith("lm_head.") or (k.startswith("model.") and not k.startswith("model.visual.")):
                text[k] = v
        load_hf_state_dict(self.language_model, text, strict=True)
        pre = "model.visual." if any(k.startswith("model.visual.") for k in sd) else "visual."
        self.visual.patch_w.copy_(sd[pre + "patch_embed.proj.weight"].reshape(self.visual.patch_w.shape))
        for i, b in enumerate(self.visual.blocks):
            for hk, ok in self._BLOCK_KEYS.items():
                getattr(b, ok).copy_(sd[f"{pre}blocks.{i}.{hk}"])
        for hk, ok in self._TOWER_KEYS.items():
            getattr(self.visual, ok).copy_(sd[pre + hk])

    def state_dict_for_save(self):
        return self.hf_state_dict()

    def save_pretrained(self, path: str, state_dict=None, safe_serialization: bool = True, **unused):
        from .hf_io import save_state_dict_sharded

        self.config.save_pretrained(path)
        save_state_dict_sharded(state_dict if state_dict is not None else self.hf_state_dict(), path)

    @classmethod
    def from_pretrained(cls, path: str, dtype=None, device=None, **unused) -> "Qwen2VLModel":
        from .hf_io import load_state_dict_dir, resolve_dtype

        cfg = Qwen2VLArch.from_pretrained(path)
        model = cls(cfg, dtype=resolve_dtype(dtype) or torch.float32, device=device, init=False)
        model.load_hf_state_dict(load_state_dict_dir(path))
        model.name_or_path = path
        return model


def patchify(images: torch.Tensor, cfg: QwenVisionArch):
    """Images [n, C, H, W] (H and W multiples of ``patch_size * spatial_merge_size``; already normalised) ->
    (pixel_values [sum patches, C * T * P * P], image_grid_thw [n, 3]) in the order the tower expects: a still image
    is repeated ``temporal_patch_size`` times along time, patches of one 2 x 2 merge window are contiguous."""
    n, C, H, W = images.shape
    P, m, T = cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size
    if H % (P * m) or W % (P * m):
        raise ValueError(f"image sides must be multiples of {P * m}")
    gh, gw = H // P, W // P
    x = images[:, None].expand(n, T, C, H, W)                                   # one temporal patch per still image
    x = x.reshape(n, T, C, gh // m, m, P, gw // m, m, P)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                                    # [n, gh/m, gw/m, m, m, C, T, P, P]
    pixel_values = x.reshape(n * gh * gw, C * T * P * P)
    grid = torch.tensor([[1, gh, gw]] * n, dtype=torch.long)
    return pixel_values, grid


def tiny_qwen2_vl_arch() -> Qwen2VLArch:
    text = ModelArch(model_type="qwen2", vocab_size=1024, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, rope_theta=10000.0, extra={"mrope_section": [2, 3, 3]})
    return Qwen2VLArch(text, QwenVisionArch(depth=2, embed_dim=32, hidden_size=64, num_heads=2, mlp_ratio=2))
