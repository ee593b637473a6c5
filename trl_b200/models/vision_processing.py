"""Image + text processor for the native vision-language model.

Same call contract as a transformers ``ProcessorMixin`` (the object the reference's vision collator is written
against, trl/trainer/sft_trainer.py:617-760): ``processor(images=..., text=..., padding=..., padding_side=...,
return_tensors="pt")`` returns ``input_ids`` / ``attention_mask`` / ``pixel_values``, ``apply_chat_template`` renders
conversations whose user turns carry ``{"type": "image"}`` blocks, and ``.tokenizer`` is the text tokenizer.  A
transformers processor (for example ``LlavaProcessor``) can be passed to the trainers instead; this one exists so
that the pipeline runs without the Hub.

Every image placeholder in the text is expanded to ``image_seq_length`` copies of the image token, which the model
replaces by the projected patch features.  Images (PIL, numpy HWC uint8, or tensors CHW) are resized to
``image_size`` x ``image_size`` with bilinear interpolation and normalised with the CLIP mean / std.
"""
from __future__ import annotations

import json
import os
from typing import Any

import numpy as np
import torch

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


class VisionProcessor:
    def __init__(self, tokenizer, image_size: int, image_seq_length: int, image_token: str = "<image>",
                 image_mean=CLIP_MEAN, image_std=CLIP_STD):
        self.tokenizer = tokenizer
        self.image_size, self.image_seq_length = int(image_size), int(image_seq_length)
        self.image_token = image_token
        if tokenizer.convert_tokens_to_ids(image_token) in (None, tokenizer.unk_token_id):
            tokenizer.add_special_tokens({"additional_special_tokens": [image_token]})
        self.image_token_id = tokenizer.convert_tokens_to_ids(image_token)
        self.image_mean, self.image_std = tuple(image_mean), tuple(image_std)

    @classmethod
    def for_model(cls, tokenizer, model, **kw) -> "VisionProcessor":
        """Processor matching a ``VisionLanguageModel``; the image token id must agree with the model's config."""
        c = model.config
        p = cls(tokenizer, c.vision.image_size, c.image_seq_length, **kw)
        if p.image_token_id != c.image_token_index:
            raise ValueError(f"tokenizer maps {p.image_token!r} to {p.image_token_id}, the model expects "
                             f"image_token_index={c.image_token_index}")
        return p

    # ---- tokenizer pass-throughs the trainers use -----------------------------------------------------------------
    def __getattr__(self, name):
        if name in ("tokenizer", "__setstate__", "__getstate__"):
            raise AttributeError(name)
        return getattr(self.tokenizer, name)

    @property
    def chat_template(self):
        return self.tokenizer.chat_template

    # ---- images -----------------------------------------------------------------------------------------------------
    def _load(self, img: Any) -> torch.Tensor:
        """Any accepted image form -> float tensor [3, H, W] in [0, 1]."""
        # file paths and the {"path": ..., "bytes": ...} records of an undecoded datasets.Image column are opened here
        if isinstance(img, dict) and ("bytes" in img or "path" in img):
            import io

            from PIL import Image

            img = Image.open(io.BytesIO(img["bytes"])) if img.get("bytes") else Image.open(img["path"])
        elif isinstance(img, (str, os.PathLike)):
            from PIL import Image

            img = Image.open(img)
        if isinstance(img, torch.Tensor):
            t = img.float()
            if t.ndim == 3 and t.shape[0] not in (1, 3) and t.shape[-1] in (1, 3):
                t = t.permute(2, 0, 1)
            if t.max() > 1.5:
                t = t / 255.0
        else:
            a = np.asarray(img.convert("RGB") if hasattr(img, "convert") else img)
            t = torch.from_numpy(a.copy()).float()
            if t.ndim == 2:
                t = t[..., None]
            t = t.permute(2, 0, 1)
            if a.dtype == np.uint8 or t.max() > 1.5:
                t = t / 255.0
        if t.shape[0] == 1:
            t = t.expand(3, -1, -1)
        return t

    def _one_image(self, img: Any) -> torch.Tensor:
        t = self._load(img)
        S = self.image_size
        if t.shape[1:] != (S, S):
            t = torch.nn.functional.interpolate(t[None], size=(S, S), mode="bilinear", align_corners=False,
                                                antialias=True)[0]
        mean = torch.tensor(self.image_mean)[:, None, None]
        std = torch.tensor(self.image_std)[:, None, None]
        return (t - mean) / std

    def preprocess_images(self, images) -> torch.Tensor:
        """A flat list (or list of per-example lists) of images -> [N, 3, S, S]."""
        flat = []
        for x in images:
            flat.extend(x) if isinstance(x, (list, tuple)) else flat.append(x)
        if not flat:
            return torch.zeros(0, 3, self.image_size, self.image_size)
        return torch.stack([self._one_image(i) for i in flat])

    # ---- text -------------------------------------------------------------------------------------------------------
    def apply_chat_template(self, conversation, tokenize: bool = False, **kw):
        """Content blocks become text: ``{"type": "image"}`` -> the image token, ``{"type": "text"}`` -> its text."""
        batched = bool(conversation) and isinstance(conversation[0], list)
        convs = conversation if batched else [conversation]
        out = []
        for msgs in convs:
            flat = []
            for m in msgs:
                c = m.get("content")
                if isinstance(c, list):
                    c = "".join(self.image_token if b.get("type") == "image" else (b.get("text") or "") for b in c)
                flat.append({**m, "content": c})
            out.append(self.tokenizer.apply_chat_template(flat, tokenize=tokenize, **kw))
        return out if batched else out[0]

    def __call__(self, images=None, text=None, padding=False, padding_side=None, pad_to_multiple_of=None,
                 truncation=False, max_length=None, return_tensors=None, add_special_tokens=True, **kw):
        texts = [text] if isinstance(text, str) else list(text)
        vis = self._convert(images, texts) if images is not None else {}
        expanded = self._expand(texts, vis)
        tk = dict(padding=padding, truncation=truncation, max_length=max_length, return_tensors=return_tensors,
                  add_special_tokens=add_special_tokens, pad_to_multiple_of=pad_to_multiple_of)
        if padding_side is not None:
            tk["padding_side"] = padding_side
        out = dict(self.tokenizer(expanded, **tk))
        out.update(vis)
        return out

    def _convert(self, images, texts) -> dict:
        pv = self.preprocess_images(images)
        n_slots = sum(t.count(self.image_token) for t in texts)
        if n_slots != pv.shape[0]:
            raise ValueError(f"{pv.shape[0]} images for {n_slots} image placeholders in the text")
        return {"pixel_values": pv}

    def _expand(self, texts, pv):
        """Image placeholders of the texts -> the run of image tokens the model replaces."""
        return [t.replace(self.image_token, self.image_token * self.image_seq_length) for t in texts]

    def batch_decode(self, *a, **kw):
        return self.tokenizer.batch_decode(*a, **kw)

    def decode(self, *a, **kw):
        return self.tokenizer.decode(*a, **kw)

    def save_pretrained(self, path: str, **kw):
        os.makedirs(path, exist_ok=True)
        self.tokenizer.save_pretrained(path)
        with open(os.path.join(path, "preprocessor_config.json"), "w") as f:
            json.dump({"processor_class": "VisionProcessor", "image_size": self.image_size,
                       "image_seq_length": self.image_seq_length, "image_token": self.image_token,
                       "image_mean": list(self.image_mean), "image_std": list(self.image_std)}, f, indent=2)

    @classmethod
    def from_pretrained(cls, path: str, **kw) -> "VisionProcessor":
        from transformers import AutoTokenizer

        with open(os.path.join(path, "preprocessor_config.json")) as f:
            d = json.load(f)
        return cls(AutoTokenizer.from_pretrained(path), d["image_size"], d["image_seq_length"], d["image_token"],
                   d["image_mean"], d["image_std"])


class DynamicResolutionProcessor(VisionProcessor):
    """Processor of towers that take images of any size as a flat list of patches (Qwen2-VL layout): every image keeps
    its aspect ratio, its sides are rounded to multiples of ``patch_size * merge_size`` with the pixel count kept inside
    ``[min_pixels, max_pixels]``, and it contributes ``(h / patch / merge) * (w / patch / merge)`` image tokens.
    Returns ``pixel_values`` [sum patches, C * temporal * patch * patch] and ``image_grid_thw`` [n_images, 3]."""

    def __init__(self, tokenizer, patch_size: int = 14, merge_size: int = 2, temporal_patch_size: int = 2,
                 min_pixels: int = 56 * 56, max_pixels: int = 28 * 28 * 1280, image_token: str = "<image>",
                 image_mean=CLIP_MEAN, image_std=CLIP_STD):
        super().__init__(tokenizer, image_size=0, image_seq_length=0, image_token=image_token, image_mean=image_mean,
                         image_std=image_std)
        self.patch_size, self.merge_size, self.temporal_patch_size = int(patch_size), int(merge_size), int(temporal_patch_size)
        self.min_pixels, self.max_pixels = int(min_pixels), int(max_pixels)

    @classmethod
    def for_model(cls, tokenizer, model, **kw) -> "DynamicResolutionProcessor":
        v = model.config.vision
        p = cls(tokenizer, v.patch_size, v.spatial_merge_size, v.temporal_patch_size, **kw)
        if p.image_token_id != model.config.image_token_id:
            raise ValueError(f"tokenizer maps {p.image_token!r} to {p.image_token_id}, the model expects "
                             f"image_token_id={model.config.image_token_id}")
        return p

    def target_size(self, h: int, w: int) -> tuple[int, int]:
        """Sides rounded to the merge window, scaled (aspect kept) into the pixel budget."""
        f = self.patch_size * self.merge_size
        if max(h, w) / max(1, min(h, w)) > 200:
            raise ValueError("aspect ratio above 200")
        H, W = max(f, round(h / f) * f), max(f, round(w / f) * f)
        if H * W > self.max_pixels:
            s = (h * w / self.max_pixels) ** 0.5
            H, W = max(f, int(h / s / f) * f), max(f, int(w / s / f) * f)
        elif H * W < self.min_pixels:
            s = (self.min_pixels / (h * w)) ** 0.5
            H, W = -int(-h * s // f) * f, -int(-w * s // f) * f
        return H, W

    def _one_image(self, img: Any) -> torch.Tensor:
        t = self._load(img)
        H, W = self.target_size(t.shape[1], t.shape[2])
        if t.shape[1:] != (H, W):
            t = torch.nn.functional.interpolate(t[None], size=(H, W), mode="bicubic", align_corners=False,
                                                antialias=True)[0].clamp(0.0, 1.0)
        mean = torch.tensor(self.image_mean)[:, None, None]
        std = torch.tensor(self.image_std)[:, None, None]
        return (t - mean) / std

    def preprocess_images(self, images):
        """-> (patches [N, C * T * P * P], grid [n, 3])."""
        from .vision_qwen import QwenVisionArch, patchify

        flat = []
        for x in images:
            flat.extend(x) if isinstance(x, (list, tuple)) else flat.append(x)
        arch = QwenVisionArch(patch_size=self.patch_size, spatial_merge_size=self.merge_size,
                              temporal_patch_size=self.temporal_patch_size)
        if not flat:
            return torch.zeros(0, arch.patch_dim), torch.zeros(0, 3, dtype=torch.long)
        parts = [patchify(self._one_image(i)[None], arch) for i in flat]
        return torch.cat([p for p, _ in parts]), torch.cat([g for _, g in parts])

    def _convert(self, images, texts) -> dict:
        pv, grid = self.preprocess_images(images)
        n_slots = sum(t.count(self.image_token) for t in texts)
        if n_slots != grid.shape[0]:
            raise ValueError(f"{grid.shape[0]} images for {n_slots} image placeholders in the text")
        return {"pixel_values": pv, "image_grid_thw": grid}

    def _expand(self, texts, vis):
        if not vis:
            return list(texts)
        counts = (vis["image_grid_thw"].prod(-1) // (self.merge_size ** 2)).tolist()
        out, k = [], 0
        for t in texts:
            parts = t.split(self.image_token)
            s = parts[0]
            for p in parts[1:]:
                s += self.image_token * int(counts[k]) + p
                k += 1
            out.append(s)
        return out

    def save_pretrained(self, path: str, **kw):
        os.makedirs(path, exist_ok=True)
        self.tokenizer.save_pretrained(path)
        with open(os.path.join(path, "preprocessor_config.json"), "w") as f:
            json.dump({"processor_class": "DynamicResolutionProcessor", "patch_size": self.patch_size,
                       "merge_size": self.merge_size, "temporal_patch_size": self.temporal_patch_size,
                       "min_pixels": self.min_pixels, "max_pixels": self.max_pixels, "image_token": self.image_token,
                       "image_mean": list(self.image_mean), "image_std": list(self.image_std)}, f, indent=2)

    @classmethod
    def from_pretrained(cls, path: str, **kw) -> "DynamicResolutionProcessor":
        from transformers import AutoTokenizer

        with open(os.path.join(path, "preprocessor_config.json")) as f:
            d = json.load(f)
        d.pop("processor_class", None)
        return cls(AutoTokenizer.from_pretrained(path), **d)
