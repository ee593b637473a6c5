"""Native LoRA with PEFT-compatible artefacts.

peft is not importable here, so adapters are implemented on the native decoder
(`DecoderLayer.lora`) and saved the PEFT way: ``adapter_config.json`` +
``adapter_model.safetensors`` with keys
``base_model.model.model.layers.N.self_attn.q_proj.lora_{A,B}.weight``.
Mirrors how the reference obtains adapters through ``peft.get_peft_model``
(trl/trainer/sft_trainer.py:1039-1130) and its ``get_peft_config``
(trl/trainer/utils.py:254-277).
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Optional

import torch

_ATTN = ("q_proj", "k_proj", "v_proj", "o_proj")
_MLP = ("gate_proj", "up_proj", "down_proj")


@dataclass
class LoraConfig:
    r: int = 16
    lora_alpha: int = 32
    lora_dropout: float = 0.05
    target_modules: Optional[list] = None
    target_parameters: Optional[list] = None
    bias: str = "none"
    task_type: str = "CAUSAL_LM"
    use_rslora: bool = False
    use_dora: bool = False
    modules_to_save: Optional[list] = None
    peft_type: str = "LORA"
    base_model_name_or_path: Optional[str] = None
    inference_mode: bool = False

    def __post_init__(self):
        if self.use_dora:
            raise NotImplementedError("DoRA adapters are not implemented")
        if isinstance(self.target_modules, str):
            self.target_modules = list(_ATTN + _MLP) if self.target_modules == "all-linear" else [self.target_modules]
        if self.target_modules is None:
            self.target_modules = ["q_proj", "v_proj"]

    def to_dict(self):
        return asdict(self)


def _as_config(cfg) -> LoraConfig:
    if isinstance(cfg, LoraConfig):
        return cfg
    d = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(cfg)
    keep = {f for f in LoraConfig.__dataclass_fields__}
    d = {k: (list(v) if isinstance(v, set) else v) for k, v in d.items() if k in keep}
    return LoraConfig(**d)


def get_peft_model(model, peft_config, adapter_name: str = "default"):
    """Freeze the base weights and attach trainable low-rank slots to the targeted projections."""
    from .decoder import LoraSlot

    cfg = _as_config(peft_config)
    if "lm_head" in (cfg.target_modules or []):
        # every loss here reads lm_head.weight inside a fused GEMM + log-softmax kernel: a low-rank delta on the head
        # would be silently ignored (the reference raises for its fused losses too: trl/trainer/sft_trainer.py:1306-1318)
        raise ValueError("LoRA on lm_head is not supported: the fused lm_head losses read lm_head.weight directly; "
                         "train the head fully with modules_to_save=['lm_head'] instead")
    if getattr(cfg, "peft_type", "LORA") not in ("LORA", None):
        raise ValueError("only LoRA adapters are supported (prompt-learning methods change the input sequence)")
    save = set(cfg.modules_to_save or [])
    for n, p in model.named_parameters():
        top = n.split(".")[0]
        p.requires_grad_(top in save or (top == "lm_head" and "lm_head" in save) or (top == "score" and "score" in save))
    for layer in model.layers:
        slices = layer.proj_slices()
        for name in cfg.target_modules:
            if name not in slices:
                continue
            pname, sl = slices[name]
            w = getattr(layer, pname)
            out_f = w.shape[0] if sl == slice(None) else (sl.stop - sl.start)
            layer.lora[name] = LoraSlot(w.shape[1], out_f, cfg.r, cfg.lora_alpha, cfg.lora_dropout, cfg.use_rslora,
                                        dtype=torch.float32 if w.dtype == torch.float32 else w.dtype, device=w.device)
    if not any(len(l.lora) for l in model.layers):
        raise ValueError(f"target_modules={cfg.target_modules} matched no projection of the model")
    model.peft_config = {adapter_name: cfg}
    model.active_adapter = adapter_name
    model.save_adapter = lambda path, **k: save_adapter(model, path)
    model.load_adapter = lambda path, **k: load_adapter(model, path)
    model.disable_adapter = lambda: _disable(model)
    model.print_trainable_parameters = lambda: print(
        f"trainable params: {sum(p.numel() for p in model.parameters() if p.requires_grad):,} || "
        f"all params: {sum(p.numel() for p in model.parameters()):,}")
    return model


import contextlib


@contextlib.contextmanager
def _disable(model):
    model.set_adapter_enabled(False)
    try:
        yield
    finally:
        model.set_adapter_enabled(True)


def adapter_state_dict(model) -> dict[str, torch.Tensor]:
    sd = {}
    for i, layer in enumerate(model.layers):
        for name, slot in layer.lora.items():
            block = "self_attn" if name in _ATTN else "mlp"
            base = f"base_model.model.model.layers.{i}.{block}.{name}"
            sd[f"{base}.lora_A.weight"] = slot.lora_A.detach()
            sd[f"{base}.lora_B.weight"] = slot.lora_B.detach()
    cfg = next(iter(model.peft_config.values()))
    for mname in cfg.modules_to_save or []:
        w = getattr(model, mname, None)
        if w is not None:
            key = {"lm_head": "lm_head", "score": "score", "embed_tokens": "model.embed_tokens"}.get(mname, mname)
            sd[f"base_model.model.{key}.weight"] = w.detach()
    return sd


def save_adapter(model, path: str):
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    cfg = next(iter(model.peft_config.values()))
    d = cfg.to_dict()
    d["base_model_name_or_path"] = d.get("base_model_name_or_path") or getattr(model, "name_or_path", None)
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump(d, f, indent=2)
    save_file({k: v.cpu().contiguous().clone() for k, v in adapter_state_dict(model).items()},
              os.path.join(path, "adapter_model.safetensors"), metadata={"format": "pt"})


@torch.no_grad()
def load_adapter(model, path: str):
    from safetensors.torch import load_file

    if getattr(model, "peft_config", None) is None:
        with open(os.path.join(path, "adapter_config.json")) as f:
            get_peft_model(model, LoraConfig(**{k: v for k, v in json.load(f).items()
                                                if k in LoraConfig.__dataclass_fields__}))
    sd = load_file(os.path.join(path, "adapter_model.safetensors"))
    mine = adapter_state_dict(model)
    for k, v in mine.items():
        if k in sd:
            v.copy_(sd[k].to(v.dtype))
    return model


@torch.no_grad()
def export_merged_weights(model, target) -> None:
    """Writes ``model``'s weights with every adapter folded in (``W + scaling * B @ A`` on the adapted slices, in fp32,
    rounded once) into ``target``, a plain copy of the same architecture without adapters.  The generation engines
    read ``target``; the trained model is never touched, so nothing drifts the way a merge / unmerge round trip in
    bf16 would (the reference merges into the model itself before each weight sync and unmerges afterwards:
    trl/generation/vllm_generation.py:459-486)."""
    src = dict(model.named_parameters())
    for n, p in target.named_parameters():
        if n in src and src[n].shape == p.shape:
            p.copy_(src[n])
    for l_src, l_dst in zip(model.layers, target.layers):
        if not getattr(l_src, "lora_enabled", True):
            continue
        slices = l_src.proj_slices()
        for name, slot in l_src.lora.items():
            pname, sl = slices[name]
            w_src, w_dst = getattr(l_src, pname), getattr(l_dst, pname)
            w_dst[sl] = (w_src[sl].float() + slot.delta_weight().to(w_src.device)).to(w_dst.dtype)
