"""Hugging Face checkpoint layout <-> native fused parameters.

On disk: ``config.json`` + ``model.safetensors`` (or shards with
``model.safetensors.index.json``) using the transformers parameter names, so a
checkpoint written here loads with ``AutoModelForCausalLM.from_pretrained`` and
checkpoints from the Hub load here.  Qwen3-MoE experts are stored per expert
(``mlp.experts.E.{gate,up,down}_proj.weight``) like the Hub checkpoints.
"""
from __future__ import annotations

import json
import os
import re

import torch

from .configuration import PRESETS, ModelArch, preset

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16,
           "fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16, "auto": None, None: None}


def resolve_dtype(dtype):
    if isinstance(dtype, torch.dtype) or dtype is None:
        return dtype
    if dtype in _DTYPES:
        return _DTYPES[dtype]
    raise ValueError(f"Invalid dtype {dtype!r}; expected one of {sorted(k for k in _DTYPES if k)}")


def to_hf_state_dict(model, include_lora: bool = False, before_layer=None, copy_to=None) -> dict[str, torch.Tensor]:
    """Checkpoint names -> tensors.  ``before_layer(i)`` is called before layer i is read and ``copy_to`` (a device)
    makes a copy of every layer's tensors right after: the streamed full-shard engine holds one layer at a time.  With
    ``before_layer`` set and ``copy_to`` None the layers are visited (the gathers are collective) but not kept."""
    c = model.config
    sd = {"model.embed_tokens.weight": model.embed_tokens.detach()}
    for i, l in enumerate(model.layers):
        p = f"model.layers.{i}."
        if before_layer is not None:
            before_layer(i)
            if copy_to is None:
                continue
        n_before = len(sd)
        qkv = l.qkv_proj.detach()
        fused_on_disk = c.model_type == "phi3"  # Phi-3 checkpoints keep qkv_proj and gate_up_proj fused, like memory here
        if fused_on_disk:
            sd[p + "self_attn.qkv_proj.weight"] = qkv
        else:
            q, k, v = qkv.split([c.q_size, c.kv_size, c.kv_size], dim=0)
            sd[p + "self_attn.q_proj.weight"], sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.v_proj.weight"] = q, k, v
        if l.qkv_bias is not None:
            bq, bk, bv = l.qkv_bias.detach().split([c.q_size, c.kv_size, c.kv_size])
            sd[p + "self_attn.q_proj.bias"], sd[p + "self_attn.k_proj.bias"], sd[p + "self_attn.v_proj.bias"] = bq, bk, bv
        if c.qk_norm:
            sd[p + "self_attn.q_norm.weight"] = l.q_norm.detach()
            sd[p + "self_attn.k_norm.weight"] = l.k_norm.detach()
        sd[p + "self_attn.o_proj.weight"] = l.o_proj.detach()
        sd[p + "input_layernorm.weight"] = l.input_layernorm.detach()
        sd[p + "post_attention_layernorm.weight"] = l.post_attention_layernorm.detach()
        if c.is_moe:
            I = c.moe_intermediate_size
            sd[p + "mlp.gate.weight"] = l.router.detach()
            # an expert-parallel layer holds a slice of the experts; ``_ep_full`` is set (by the gather that runs in
            # ``before_layer``) to the complete tensors while the layer is exported
            gu_all, dn_all = getattr(l, "_ep_full", None) or (l.experts_gate_up.detach(), l.experts_down.detach())
            if gu_all.shape[0] != c.num_experts:
                raise RuntimeError("expert-parallel model: export through parallel.expert_parallel.ep_hf_state_dict "
                                   "(a collective that gathers the experts layer by layer)")
            for e in range(c.num_experts):
                sd[p + f"mlp.experts.{e}.gate_proj.weight"] = gu_all[e, :I]
                sd[p + f"mlp.experts.{e}.up_proj.weight"] = gu_all[e, I:]
                sd[p + f"mlp.experts.{e}.down_proj.weight"] = dn_all[e]
        else:
            I = c.intermediate_size
            if fused_on_disk:
                sd[p + "mlp.gate_up_proj.weight"] = l.gate_up_proj.detach()
            else:
                sd[p + "mlp.gate_proj.weight"] = l.gate_up_proj.detach()[:I]
                sd[p + "mlp.up_proj.weight"] = l.gate_up_proj.detach()[I:]
            sd[p + "mlp.down_proj.weight"] = l.down_proj.detach()
        if before_layer is not None:
            for k in list(sd)[n_before:]:
                sd[k] = sd[k].to(copy_to, copy=True)
    sd["model.norm.weight"] = model.norm.detach()
    if c.num_labels:
        sd["score.weight"] = model.score.detach()
    elif model.lm_head is not None:
        sd["lm_head.weight"] = model.lm_head.detach()
    return sd


@torch.no_grad()
def load_hf_state_dict(model, sd: dict[str, torch.Tensor], strict: bool = True, after_layer=None) -> list[str]:
    """Copy tensors named the HF way into the fused native parameters.  ``after_layer(i)`` runs once layer i is
    complete (the streamed full-shard engine re-slices its shard there, before the slot is reused)."""
    c = model.config
    used = set()

    def take(name, required=True):
        if name in sd:
            used.add(name)
            return sd[name]
        if required and strict:
            raise KeyError(f"missing tensor {name} in checkpoint")
        return None

    def put(dst, src):
        if src is not None:
            dst.copy_(src.to(dst.dtype))

    put(model.embed_tokens, take("model.embed_tokens.weight"))
    for i, l in enumerate(model.layers):
        p = f"model.layers.{i}."
        fused_qkv = take(p + "self_attn.qkv_proj.weight", required=False)
        if fused_qkv is not None:  # Phi-3 layout
            put(l.qkv_proj, fused_qkv)
        else:
            put(l.qkv_proj[: c.q_size], take(p + "self_attn.q_proj.weight"))
            put(l.qkv_proj[c.q_size: c.q_size + c.kv_size], take(p + "self_attn.k_proj.weight"))
            put(l.qkv_proj[c.q_size + c.kv_size:], take(p + "self_attn.v_proj.weight"))
        if l.qkv_bias is not None:
            put(l.qkv_bias[: c.q_size], take(p + "self_attn.q_proj.bias"))
            put(l.qkv_bias[c.q_size: c.q_size + c.kv_size], take(p + "self_attn.k_proj.bias"))
            put(l.qkv_bias[c.q_size + c.kv_size:], take(p + "self_attn.v_proj.bias"))
        if c.qk_norm:
            put(l.q_norm, take(p + "self_attn.q_norm.weight"))
            put(l.k_norm, take(p + "self_attn.k_norm.weight"))
        put(l.o_proj, take(p + "self_attn.o_proj.weight"))
        put(l.input_layernorm, take(p + "input_layernorm.weight"))
        put(l.post_attention_layernorm, take(p + "post_attention_layernorm.weight"))
        if c.is_moe:
            I = c.moe_intermediate_size
            put(l.router, take(p + "mlp.gate.weight"))
            fused_gu = take(p + "mlp.experts.gate_up_proj", required=False)
            # expert-parallel layers keep experts [e0, e0 + n_loc) only; the other experts' tensors are skipped
            e0, n_loc = getattr(l, "ep_first_expert", 0), l.experts_gate_up.shape[0]
            if fused_gu is not None:  # transformers>=5 in-memory fused layout
                put(l.experts_gate_up, fused_gu[e0:e0 + n_loc])
                put(l.experts_down, take(p + "mlp.experts.down_proj")[e0:e0 + n_loc])
            else:
                for e in range(c.num_experts):
                    if e0 <= e < e0 + n_loc:
                        put(l.experts_gate_up[e - e0, :I], take(p + f"mlp.experts.{e}.gate_proj.weight"))
                        put(l.experts_gate_up[e - e0, I:], take(p + f"mlp.experts.{e}.up_proj.weight"))
                        put(l.experts_down[e - e0], take(p + f"mlp.experts.{e}.down_proj.weight"))
                    else:
                        for leaf in ("gate_proj", "up_proj", "down_proj"):
                            take(p + f"mlp.experts.{e}.{leaf}.weight", required=False)
        else:
            I = c.intermediate_size
            fused_gate_up = take(p + "mlp.gate_up_proj.weight", required=False)
            if fused_gate_up is not None:
                put(l.gate_up_proj, fused_gate_up)
            else:
                put(l.gate_up_proj[:I], take(p + "mlp.gate_proj.weight"))
                put(l.gate_up_proj[I:], take(p + "mlp.up_proj.weight"))
            put(l.down_proj, take(p + "mlp.down_proj.weight"))
        if after_layer is not None:
            after_layer(i)
    put(model.norm, take("model.norm.weight"))
    if c.num_labels:
        put(model.score, take("score.weight", required=False))
    elif model.lm_head is not None:
        w = take("lm_head.weight", required=False)
        put(model.lm_head, w if w is not None else sd.get("model.embed_tokens.weight"))
    return [k for k in sd if k not in used]


def save_state_dict_sharded(sd: dict[str, torch.Tensor], path: str, max_shard_bytes: int = 5 * 2**30,
                            prefix: str = "model"):
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    sd = {k: v.detach().to("cpu").contiguous().clone() for k, v in sd.items()}
    total = sum(v.numel() * v.element_size() for v in sd.values())
    if total <= max_shard_bytes:
        save_file(sd, os.path.join(path, f"{prefix}.safetensors"), metadata={"format": "pt"})
        return
    shards, cur, cur_b = [], {}, 0
    for k, v in sd.items():
        b = v.numel() * v.element_size()
        if cur and cur_b + b > max_shard_bytes:
            shards.append(cur)
            cur, cur_b = {}, 0
        cur[k] = v
        cur_b += b
    shards.append(cur)
    index = {"metadata": {"total_size": total}, "weight_map": {}}
    for i, sh in enumerate(shards):
        fn = f"{prefix}-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(path, fn), metadata={"format": "pt"})
        for k in sh:
            index["weight_map"][k] = fn
    with open(os.path.join(path, f"{prefix}.safetensors.index.json"), "w") as f:
        json.dump(index, f, indent=2)


def load_state_dict_dir(path: str, prefix: str = "model") -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    single = os.path.join(path, f"{prefix}.safetensors")
    if os.path.exists(single):
        return load_file(single)
    idx = os.path.join(path, f"{prefix}.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        sd = {}
        for fn in files:
            sd.update(load_file(os.path.join(path, fn)))
        return sd
    binf = os.path.join(path, "pytorch_model.bin")
    if os.path.exists(binf):
        return torch.load(binf, map_location="cpu", weights_only=True)
    raise FileNotFoundError(f"no {prefix}.safetensors[.index.json] under {path}")


def save_model(model, path: str, state_dict=None):
    os.makedirs(path, exist_ok=True)
    model.config.save_pretrained(path)
    sd = state_dict if state_dict is not None else to_hf_state_dict(model)
    save_state_dict_sharded(sd, path)
    gen = {"_from_model_config": True, "bos_token_id": model.config.bos_token_id,
           "eos_token_id": model.config.eos_token_id, "pad_token_id": model.config.pad_token_id}
    with open(os.path.join(path, "generation_config.json"), "w") as f:
        json.dump(gen, f, indent=2)


def load_model(path_or_name, dtype=None, device=None, num_labels: int | None = None, config: ModelArch | None = None,
               seed: int | None = None, **unused):
    """Load from a local HF directory, or random-init a named preset (``"preset:qwen2.5-7b"``)."""
    from .decoder import CausalLM

    dtype = resolve_dtype(dtype) or torch.float32
    if isinstance(path_or_name, ModelArch):
        config, path_or_name = path_or_name, ""
    name = str(path_or_name)
    is_dir = os.path.isdir(name)
    if is_dir and config is None and os.path.exists(os.path.join(name, "config.json")):
        with open(os.path.join(name, "config.json")) as f:
            mt = json.load(f).get("model_type")
        if mt == "llava":  # vision tower + projector + decoder
            from .vision import VisionLanguageModel

            return VisionLanguageModel.from_pretrained(name, dtype=dtype, device=device)
        if mt == "qwen2_vl":  # dynamic-resolution tower + decoder with multimodal RoPE
            from .vision_qwen import Qwen2VLModel

            return Qwen2VLModel.from_pretrained(name, dtype=dtype, device=device)
    if config is None:
        if is_dir:
            config = ModelArch.from_pretrained(name)
        else:
            key = name.split(":", 1)[1] if name.startswith("preset:") else name
            if key not in PRESETS:
                raise FileNotFoundError(
                    f"{name!r} is neither a local checkpoint directory nor a preset "
                    f"({sorted(PRESETS)}); there is no network access to fetch Hub models."
                )
            config = preset(key)
    if num_labels is not None:
        config.num_labels = num_labels
    if seed is not None:
        torch.manual_seed(seed)
    model = CausalLM(config, dtype=dtype, device=device)
    if is_dir:
        has_weights = any(re.match(r"(model.*\.safetensors.*|pytorch_model\.bin)$", f) for f in os.listdir(name))
        if has_weights:
            load_hf_state_dict(model, load_state_dict_dir(name), strict=True)
    model.name_or_path = name
    config.extra["_name_or_path"] = name
    return model
