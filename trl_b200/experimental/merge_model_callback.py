"""Merging the trained policy with another checkpoint at save time (trl/experimental/merge_model_callback.py:
MergeConfig :48-268, merge_models :271-291, MergeModelCallback :294-352).

The reference delegates to mergekit; here the four methods are applied tensor by tensor on the safetensors
checkpoints this framework writes (HF names), in fp32, and saved in the configured dtype:
``linear``  w_p * P + w_t * T (normalised weights);  ``slerp``  spherical interpolation per tensor with factor t;
``ties`` / ``dare_ties``  task vectors against the target as base, sparsified (magnitude top-density / random drop with
rescale), sign-elected and merged back."""
from __future__ import annotations

import json
import os
import shutil

import torch

from ..loop.state import TrainerCallback


class MergeConfig:
    def __init__(self, method: str = "linear"):
        if method not in ("linear", "ties", "dare_ties", "slerp"):
            raise ValueError(f"Unsupported merge method: {method}")
        self.method = method
        self.policy_model_path = None
        self.target_model_path = None
        self.dtype = "float16"
        if method == "linear":
            self.policy_model_weight, self.target_model_weight = 0.5, 0.5
        elif method in ("ties", "dare_ties"):
            self.policy_model_weight, self.policy_model_density = 1.0, [1.0, 0.7, 0.1]
            self.target_model_weight, self.target_model_density = 1.0, [1.0]
            self.normalize = 1.0
        else:
            self.t_values = 0.5

    def create(self):
        return self


def _load_tensors(path: str) -> dict:
    from safetensors.torch import load_file

    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        out = {}
        for shard in sorted(set(json.load(open(idx))["weight_map"].values())):
            out.update(load_file(os.path.join(path, shard)))
        return out
    return load_file(os.path.join(path, "model.safetensors"))


def _density_for(name: str, densities: list, n_layers: int) -> float:
    """mergekit-style gradient: the list is interpolated over the layer index; non-layer tensors use the first value."""
    if len(densities) == 1:
        return float(densities[0])
    parts = name.split(".")
    if "layers" in parts:
        li = int(parts[parts.index("layers") + 1])
        x = li / max(1, n_layers - 1) * (len(densities) - 1)
        lo = int(x)
        hi = min(lo + 1, len(densities) - 1)
        return float(densities[lo] + (densities[hi] - densities[lo]) * (x - lo))
    return float(densities[0])


def _sparsify(delta: torch.Tensor, density: float, random: bool, gen) -> torch.Tensor:
    if density >= 1.0:
        return delta
    if random:  # DARE: drop at random, rescale the survivors
        keep = torch.rand(delta.shape, generator=gen) < density
        return delta * keep / density
    k = max(1, int(density * delta.numel()))
    thresh = delta.abs().flatten().kthvalue(delta.numel() - k + 1).values
    return delta * (delta.abs() >= thresh)


def merge_models(config: MergeConfig, out_path: str):
    from safetensors.torch import save_file

    P, T = _load_tensors(config.policy_model_path), _load_tensors(config.target_model_path)
    dtype = getattr(torch, config.dtype)
    n_layers = 1 + max([int(k.split(".")[k.split(".").index("layers") + 1]) for k in P if ".layers." in k] or [0])
    gen = torch.Generator().manual_seed(0)
    out = {}
    for name, p in P.items():
        if name not in T or T[name].shape != p.shape:
            out[name] = p.to(dtype)
            continue
        a, b = p.float(), T[name].float()
        if config.method == "linear":
            w = config.policy_model_weight + config.target_model_weight
            m = (config.policy_model_weight * a + config.target_model_weight * b) / w
        elif config.method == "slerp":
            t = float(config.t_values)
            na, nb = a.flatten() / (a.norm() + 1e-12), b.flatten() / (b.norm() + 1e-12)
            omega = torch.acos(torch.clamp((na * nb).sum(), -1.0, 1.0))
            if float(omega.abs()) < 1e-4:
                m = (1 - t) * a + t * b
            else:
                so = torch.sin(omega)
                m = torch.sin((1 - t) * omega) / so * a + torch.sin(t * omega) / so * b
        else:
            # the target is the base; the policy contributes its task vector
            delta = _sparsify(a - b, _density_for(name, config.policy_model_density, n_layers),
                              config.method == "dare_ties", gen) * config.policy_model_weight
            sign = torch.sign(delta)  # one task vector: its own signs are the elected signs
            scale = config.policy_model_weight if config.normalize else 1.0
            m = b + torch.where(sign != 0, delta, torch.zeros_like(delta)) / (scale if scale else 1.0)
        out[name] = m.to(dtype).contiguous()
    os.makedirs(out_path, exist_ok=True)
    save_file(out, os.path.join(out_path, "model.safetensors"), metadata={"format": "pt"})
    for f in os.listdir(config.policy_model_path):
        if f.endswith(".json") and not f.startswith(("model.safetensors", "trainer_state", "entropy_ctrl")) \
                or f.endswith((".jinja", ".model", ".txt")):
            shutil.copy(os.path.join(config.policy_model_path, f), os.path.join(out_path, f))


def upload_model_to_hf(folder_path: str, repo_id: str):
    raise RuntimeError("pushing to the Hub needs network access; the merged model is in " + folder_path)


class MergeModelCallback(TrainerCallback):
    def __init__(self, merge_config: MergeConfig | None = None, merge_at_every_checkpoint: bool = False,
                 push_to_hub: bool = False):
        self.merge_config = merge_config or MergeConfig()
        self.merge_at_every_checkpoint, self.push_to_hub = merge_at_every_checkpoint, push_to_hub

    def _merge_and_maybe_push(self, output_dir, global_step, model):
        ckpt = os.path.join(output_dir, f"checkpoint-{global_step}")
        if not os.path.isdir(ckpt):
            return
        self.merge_config.policy_model_path = ckpt
        if self.merge_config.target_model_path is None:
            self.merge_config.target_model_path = getattr(model, "name_or_path", None) or getattr(model.config, "_name_or_path", None)
        if not self.merge_config.target_model_path:
            raise ValueError("MergeConfig.target_model_path is not set and the model does not know where it came from")
        merged = os.path.join(ckpt, "merged")
        merge_models(self.merge_config.create(), merged)
        if self.push_to_hub:
            upload_model_to_hf(merged, f"{output_dir}_checkpoint-{global_step}_merged")

    def on_save(self, args, state, control, model=None, **kw):
        if self.merge_at_every_checkpoint and state.is_world_process_zero:
            self._merge_and_maybe_push(args.output_dir, state.global_step, model)

    def on_train_end(self, args, state, control, model=None, **kw):
        if not self.merge_at_every_checkpoint and state.is_world_process_zero:
            self._merge_and_maybe_push(args.output_dir, state.global_step, model)
