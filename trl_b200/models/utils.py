"""Model helpers named like trl/models/utils.py.

The reference wraps models in DeepSpeed / FSDP engines and needs hook juggling around generation
(:47-233) and special preparation of frozen reference/reward models (:236-321).  The native engine keeps
parameters as plain (flat-bucket) tensors, so these entry points reduce to what is still meaningful:
turning off gradient checkpointing for generation, gathering parameters of a fully sharded model, and
freezing + placing auxiliary models.
"""
from __future__ import annotations

import contextlib
import copy

import torch


@contextlib.contextmanager
def disable_gradient_checkpointing(model, gradient_checkpointing_kwargs=None):
    was = getattr(model, "gradient_checkpointing", False)
    if was:
        model.gradient_checkpointing_disable()
    try:
        yield
    finally:
        if was:
            model.gradient_checkpointing_enable(gradient_checkpointing_kwargs)


@contextlib.contextmanager
def unwrap_model_for_generation(model, accelerator=None, gather_deepspeed3_params: bool = True, generation_kwargs=None):
    """Yield a model whose parameters are complete and whose forward is cheap: gradient checkpointing off;
    under the full-shard engine all buckets are materialised for the duration of the block."""
    engine = getattr(model, "_trl_b200_engine", None)
    ctx = engine.gathered(None) if (engine is not None and gather_deepspeed3_params and hasattr(engine, "gathered")) \
        else contextlib.nullcontext()
    with ctx, disable_gradient_checkpointing(model):
        yield model


def _freeze(model, device=None, dtype=None):
    model = model.eval().requires_grad_(False)
    if device is not None or dtype is not None:
        model = model.to(device=device, dtype=dtype)
    return model


def prepare_deepspeed(model, accelerator=None):
    """Inference placement of a frozen reference / reward model (no ZeRO engine is created)."""
    return _freeze(model, getattr(accelerator, "device", None))


def prepare_fsdp(model, accelerator=None):
    return _freeze(model, getattr(accelerator, "device", None))


def create_reference_model(model, num_shared_layers=None, pattern=None):
    """Frozen deep copy of ``model``; with ``num_shared_layers`` the first N decoder layers are shared
    (same tensors, frozen in both) instead of copied."""
    ref = copy.deepcopy(model)
    if num_shared_layers:
        for i in range(num_shared_layers):
            ref.layers[i] = model.layers[i]
            for p in model.layers[i].parameters():
                p.requires_grad_(False)
    for p in ref.parameters():
        p.requires_grad_(False)
    return ref.eval()


def remove_hooks(model):  # the native engine installs no forward hooks
    return None


def add_hooks(model):
    return None


class _ForwardRedirection:
    """Runs an arbitrary method through a wrapper module's ``forward`` so that the wrapper's pre/post hooks fire
    (counterpart of trl/models/utils.py:324-372, where FSDP / ZeRO-3 hooks gather parameters).  The native engines hang
    no hooks on ``forward`` (full-shard gathers happen inside the layer's QKV GEMM), so this only swaps the call."""

    def __call__(self, wrapper_module, original_module, method, *args, **kwargs):
        original_forward = original_module.forward

        def wrapped_forward(*a, **k):
            original_module.forward = original_forward
            out = method(*a, **k)
            self.on_after_inner_forward(wrapper_module, original_module)
            return out
        original_module.forward = wrapped_forward
        try:
            out = wrapper_module(*args, **kwargs)
        finally:
            original_module.forward = original_forward
        self.on_after_outer_forward(wrapper_module, original_module)
        return out

    def on_after_inner_forward(self, wrapper_module, original_module):
        pass

    def on_after_outer_forward(self, wrapper_module, original_module):
        pass
