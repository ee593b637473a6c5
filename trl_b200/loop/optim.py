"""Learning-rate schedules and the AdamW update rule on flat shards.

The schedules reproduce ``transformers.get_scheduler`` names used by the
reference configs (``lr_scheduler_type`` in trl/trainer/*_config.py).  The
update itself runs on flat fp32 master/moment shards: on GPUs through the fused
sm_100a kernel (``ops.cuda.adamw_flat``), on CPU through the PyTorch expression
below, which is also the kernel's oracle.
"""
from __future__ import annotations

import math

import torch


def lr_lambda_for(name: str, warmup: int, total: int, **kw):
    name = str(name).lower().replace("schedulertype.", "")

    def warm(step):
        return float(step) / float(max(1, warmup))

    if name == "linear":
        return lambda s: warm(s) if s < warmup else max(0.0, float(total - s) / float(max(1, total - warmup)))
    if name == "cosine":
        cycles = kw.get("num_cycles", 0.5)
        return lambda s: warm(s) if s < warmup else max(
            0.0, 0.5 * (1.0 + math.cos(math.pi * cycles * 2.0 * (s - warmup) / max(1, total - warmup))))
    if name == "cosine_with_restarts":
        cycles = kw.get("num_cycles", 1)

        def f(s):
            if s < warmup:
                return warm(s)
            p = (s - warmup) / max(1, total - warmup)
            return 0.0 if p >= 1 else max(0.0, 0.5 * (1.0 + math.cos(math.pi * ((cycles * p) % 1.0))))
        return f
    if name == "polynomial":
        power, end = kw.get("power", 1.0), kw.get("lr_end", 1e-7)
        return lambda s: warm(s) if s < warmup else max(end, (1 - (s - warmup) / max(1, total - warmup)) ** power)
    if name == "constant":
        return lambda s: 1.0
    if name == "constant_with_warmup":
        return lambda s: warm(s) if s < warmup else 1.0
    if name == "inverse_sqrt":
        ts = kw.get("timescale", warmup or 10000)
        return lambda s: warm(s) if s < warmup else 1.0 / math.sqrt((s + ts - warmup) / ts)
    if name == "cosine_with_min_lr":
        mr = kw.get("min_lr_rate", 0.0)
        return lambda s: warm(s) if s < warmup else mr + (1 - mr) * 0.5 * (
            1.0 + math.cos(math.pi * (s - warmup) / max(1, total - warmup)))
    if name in ("warmup_stable_decay", "wsd"):
        decay = kw.get("num_decay_steps", max(1, total // 10))
        stable = total - warmup - decay
        mr = kw.get("min_lr_ratio", 0.0)

        def f(s):
            if s < warmup:
                return warm(s)
            if s < warmup + stable:
                return 1.0
            p = min(1.0, (s - warmup - stable) / max(1, decay))
            return mr + (1 - mr) * (1 - p)
        return f
    raise ValueError(f"unknown lr_scheduler_type {name!r}")


class LRScheduler:
    """Minimal LambdaLR clone that does not need a torch optimizer."""

    def __init__(self, base_lr: float, lr_lambda, last_step: int = 0):
        self.base_lr, self.fn, self.step_count = base_lr, lr_lambda, last_step

    def step(self):
        self.step_count += 1

    def get_last_lr(self):
        return [self.base_lr * self.fn(self.step_count)]

    def state_dict(self):
        return {"step_count": self.step_count, "base_lr": self.base_lr}

    def load_state_dict(self, sd):
        self.step_count = sd["step_count"]
        self.base_lr = sd.get("base_lr", self.base_lr)


def adamw_reference(master, grad, m, v, step, lr, beta1, beta2, eps, weight_decay, grad_scale=1.0):
    """Decoupled-weight-decay Adam on fp32 tensors, in place.  ``step`` counts from 1."""
    g = grad.float() * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    master.mul_(1 - lr * weight_decay)
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    master.addcdiv_(m, denom, value=-lr / bc1)


def adamw_flat(master, grad, m, v, step, lr, beta1, beta2, eps, weight_decay, grad_scale=1.0, shadow=None):
    """Update a flat shard; ``shadow`` (bf16 compute copy of the same slice) is refreshed."""
    if master.is_cuda:
        from ..ops import cuda as K

        K.adamw_flat(master, grad, m, v, step, lr, beta1, beta2, eps, weight_decay, grad_scale, shadow)
        return
    adamw_reference(master, grad, m, v, step, lr, beta1, beta2, eps, weight_decay, grad_scale)
    if shadow is not None and shadow.data_ptr() != master.data_ptr():
        shadow.copy_(master)
