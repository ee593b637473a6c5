"""GMPOConfig (trl/experimental/gmpo/gmpo_config.py:22-47): GRPO with the geometric-mean objective."""
from __future__ import annotations

from dataclasses import dataclass

from ...trainer.grpo_config import GRPOConfig


@dataclass
class GMPOConfig(GRPOConfig):
    _LOSS_TYPES = GRPOConfig._LOSS_TYPES + ("gmpo",)

    loss_type: str = "gmpo"
    gmpo_log_clip: float = 0.4  # token log-ratios are clipped to [-0.4, 0.4], i.e. ratios to (e^-0.4, e^0.4)
    beta: float = 0.0
