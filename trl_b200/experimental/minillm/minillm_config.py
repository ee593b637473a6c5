"""MiniLLMConfig (trl/experimental/minillm/minillm_config.py:20-137)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from ...trainer.grpo_config import GRPOConfig


@dataclass
class MiniLLMConfig(GRPOConfig):
    _VALID_DICT_FIELDS = GRPOConfig._VALID_DICT_FIELDS + ["teacher_model_init_kwargs"]

    teacher_model_init_kwargs: Optional[Any] = None
    disable_dropout: bool = True
    rkl_advantage: bool = True              # add the reverse-KL return to the reward advantage
    single_step_decomposition: bool = True  # add the per-token reverse KL over the full vocabulary
    kd_temperature: float = 1.0
    gamma: float = 0.0                      # discount of future per-token reverse-KL rewards
    length_normalization: bool = True

    def __post_init__(self):
        super().__post_init__()
        if self.kd_temperature <= 0:
            raise ValueError("kd_temperature must be positive")
