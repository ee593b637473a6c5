"""BCOConfig (fields/defaults of trl/experimental/bco/bco_config.py:24-164)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ...trainer.kto_trainer import KTOConfig


@dataclass
class BCOConfig(KTOConfig):
    _LOSS_TYPES = ("bco",)

    learning_rate: float = 5e-7
    loss_type: str = "bco"
    train_sampling_strategy: str = "random"
    max_completion_length: Optional[int] = None
    generate_during_eval: bool = False
    is_encoder_decoder: Optional[bool] = None
    prompt_sample_size: int = 1024   # prompts embedded to fit the density-ratio classifier (UDM)
    min_density_ratio: float = 0.5
    max_density_ratio: float = 10.0
