"""SSDConfig (fields/defaults of trl/experimental/ssd/ssd_config.py:24-263)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ...trainer.grpo_config import _OnlineConfig


@dataclass
class SSDConfig(_OnlineConfig):
    _MIN_GENERATIONS = 1

    learning_rate: float = 1e-5
    max_prompt_length: Optional[int] = 512
    max_completion_length: Optional[int] = 256
    num_generations: Optional[int] = 1
    temperature: float = 1.0   # T_train: the sampling temperature of the self-generated training data
    filter_empty: bool = True  # drop samples that are empty after decoding
    disable_dropout: bool = True

    def __post_init__(self):
        super().__post_init__()
        self._derive_generation_batch()
