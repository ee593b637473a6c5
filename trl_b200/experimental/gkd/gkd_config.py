"""GKDConfig (fields/defaults of trl/experimental/gkd/gkd_config.py:24-110)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from ...trainer.sft_config import SFTConfig


@dataclass
class GKDConfig(SFTConfig):
    _VALID_DICT_FIELDS = SFTConfig._VALID_DICT_FIELDS + ["teacher_model_init_kwargs"]

    temperature: float = 0.9
    lmbda: float = 0.5          # fraction of steps trained on completions sampled from the student
    beta: float = 0.5           # JSD interpolation: 0 = forward KL, 1 = reverse KL
    max_new_tokens: int = 128
    teacher_model_name_or_path: Optional[str] = None
    teacher_model_init_kwargs: Optional[Any] = None
    disable_dropout: bool = True
    seq_kd: bool = False        # off-policy steps train on completions sampled from the teacher

    def __post_init__(self):
        super().__post_init__()
        if not 0.0 <= self.lmbda <= 1.0:
            raise ValueError("lmbda must be in the range [0.0, 1.0].")
        if not 0.0 <= self.beta <= 1.0:
            raise ValueError("beta must be in the range [0.0, 1.0].")
