"""ORPOConfig (fields/defaults of trl/experimental/orpo/orpo_config.py:24-134)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from ...trainer.base_config import _BaseConfig


@dataclass
class ORPOConfig(_BaseConfig):
    _VALID_DICT_FIELDS = _BaseConfig._VALID_DICT_FIELDS + ["model_init_kwargs"]

    learning_rate: float = 1e-6
    max_length: Optional[int] = 1024
    max_completion_length: Optional[int] = None
    beta: float = 0.1  # the paper's lambda: weight of the odds-ratio term
    disable_dropout: bool = True
    generate_during_eval: bool = False
    is_encoder_decoder: Optional[bool] = None
    model_init_kwargs: Optional[Any] = None
    trust_remote_code: bool = False
    dataset_num_proc: Optional[int] = None
