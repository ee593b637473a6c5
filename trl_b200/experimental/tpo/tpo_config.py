"""TPOConfig (fields/defaults of trl/experimental/tpo/tpo_config.py:24-174)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from ...trainer.base_config import _BaseConfig


@dataclass
class TPOConfig(_BaseConfig):
    _VALID_DICT_FIELDS = _BaseConfig._VALID_DICT_FIELDS + ["model_init_kwargs"]

    learning_rate: float = 5e-7
    model_init_kwargs: Optional[Any] = None
    trust_remote_code: bool = False
    disable_dropout: bool = True
    dataset_num_proc: Optional[int] = None
    max_length: Optional[int] = 1024
    truncation_mode: str = "keep_start"
    pad_to_multiple_of: Optional[int] = None
    loss_type: str = "sigmoid"  # sigmoid | hinge | ipo | tpo-l
    beta: float = 0.01
    label_smoothing: float = 0.0
    tpo_alpha: float = 1.0      # weight of the NLL term on the gold ("reference") response
    tpo_l_gamma: float = 0.5    # target margin of the length-normalised variant

    def __post_init__(self):
        super().__post_init__()
        if self.loss_type not in ("sigmoid", "hinge", "ipo", "tpo-l"):
            raise ValueError(f"Unknown loss type: {self.loss_type}. Should be one of ['sigmoid', 'hinge', 'ipo', 'tpo-l']")
