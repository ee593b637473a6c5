"""CPOConfig (fields/defaults of trl/experimental/cpo/cpo_config.py:24-182)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from ...trainer.base_config import _BaseConfig


@dataclass
class CPOConfig(_BaseConfig):
    _VALID_DICT_FIELDS = _BaseConfig._VALID_DICT_FIELDS + ["model_init_kwargs"]

    learning_rate: float = 1e-6
    max_length: Optional[int] = 1024
    max_completion_length: Optional[int] = None
    beta: float = 0.1
    label_smoothing: float = 0.0
    loss_type: str = "sigmoid"  # sigmoid | hinge | ipo | simpo
    disable_dropout: bool = True
    cpo_alpha: float = 1.0      # weight of the NLL term on the chosen completion (0 with simpo = pure SimPO)
    simpo_gamma: float = 0.5    # target reward margin of SimPO
    alpha: float = 0.0          # AlphaPO reward shape; 0 = log-prob rewards
    generate_during_eval: bool = False
    is_encoder_decoder: Optional[bool] = None
    model_init_kwargs: Optional[Any] = None
    trust_remote_code: bool = False
    dataset_num_proc: Optional[int] = None
    truncation_mode: str = "keep_start"
    pad_to_multiple_of: Optional[int] = None
    router_aux_loss_coef: float = 0.001
    eos_token: Optional[str] = None
    pad_token: Optional[str] = None
    padding_free: bool = False

    def __post_init__(self):
        super().__post_init__()
        if self.loss_type not in ("sigmoid", "hinge", "ipo", "simpo"):
            raise ValueError(f"Unknown loss type: {self.loss_type}. Should be one of ['sigmoid', 'hinge', 'ipo', 'simpo']")
        if self.loss_type == "simpo" and self.cpo_alpha != 0.0:
            import warnings

            warnings.warn("You are using CPO-SimPO (simpo loss with cpo_alpha > 0): set cpo_alpha=0.0 for plain SimPO.")
