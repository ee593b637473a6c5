"""DPOConfig: fields and defaults of trl/trainer/dpo_config.py:22-366."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from .base_config import _BaseConfig

DPO_LOSS_TYPES = ["sigmoid", "hinge", "ipo", "exo_pair", "nca_pair", "robust", "bco_pair", "sppo_hard", "aot",
                  "aot_unpaired", "apo_zero", "apo_down", "discopop", "sft", "sigmoid_norm"]


@dataclass
class DPOConfig(_BaseConfig):
    _VALID_DICT_FIELDS = _BaseConfig._VALID_DICT_FIELDS + ["model_init_kwargs"]

    learning_rate: float = 1e-6
    model_init_kwargs: Optional[Any] = None
    trust_remote_code: bool = False
    router_aux_loss_coef: float = 0.001
    disable_dropout: bool = True
    dataset_num_proc: Optional[int] = None
    eos_token: Optional[str] = None
    pad_token: Optional[str] = None
    max_length: Optional[int] = 1024
    truncation_mode: str = "keep_start"
    padding_free: bool = False
    pad_to_multiple_of: Optional[int] = None
    precompute_ref_log_probs: bool = False
    precompute_ref_batch_size: Optional[int] = None
    loss_type: Any = field(default_factory=lambda: ["sigmoid"])
    loss_weights: Optional[list] = None
    ld_alpha: Optional[float] = None
    f_divergence_type: str = "reverse_kl"
    f_alpha_divergence_coef: float = 0.5
    label_smoothing: float = 0.0
    beta: float = 0.1
    use_weighting: bool = False
    discopop_tau: float = 0.05
    activation_offloading: bool = False
    sync_ref_model: bool = False
    ref_model_mixup_alpha: float = 0.6
    ref_model_sync_steps: int = 512

    def __post_init__(self):
        super().__post_init__()
        if isinstance(self.loss_type, str):
            self.loss_type = [self.loss_type]
        for lt in self.loss_type:
            if lt not in DPO_LOSS_TYPES:
                raise ValueError(f"Unknown loss type: {lt}. Should be one of {DPO_LOSS_TYPES}")
        if self.loss_weights is not None and len(self.loss_weights) != len(self.loss_type):
            raise ValueError("loss_weights must have one entry per loss_type")
        if self.f_divergence_type not in ("reverse_kl", "forward_kl", "js_divergence", "alpha_divergence"):
            raise ValueError(f"Unknown f_divergence_type: {self.f_divergence_type}")
        if self.truncation_mode not in ("keep_start", "keep_end"):
            raise ValueError("truncation_mode must be 'keep_start' or 'keep_end'")
        if self.ld_alpha is not None and not 0.0 <= self.ld_alpha <= 1.0:
            raise ValueError("ld_alpha must be in [0, 1]")
        if self.sync_ref_model and self.precompute_ref_log_probs:
            raise ValueError("sync_ref_model and precompute_ref_log_probs cannot both be enabled")
