"""IWOPDConfig (fields/defaults of trl/experimental/iw_opd/iw_opd_config.py:24-501)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..distillation.distillation_config import DistillationConfig


@dataclass
class IWOPDConfig(DistillationConfig):
    distillation_objective: str = "iw_opd"  # iw_opd | jsd
    iw_opd_gamma: float = 0.5               # amplification of early-token weights
    iw_opd_epsilon: float = 1e-8
    reverse_kl_top_1_mode: str = "sampled"
    max_prompt_length: Optional[int] = None
    use_teacher_server: bool = False
    teacher_model_server_url: Optional[str] = None
    loss_top_k: int = 0
    loss_add_tail: bool = True

    def __post_init__(self):
        super().__post_init__()
        if self.distillation_objective not in ("iw_opd", "jsd"):
            raise ValueError("distillation_objective must be 'iw_opd' or 'jsd'")
        if self.reverse_kl_top_1_mode not in ("sampled", "argmax"):
            raise ValueError("reverse_kl_top_1_mode must be 'sampled' or 'argmax'")
