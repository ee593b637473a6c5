"""ServerDistillationConfig (trl/experimental/server_distillation/server_distillation_config.py:20-102)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..distillation.distillation_config import DistillationConfig


@dataclass
class ServerDistillationConfig(DistillationConfig):
    teacher_model_server_url: Optional[str] = None
    loss_top_k: int = 1
    loss_add_tail: bool = True
    reverse_kl_top_1_mode: str = "sampled"

    def __post_init__(self):
        super().__post_init__()
        if self.teacher_model_server_url is None:
            raise ValueError("teacher_model_server_url is required: the teacher is only reachable through the server")
        if self.beta > 0 and self.loss_top_k != 1:
            raise ValueError("with beta > 0 the server teacher supports loss_top_k == 1 only (top-1 support)")
        if self.reverse_kl_top_1_mode == "argmax":
            raise ValueError("the server cannot score student-selected tokens: reverse_kl_top_1_mode must be 'sampled'")
