"""DistillationConfig (fields/defaults of trl/experimental/distillation/distillation_config.py:24-304)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from ..gkd.gkd_config import GKDConfig


@dataclass
class DistillationConfig(GKDConfig):
    temperature: float = 1.0
    beta: float = 1.0                  # 1.0 = reverse KL on the student's own samples
    lmbda: float = 1.0                 # fully on-policy by default
    max_completion_length: int = 512
    teacher_model_revision: Optional[str] = None
    num_generations: int = 1
    generation_batch_size: Optional[int] = None
    top_p: float = 0.95
    top_k: int = 0
    use_vllm: bool = False
    vllm_mode: str = "colocate"
    vllm_sync_frequency: int = 1
    log_completions: bool = False
    log_completions_steps: int = 100
    num_completions_to_print: Optional[int] = None

    def __post_init__(self):
        super().__post_init__()
        self.max_new_tokens = self.max_completion_length
