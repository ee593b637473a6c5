"""A2POConfig (trl/experimental/a2po/a2po_config.py:24-156)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ...trainer.grpo_config import _OnlineConfig


@dataclass
class A2POConfig(_OnlineConfig):
    _MIN_GENERATIONS = 1

    learning_rate: float = 1e-6
    max_prompt_length: Optional[int] = 512
    max_completion_length: Optional[int] = 256
    num_value_samples: int = 8      # reference-policy samples per prompt for the V* estimate (stage 1)
    beta1: float = 0.5              # KL temperature of the V* estimate
    filter_all_incorrect: bool = True
    beta2: float = 1e-3             # scale of the implicit reward beta2 * log(pi / pi_ref) (stage 2)
    num_generations: Optional[int] = 1

    def __post_init__(self):
        super().__post_init__()
        self.num_generations, self.num_iterations = 1, 1
        self._needs_ref = True
        self._derive_generation_batch()
