"""OnlineDPOConfig (fields/defaults of trl/experimental/online_dpo/online_dpo_config.py:24-390).

Every dataloader row is one prompt; the trainer samples the two candidate completions itself, so
``num_generations`` stays 1 and the ``vllm_*`` names select the in-box rollout engine as in GRPO."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ...trainer.grpo_config import _OnlineConfig


@dataclass
class OnlineDPOConfig(_OnlineConfig):
    _MIN_GENERATIONS = 1

    learning_rate: float = 5e-7
    reward_model_path: Optional[str] = None
    judge: Optional[str] = None
    max_new_tokens: int = 64
    max_length: int = 512
    temperature: float = 0.9
    missing_eos_penalty: Optional[float] = None
    beta: Any = field(default_factory=lambda: [0.1])  # a list selects one value per epoch
    loss_type: str = "sigmoid"  # sigmoid | ipo
    disable_dropout: bool = True
    num_generations: Optional[int] = 1
    logging_steps: float = 10

    def __post_init__(self):
        super().__post_init__()
        if hasattr(self.beta, "__len__") and len(self.beta) == 1:
            self.beta = self.beta[0]
        if self.loss_type not in ("sigmoid", "ipo"):
            raise ValueError("loss_type must be 'sigmoid' or 'ipo'")
        self.max_completion_length = self.max_new_tokens
        self.num_generations = 1
        self.num_iterations = 1
        self._needs_ref = True
        self._derive_generation_batch()
