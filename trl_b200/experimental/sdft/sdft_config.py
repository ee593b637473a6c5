"""SDFTConfig (fields/defaults of trl/experimental/sdft/sdft_config.py:24-472)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ...trainer.grpo_config import _OnlineConfig


@dataclass
class SDFTConfig(_OnlineConfig):
    _MIN_GENERATIONS = 1

    distillation_alpha: float = 0.5
    distillation_mode: str = "topk_logits"  # sampled_token | full_logits | topk_logits
    distillation_topk: Optional[int] = 100
    distillation_is_clip: Optional[float] = 2.0
    distillation_add_tail: bool = False
    num_loss_tokens_to_skip: int = 0
    teacher_model_kind: str = "base"        # base | ema | student
    teacher_update_rate: float = 0.05
    teacher_sync_steps: int = 1
    generate_from_teacher: bool = False
    teacher_prompt_template: str = "{prompt}\n\n{privileged_context}"
    disable_dropout: bool = True
    max_prompt_length: Optional[int] = 512
    max_completion_length: Optional[int] = 256
    num_generations: Optional[int] = 8
    use_teacher_server: bool = False

    def __post_init__(self):
        super().__post_init__()
        if self.distillation_mode not in ("sampled_token", "full_logits", "topk_logits"):
            raise ValueError("distillation_mode must be 'sampled_token', 'full_logits' or 'topk_logits'")
        if self.distillation_mode == "sampled_token" and self.distillation_alpha != 1.0:
            raise ValueError("distillation_mode='sampled_token' needs distillation_alpha=1.0 (reverse KL)")
        if self.use_teacher_server:
            raise NotImplementedError("use_teacher_server needs a remote teacher endpoint; the teacher runs in-process here")
        self._derive_generation_batch()
