"""SDPOConfig (fields/defaults of trl/experimental/sdpo/sdpo_config.py:24-644)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ...trainer.grpo_config import GRPOConfig


@dataclass
class SDPOConfig(GRPOConfig):
    distillation_weight: float = 1.0        # loss = (1 - w) * policy loss + w * self-distillation loss
    distillation_alpha: float = 0.5
    distillation_mode: str = "topk_logits"
    distillation_topk: Optional[int] = 100
    distillation_is_clip: Optional[float] = 2.0
    distillation_add_tail: bool = False
    num_loss_tokens_to_skip: int = 0
    teacher_model_kind: str = "base"
    teacher_update_rate: float = 0.05
    teacher_sync_steps: int = 1
    use_successful_as_teacher: bool = True  # a successful rollout of the same prompt becomes the demonstration
    success_reward_threshold: float = 1.0
    dont_reprompt_on_self_success: bool = True
    max_reprompt_len: int = 10240
    reprompt_template: str = "{prompt}{solution}{feedback}\n\nCorrectly solve the original question.\n"
    solution_template: str = "\nCorrect solution:\n\n{successful_previous_attempt}\n\n"
    feedback_template: str = "\nThe following is feedback from your unsuccessful earlier attempt:\n\n{feedback_raw}\n\n"
    include_environment_feedback: bool = False
    environment_feedback_only_without_solution: bool = False
    remove_thinking_from_demonstration: bool = False
    diagnostics_warning_interval: int = 10
    diagnostics_flat_tolerance: float = 1e-8
    use_teacher_server: bool = False

    def __post_init__(self):
        super().__post_init__()
        if not 0.0 <= self.distillation_weight <= 1.0:
            raise ValueError("distillation_weight must be in [0, 1]")
        if self.distillation_mode not in ("sampled_token", "full_logits", "topk_logits"):
            raise ValueError("distillation_mode must be 'sampled_token', 'full_logits' or 'topk_logits'")
        if self.use_teacher_server:
            raise NotImplementedError("use_teacher_server needs a remote teacher endpoint; the teacher runs in-process here")
