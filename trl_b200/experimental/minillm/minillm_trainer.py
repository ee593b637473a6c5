"""MiniLLM: reverse-KL distillation by policy gradient (trl/experimental/minillm/minillm_trainer.py: single-step loss
:246-289, advantage :291-346, compute_loss :348-400).

GRPO machinery with a teacher: per-token reward r_t = log p_teacher(y_t) - log p_student(y_t) turned into a (discounted,
length-normalised) return and added to the reward advantage; plus the exact single-step reverse KL between the
student's and the teacher's next-token distributions on the sampled prefixes."""
from __future__ import annotations

import torch

from ...trainer.grpo_trainer import GRPOTrainer
from ...trainer.utils import create_model_from_path
from .._distill import chunked_token_divergence
from .minillm_config import MiniLLMConfig


def dummy_reward_func(completions: list, **kwargs):
    """Pure distillation: no task reward."""
    return [1.0 for _ in completions]


class MiniLLMTrainer(GRPOTrainer):
    _tag_names = ["trl", "minillm"]
    _name = "MiniLLM"

    def __init__(self, model, teacher_model, reward_funcs=None, args: MiniLLMConfig | None = None, **kw):
        args = args or MiniLLMConfig("model-MiniLLM")
        super().__init__(model, reward_funcs if reward_funcs is not None else [dummy_reward_func], args, **kw)
        if isinstance(teacher_model, str):
            teacher_model = create_model_from_path(teacher_model, **dict(args.teacher_model_init_kwargs or {}))
        self.teacher_model = teacher_model.to(self.args.device, dtype=self.model.dtype).eval().requires_grad_(False)
        self.rkl_advantage, self.single_step = args.rkl_advantage, args.single_step_decomposition
        self.kd_temperature, self.gamma, self.length_normalization = args.kd_temperature, args.gamma, args.length_normalization

    def _compute_advantage(self, student_lp, teacher_lp, mask):
        mask = mask.float()
        rewards = (teacher_lp - student_lp) * mask
        if self.gamma > 0.0:
            T = rewards.shape[1]
            gp = torch.pow(self.gamma, torch.arange(T, device=rewards.device))
            adv = (rewards * gp).flip(1).cumsum(1).flip(1)
            if self.length_normalization:
                lengths = (torch.where(mask < 0.5, torch.full_like(mask, 1e-4), mask) * gp).flip(1).cumsum(1).flip(1)
                adv = adv / lengths
            return adv
        return rewards

    def _compute_loss(self, model, inputs):
        p, c = inputs["prompt_ids"], inputs["completion_ids_list"]
        mask = inputs["completion_mask"].float()
        with torch.no_grad():
            self._keep_selected_hidden = True
            t_lp, _ = self._get_per_token_logps_and_entropies(self.teacher_model, p, c, temperature=self.kd_temperature)
            t_hidden = self._selected_hidden[0]
            self._keep_selected_hidden = False
            if self.rkl_advantage:
                s_lp, _ = self._get_per_token_logps_and_entropies(model, p, c, temperature=self.kd_temperature)
                Tc = s_lp.shape[1]
                mk = mask[:, :Tc] if mask.shape[1] >= Tc else torch.nn.functional.pad(mask, (0, Tc - mask.shape[1]))
                rkl = self._compute_advantage(s_lp, t_lp, mk)
                adv = inputs["advantages"]
                inputs = dict(inputs, advantages=(adv[:, None] if adv.ndim == 1 else adv[:, :Tc]) + rkl)
        self._keep_selected_hidden = self.single_step
        try:
            loss = super()._compute_loss(model, inputs)
            if self.single_step:
                h_s = self._selected_hidden[0]
                kl_sum, per_row = chunked_token_divergence(h_s, model.lm_head_weight, t_hidden,
                                                           self.teacher_model.lm_head_weight, beta=1.0,
                                                           temperature=self.kd_temperature)
                n = max(1, h_s.shape[0])
                loss = loss + kl_sum / n / self.current_gradient_accumulation_steps
                self._metrics["train" if model.training else "eval"]["single_step_rkl"].append(per_row.mean())
        finally:
            self._keep_selected_hidden = False
            self._selected_hidden = None
        return loss
