"""Self-distillation policy optimisation (trl/experimental/sdpo/sdpo_trainer.py: re-prompting :700-1000, loss mix
:1300-1500).

GRPO rollouts with rewards.  For every rollout a teacher prompt is built from the original prompt plus a successful
rollout of the same prompt (reward >= ``success_reward_threshold``; not the rollout itself unless allowed) and,
optionally, environment feedback; the student is distilled towards the teacher's token distributions under that
re-prompt.  Rollouts with nothing to show the teacher take no distillation loss.
loss = (1 - distillation_weight) * GRPO loss + distillation_weight * distillation loss."""
from __future__ import annotations

import re
import warnings

import torch

from ...parallel import dist as D
from ...trainer.grpo_trainer import GRPOTrainer
from .._self_distill import SelfDistillMixin
from .sdpo_config import SDPOConfig
from ..sdft.teacher_sync import build_teacher

_THINK = re.compile(r"<think>.*?</think>", re.S)


class SDPOTrainer(SelfDistillMixin, GRPOTrainer):
    _tag_names = ["trl", "sdpo"]
    _name = "SDPO"
    config_cls = SDPOConfig

    def __init__(self, model, reward_funcs, args: SDPOConfig | None = None, **kw):
        args = args or SDPOConfig("model-SDPO")
        super().__init__(model, reward_funcs, args, **kw)
        self.teacher = build_teacher(self, args.teacher_model_kind, args.teacher_update_rate, args.teacher_sync_steps)
        self._flat_steps = 0

    def _reprompt(self, prompt, solution_text, feedback_text):
        a = self.args
        sol = a.solution_template.format(successful_previous_attempt=solution_text) if solution_text else ""
        fb = a.feedback_template.format(feedback_raw=feedback_text) if feedback_text else ""
        if isinstance(prompt, str):
            return a.reprompt_template.format(prompt=prompt, solution=sol, feedback=fb)
        msgs = [dict(m) for m in prompt]
        for m in reversed(msgs):
            if m["role"] == "user":
                m["content"] = a.reprompt_template.format(prompt=m["content"], solution=sol, feedback=fb)
                break
        return msgs

    def _calculate_rewards(self, inputs, prompts, completions, completion_ids_list):
        out = super()._calculate_rewards(inputs, prompts, completions, completion_ids_list)
        self._last_inputs, self._last_prompts, self._last_completions = inputs, prompts, completions
        return out

    def _generate_and_score_completions(self, inputs):
        out = super()._generate_and_score_completions(inputs)
        a = self.args
        B = len(out["prompt_ids"])
        ng = self.num_generations if self.model.training else self.num_generations_eval
        tok = self.processing_class
        texts = tok.batch_decode(out["completion_ids_list"], skip_special_tokens=True)
        if a.remove_thinking_from_demonstration:
            demo_texts = [_THINK.sub("", t).strip() for t in texts]
        else:
            demo_texts = texts
        local_r = self._local_total_rewards
        t_prompts, has_teacher = [], []
        for i in range(B):
            g0 = i // ng * ng
            sol = None
            if a.use_successful_as_teacher:
                cands = [j for j in range(g0, min(g0 + ng, B)) if float(local_r[j]) >= a.success_reward_threshold
                         and (j != i or not a.dont_reprompt_on_self_success)]
                if cands:
                    sol = demo_texts[max(cands, key=lambda j: float(local_r[j]))]
            fb = None
            if a.include_environment_feedback and not (a.environment_feedback_only_without_solution and sol):
                fb = self._last_inputs[i].get("feedback") if isinstance(self._last_inputs[i], dict) else None
            has_teacher.append(sol is not None or fb is not None)
            t_prompts.append(self._reprompt(self._last_prompts[i], sol, fb))
        t_ids = [ids[-a.max_reprompt_len:] for ids in self._tokenize_prompts(t_prompts)]
        out["teacher_prompt_ids"] = t_ids
        out["has_teacher"] = torch.tensor(has_teacher, dtype=torch.float32, device=out["advantages"].device)
        frac = D.gather(out["has_teacher"].mean().reshape(1)).mean()
        self._metrics["train" if self.model.training else "eval"]["sdpo/teacher_coverage"].append(frac)
        if float(frac) == 0.0:
            self._flat_steps += 1
            if self._flat_steps % max(1, a.diagnostics_warning_interval) == 0:
                warnings.warn("SDPO: no rollout reached success_reward_threshold for a while; the distillation term is idle")
        return out

    def _advantages(self, rewards_per_func, ng):
        adv, rewards, std, is_zero = super()._advantages(rewards_per_func, ng)
        n = rewards.shape[0] // D.world_size()
        self._local_total_rewards = torch.nan_to_num(rewards[D.rank() * n:(D.rank() + 1) * n], nan=float("-inf"))
        return adv, rewards, std, is_zero

    def _compute_loss(self, model, inputs):
        w = self.args.distillation_weight
        m = self._metrics["train" if model.training else "eval"]
        policy = super()._compute_loss(model, inputs) if w < 1.0 else None
        loss = 0.0 if policy is None else (1 - w) * policy
        if w > 0.0:
            d, per_tok = self.self_distillation_loss(model, inputs["prompt_ids"], inputs["teacher_prompt_ids"],
                                                     inputs["completion_ids_list"], inputs.get("old_per_token_logps"),
                                                     row_weight=inputs["has_teacher"])
            m["sdpo/distillation_loss"].append(d.detach())
            loss = loss + w * d / self.current_gradient_accumulation_steps
        return loss
