"""Self-distillation fine-tuning (trl/experimental/sdft/sdft_trainer.py: teacher prompts :300-420, loss :900-1100).

Rows carry ``prompt`` and ``privileged_context`` (a demonstration, a hint, ...).  The student samples completions from
the plain prompt; the teacher (initial weights, an EMA of the student, or the live student) scores the same completion
under ``teacher_prompt_template.format(prompt, privileged_context)``; the student is pulled towards the teacher's
token distributions on its own samples."""
from __future__ import annotations

from typing import Any

import torch

from ...data_utils import is_conversational
from ...parallel import dist as D
from ...trainer.online_base import OnlineTrainer
from .._self_distill import SelfDistillMixin
from .sdft_config import SDFTConfig
from .teacher_sync import build_teacher


def _no_reward(completions, **kw):
    return [0.0] * len(completions)


def privileged_prompt(prompt, context, template: str):
    if isinstance(prompt, str):
        return template.format(prompt=prompt, privileged_context=context)
    msgs = [dict(m) for m in prompt]
    for m in reversed(msgs):
        if m["role"] == "user":
            m["content"] = template.format(prompt=m["content"], privileged_context=context)
            break
    return msgs


class SDFTTrainer(SelfDistillMixin, OnlineTrainer):
    _tag_names = ["trl", "sdft"]
    _name = "SDFT"
    config_cls = SDFTConfig

    def __init__(self, model, args: SDFTConfig | None = None, train_dataset=None, eval_dataset=None,
                 processing_class=None, callbacks=None, peft_config=None, **kw):
        args = args or SDFTConfig("model-SDFT")
        super().__init__(model, [_no_reward], args, train_dataset=train_dataset, eval_dataset=eval_dataset,
                         processing_class=processing_class, callbacks=callbacks, peft_config=peft_config)
        self.teacher = build_teacher(self, args.teacher_model_kind, args.teacher_update_rate, args.teacher_sync_steps)

    def _generate_and_score_completions(self, inputs: list[dict]) -> dict[str, Any]:
        a = self.args
        prompts = [x["prompt"] for x in inputs]
        t_prompts = [privileged_prompt(x["prompt"], x.get("privileged_context", ""), a.teacher_prompt_template)
                     if x.get("privileged_context") else x["prompt"] for x in inputs]
        t_ids = self._tokenize_prompts(t_prompts)
        if a.generate_from_teacher:
            _, completion_ids, _, _ = self._generate(t_prompts)
            prompt_ids = self._tokenize_prompts(prompts)
        else:
            prompt_ids, completion_ids, _, _ = self._generate(prompts)
        if a.max_prompt_length:
            prompt_ids = [p[-a.max_prompt_length:] for p in prompt_ids]
        with torch.no_grad():
            old, _ = self._get_per_token_logps_and_entropies(self.model, prompt_ids, completion_ids)
        lens = torch.tensor([len(c) for c in completion_ids], device=old.device, dtype=torch.float32)
        m = self._metrics["train" if self.model.training else "eval"]
        m["completions/mean_length"].append(D.gather(lens.mean().reshape(1)).mean())
        return {"prompt_ids": prompt_ids, "teacher_prompt_ids": t_ids, "completion_ids_list": completion_ids,
                "old_per_token_logps": old}

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        loss, per_tok = self.self_distillation_loss(model, inputs["prompt_ids"], inputs["teacher_prompt_ids"],
                                                    inputs["completion_ids_list"], inputs.get("old_per_token_logps"))
        self._metrics["train" if model.training else "eval"]["distillation_loss"].append(per_tok.mean())
        loss = loss / self.current_gradient_accumulation_steps
        return (loss, None) if return_outputs else loss
