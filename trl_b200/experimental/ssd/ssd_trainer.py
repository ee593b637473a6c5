"""Simple self-distillation (trl/experimental/ssd/ssd_trainer.py:74-533): sample completions from the model at a
training-time temperature / truncation setting and fine-tune on those raw, unverified samples with plain
cross-entropy.  The dataset only needs a ``prompt`` column."""
from __future__ import annotations

from typing import Any

import torch

from ...parallel import dist as D
from ...trainer.online_base import OnlineTrainer
from .ssd_config import SSDConfig


def _no_reward(completions, **kw):
    return [0.0] * len(completions)


class SSDTrainer(OnlineTrainer):
    _tag_names = ["trl", "ssd"]
    _name = "SSD"
    config_cls = SSDConfig

    def __init__(self, model, args: SSDConfig | None = None, train_dataset=None, eval_dataset=None, processing_class=None,
                 callbacks=None, peft_config=None, **kw):
        super().__init__(model, [_no_reward], args or SSDConfig("model-SSD"), train_dataset=train_dataset,
                         eval_dataset=eval_dataset, processing_class=processing_class, callbacks=callbacks,
                         peft_config=peft_config)

    def _generate_and_score_completions(self, inputs: list[dict]) -> dict[str, Any]:
        a = self.args
        prompt_ids, completion_ids, _, _ = self._generate([x["prompt"] for x in inputs])
        if a.max_prompt_length:
            prompt_ids = [p[-a.max_prompt_length:] for p in prompt_ids]
        keep = torch.tensor([1.0 if (len(c) > 0 or not a.filter_empty) else 0.0 for c in completion_ids],
                            device=self.args.device)
        lens = torch.tensor([float(len(c)) for c in completion_ids], device=self.args.device)
        m = self._metrics["train" if self.model.training else "eval"]
        m["completions/mean_length"].append(D.gather(lens.mean().reshape(1)).mean())
        return {"prompt_ids": prompt_ids, "completion_ids_list": completion_ids, "keep": keep}

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        lp, ent = self._get_per_token_logps_and_entropies(model, inputs["prompt_ids"], inputs["completion_ids_list"],
                                                          compute_entropy=True, temperature=1.0)
        lens = torch.tensor([len(c) for c in inputs["completion_ids_list"]], device=lp.device)
        mask = (torch.arange(lp.shape[1], device=lp.device)[None] < lens[:, None]).float() * inputs["keep"][:, None]
        s = torch.stack([mask.sum()])
        if D.world_size() > 1:
            D.all_reduce(s, "sum")
        # token mean over the whole job, like num_items_in_batch of the SFT loss
        loss = -(lp * mask).sum() / (s[0].clamp(min=1) / D.world_size()) / self.current_gradient_accumulation_steps
        m = self._metrics["train" if model.training else "eval"]
        m["entropy"].append(((ent * mask).sum() / mask.sum().clamp(min=1)).detach())
        return (loss, None) if return_outputs else loss
