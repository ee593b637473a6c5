"""On-policy distillation (trl/experimental/distillation/distillation_trainer.py: buffer :627-860, loss :886-997).

The GKD objective with the generation settings of an online trainer: completions are sampled from the student
(fraction ``lmbda`` of the steps) with top-p / top-k, several per prompt when ``num_generations > 1``, and the
student is trained with JSD(beta) against the teacher on them."""
from __future__ import annotations

from ...trainer.utils import pad
from .._distill import sample_completions
from ..gkd.gkd_trainer import GKDTrainer
from .distillation_config import DistillationConfig

import torch


class DistillationTrainer(GKDTrainer):
    _tag_names = ["trl", "distillation"]
    _name = "Distillation"

    def __init__(self, model=None, teacher_model=None, args: DistillationConfig | None = None, **kw):
        super().__init__(model, teacher_model, args or DistillationConfig("model-Distillation"), **kw)

    def generate_on_policy_outputs(self, model, inputs):
        a, tok = self.args, self.processing_class
        prompts = [p for p in self._prompts_of(inputs) for _ in range(max(1, a.num_generations))]
        comps = sample_completions(model, prompts, a.max_completion_length, temperature=self.temperature, top_p=a.top_p,
                                   top_k=a.top_k, eos_token_id=tok.eos_token_id, seed=self._rng.randrange(1 << 30),
                                   engine_cache=self._gen_cache)
        dev = inputs["input_ids"].device
        seqs = [torch.tensor(p + c, dtype=torch.long) for p, c in zip(prompts, comps)]
        labs = [torch.tensor([-100] * len(p) + c, dtype=torch.long) for p, c in zip(prompts, comps)]
        return (pad(seqs, tok.pad_token_id, "right").to(dev), pad([torch.ones_like(s) for s in seqs], 0, "right").to(dev),
                pad(labs, -100, "right").to(dev))
