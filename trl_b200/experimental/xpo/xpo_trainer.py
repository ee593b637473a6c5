"""Exploratory preference optimisation (trl/experimental/xpo/xpo_trainer.py: generation :188-253, losses :324-372).

The opponent completion is sampled from the reference model; the loss is the online DPO loss on the (policy sample,
reference sample) pair plus the optimism term  alpha * log pi(y_ref | x)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...parallel import dist as D
from .._distill import sample_completions
from ..online_dpo.online_dpo_trainer import OnlineDPOTrainer
from .xpo_config import XPOConfig


class XPOTrainer(OnlineDPOTrainer):
    _tag_names = ["trl", "xpo"]
    _name = "XPO"

    def __init__(self, model, ref_model=None, reward_funcs=None, judge=None, args: XPOConfig | None = None, **kw):
        args = args or XPOConfig("model-XPO")
        super().__init__(model, ref_model, reward_funcs, judge, args, **kw)
        self._alpha_schedule = args.alpha

    @property
    def alpha(self):
        return self._per_epoch(self._alpha_schedule)

    def _second_candidates(self, prompt_ids, first):
        ref = self.ref_model if self.ref_model is not None else self.model
        a = self.args
        return sample_completions(ref, prompt_ids, self.max_completion_length, temperature=a.temperature, top_p=a.top_p,
                                  top_k=a.top_k, eos_token_id=self.eos_token_id, seed=a.seed + self.state.global_step,
                                  engine_cache=self._gen_cache)

    def _compute_loss(self, model, inputs):
        mode = "train" if model.training else "eval"
        m = self._metrics[mode]
        p, a, b, a_wins = inputs["prompt_ids"], inputs["cand_a"], inputs["cand_b"], inputs["a_wins"]
        n = len(p)
        lp, mask, ent = self._seq_logps(model, p + p, a + b)  # a: policy data, b: reference data
        with torch.no_grad():
            ref = self._ref_seq_logps(p + p, a + b)
        pol_sum, ref_sum = lp.sum(1), ref.sum(1)
        lr_a, lr_b = pol_sum[:n] - ref_sum[:n], pol_sum[n:] - ref_sum[n:]
        logits = torch.where(a_wins, lr_a - lr_b, lr_b - lr_a)
        beta = self.beta
        dpo = -F.logsigmoid(beta * logits) if self.args.loss_type == "sigmoid" else (logits - 1 / (2 * beta)) ** 2
        xpo = self.alpha * pol_sum[n:]
        loss = (dpo + xpo).mean() / self.current_gradient_accumulation_steps
        with torch.no_grad():
            vals = torch.stack([dpo.mean(), xpo.mean(), (lp.detach() - ref)[:n].sum(1).mean(),
                                (ent * mask)[:n].sum() / mask[:n].sum().clamp(min=1),
                                (beta * torch.where(a_wins, lr_a, lr_b)).mean(), (beta * torch.where(a_wins, lr_b, lr_a)).mean()])
            if D.world_size() > 1:
                D.all_reduce(vals, "mean")
            for k, v in zip(["loss/dpo", "loss/xpo", "objective/kl", "objective/entropy", "rewards/chosen",
                             "rewards/rejected"], vals):
                m[k].append(v)
            m["objective/model_scores"].append(inputs["scores"][:, 0].mean())
            m["objective/ref_scores"].append(inputs["scores"][:, 1].mean())
            m["alpha"].append(float(self.alpha))
            m["beta"].append(float(beta))
        return loss
