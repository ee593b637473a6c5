"""CPO / SimPO / AlphaPO (trl/experimental/cpo/cpo_trainer.py: loss :671-737, NLL term :838-845, total :889).

Reference-free: loss = pair_loss(logp_chosen, logp_rejected) + cpo_alpha * NLL(chosen); ``simpo`` and ``ipo`` use
length-normalised log-probs, ``simpo`` subtracts the margin gamma/beta; ``alpha != 0`` reshapes rewards as
(1 - p^-alpha) / alpha."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .._pairwise import PairwiseTrainer
from .cpo_config import CPOConfig


class CPOTrainer(PairwiseTrainer):
    _tag_names = ["trl", "cpo"]
    _name = "CPO"

    def __init__(self, model, args: CPOConfig | None = None, **kw):
        args = args or CPOConfig("model-CPO")
        self._average_logps = args.loss_type in ("ipo", "simpo")
        super().__init__(model, args, **kw)
        self.cpo_alpha, self.simpo_gamma, self.alpha = args.cpo_alpha, args.simpo_gamma, args.alpha

    def _shaped(self, logps):
        if self.alpha != 0.0:
            return (1 - torch.exp(logps).pow(-self.alpha)) / self.alpha
        return logps

    def _rewards(self, logps):
        return self.args.beta * self._shaped(logps)

    def pair_loss(self, pc, pr, nll, ex, P):
        beta, ls = self.args.beta, self.args.label_smoothing
        logits = self._shaped(pc) - self._shaped(pr)
        if self.loss_type == "simpo":
            logits = logits - self.simpo_gamma / beta
        if self.loss_type in ("simpo", "sigmoid"):
            per = -F.logsigmoid(beta * logits) * (1 - ls) - F.logsigmoid(-beta * logits) * ls
        elif self.loss_type == "hinge":
            per = torch.relu(1 - beta * logits)
        else:  # ipo
            per = (logits - 1 / (2 * beta)) ** 2
        extra = self.cpo_alpha * nll if self.cpo_alpha != 0 else nll * 0.0
        return per, extra, {}
