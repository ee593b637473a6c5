"""ORPO (trl/experimental/orpo/orpo_trainer.py: odds_ratio_loss :693-735, total loss :851).

loss = NLL(chosen) - beta * mean(log sigmoid(log_odds)), log_odds = (lc - lr) - (log(1-e^lc) - log(1-e^lr)) on
length-normalised log-probs; no reference model."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .._pairwise import PairwiseTrainer
from .orpo_config import ORPOConfig


def log1mexp(x: torch.Tensor) -> torch.Tensor:
    """log(1 - exp(x)) for x < 0, stable on both ends."""
    x = x.clamp(max=-1e-7)
    return torch.where(x > -0.6931471805599453, torch.log(-torch.expm1(x)), torch.log1p(-torch.exp(x)))


class ORPOTrainer(PairwiseTrainer):
    _tag_names = ["trl", "orpo"]
    _name = "ORPO"
    _average_logps = True

    def __init__(self, model, args: ORPOConfig | None = None, **kw):
        super().__init__(model, args or ORPOConfig("model-ORPO"), **kw)

    def pair_loss(self, pc, pr, nll, ex, P):
        pc, pr = pc.float(), pr.float()
        log_odds = (pc - pr) - (log1mexp(pc) - log1mexp(pr))
        ratio = F.logsigmoid(log_odds)
        return -self.args.beta * ratio, nll, {"log_odds_ratio": ratio.mean(), "log_odds_chosen": log_odds.mean()}
