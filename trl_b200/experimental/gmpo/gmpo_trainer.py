"""Geometric-mean policy optimisation (trl/experimental/gmpo/gmpo_trainer.py:25-155).

GRPO maximises the arithmetic mean of clipped token ratios times the advantage; GMPO takes the geometric mean:
per sequence  -A * exp( mean_t clip_sign(log pi/pi_old) ), clipping in log space on the side the advantage pushes
towards.  The objective itself is the ``gmpo`` branch of ``GRPOTrainer._compute_loss``."""
from __future__ import annotations

from ...trainer.grpo_trainer import GRPOTrainer
from .gmpo_config import GMPOConfig


class GMPOTrainer(GRPOTrainer):
    _tag_names = ["trl", "gmpo"]
    _name = "GMPO"

    def __init__(self, model, reward_funcs, args: GMPOConfig | None = None, **kw):
        args = args or GMPOConfig("model-GMPO")
        if args.loss_type != "gmpo":
            raise ValueError("GMPOTrainer needs loss_type='gmpo'")
        super().__init__(model, reward_funcs, args, **kw)
