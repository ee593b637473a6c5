"""GSPO-token (trl/experimental/gspo_token/grpo_trainer.py:24-159): sequence-level importance weights whose gradient
flows through each token's own log-prob, s_{i,t} = sg[s_i] * pi(y_t) / sg[pi(y_t)].  Implemented as
``importance_sampling_level="sequence_token"`` in the stable loss; this class only selects it."""
from __future__ import annotations

from ...trainer.grpo_trainer import GRPOTrainer as _GRPOTrainer


class GRPOTrainer(_GRPOTrainer):
    _tag_names = ["trl", "gspo-token"]

    def __init__(self, model, reward_funcs, args=None, **kw):
        if args is not None and args.importance_sampling_level == "token":
            args.importance_sampling_level = "sequence_token"
        super().__init__(model, reward_funcs, args, **kw)
        self.importance_sampling_level = "sequence_token"
