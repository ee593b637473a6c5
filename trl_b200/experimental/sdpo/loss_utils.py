"""SDPO scores its distillation term with the same divergences as SDFT (trl/experimental/sdpo/loss_utils.py is a copy of
the SDFT module in the reference); they live in ``experimental/sdft/loss_utils.py``."""
from ..sdft.loss_utils import *  # noqa: F401,F403
from ..sdft.loss_utils import (add_tail_bucket, apply_importance_sampling_clipping, compute_divergence,  # noqa: F401
                               compute_full_logit_self_distillation_loss, compute_sampled_token_self_distillation_loss,
                               compute_topk_self_distillation_loss, support_divergence)
