"""BEMA that also refreshes the DPO reference model (trl/experimental/bema_for_ref_model/callback.py:24-223).

Same bias-corrected EMA as ``trl_b200.trainer.callbacks.BEMACallback``; every update additionally copies the BEMA
weights into ``trainer.ref_model`` (``update_ref_model=True``, every ``ref_model_update_freq`` updates)."""
from __future__ import annotations

import torch

from ...trainer.callbacks import BEMACallback as _BEMA


class BEMACallback(_BEMA):
    def __init__(self, *a, update_ref_model: bool = False, ref_model_update_freq: int = 400,
                 ref_model_update_after: int = 0, **kw):
        super().__init__(*a, **kw)
        self.update_ref_model = update_ref_model
        self.ref_model_update_freq, self.ref_model_update_after = ref_model_update_freq, ref_model_update_after
        self.ref_model = None

    def attach(self, ref_model):
        self.ref_model = ref_model

    @torch.no_grad()
    def on_step_end(self, args, state, control, model=None, **kw):
        super().on_step_end(args, state, control, model=model, **kw)
        step = state.global_step
        if (self.update_ref_model and self.ref_model is not None and self.running is not None
                and step >= self.ref_model_update_after
                and (step - self.ref_model_update_after) % self.ref_model_update_freq == 0):
            named = dict(self.ref_model.named_parameters())
            for n, w in zip(self.names, self.running):
                if n in named:
                    named[n].copy_(w.to(named[n].device, named[n].dtype))
