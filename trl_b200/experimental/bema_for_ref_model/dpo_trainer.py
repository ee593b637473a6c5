"""DPOTrainer that hands its reference model to a BEMACallback (trl/experimental/bema_for_ref_model/dpo_trainer.py)."""
from __future__ import annotations

from ...trainer.dpo_trainer import DPOTrainer as _DPOTrainer
from .callback import BEMACallback


class DPOTrainer(_DPOTrainer):
    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        for cb in self.callback_handler.callbacks:
            if isinstance(cb, BEMACallback):
                cb.attach(self.ref_model)
