from .callback import BEMACallback
from .dpo_trainer import DPOTrainer

__all__ = ["BEMACallback", "DPOTrainer"]
