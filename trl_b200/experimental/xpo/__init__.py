from .xpo_config import XPOConfig
from .xpo_trainer import XPOTrainer

__all__ = ["XPOConfig", "XPOTrainer"]
