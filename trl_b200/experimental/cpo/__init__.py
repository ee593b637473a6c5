from .cpo_config import CPOConfig
from .cpo_trainer import CPOTrainer

__all__ = ["CPOConfig", "CPOTrainer"]
