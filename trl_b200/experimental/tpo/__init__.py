from .tpo_config import TPOConfig
from .tpo_trainer import TPOTrainer

__all__ = ["TPOConfig", "TPOTrainer"]
