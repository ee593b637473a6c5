from .gmpo_config import GMPOConfig
from .gmpo_trainer import GMPOTrainer

__all__ = ["GMPOConfig", "GMPOTrainer"]
