from .orpo_config import ORPOConfig
from .orpo_trainer import ORPOTrainer

__all__ = ["ORPOConfig", "ORPOTrainer"]
