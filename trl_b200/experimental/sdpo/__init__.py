from .sdpo_config import SDPOConfig
from .sdpo_trainer import SDPOTrainer

__all__ = ["SDPOConfig", "SDPOTrainer"]
