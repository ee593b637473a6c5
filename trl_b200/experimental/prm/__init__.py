from .prm_config import PRMConfig
from .prm_trainer import PRMTrainer

__all__ = ["PRMConfig", "PRMTrainer"]
