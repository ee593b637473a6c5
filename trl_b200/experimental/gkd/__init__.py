from .gkd_config import GKDConfig
from .gkd_trainer import GKDTrainer

__all__ = ["GKDConfig", "GKDTrainer"]
