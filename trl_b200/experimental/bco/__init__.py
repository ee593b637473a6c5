from .bco_config import BCOConfig
from .bco_trainer import BCOTrainer, RunningMoments

__all__ = ["BCOConfig", "BCOTrainer", "RunningMoments"]
