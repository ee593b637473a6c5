from .gold_config import GOLDConfig
from .gold_trainer import GOLDTrainer, ULDLoss

__all__ = ["GOLDConfig", "GOLDTrainer", "ULDLoss"]
