from .sdft_config import SDFTConfig
from .sdft_trainer import SDFTTrainer

__all__ = ["SDFTConfig", "SDFTTrainer"]
