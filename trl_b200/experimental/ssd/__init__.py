from .ssd_config import SSDConfig
from .ssd_trainer import SSDTrainer

__all__ = ["SSDConfig", "SSDTrainer"]
