from .nash_md_config import NashMDConfig
from .nash_md_trainer import GeometricMixtureGenerator, NashMDTrainer

__all__ = ["NashMDConfig", "NashMDTrainer", "GeometricMixtureGenerator"]
