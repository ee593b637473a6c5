from .distillation_config import DistillationConfig
from .distillation_trainer import DistillationTrainer

__all__ = ["DistillationConfig", "DistillationTrainer"]
