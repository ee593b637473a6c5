from .server_distillation_config import ServerDistillationConfig
from .server_distillation_trainer import ServerDistillationTrainer

__all__ = ["ServerDistillationConfig", "ServerDistillationTrainer"]
