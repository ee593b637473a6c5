from .server_distillation_config import ServerDistillationConfig
from .server_distillation_trainer import ServerDistillationTrainer, build_teacher_request_inputs

__all__ = ["ServerDistillationConfig", "ServerDistillationTrainer", "build_teacher_request_inputs"]
