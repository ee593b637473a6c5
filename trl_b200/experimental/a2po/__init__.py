from .a2po_config import A2POConfig
from .a2po_trainer import A2POTrainer

__all__ = ["A2POConfig", "A2POTrainer"]
