from .minillm_config import MiniLLMConfig
from .minillm_trainer import MiniLLMTrainer

__all__ = ["MiniLLMConfig", "MiniLLMTrainer"]
