from .grpo_trainer import GRPOTrainer

__all__ = ["GRPOTrainer"]
