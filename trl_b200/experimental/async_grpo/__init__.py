from .async_grpo_config import AsyncGRPOConfig
from .async_grpo_trainer import AsyncGRPOTrainer, TokenBudgetBatcher
from .async_rollout_worker import AsyncRolloutWorker, RolloutSample

__all__ = ["AsyncGRPOConfig", "AsyncGRPOTrainer", "AsyncRolloutWorker", "RolloutSample", "TokenBudgetBatcher"]
