"""Reward functions (trl/rewards/__init__.py:21-25)."""
from .accuracy_rewards import accuracy_reward, get_cosine_scaled_reward, reasoning_accuracy_reward
from .format_rewards import think_format_reward
from .other_rewards import get_repetition_penalty_reward, get_soft_overlong_punishment

__all__ = ["accuracy_reward", "get_cosine_scaled_reward", "reasoning_accuracy_reward", "think_format_reward",
           "get_repetition_penalty_reward", "get_soft_overlong_punishment"]
