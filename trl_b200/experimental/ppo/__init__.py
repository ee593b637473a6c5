from .modeling_value_head import AutoModelForCausalLMWithValueHead, ValueHead
from .ppo_config import PPOConfig
from .ppo_trainer import PPOTrainer

__all__ = ["AutoModelForCausalLMWithValueHead", "PPOConfig", "PPOTrainer", "ValueHead"]
