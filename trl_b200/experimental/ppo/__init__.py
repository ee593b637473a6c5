from .modeling_value_head import (AutoModelForCausalLMWithValueHead, AutoModelForSeq2SeqLMWithValueHead,
                                  PreTrainedModelWrapper, ValueHead)
from .ppo_config import PPOConfig
from .ppo_trainer import PPOTrainer

__all__ = ["AutoModelForCausalLMWithValueHead", "AutoModelForSeq2SeqLMWithValueHead", "PPOConfig", "PPOTrainer",
           "PreTrainedModelWrapper", "ValueHead"]
