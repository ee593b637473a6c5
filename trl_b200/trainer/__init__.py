"""Trainers and configs (trl/trainer/__init__.py:20-48)."""
from .callbacks import (BEMACallback, LogCompletionsCallback, RichProgressCallback, SyncRefModelCallback,
                        WeaveCallback)
from .dpo_config import DPOConfig
from .dpo_trainer import DPOTrainer
from .grpo_config import GRPOConfig, RLOOConfig
from .grpo_trainer import GRPOTrainer
from .kto_trainer import KTOConfig, KTOTrainer
from .model_config import ModelConfig
from .reward_trainer import RewardConfig, RewardTrainer
from .rloo_trainer import RLOOTrainer
from .sft_config import SFTConfig
from .sft_trainer import SFTTrainer
from .utils import (disable_dropout_in_model, ensure_master_addr_port, get_peft_config, get_quantization_config)
from ..ops.chunked_lm_head import patch_chunked_lm_head
