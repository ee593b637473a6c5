"""Defaults shared by all trainer configs (trl/trainer/base_config.py:20-107):
``logging_steps=10``, ``gradient_checkpointing=True``, ``bf16`` defaults to
``not fp16``, ``lr_scheduler_kwargs`` accepts a dict or JSON string."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ..loop.training_args import TrainingArguments


@dataclass
class _BaseConfig(TrainingArguments):
    logging_steps: float = field(default=10, metadata={"help": "Log every N update steps (or ratio if < 1)."})
    gradient_checkpointing: bool = field(default=True, metadata={"help": "Recompute layer activations in backward."})
    bf16: Optional[bool] = field(default=None, metadata={"help": "bf16 compute; defaults to True unless fp16 is set."})
    lr_scheduler_kwargs: Optional[Any] = field(default=None, metadata={"help": "Extra scheduler parameters."})
    use_liger_kernel: bool = field(default=False, metadata={
        "help": "Accepted for compatibility: the fused sm_100a kernels are always used on GPUs."})
    torch_empty_cache_steps: Optional[int] = field(default=None, metadata={"help": "Empty the caching allocator every N steps."})
