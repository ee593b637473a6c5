"""ModelConfig: model / adapter / quantisation flags of the scripts (trl/trainer/model_config.py:18-178)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class ModelConfig:
    model_name_or_path: Optional[str] = field(default=None, metadata={"help": "Local checkpoint directory or preset name."})
    model_revision: str = "main"
    dtype: Optional[str] = field(default="float32", metadata={"help": "auto | bfloat16 | float16 | float32"})
    trust_remote_code: bool = False
    attn_implementation: Optional[str] = field(default=None, metadata={
        "help": "Accepted for compatibility; the native varlen attention is always used."})
    use_peft: bool = False
    lora_r: int = 16
    lora_alpha: int = 32
    lora_dropout: float = 0.05
    lora_target_modules: Optional[list] = None
    lora_target_parameters: Optional[list] = None
    lora_modules_to_save: Optional[list] = None
    lora_task_type: str = "CAUSAL_LM"
    use_rslora: bool = False
    use_dora: bool = False
    load_in_8bit: bool = False
    load_in_4bit: bool = False
    bnb_4bit_quant_type: str = "nf4"
    use_bnb_nested_quant: bool = False
    bnb_4bit_quant_storage: Optional[str] = None

    def __post_init__(self):
        if self.load_in_8bit and self.load_in_4bit:
            raise ValueError("You can't use 8 bit and 4 bit precision at the same time")
        if isinstance(self.lora_target_modules, list) and len(self.lora_target_modules) == 1:
            self.lora_target_modules = self.lora_target_modules[0] if self.lora_target_modules[0] == "all-linear" \
                else self.lora_target_modules
