"""GOLDConfig (fields/defaults of trl/experimental/gold/gold_config.py:24-531)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..distillation.distillation_config import DistillationConfig


@dataclass
class GOLDConfig(DistillationConfig):
    lmbda: float = 0.5
    beta: float = 0.5
    teacher_tokenizer_name_or_path: Optional[str] = None
    use_uld_loss: bool = False               # cross-tokenizer distillation (universal logit distillation)
    use_extended_uld: bool = True            # align student / teacher tokens by text spans before comparing
    uld_token_merge_strategy: str = "mean"   # how distributions of several tokens inside one span are merged
    uld_use_hybrid_loss: bool = False        # JSD on tokens both vocabularies share + sorted-L1 on the rest
    uld_hybrid_matched_weight: Optional[float] = None
    uld_hybrid_unmatched_weight: Optional[float] = None
    uld_crossentropy_weight: float = 0.0
    uld_distillation_weight: float = 1.0
    uld_student_temperature: float = 1.0
    uld_teacher_temperature: float = 1.0
    uld_skip_student_eos: bool = True
    uld_skip_teacher_eos: bool = True
    wandb_log_unique_prompts: bool = True

    def __post_init__(self):
        super().__post_init__()
        if self.uld_token_merge_strategy not in ("mean", "first", "last"):
            raise ValueError("uld_token_merge_strategy must be 'mean', 'first' or 'last'")
