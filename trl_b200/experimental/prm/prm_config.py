"""PRMConfig (fields/defaults of trl/experimental/prm/prm_config.py:24-88)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ...trainer.base_config import _BaseConfig


@dataclass
class PRMConfig(_BaseConfig):
    learning_rate: float = 1e-5
    max_length: Optional[int] = 1024
    max_completion_length: Optional[int] = None
    disable_dropout: bool = True
    step_separator: str = "\n"
    train_on_last_step_only: bool = False
    dataset_num_proc: Optional[int] = None
