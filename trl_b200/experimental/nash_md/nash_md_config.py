"""NashMDConfig (trl/experimental/nash_md/nash_md_config.py:20-46)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..online_dpo.online_dpo_config import OnlineDPOConfig


@dataclass
class NashMDConfig(OnlineDPOConfig):
    mixture_coef: Any = field(default_factory=lambda: [0.5])  # weight of the reference logits in the mixture policy

    def __post_init__(self):
        super().__post_init__()
        if hasattr(self.mixture_coef, "__len__") and len(self.mixture_coef) == 1:
            self.mixture_coef = self.mixture_coef[0]
