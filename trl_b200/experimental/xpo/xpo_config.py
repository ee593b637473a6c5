"""XPOConfig (trl/experimental/xpo/xpo_config.py:20-44)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..online_dpo.online_dpo_config import OnlineDPOConfig


@dataclass
class XPOConfig(OnlineDPOConfig):
    alpha: Any = field(default_factory=lambda: [1e-5])  # weight of the optimism term; a list selects one value per epoch

    def __post_init__(self):
        super().__post_init__()
        if hasattr(self.alpha, "__len__") and len(self.alpha) == 1:
            self.alpha = self.alpha[0]
