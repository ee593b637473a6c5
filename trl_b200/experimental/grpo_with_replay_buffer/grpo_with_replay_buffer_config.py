"""trl/experimental/grpo_with_replay_buffer/grpo_with_replay_buffer_config.py:20-34."""
from __future__ import annotations

from dataclasses import dataclass

from ...trainer.grpo_config import GRPOConfig


@dataclass
class GRPOWithReplayBufferConfig(GRPOConfig):
    replay_buffer_size: int = 64  # groups kept (highest |advantage| x reward-std first); 0 disables the buffer
