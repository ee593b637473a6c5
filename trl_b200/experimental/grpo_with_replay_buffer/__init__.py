from .grpo_with_replay_buffer_config import GRPOWithReplayBufferConfig
from .grpo_with_replay_buffer_trainer import GRPOWithReplayBufferTrainer, ReplayBuffer

__all__ = ["GRPOWithReplayBufferConfig", "GRPOWithReplayBufferTrainer", "ReplayBuffer"]
