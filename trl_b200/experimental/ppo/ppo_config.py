"""PPOConfig (fields/defaults of trl/experimental/ppo/ppo_config.py:24-280).

The rollout batch of one update is ``per_device_train_batch_size * gradient_accumulation_steps * num_mini_batches``
sequences per rank; it is split into ``num_mini_batches`` optimizer steps and revisited ``num_ppo_epochs`` times."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ...trainer.grpo_config import _OnlineConfig


@dataclass
class PPOConfig(_OnlineConfig):
    _MIN_GENERATIONS = 1

    learning_rate: float = 3e-6
    dataset_num_proc: Optional[int] = None
    num_mini_batches: int = 1
    total_episodes: Optional[int] = None
    local_rollout_forward_batch_size: int = 64
    num_sample_generations: int = 10
    response_length: int = 53
    stop_token: Optional[str] = None
    stop_token_id: Optional[int] = None
    temperature: float = 0.7
    missing_eos_penalty: Optional[float] = None
    sft_model_path: str = "EleutherAI/pythia-160m"
    reward_model_path: str = "EleutherAI/pythia-160m"
    model_adapter_name: Optional[str] = None
    ref_adapter_name: Optional[str] = None
    num_ppo_epochs: int = 4
    whiten_rewards: bool = False
    kl_coef: float = 0.05
    kl_estimator: str = "k1"
    cliprange: float = 0.2
    vf_coef: float = 0.1
    cliprange_value: float = 0.2
    gamma: float = 1.0
    lam: float = 0.95
    logging_steps: float = 1

    def __post_init__(self):
        super().__post_init__()
        if self.kl_estimator not in ("k1", "k3"):
            raise ValueError("kl_estimator must be 'k1' or 'k3'")
        self.max_completion_length = self.response_length
        self.num_generations = 1
        self.num_iterations = self.num_ppo_epochs
        self.steps_per_generation = self.num_mini_batches * self.gradient_accumulation_steps
        self.generation_batch_size = None
        self._needs_ref = True
        self._derive_generation_batch()
        from ...parallel import dist as D

        world = D.world_size()
        self.local_batch_size = self.per_device_train_batch_size * self.steps_per_generation
        self.batch_size = self.local_batch_size * world
        self.local_mini_batch_size = self.local_batch_size // self.num_mini_batches
        self.mini_batch_size = self.batch_size // self.num_mini_batches
        if self.total_episodes is not None and self.max_steps <= 0:
            updates = -(-self.total_episodes // self.batch_size)
            self.max_steps = updates * self.num_ppo_epochs * self.num_mini_batches
