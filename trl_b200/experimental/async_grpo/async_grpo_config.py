"""AsyncGRPOConfig (fields/defaults of trl/experimental/async_grpo/async_grpo_config.py:24-331)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from ...trainer.base_config import _BaseConfig


@dataclass
class AsyncGRPOConfig(_BaseConfig):
    _VALID_DICT_FIELDS = _BaseConfig._VALID_DICT_FIELDS + ["model_init_kwargs", "chat_template_kwargs"]

    learning_rate: float = 1e-6
    logging_steps: float = 1
    model_init_kwargs: Optional[Any] = None
    trust_remote_code: bool = False
    router_aux_loss_coef: float = 0.001
    num_generations: int = 8
    max_completion_length: int = 2048
    temperature: float = 1.0
    chat_template_kwargs: Optional[Any] = None
    max_tool_calling_iterations: Optional[int] = None
    fork_threshold_tokens: int = 1024
    vllm_server_base_url: Optional[str] = "http://localhost:8000"  # None: generate in-process on a worker thread
    vllm_server_timeout: float = 240.0
    request_timeout: int = 600
    epsilon: float = 0.2
    epsilon_high: Optional[float] = None
    token_budget: Optional[int] = None   # real tokens per rank and micro-batch; <= 0: fixed sample count instead
    max_inflight_tasks: int = -1
    max_staleness: int = 4               # optimizer steps a sample may lag behind the current weights
    queue_maxsize: int = 1024
    weight_sync_steps: int = 1
    heartbeat_stale_after_s: float = 300.0
    log_completions: bool = False
    num_completions_to_print: Optional[int] = None
    scale_rewards: bool = True
    # "thread": rollouts on a background thread of the training process; "process": a spawned child with its own event
    # loop that talks to the generation server (reward functions must be picklable); "auto": process when a server is
    # configured and training runs on a GPU, else thread
    rollout_worker: str = "auto"

    def __post_init__(self):
        super().__post_init__()
        if self.num_generations < 2:
            raise ValueError("AsyncGRPO needs at least 2 generations per prompt to form advantages")
        if self.epsilon_high is None:
            self.epsilon_high = self.epsilon
