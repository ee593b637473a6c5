"""GRPOConfig / RLOOConfig: field names, defaults and validation of
trl/trainer/grpo_config.py:418-1150 and trl/trainer/rloo_config.py.

``use_vllm=True`` selects the in-box rollout engine (``vllm_mode="colocate"``,
``vllm_tensor_parallel_size=k`` -> TP=k); the ``vllm_*`` names are kept so existing
configs parse.  ``rollout_*`` aliases exist for new code.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass, field
from typing import Any, Optional

from .base_config import _BaseConfig


@dataclass
class _OnlineConfig(_BaseConfig):
    _VALID_DICT_FIELDS = _BaseConfig._VALID_DICT_FIELDS + ["model_init_kwargs", "generation_kwargs", "chat_template_kwargs",
                                                            "transformers_continuous_batching_config"]

    learning_rate: float = 1e-6
    logging_steps: float = 10
    model_init_kwargs: Optional[Any] = None
    trust_remote_code: bool = False
    router_aux_loss_coef: float = 0.001
    disable_dropout: bool = False
    cast_lm_head_to_fp32: bool = False
    remove_unused_columns: Optional[bool] = False
    # accepted for configuration parity; generation always runs in this framework's own engine (paged KV, continuous
    # batching), so these select nothing (grpo_config.py / rloo_config.py "transformers continuous batching")
    use_transformers_continuous_batching: bool = False
    transformers_continuous_batching_config: Optional[Any] = None
    use_transformers_paged: bool = False
    num_generations: Optional[int] = 8
    num_generations_eval: Optional[int] = None
    max_completion_length: Optional[int] = 512
    ds3_gather_for_generation: bool = True
    shuffle_dataset: Optional[bool] = True
    # after scoring, deal the job's completions to the ranks by length so that every rank trains on equal work
    # (token ids are exchanged; no counterpart in the reference's synchronous trainer)
    balance_completions: bool = True
    pad_to_multiple_of: Optional[int] = None
    generation_batch_size: Optional[int] = None
    steps_per_generation: Optional[int] = None
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: Optional[float] = None
    generation_kwargs: Optional[Any] = None
    chat_template_kwargs: Optional[Any] = None
    repetition_penalty: float = 1.0
    cache_implementation: Optional[str] = None
    use_vllm: bool = False
    vllm_mode: str = "colocate"
    vllm_model_impl: str = "vllm"
    vllm_enable_sleep_mode: bool = False
    vllm_structured_outputs_regex: Optional[str] = None
    vllm_server_base_url: Optional[str] = None
    vllm_server_host: str = "0.0.0.0"
    vllm_server_port: int = 8000
    vllm_server_timeout: float = 240.0
    vllm_group_port: int = 51216
    vllm_gpu_memory_utilization: float = 0.3
    vllm_max_model_length: Optional[int] = None
    vllm_tensor_parallel_size: int = 1
    beta: float = 0.0
    num_iterations: int = 1
    epsilon: float = 0.2
    epsilon_high: Optional[float] = None
    reward_weights: Optional[list] = None
    mask_truncated_completions: bool = False
    sync_ref_model: bool = False
    ref_model_mixup_alpha: float = 0.6
    ref_model_sync_steps: int = 512
    log_completions: bool = False
    log_multimodal: bool = True
    num_completions_to_print: Optional[int] = None
    log_unique_prompts: bool = False
    log_completions_hub_repo: Optional[str] = None
    # synthetic-benchmark knob: floor on the end-of-sequence probability during sampling
    eos_prob_floor: float = 0.0
    rollout_block_size: int = 0  # 0 = chosen by the engine (64-token pages for the tensor-core decode attention)
    rollout_poll_every: int = 16

    def _derive_generation_batch(self):
        from ..parallel import dist as D

        world = D.world_size()
        if self.generation_batch_size is None and self.steps_per_generation is None:
            self.steps_per_generation = self.gradient_accumulation_steps
            self.generation_batch_size = self.per_device_train_batch_size * world * self.steps_per_generation
        elif self.generation_batch_size is not None and self.steps_per_generation is None:
            gbs = self.per_device_train_batch_size * world
            if self.generation_batch_size % gbs != 0:
                raise ValueError(f"generation_batch_size ({self.generation_batch_size}) must be divisible by the global "
                                 f"batch size ({gbs}).")
            self.steps_per_generation = self.generation_batch_size // gbs
        elif self.generation_batch_size is None:
            self.generation_batch_size = self.per_device_train_batch_size * world * self.steps_per_generation
        else:
            raise ValueError("'generation_batch_size' and 'steps_per_generation' can not be both configured at the same time")
        if self.num_generations < getattr(self, "_MIN_GENERATIONS", 2):
            raise ValueError(f"{type(self).__name__[:-6]} requires at least 2 generations per prompt to calculate the "
                             f"advantages. You provided {self.num_generations}, which is less than the minimum required.")
        if self.generation_batch_size % self.num_generations != 0:
            raise ValueError(f"generation_batch_size ({self.generation_batch_size}) must be divisible by num_generations "
                             f"({self.num_generations}).")
        if self.do_eval and self.eval_strategy != "no":
            ng = self.num_generations_eval or self.num_generations
            if (self.per_device_eval_batch_size * world) % ng != 0:
                raise ValueError(f"The global eval batch size ({self.per_device_eval_batch_size} * {world}) must be "
                                 f"divisible by the number of generations used for evaluation ({ng}).")

    def _reject_seq_parallel(self):
        pc = self.parallelism_config
        if isinstance(pc, dict) and (pc.get("cp_size", 1) > 1 or pc.get("sp_size", 1) > 1):
            raise ValueError(f"{type(self).__name__[:-6]} does not support context or sequence parallelism.")
        if self.use_transformers_paged:
            warnings.warn("`use_transformers_paged` is deprecated and will be removed in v2.0.0. Use "
                          "`use_transformers_continuous_batching` instead.", FutureWarning)
            self.use_transformers_continuous_batching = True


@dataclass
class GRPOConfig(_OnlineConfig):
    _LOSS_TYPES = ("grpo", "bnpo", "dr_grpo", "dapo", "cispo", "sapo", "luspo", "vespo")

    delta: Optional[float] = None
    sapo_temperature_neg: float = 1.05
    sapo_temperature_pos: float = 1.0
    vespo_k_pos: float = 2.0
    vespo_lambda_pos: float = 3.0
    vespo_k_neg: float = 3.0
    vespo_lambda_neg: float = 2.0
    importance_sampling_level: str = "token"
    multi_objective_aggregation: str = "sum_then_normalize"
    scale_rewards: Any = "group"
    loss_type: str = "dapo"
    top_entropy_quantile: float = 1.0
    entropy_coef: float = 0.0
    use_adaptive_entropy: bool = False
    entropy_coef_min: float = 0.0
    entropy_coef_max: float = 1.0
    entropy_coef_delta: float = 0.005
    entropy_target: float = 0.2
    max_tool_calling_iterations: Optional[int] = None
    vllm_importance_sampling_correction: bool = True
    vllm_importance_sampling_mode: str = "sequence_mask"
    vllm_importance_sampling_clip_max: float = 3.0
    vllm_importance_sampling_clip_min: Optional[float] = None
    off_policy_mask_threshold: Optional[float] = None
    use_bias_correction_kl: bool = False
    vllm_importance_sampling_cap: Optional[float] = None

    def __post_init__(self):
        super().__post_init__()
        self._reject_seq_parallel()
        if isinstance(self.scale_rewards, bool):
            self.scale_rewards = "group" if self.scale_rewards else "none"
        if self.scale_rewards not in ("group", "batch", "none"):
            raise ValueError("scale_rewards must be one of 'group', 'batch', 'none'")
        if getattr(self, "vllm_structured_outputs_regex", None):
            raise NotImplementedError("vllm_structured_outputs_regex: the rollout engine has no regex-constrained sampler")
        if self.use_vllm and self.vllm_mode not in ("colocate", "server"):
            raise ValueError("vllm_mode must be 'colocate' (the in-process engine) or 'server'")
        if self.loss_type not in self._LOSS_TYPES:
            raise ValueError(f"Unknown loss type: {self.loss_type}")
        if self.importance_sampling_level not in ("token", "sequence", "sequence_token"):
            raise ValueError("importance_sampling_level must be 'token', 'sequence' or 'sequence_token'")
        if self.vllm_importance_sampling_cap is not None:
            warnings.warn("vllm_importance_sampling_cap is deprecated; use vllm_importance_sampling_clip_max.", FutureWarning)
            self.vllm_importance_sampling_clip_max = self.vllm_importance_sampling_cap
        if self.vllm_importance_sampling_mode not in ("token_truncate", "token_mask", "sequence_truncate", "sequence_mask"):
            raise ValueError("vllm_importance_sampling_mode must be token_truncate|token_mask|sequence_truncate|sequence_mask")
        cmin, cmax = self.vllm_importance_sampling_clip_min, self.vllm_importance_sampling_clip_max
        if cmin is not None and cmin > cmax:
            raise ValueError("vllm_importance_sampling_clip_min must not exceed vllm_importance_sampling_clip_max")
        if self.delta is not None and self.use_liger_kernel and False:
            raise ValueError("delta is not supported with the fused loss")
        self._derive_generation_batch()


@dataclass
class RLOOConfig(_OnlineConfig):
    beta: float = 0.05
    normalize_advantages: bool = False
    reward_clip_range: Optional[Any] = None
    vllm_importance_sampling_correction: bool = False

    def __post_init__(self):
        super().__post_init__()
        self._reject_seq_parallel()
        if self.reward_clip_range is not None:
            if len(self.reward_clip_range) != 2 or self.reward_clip_range[0] >= self.reward_clip_range[1]:
                raise ValueError("reward_clip_range must be (min, max) with min < max")
        self._derive_generation_batch()
