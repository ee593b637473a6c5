"""Standalone ``TrainingArguments``.

``transformers.TrainingArguments`` cannot be instantiated without accelerate,
so the field names and defaults the reference inherits
(trl/trainer/base_config.py:20-107 on top of transformers/training_args.py) are
replicated here.  Fields that select machinery this framework does not have
(hub push, torch.compile, ...) are accepted and stored so user code keeps
working; the ones that matter are honoured by :class:`trl_b200.loop.Trainer`.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Optional


def _env_int(k, d):
    try:
        return int(os.environ.get(k, d))
    except ValueError:
        return d


@dataclass
class TrainingArguments:
    _VALID_DICT_FIELDS = ["lr_scheduler_kwargs", "gradient_checkpointing_kwargs", "accelerator_config",
                          "fsdp_config", "parallelism_config"]

    output_dir: Optional[str] = field(default=None, metadata={"help": "Where checkpoints and the final model go."})
    overwrite_output_dir: bool = False
    do_train: bool = False
    do_eval: bool = False
    do_predict: bool = False
    eval_strategy: str = "no"
    prediction_loss_only: bool = False
    per_device_train_batch_size: int = 8
    per_device_eval_batch_size: int = 8
    gradient_accumulation_steps: int = 1
    eval_accumulation_steps: Optional[int] = None
    eval_delay: float = 0
    torch_empty_cache_steps: Optional[int] = None
    learning_rate: float = 5e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    num_train_epochs: float = 3.0
    max_steps: int = -1
    lr_scheduler_type: str = "linear"
    lr_scheduler_kwargs: Optional[Any] = None
    warmup_ratio: Optional[float] = None
    warmup_steps: float = 0
    log_level: str = "passive"
    log_level_replica: str = "warning"
    log_on_each_node: bool = True
    logging_dir: Optional[str] = None
    logging_strategy: str = "steps"
    logging_first_step: bool = False
    logging_steps: float = 10
    logging_nan_inf_filter: bool = True
    save_strategy: str = "steps"
    save_steps: float = 500
    save_total_limit: Optional[int] = None
    save_safetensors: bool = True
    save_on_each_node: bool = False
    save_only_model: bool = False
    restore_callback_states_from_checkpoint: bool = False
    use_cpu: bool = False
    seed: int = 42
    data_seed: Optional[int] = None
    bf16: Optional[bool] = None
    fp16: bool = False
    bf16_full_eval: bool = False
    fp16_full_eval: bool = False
    tf32: Optional[bool] = None
    local_rank: int = -1
    ddp_backend: Optional[str] = None
    ddp_timeout: int = 1800
    ddp_find_unused_parameters: Optional[bool] = None
    ddp_bucket_cap_mb: Optional[int] = None
    ddp_broadcast_buffers: Optional[bool] = None
    dataloader_drop_last: bool = False
    eval_steps: Optional[float] = None
    eval_on_start: bool = False
    dataloader_num_workers: int = 0
    dataloader_prefetch_factor: Optional[int] = None
    dataloader_pin_memory: bool = True
    dataloader_persistent_workers: bool = False
    run_name: Optional[str] = None
    disable_tqdm: Optional[bool] = None
    remove_unused_columns: Optional[bool] = True
    label_names: Optional[list] = None
    load_best_model_at_end: bool = False
    metric_for_best_model: Optional[str] = None
    greater_is_better: Optional[bool] = None
    ignore_data_skip: bool = False
    fsdp: Optional[Any] = None
    fsdp_config: Optional[Any] = None
    deepspeed: Optional[Any] = None
    accelerator_config: Optional[Any] = None
    parallelism_config: Optional[Any] = None
    label_smoothing_factor: float = 0.0
    optim: str = "adamw_torch_fused"
    optim_args: Optional[str] = None
    optim_target_modules: Optional[Any] = None
    group_by_length: bool = False
    length_column_name: str = "length"
    report_to: Any = "none"
    project: str = "huggingface"
    trackio_space_id: Optional[str] = None
    skip_memory_metrics: bool = True
    # save a checkpoint and stop at the next step boundary when the job receives SIGTERM (preemption)
    enable_jit_checkpoint: bool = False
    # "underflow_overflow": stop with an error at the first non-finite loss or gradient norm (one device sync per step)
    debug: Any = ""
    push_to_hub: bool = False
    resume_from_checkpoint: Optional[str] = None
    hub_model_id: Optional[str] = None
    hub_strategy: str = "every_save"
    hub_token: Optional[str] = None
    hub_private_repo: Optional[bool] = None
    hub_always_push: bool = False
    hub_revision: Optional[str] = None
    gradient_checkpointing: bool = True
    gradient_checkpointing_kwargs: Optional[Any] = None
    include_for_metrics: list = field(default_factory=list)
    include_num_input_tokens_seen: Any = "no"
    eval_do_concat_batches: bool = True
    auto_find_batch_size: bool = False
    full_determinism: bool = False
    torch_compile: bool = False
    torch_compile_backend: Optional[str] = None
    torch_compile_mode: Optional[str] = None
    neftune_noise_alpha: Optional[float] = None
    batch_eval_metrics: bool = False
    eval_use_gather_object: bool = False
    average_tokens_across_devices: bool = True
    use_liger_kernel: bool = False
    liger_kernel_config: Optional[dict] = None
    use_cache: bool = False
    train_sampling_strategy: str = "random"
    # ---- engine selection (maps the reference's accelerate profiles) --------
    shard_mode: str = field(default="auto", metadata={
        "help": "auto | ddp | zero1 | zero2 | full_shard | full_shard_stream.  The packaged accelerate profiles "
                "(multi_gpu, zero1/2/3, fsdp1/2) map onto these.  full_shard keeps a full-size buffer per layer and "
                "gathers once per optimizer step (fast, the model must fit one GPU in bf16); full_shard_stream holds "
                "1 / world of every layer and gathers layer by layer (needs gradient_checkpointing)."})
    ep_size: int = field(default=1, metadata={
        "help": "Expert parallelism for mixture-of-experts models: 1 keeps every expert on every rank; a value equal to "
                "the number of processes gives each rank num_experts / ep_size experts (tokens travel to the experts; "
                "data parallelism for everything else).  Works with shard_mode ddp, zero1 and zero2."})
    activation_offloading: bool = False

    def __post_init__(self):
        if self.output_dir is None:
            self.output_dir = "trainer_output"
        for f in self._VALID_DICT_FIELDS:
            v = getattr(self, f, None)
            if isinstance(v, str) and v.strip().startswith("{"):
                setattr(self, f, json.loads(v))
        if self.lr_scheduler_kwargs is None:
            self.lr_scheduler_kwargs = {}
        self.bf16 = (not self.fp16) if self.bf16 is None else self.bf16
        if self.bf16 and self.fp16:
            raise ValueError("At most one of fp16 and bf16 can be True.")
        if self.eval_strategy != "no" and self.eval_steps is None and self.eval_strategy == "steps":
            self.eval_steps = self.logging_steps
        if isinstance(self.report_to, str):
            self.report_to = [] if self.report_to in ("none", "") else (
                ["tensorboard"] if self.report_to == "all" else [self.report_to])
        if self.disable_tqdm is None:
            self.disable_tqdm = True
        if self.auto_find_batch_size and type(self).__name__ in ("GRPOConfig", "RLOOConfig"):
            raise ValueError("auto_find_batch_size is not supported for online methods")
        if self.deepspeed or self.fsdp:
            prof = str(self.deepspeed or self.fsdp)
            if self.shard_mode == "auto":
                self.shard_mode = "full_shard" if ("3" in prof or "full_shard" in prof or "fsdp" in prof) else "zero2"

    # ---- process topology (duck-typed like transformers) ---------------------
    @property
    def world_size(self) -> int:
        from ..parallel import dist as D

        return D.world_size()

    @property
    def process_index(self) -> int:
        from ..parallel import dist as D

        return D.rank()

    @property
    def local_process_index(self) -> int:
        return _env_int("LOCAL_RANK", 0)

    @property
    def should_save(self) -> bool:
        return self.process_index == 0

    @property
    def should_log(self) -> bool:
        return self.process_index == 0

    @property
    def device(self):
        import torch

        if self.use_cpu or not torch.cuda.is_available():
            return torch.device("cpu")
        return torch.device("cuda", self.local_process_index)

    @property
    def n_gpu(self) -> int:
        return 1

    @property
    def train_batch_size(self) -> int:
        return self.per_device_train_batch_size

    @property
    def eval_batch_size(self) -> int:
        return self.per_device_eval_batch_size

    @property
    def parallel_mode(self):
        return "distributed" if self.world_size > 1 else "not_parallel"

    def get_warmup_steps(self, num_training_steps: int) -> int:
        if self.warmup_ratio:
            return int(num_training_steps * self.warmup_ratio + 0.999999)
        w = self.warmup_steps
        return int(w) if w >= 1 else int(num_training_steps * w + 0.999999)

    def to_dict(self) -> dict:
        d = {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}
        for k, v in d.items():
            if k.endswith("_token") and v is not None:
                d[k] = f"<{k.upper()}>"
        return d

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, default=str)

    def to_sanitized_dict(self) -> dict:
        return {k: (v if isinstance(v, (bool, int, float, str)) else str(v)) for k, v in self.to_dict().items()}

    def set_training(self, **kw):
        for k, v in kw.items():
            setattr(self, k, v)
        return self
