"""SFTConfig: field names/defaults of trl/trainer/sft_config.py:22-336."""
from __future__ import annotations

import warnings
from dataclasses import dataclass, field
from typing import Any, Optional

from .base_config import _BaseConfig


@dataclass
class SFTConfig(_BaseConfig):
    _VALID_DICT_FIELDS = _BaseConfig._VALID_DICT_FIELDS + ["model_init_kwargs"]

    learning_rate: float = field(default=2e-5, metadata={"help": "Initial AdamW learning rate."})
    model_init_kwargs: Optional[Any] = field(default=None, metadata={"help": "kwargs for loading the model from a path."})
    router_aux_loss_coef: float = field(default=0.001, metadata={"help": "MoE load-balancing loss coefficient."})
    trust_remote_code: bool = False
    chat_template_path: Optional[str] = field(default=None, metadata={"help": "Jinja file or tokenizer dir to copy a chat template from."})
    dataset_text_field: str = "text"
    dataset_kwargs: Optional[dict] = None
    dataset_num_proc: Optional[int] = None
    eos_token: Optional[str] = None
    pad_token: Optional[str] = None
    max_length: Optional[int] = field(default=1024, metadata={"help": "Truncate tokenised sequences to this length."})
    truncation_mode: str = field(default="keep_start", metadata={"help": "keep_start | keep_end"})
    shuffle_dataset: bool = False
    packing: bool = False
    packing_strategy: str = field(default="bfd", metadata={"help": "bfd | bfd_split | wrapped"})
    padding_free: bool = field(default=False, metadata={"help": "Flatten each batch into one row with restarting position_ids."})
    pad_to_multiple_of: Optional[int] = None
    eval_packing: Optional[bool] = None
    completion_only_loss: Optional[bool] = None
    assistant_only_loss: bool = False
    loss_type: Optional[str] = field(default=None, metadata={"help": "nll | dft | chunked_nll (default)"})
    activation_offloading: bool = False

    def __post_init__(self):
        super().__post_init__()
        if self.packing_strategy == "bfd-requeue":
            warnings.warn("packing_strategy='bfd-requeue' is deprecated; use 'bfd_split'.", FutureWarning)
            self.packing_strategy = "bfd_split"
        if self.loss_type is None:
            self.loss_type = "chunked_nll"
        if self.loss_type not in ("nll", "dft", "chunked_nll"):
            raise ValueError(f"Invalid loss_type {self.loss_type!r}; expected nll, dft or chunked_nll")
        if self.truncation_mode not in ("keep_start", "keep_end"):
            raise ValueError("truncation_mode must be 'keep_start' or 'keep_end'")
        if self.pad_token is not None:
            warnings.warn("`pad_token` is deprecated; set it on the tokenizer instead.", FutureWarning)
