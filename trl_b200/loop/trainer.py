"""The training loop: own implementation of what the reference inherits from
``transformers.Trainer`` (trl/trainer/base_trainer.py:67 ``class _BaseTrainer(Trainer)``).

Hook names are kept (``compute_loss``, ``training_step``, ``_prepare_inputs``,
``get_train_dataloader``, ``_get_train_sampler``, ``prediction_step``, ``log``,
``_save_checkpoint``, ``evaluate``, ``save_model``) so subclasses written for the
reference's loop read the same.  Checkpoints use the Hugging Face layout:
``checkpoint-<step>/{config.json, model.safetensors, trainer_state.json,
optimizer*.pt, scheduler.pt, rng_state_<rank>.pth, training_args.json}``.
"""
from __future__ import annotations

import contextlib

import json
import math
import os
import random
import re
import shutil
import time
import warnings
from collections import defaultdict
from typing import Any, Callable, Optional

import numpy as np
import torch
import torch.nn as nn

from ..parallel import dist as D
from ..parallel.engine import TrainEngine
from .optim import LRScheduler, lr_lambda_for
from .state import (CallbackHandler, DefaultFlowCallback, PrinterCallback, TrainerCallback, TrainerControl,
                    TrainerState)
from .training_args import TrainingArguments

PREFIX_CHECKPOINT_DIR = "checkpoint"


def set_seed(seed: int, deterministic: bool = False):
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if deterministic:
        torch.use_deterministic_algorithms(True, warn_only=True)


class TrainOutput(tuple):
    def __new__(cls, global_step, training_loss, metrics):
        o = super().__new__(cls, (global_step, training_loss, metrics))
        o.global_step, o.training_loss, o.metrics = global_step, training_loss, metrics
        return o


class ShardedBatchSampler:
    """Global batches of ``batch_size * world`` indices; rank r takes slice r (what
    accelerate's BatchSamplerShard does with ``split_batches=False``)."""

    def __init__(self, sampler, batch_size: int, drop_last: bool, rank: int, world: int, shard: bool = True):
        self.sampler, self.bs, self.drop_last = sampler, batch_size, drop_last
        self.rank, self.world = (rank, world) if shard else (0, 1)

    def __iter__(self):
        g = self.bs * self.world
        buf = []
        first = None
        for i in self.sampler:
            buf.append(i)
            if len(buf) == g:
                first = first or list(buf)
                yield buf[self.rank * self.bs:(self.rank + 1) * self.bs]
                buf = []
        if buf and not self.drop_last:
            # pad the tail by cycling from the start so every rank gets a (non-empty) batch
            src = first or list(buf)
            while len(buf) % self.world != 0 or len(buf) < self.world:
                buf.append(src[len(buf) % len(src)])
            per = len(buf) // self.world
            yield buf[self.rank * per:(self.rank + 1) * per]

    def __len__(self):
        n = len(self.sampler)
        g = self.bs * self.world
        return n // g if self.drop_last else math.ceil(n / g)


class SeededRandomSampler:
    def __init__(self, n: int, seed: int):
        self.n, self.seed, self.epoch = n, seed, 0

    def set_epoch(self, e):
        self.epoch = e

    def __iter__(self):
        g = torch.Generator()
        g.manual_seed(self.seed + self.epoch)
        return iter(torch.randperm(self.n, generator=g).tolist())

    def __len__(self):
        return self.n


class LengthGroupedSampler(SeededRandomSampler):
    """``group_by_length``: a random order in which every global batch holds samples of similar length, so that padded
    batches waste little.  As in transformers: shuffle, cut into mega-batches of 50 global batches, sort each by
    length (longest first), and put the mega-batch with the longest sample first (an out-of-memory shows at step 1)."""

    def __init__(self, lengths, batch_size: int, seed: int, mega: int = 50):
        super().__init__(len(lengths), seed)
        self.lengths, self.batch = [int(x) for x in lengths], max(1, int(batch_size))
        self.mega = self.batch * mega

    def __iter__(self):
        g = torch.Generator()
        g.manual_seed(self.seed + self.epoch)
        order = torch.randperm(self.n, generator=g).tolist()
        chunks = [sorted(order[i:i + self.mega], key=lambda j: -self.lengths[j]) for i in range(0, self.n, self.mega)]
        if chunks:
            k = max(range(len(chunks)), key=lambda c: self.lengths[chunks[c][0]])
            chunks[0], chunks[k] = chunks[k], chunks[0]
        return iter([j for c in chunks for j in c])


class DataLoaderLite:
    """Minimal map-style / iterable loader (single process; collate on the host)."""

    def __init__(self, dataset, batch_sampler=None, collate_fn=None, batch_size=None, rank=0, world=1,
                 pin_memory=False):
        self.dataset, self.batch_sampler, self.collate_fn = dataset, batch_sampler, collate_fn or (lambda x: x)
        self.batch_size, self.rank, self.world, self.pin = batch_size, rank, world, pin_memory

    def __iter__(self):
        if self.batch_sampler is not None:
            for idxs in self.batch_sampler:
                yield self._finish(self.collate_fn([self.dataset[int(i)] for i in idxs]))
        else:  # iterable dataset: every rank reads the stream, keeps its slice
            buf = []
            g = self.batch_size * self.world
            for ex in self.dataset:
                buf.append(ex)
                if len(buf) == g:
                    yield self._finish(self.collate_fn(buf[self.rank * self.batch_size:(self.rank + 1) * self.batch_size]))
                    buf = []

    def _finish(self, batch):
        if self.pin and isinstance(batch, dict):
            batch = {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in batch.items()}
        return batch

    def __len__(self):
        if self.batch_sampler is not None:
            return len(self.batch_sampler)
        raise TypeError("iterable dataset has no length")

    def set_epoch(self, e):
        s = getattr(self.batch_sampler, "sampler", None)
        if hasattr(s, "set_epoch"):
            s.set_epoch(e)


class JsonlSink(TrainerCallback):
    """``report_to=["jsonl"]``: one JSON object per log call under ``output_dir/logs.jsonl``."""

    def on_log(self, args, state, control, logs=None, **kw):
        if state.is_world_process_zero and logs:
            os.makedirs(args.output_dir, exist_ok=True)
            with open(os.path.join(args.output_dir, "logs.jsonl"), "a") as f:
                f.write(json.dumps({"step": state.global_step, **logs}, default=float) + "\n")


class TensorBoardSink(TrainerCallback):
    def __init__(self):
        self.w = None

    def on_log(self, args, state, control, logs=None, **kw):
        if not state.is_world_process_zero or not logs:
            return
        if self.w is None:
            try:
                from torch.utils.tensorboard import SummaryWriter

                self.w = SummaryWriter(args.logging_dir or os.path.join(args.output_dir, "runs"))
            except Exception:
                self.w = False
        if self.w:
            for k, v in logs.items():
                if isinstance(v, (int, float)):
                    self.w.add_scalar(k, v, state.global_step)


_SINKS = {"jsonl": JsonlSink, "tensorboard": TensorBoardSink}


class Trainer:
    _tag_names: list[str] = []
    _name = "Trainer"
    model_accepts_loss_kwargs = True

    def __init__(self, model=None, args: TrainingArguments | None = None, data_collator=None, train_dataset=None,
                 eval_dataset=None, processing_class=None, compute_loss_func=None, compute_metrics=None,
                 callbacks=None, optimizers=(None, None), optimizer_cls_and_kwargs=None,
                 preprocess_logits_for_metrics=None, model_init=None, tokenizer=None):
        self.args = args or TrainingArguments()
        D.init_process_group(self.args.use_cpu, self.args.ddp_timeout)
        set_seed(self.args.seed, self.args.full_determinism)
        self.model = model
        self.data_collator = data_collator
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self.processing_class = processing_class or tokenizer
        self.compute_loss_func, self.compute_metrics = compute_loss_func, compute_metrics
        self.preprocess_logits_for_metrics = preprocess_logits_for_metrics
        self.state = TrainerState(is_local_process_zero=D.local_rank() == 0, is_world_process_zero=D.is_main())
        self.control = TrainerControl()
        self.engine: TrainEngine | None = None
        self.lr_scheduler: LRScheduler | None = None
        self.optimizer = None
        if optimizers is not None and (optimizers[0] is not None or optimizers[1] is not None):
            # parameters live in the engine's flat buffers (bf16 compute copy + fp32 master slices), which do not exist
            # yet when a caller builds an optimizer over model.parameters()
            raise NotImplementedError("a ready-made (optimizer, scheduler) pair is not supported: pass "
                                      "optimizer_cls_and_kwargs=(cls, kwargs) or set args.optim / args.lr_scheduler_type")
        self._optimizer_cls_and_kwargs = optimizer_cls_and_kwargs
        self._metrics = {"train": defaultdict(list), "eval": defaultdict(list)}
        self._watchdog_dir = os.environ.get("TRL_B200_WATCHDOG_DIR")
        self._train_batch_size = self.args.per_device_train_batch_size
        self.is_in_train = False
        self._place_model()
        cbs = [DefaultFlowCallback()] + list(callbacks or [])
        for r in self.args.report_to:
            if r in _SINKS:
                cbs.append(_SINKS[r]())
        if not any(isinstance(c, PrinterCallback) for c in cbs) and self.args.disable_tqdm:
            cbs.append(PrinterCallback())
        if self.args.enable_jit_checkpoint:
            from ..trainer.callbacks import JITCheckpointCallback

            cbs.append(JITCheckpointCallback())
        if self._watchdog_dir:
            from ..trainer.callbacks import WatchdogCallback

            cbs.append(WatchdogCallback(self._watchdog_dir, stale_after_s=float(os.environ.get("TRL_B200_WATCHDOG_STALE_S", 60))))
        self.callback_handler = CallbackHandler(cbs, self.model, self.processing_class, None, None)
        self.control = self.callback_handler.call_event("on_init_end", self.args, self.state, self.control)

    # ---- model placement / precision ---------------------------------------------
    def _place_model(self):
        if self.model is None:
            return
        dev = self.args.device
        first = next(self.model.parameters(), None)
        on_meta = first is not None and first.is_meta  # materialised slice by slice by the streamed engine
        if on_meta and self.args.shard_mode != "full_shard_stream":
            raise ValueError("a model on the meta device can only be trained with shard_mode='full_shard_stream'")
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        if dev.type == "cuda" and not on_meta:
            dt = torch.bfloat16 if self.args.bf16 else (torch.float16 if self.args.fp16 else None)
            self.model.to(device=dev, dtype=dt) if dt is not None else self.model.to(dev)
        if self.args.gradient_checkpointing and hasattr(self.model, "gradient_checkpointing_enable"):
            kw = self.args.gradient_checkpointing_kwargs
            # {"num_layers": "auto"}: start with every layer recomputed and let the first optimizer steps measure how
            # many layers can keep their activations (see _autotune_checkpointing)
            self._ckpt_auto = 0 if isinstance(kw, dict) and kw.get("num_layers") == "auto" else None
            if self._ckpt_auto is not None:
                kw = {k: v for k, v in kw.items() if k != "num_layers"} or None
            self.model.gradient_checkpointing_enable(kw)

    @property
    def accelerator(self):
        """Small shim exposing the accelerate calls subclasses and callbacks use."""
        return _AcceleratorShim(self)

    @property
    def tokenizer(self):
        return self.processing_class

    def add_callback(self, cb):
        self.callback_handler.add_callback(cb)

    def pop_callback(self, cb):
        return self.callback_handler.pop_callback(cb)

    def remove_callback(self, cb):
        self.callback_handler.remove_callback(cb)

    def is_world_process_zero(self):
        return D.is_main()

    def is_local_process_zero(self):
        return D.local_rank() == 0

    # ---- data -----------------------------------------------------------------------
    def _get_train_sampler(self, dataset=None):
        ds = dataset if dataset is not None else self.train_dataset
        if getattr(self.args, "train_sampling_strategy", "random") == "sequential":
            return range(len(ds))
        seed = self.args.data_seed if self.args.data_seed is not None else self.args.seed
        if getattr(self.args, "group_by_length", False):
            col = self.args.length_column_name or "length"
            names = getattr(ds, "column_names", None) or (list(ds[0].keys()) if len(ds) and isinstance(ds[0], dict) else [])
            if col in names:
                lengths = ds[col] if hasattr(ds, "column_names") else [r[col] for r in ds]
            elif "input_ids" in names:
                lengths = [len(r["input_ids"]) for r in ds]
            else:
                raise ValueError(f"group_by_length needs a {col!r} or an 'input_ids' column in the (prepared) dataset")
            return LengthGroupedSampler(lengths, self._train_batch_size * max(1, D.world_size() // self.sp_size), seed)
        return SeededRandomSampler(len(ds), seed)

    def _get_eval_sampler(self, dataset):
        return range(len(dataset))

    def _shard_train_batches(self) -> bool:
        return True

    @property
    def sp_size(self) -> int:
        """Ranks per sequence-sharded group: ``parallelism_config["sp_size"]`` (Ulysses, heads are exchanged) or
        ``["cp_size"]`` (context parallel, keys / values are gathered); one of the two."""
        pc = self.args.parallelism_config
        pc = pc if isinstance(pc, dict) else {}
        sp, cp = int(pc.get("sp_size", 1) or 1), int(pc.get("cp_size", 1) or 1)
        if sp > 1 and cp > 1:
            raise ValueError("sp_size and cp_size cannot be combined: pick Ulysses (sp_size) or context parallel (cp_size)")
        sp = max(sp, cp)
        if sp > 1 and D.world_size() % sp:
            raise ValueError(f"sp_size / cp_size ({sp}) must divide the world size ({D.world_size()})")
        return sp if D.world_size() > 1 else 1

    def sp_info(self):
        """Sequence-parallel group of this rank (consecutive ranks), or None."""
        sp = self.sp_size
        if sp <= 1:
            return None
        if getattr(self, "_sp_info", None) is None:
            from ..parallel.ulysses import SpInfo

            groups = [list(range(i, i + sp)) for i in range(0, D.world_size(), sp)]
            pc = self.args.parallelism_config
            mode = "allgather_kv" if isinstance(pc, dict) and int(pc.get("cp_size", 1) or 1) > 1 else "ulysses"
            self._sp_info = SpInfo(D.new_subgroups_by_enumeration(groups), sp, D.rank() % sp, mode)
        return self._sp_info

    def get_train_dataloader(self):
        ds = self.train_dataset
        if ds is None:
            raise ValueError("Trainer: training requires a train_dataset.")
        if not hasattr(ds, "__len__") or not hasattr(ds, "__getitem__"):
            return DataLoaderLite(ds, None, self.data_collator, self._train_batch_size, D.rank(), D.world_size())
        sp = self.sp_size  # ranks of one sequence-parallel group read the same batches
        bs = ShardedBatchSampler(self._get_train_sampler(ds), self._train_batch_size, self.args.dataloader_drop_last,
                                 D.rank() // sp, D.world_size() // sp, self._shard_train_batches())
        return DataLoaderLite(ds, bs, self.data_collator,
                              pin_memory=self.args.dataloader_pin_memory and self.args.device.type == "cuda")

    def get_eval_dataloader(self, eval_dataset=None):
        ds = eval_dataset if eval_dataset is not None else self.eval_dataset
        if isinstance(ds, str):
            ds = self.eval_dataset[ds]
        bs = ShardedBatchSampler(self._get_eval_sampler(ds), self.args.per_device_eval_batch_size, False,
                                 D.rank(), D.world_size())
        return DataLoaderLite(ds, bs, self.data_collator)

    def _prepare_input(self, v):
        if torch.is_tensor(v):
            return v.to(self.args.device, non_blocking=True)
        if isinstance(v, dict):
            return {k: self._prepare_input(x) for k, x in v.items()}
        if isinstance(v, (list, tuple)) and v and torch.is_tensor(v[0]):
            return type(v)(self._prepare_input(x) for x in v)
        return v

    def _prepare_inputs(self, inputs):
        return self._prepare_input(inputs)

    # ---- optimizer --------------------------------------------------------------------
    def create_optimizer_and_scheduler(self, num_training_steps: int):
        a = self.args
        if self.engine is None:
            self.engine = self._create_engine()
        self.optimizer = self.engine
        warm = a.get_warmup_steps(num_training_steps)
        self.lr_scheduler = LRScheduler(a.learning_rate, lr_lambda_for(a.lr_scheduler_type, warm, num_training_steps,
                                                                       **(a.lr_scheduler_kwargs or {})))
        self.callback_handler.optimizer, self.callback_handler.lr_scheduler = self.engine, self.lr_scheduler

    def _optimizer_factory(self):
        """None for the built-in AdamW (every ``adamw_*`` name of ``optim``); else a function building the optimizer
        from parameter groups: ``optimizer_cls_and_kwargs`` (trainer argument, as in transformers), or ``optim`` in
        ``sgd`` / ``adagrad`` / ``rmsprop`` / ``adafactor`` with ``optim_args`` ("key=value,..." or a dict)."""
        a = self.args
        if self._optimizer_cls_and_kwargs is not None:
            cls, kw = self._optimizer_cls_and_kwargs
            return lambda groups: cls(groups, **{"lr": a.learning_rate, **(kw or {})})
        name = (a.optim or "adamw_torch_fused").lower()
        if name.startswith("adamw"):
            return None
        extra = a.optim_args if isinstance(getattr(a, "optim_args", None), dict) else dict(
            kv.split("=") for kv in (getattr(a, "optim_args", None) or "").replace(" ", "").split(",") if kv)
        extra = {k: (float(v) if isinstance(v, str) else v) for k, v in extra.items()}
        table = {"sgd": torch.optim.SGD, "adagrad": torch.optim.Adagrad, "rmsprop": torch.optim.RMSprop}
        if name in table:
            return lambda groups: table[name](groups, lr=a.learning_rate, **extra)
        if name == "adafactor":
            from transformers.optimization import Adafactor

            return lambda groups: Adafactor(groups, lr=a.learning_rate, scale_parameter=False, relative_step=False, **extra)
        raise ValueError(f"optim={a.optim!r} is not available; use an adamw_* name, sgd, adagrad, rmsprop, adafactor, or "
                         "pass optimizer_cls_and_kwargs=(cls, kwargs)")

    def _create_engine(self) -> TrainEngine:
        a = self.args
        mode = a.shard_mode
        factory = self._optimizer_factory()
        if factory is not None and mode in ("full_shard", "full_shard_stream") and D.world_size() > 1:
            raise NotImplementedError("a custom optimizer runs with shard_mode ddp, zero1 or zero2")
        if getattr(a, "ep_size", 1) > 1:
            if a.ep_size != D.world_size():
                raise ValueError(f"ep_size={a.ep_size} must equal the number of processes ({D.world_size()})")
            if mode in ("full_shard", "full_shard_stream"):
                raise ValueError("expert parallelism goes with shard_mode ddp, zero1 or zero2: the experts are already "
                                 "split over the ranks, the rest of the model is small")
            lm = getattr(self.model, "language_model", self.model)
            if getattr(lm, "ep_world", 1) == 1:
                from ..parallel.expert_parallel import shard_experts

                shard_experts(self.model, max_tokens=int(os.environ.get("TRL_B200_EP_MAX_TOKENS", "16384")))
        if mode == "full_shard" and D.world_size() > 1:
            from ..parallel.symm import symmetric_available

            first = next(self.model.parameters())
            if first.is_cuda and first.dtype == torch.bfloat16 and symmetric_available():
                from ..parallel.fullshard import FullShardEngine

                return FullShardEngine(self.model, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                                       weight_decay=a.weight_decay)
            # CPU / fp32: same sharding of gradients and optimizer state through the backend collectives
        if mode == "full_shard_stream":
            from ..parallel.streamshard import StreamShardEngine

            # TRL_B200_STREAM_GRAD_DTYPE=bf16: keep the reduced layer gradients in bf16 (2 bytes / parameter less per
            # rank; exact when gradient_accumulation_steps == 1, where the reduce-scatter already delivers bf16)
            gd = {"bf16": torch.bfloat16, "fp32": torch.float32}[os.environ.get("TRL_B200_STREAM_GRAD_DTYPE", "fp32")]
            return StreamShardEngine(self.model, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                                     weight_decay=a.weight_decay, device=a.device, init_seed=a.seed, grad_dtype=gd)
        return TrainEngine(self.model, mode=mode, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                           weight_decay=a.weight_decay, optimizer_factory=factory)

    def _get_learning_rate(self) -> float:
        return self.lr_scheduler.get_last_lr()[0]

    # ---- loss ---------------------------------------------------------------------------
    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        labels = inputs.get("labels") if self.compute_loss_func is not None else None
        outputs = model(**inputs)
        if self.compute_loss_func is not None:
            loss = self.compute_loss_func(outputs, labels, num_items_in_batch=num_items_in_batch)
        else:
            loss = outputs["loss"] if isinstance(outputs, dict) else outputs.loss
        return (loss, outputs) if return_outputs else loss

    def training_step(self, model, inputs, num_items_in_batch=None):
        from ..extras.profiling import profiling_context

        model.train()
        inputs = self._prepare_inputs(inputs)
        with profiling_context(self, "forward_backward"):  # the micro-batch itself: loss forward + backward
            with self._activation_offload_context():
                loss = self.compute_loss(model, inputs, num_items_in_batch=num_items_in_batch)
            if (not self.model_accepts_loss_kwargs or num_items_in_batch is None) and self.compute_loss_func is None:
                loss = loss / self.current_gradient_accumulation_steps
            self.engine.backward(loss)
        return loss.detach()

    def _activation_offload_context(self):
        """Saved activations of the forward go to pinned host memory when ``args.activation_offloading`` is set
        (every trainer: trl/trainer/sft_trainer.py:1840-1842 and the same lines of the DPO / KTO / reward trainers).
        The context is built once; trainers that wrap only part of their forward themselves set
        ``self._own_offload_scope``."""
        if not getattr(self.args, "activation_offloading", False) or getattr(self, "_own_offload_scope", False):
            return contextlib.nullcontext()
        ctx = getattr(self, "_offload_ctx", None)
        if ctx is None:
            from ..models.activation_offloading import get_act_offloading_ctx_manager

            ctx = self._offload_ctx = get_act_offloading_ctx_manager(self.model)
        return ctx

    def _count_items(self, batches) -> Optional[torch.Tensor]:
        """Global number of supervised tokens over the accumulation window (HF ``num_items_in_batch``)."""
        try:
            n = sum(int((b["labels"] != -100).sum()) for b in batches)
        except (TypeError, KeyError):
            return None
        t = torch.tensor(n, dtype=torch.long, device=self.args.device)
        if self.args.average_tokens_across_devices and D.world_size() > 1:
            D.all_reduce(t, "sum")
            if self.sp_size > 1:  # every batch was counted once per rank of its sequence-parallel group
                t = t // self.sp_size
        return t

    # ---- main loop ------------------------------------------------------------------------
    def train(self, resume_from_checkpoint: str | bool | None = None, **kw):
        a = self.args
        self.is_in_train = True
        resume_from_checkpoint = resume_from_checkpoint if resume_from_checkpoint is not None else a.resume_from_checkpoint
        if resume_from_checkpoint is True:
            resume_from_checkpoint = get_last_checkpoint(a.output_dir)
            if resume_from_checkpoint is None:
                raise ValueError(f"No valid checkpoint found in output directory ({a.output_dir})")
        loader = self.get_train_dataloader()
        self.callback_handler.train_dataloader = loader
        self._apply_runtime_arguments()
        ga = a.gradient_accumulation_steps
        try:
            n_batches = len(loader)
            steps_per_epoch = max(1, n_batches // ga + int(n_batches % ga > 0))
        except TypeError:
            n_batches, steps_per_epoch = None, None
        if a.max_steps > 0:
            max_steps = a.max_steps
            epochs = math.ceil(max_steps / steps_per_epoch) if steps_per_epoch else 10**9
        else:
            if steps_per_epoch is None:
                raise ValueError("max_steps must be set for datasets without a length")
            max_steps = math.ceil(a.num_train_epochs * steps_per_epoch)
            epochs = math.ceil(a.num_train_epochs)
        st = self.state
        st.max_steps, st.num_train_epochs = max_steps, epochs
        st.train_batch_size = self._train_batch_size
        for name in ("logging_steps", "eval_steps", "save_steps"):
            v = getattr(a, name)
            if v is not None:
                setattr(st, name, max(1, int(v * max_steps)) if v < 1 else int(v))
        self.create_optimizer_and_scheduler(max_steps)
        start_epoch, skip_batches = 0, 0
        if resume_from_checkpoint:
            self._load_from_checkpoint(resume_from_checkpoint)
            st = self.state
            st.max_steps, st.num_train_epochs = max_steps, epochs
            if steps_per_epoch and not a.ignore_data_skip:
                start_epoch = st.global_step // steps_per_epoch
                skip_batches = (st.global_step % steps_per_epoch) * ga
            elif steps_per_epoch:
                start_epoch = st.global_step // steps_per_epoch
        self.control = self.callback_handler.call_event("on_train_begin", a, st, self.control)
        if a.eval_on_start:
            self.evaluate()
        tr_loss = torch.zeros((), device=a.device)
        self._total_loss_scalar, self._logged_step = 0.0, st.global_step
        t_start = time.time()
        self.engine.zero_grad()
        grad_norm = None
        for epoch in range(start_epoch, epochs):
            loader.set_epoch(epoch) if hasattr(loader, "set_epoch") else None
            self.control = self.callback_handler.call_event("on_epoch_begin", a, st, self.control)
            it = iter(loader)
            if epoch == start_epoch and skip_batches:
                for _ in range(skip_batches):
                    next(it, None)
            step_in_epoch = skip_batches // ga if epoch == start_epoch else 0
            exhausted = False
            while not exhausted:
                batches = []
                for _ in range(ga):
                    b = next(it, None)
                    if b is None:
                        exhausted = True
                        break
                    batches.append(b)
                if not batches:
                    break
                loss_sum, grad_norm, lr = self.optimizer_step(batches)
                tr_loss += loss_sum
                st.global_step += 1
                step_in_epoch += 1
                st.epoch = epoch + (step_in_epoch / steps_per_epoch if steps_per_epoch else 0)
                self.control = self.callback_handler.call_event("on_step_end", a, st, self.control)
                tr_loss = self._maybe_log_save_evaluate(tr_loss, grad_norm, lr, t_start)
                if a.torch_empty_cache_steps and st.global_step % a.torch_empty_cache_steps == 0 and torch.cuda.is_available():
                    torch.cuda.empty_cache()
                if self.control.should_training_stop or self.control.should_epoch_stop:
                    break
            self.control = self.callback_handler.call_event("on_epoch_end", a, st, self.control)
            tr_loss = self._maybe_log_save_evaluate(tr_loss, grad_norm, self._get_learning_rate(), t_start)
            if self.control.should_training_stop:
                break
        self._total_loss_scalar += float(tr_loss)
        train_loss = self._total_loss_scalar / max(1, st.global_step)
        runtime = time.time() - t_start
        metrics = {"train_runtime": round(runtime, 4), "train_steps_per_second": round(st.global_step / max(runtime, 1e-9), 3),
                   "train_loss": train_loss, "epoch": st.epoch}
        self.log(metrics)
        lm = getattr(self.model, "language_model", self.model)
        if getattr(lm, "neftune_noise_alpha", None) is not None:
            lm.neftune_noise_alpha = None
        if a.load_best_model_at_end and st.best_model_checkpoint and os.path.isdir(st.best_model_checkpoint):
            # weights of the checkpoint that scored best on `metric_for_best_model` (optimizer state is left as it is)
            self._load_weights_only(st.best_model_checkpoint)
        self.control = self.callback_handler.call_event("on_train_end", a, st, self.control)
        from ..extras import profiling

        if profiling.TRACE_PATH:  # TRL_B200_TRACE=<file>: Chrome trace of the phase timers, one file per rank
            profiling.dump_trace(rank=D.rank())
        self.is_in_train = False
        return TrainOutput(st.global_step, train_loss, metrics)

    _IGNORED_WHEN_SET = {
        "torch_compile": "kernels are hand-written; nothing is traced or compiled",
        "label_smoothing_factor": "the fused lm_head losses have no label smoothing",
        "optim_target_modules": "layer-wise optimizers are not available",
        "hub_model_id": "there is no network: nothing is pushed to the Hub",
        "fsdp_config": "sharding is chosen with shard_mode", "accelerator_config": "there is no accelerate layer",
        "liger_kernel_config": "the fused kernels are always on",
    }

    def _apply_runtime_arguments(self):
        """Arguments that act on the process or the model rather than on the loop: ``tf32``, ``neftune_noise_alpha``;
        and one warning for arguments that were set but have no effect here."""
        a = self.args
        if a.tf32 is not None and torch.cuda.is_available():
            torch.backends.cuda.matmul.allow_tf32 = bool(a.tf32)
            torch.backends.cudnn.allow_tf32 = bool(a.tf32)
        if a.neftune_noise_alpha:
            lm = getattr(self.model, "language_model", self.model)
            lm.neftune_noise_alpha = float(a.neftune_noise_alpha)
        if not getattr(self, "_warned_ignored", False):
            self._warned_ignored = True
            base = TrainingArguments()
            hit = [f"{k} ({why})" for k, why in self._IGNORED_WHEN_SET.items()
                   if getattr(a, k, None) not in (None, False, 0, 0.0, "") and getattr(a, k, None) != getattr(base, k, None)]
            if hit:
                warnings.warn("training arguments without effect in this framework: " + "; ".join(hit))

    def _load_weights_only(self, folder: str):
        from ..models.hf_io import load_hf_state_dict, load_state_dict_dir

        m = self.model
        if hasattr(m, "load_adapter") and os.path.exists(os.path.join(folder, "adapter_model.safetensors")):
            m.load_adapter(folder)
        elif getattr(m, "_is_native", False) and hasattr(self.engine, "load_weights"):
            self.engine.load_weights(load_state_dict_dir(folder))
        elif hasattr(m, "load_hf_state_dict"):  # composite models (vision-language) map their own key layout
            m.load_hf_state_dict(load_state_dict_dir(folder))
        elif getattr(m, "_is_native", False):
            load_hf_state_dict(m, load_state_dict_dir(folder), strict=True)
        if self.engine is not None and hasattr(self.engine, "sync_master_from_params"):
            self.engine.sync_master_from_params()

    def optimizer_step(self, batches: list):
        """One optimizer step over ``batches`` (the accumulation window): forward/backward of every
        micro-batch, gradient reduction, clipping, AdamW, scheduler.  Returns (summed loss, grad norm, lr)."""
        a, st = self.args, self.state
        self.current_gradient_accumulation_steps = len(batches)
        n_items = self._count_items(batches)
        self.control = self.callback_handler.call_event("on_step_begin", a, st, self.control)
        total = torch.zeros((), device=a.device)
        for i, b in enumerate(batches):
            # True while the last micro-batch of the accumulation window runs (accelerate's ``sync_gradients``)
            self.sync_gradients = i == len(batches) - 1
            loss = self.training_step(self.model, b, n_items)
            keep_nan = not a.logging_nan_inf_filter or "underflow_overflow" in str(a.debug)
            total += loss if keep_nan else torch.nan_to_num(loss.float(), nan=0.0, posinf=0.0, neginf=0.0)
            if i < len(batches) - 1:
                self.control = self.callback_handler.call_event("on_substep_end", a, st, self.control)
        self.control = self.callback_handler.call_event("on_pre_optimizer_step", a, st, self.control)
        lr = self._get_learning_rate()
        from ..extras.profiling import profiling_context

        with profiling_context(self, "optimizer"):
            grad_norm = self.engine.step(lr, a.max_grad_norm)
        if "underflow_overflow" in str(a.debug):  # costs a device sync per step: a debugging aid, off by default
            if not (bool(torch.isfinite(total)) and bool(torch.isfinite(torch.as_tensor(grad_norm)))):
                raise FloatingPointError(f"non-finite loss ({float(total)}) or gradient norm ({float(grad_norm)}) at "
                                         f"optimizer step {st.global_step + 1}")
        self.control = self.callback_handler.call_event("on_optimizer_step", a, st, self.control)
        self.lr_scheduler.step()
        self.engine.zero_grad()
        if getattr(self, "_ckpt_auto", None) is not None:
            self._autotune_checkpointing()
        return total, grad_norm, lr

    def _autotune_checkpointing(self, probe: int = 4):
        """``gradient_checkpointing_kwargs={"num_layers": "auto"}``: how many layers may keep their activations.

        Optimizer step 1 runs with every layer recomputed and gives the peak memory of the whole step (generation and
        reference passes of the online trainers included).  Step 2 keeps the activations of the last ``probe`` layers;
        the growth of the peak is what one layer costs.  From step 3 on as many layers keep theirs as fit into the
        memory that was free at the first peak, less a reserve of 12 % of the device + 4 GiB (allocator slack,
        variation between batches: a step that runs close to the limit loses more in allocator retries than it saves
        in recomputation), the minimum over all ranks.  Engines that need every layer recomputed (streamed
        shards) and CPU runs leave the setting alone."""
        m, dev = self.model, self.args.device
        lm = getattr(m, "language_model", m)
        L = len(getattr(lm, "layers", []))
        if dev.type != "cuda" or L == 0 or getattr(self.engine, "mode", "") == "full_shard_stream":
            self._ckpt_auto = None
            return
        stage = self._ckpt_auto
        peak = torch.cuda.max_memory_allocated(dev)
        if stage == 0:
            self._ckpt_peak0 = peak
            lm.checkpoint_num_layers = max(0, L - min(probe, L))
            torch.cuda.reset_peak_memory_stats(dev)
            self._ckpt_auto = 1
            return
        total_mem = torch.cuda.get_device_properties(dev).total_memory
        kept = L - lm.checkpoint_num_layers
        per_layer = max((peak - self._ckpt_peak0) / max(kept, 1), 1.0)
        # a step whose peak lies outside the training pass hides the cost of the probe: fall back to an estimate of
        # what a layer saves for backward (about 34 values of hidden size per token for a SwiGLU decoder, in bf16)
        c = lm.config
        tokens = getattr(self, "_last_micro_batch_tokens", None) or 8192
        floor = tokens * (10 * c.hidden_size + 4 * (getattr(c, "moe_intermediate_size", None) or c.intermediate_size)) * 2
        per_layer = max(per_layer, floor / 2)
        headroom = total_mem - self._ckpt_peak0 - int(0.12 * total_mem) - (4 << 30)
        k = int(max(0, min(L, headroom // per_layer)))
        t = torch.tensor([k], device=dev)
        if D.world_size() > 1:
            D.all_reduce(t, "min")
        k = int(t)
        lm.checkpoint_num_layers = L - k
        self._ckpt_auto = None
        self._ckpt_auto_result = {"layers_keeping_activations": k, "layers": L, "bytes_per_layer": int(per_layer),
                                  "peak_all_recomputed": int(self._ckpt_peak0)}

    def _maybe_log_save_evaluate(self, tr_loss, grad_norm, lr, t_start):
        st, a = self.state, self.args
        if self.control.should_log and st.global_step > self._logged_step:
            t = tr_loss.clone()
            if D.world_size() > 1:
                D.all_reduce(t, "mean")
            scalar = float(t)
            logs = {"loss": round(scalar / (st.global_step - self._logged_step), 4)}
            if grad_norm is not None:
                logs["grad_norm"] = float(grad_norm)
            logs["learning_rate"] = lr
            self._total_loss_scalar += scalar
            self._logged_step = st.global_step
            tr_loss = torch.zeros_like(tr_loss)
            self.log(logs, t_start)
            self.control.should_log = False
        metrics = None
        if self.control.should_evaluate:
            metrics = self.evaluate()
            self.control.should_evaluate = False
        if self.control.should_save:
            self._save_checkpoint(self.model, metrics=metrics)
            self.control = self.callback_handler.call_event("on_save", a, st, self.control)
            self.control.should_save = False
        return tr_loss

    def log(self, logs: dict, start_time: float | None = None):
        mode = "train" if self.model is None or self.model.training else "eval"
        own = self._metrics[mode]
        if own:
            from ..trainer.utils import resolve_deferred_metrics

            resolve_deferred_metrics(own)  # one collective for everything the micro-batches recorded
            avg = {k: sum(v) / len(v) for k, v in own.items() if len(v)}
            if D.world_size() > 1 and os.environ.get("TRL_B200_PROFILE_MAX_OVER_RANKS", "0") == "1":
                # a phase is as slow as its slowest rank: report the maximum of the phase timers (one small object
                # gather per log call; every rank logs at the same steps)
                prof = {k: float(v) for k, v in avg.items() if k.startswith("profiling/")}
                for other in D.gather_object([prof]):
                    for k, v in other.items():
                        if k in avg:
                            avg[k] = max(float(avg[k]), v)
            if mode == "eval":
                avg = {f"eval_{k}": v for k, v in avg.items()}
            logs = {**logs, **avg}
            own.clear()
        if self.state.epoch is not None:
            logs["epoch"] = round(self.state.epoch, 4) if isinstance(self.state.epoch, float) else self.state.epoch
        # metrics are averaged as tensors to avoid a device sync per micro-step; they leave the trainer as numbers
        logs = {k: (float(v) if torch.is_tensor(v) and v.numel() == 1 else v) for k, v in logs.items()}
        self.state.log_history.append({**logs, "step": self.state.global_step})
        self.control = self.callback_handler.call_event("on_log", self.args, self.state, self.control, logs=logs)

    # ---- evaluation ---------------------------------------------------------------------------
    def prediction_step(self, model, inputs, prediction_loss_only=True, ignore_keys=None):
        inputs = self._prepare_inputs(inputs)
        with torch.no_grad():
            loss = self.compute_loss(model, inputs)
        return loss.detach(), None, None

    def evaluate(self, eval_dataset=None, ignore_keys=None, metric_key_prefix: str = "eval"):
        if isinstance(eval_dataset, str):  # the name of one of the datasets given at construction
            eval_dataset, metric_key_prefix = self.eval_dataset[eval_dataset], f"{metric_key_prefix}_{eval_dataset}"
        elif eval_dataset is not None:
            if isinstance(eval_dataset, dict):  # also DatasetDict / IterableDatasetDict
                out = {}
                for name, ds in eval_dataset.items():
                    out.update(self.evaluate(ds, ignore_keys, f"{metric_key_prefix}_{name}"))
                return out
            prepare = getattr(self, "_prepare_given_eval_dataset", None)
            if prepare is not None:  # raw rows get the preparation of the trainer's constructor (a no-op on prepared rows)
                eval_dataset = prepare(eval_dataset)
        if eval_dataset is None and isinstance(self.eval_dataset, dict):
            out = {}
            for name, ds in self.eval_dataset.items():
                out.update(self.evaluate(ds, ignore_keys, f"{metric_key_prefix}_{name}"))
            return out
        loader = self.get_eval_dataloader(eval_dataset)
        was_training = self.model.training
        self.model.eval()
        losses, preds, labels_all = [], [], []
        t0 = time.time()
        for batch in loader:
            loss, logits, labels = self.prediction_step(self.model, batch, prediction_loss_only=self.compute_metrics is None)
            losses.append(loss.float().reshape(1))
            if logits is not None and self.compute_metrics is not None:
                if self.preprocess_logits_for_metrics is not None:
                    logits = self.preprocess_logits_for_metrics(logits, labels)
                preds.append(logits.cpu())
                labels_all.append(labels.cpu() if labels is not None else None)
            self.control = self.callback_handler.call_event("on_prediction_step", self.args, self.state, self.control)
        metrics = {}
        if losses:
            l = torch.cat(losses)
            l = D.gather(l) if D.world_size() > 1 else l
            metrics[f"{metric_key_prefix}_loss"] = float(l.mean())
        if self.compute_metrics is not None and preds:
            from types import SimpleNamespace

            def pad_cat(ts):  # batches of different width: pad the sequence dimension with -100, as transformers does
                if ts[0].ndim < 2:
                    return torch.cat(ts)
                w = max(t.shape[1] for t in ts)
                return torch.cat([t if t.shape[1] == w else torch.nn.functional.pad(
                    t, (0, 0) * (t.ndim - 2) + (0, w - t.shape[1]), value=-100) for t in ts])

            ep = SimpleNamespace(predictions=pad_cat(preds).float().numpy(),
                                 label_ids=pad_cat(labels_all).numpy() if labels_all[0] is not None else None)
            for k, v in self.compute_metrics(ep).items():
                metrics[k if k.startswith(metric_key_prefix) else f"{metric_key_prefix}_{k}"] = v
        metrics[f"{metric_key_prefix}_runtime"] = round(time.time() - t0, 4)
        self.log(metrics)
        self.control = self.callback_handler.call_event("on_evaluate", self.args, self.state, self.control, metrics=metrics)
        if was_training:
            self.model.train()
        return metrics

    # ---- persistence ------------------------------------------------------------------------------
    def _full_state_dict(self):
        """Makes the model's weights whole before saving (collective).  Engines that never hold the whole model return
        the checkpoint tensors instead (host copies on the saving rank, nothing elsewhere)."""
        if self.engine is not None and hasattr(self.engine, "gather_full_params"):
            self.engine.gather_full_params()
        if self.engine is not None and hasattr(self.engine, "streamed_hf_state_dict"):
            sd = self.engine.streamed_hf_state_dict(to_cpu=self.args.should_save)
            return sd if self.args.should_save else None
        lm = getattr(self.model, "language_model", self.model)
        if getattr(lm, "ep_world", 1) > 1:  # expert-parallel model: the experts are gathered layer by layer
            from ..parallel.expert_parallel import ep_hf_state_dict

            sd = ep_hf_state_dict(self.model, to_cpu=self.args.should_save)
            return sd if self.args.should_save else None
        return None

    def save_model(self, output_dir: str | None = None, _internal_call: bool = False):
        output_dir = output_dir or self.args.output_dir
        state_dict = self._full_state_dict()
        if self.args.should_save:
            os.makedirs(output_dir, exist_ok=True)
            self._save(output_dir, state_dict)
        D.barrier()

    def _save(self, output_dir: str, state_dict=None):
        m = self.model
        if getattr(m, "peft_config", None) is not None and hasattr(m, "save_adapter"):
            m.save_adapter(output_dir)
        elif hasattr(m, "save_pretrained"):
            m.save_pretrained(output_dir, **({"state_dict": state_dict} if state_dict is not None else {}))
        else:
            torch.save(m.state_dict(), os.path.join(output_dir, "pytorch_model.bin"))
        if self.processing_class is not None and hasattr(self.processing_class, "save_pretrained"):
            self.processing_class.save_pretrained(output_dir)
        with open(os.path.join(output_dir, "training_args.json"), "w") as f:
            f.write(self.args.to_json_string())

    def _save_checkpoint(self, model, trial=None, metrics=None):
        a, st = self.args, self.state
        folder = os.path.join(a.output_dir, f"{PREFIX_CHECKPOINT_DIR}-{st.global_step}")
        self.save_model(folder, _internal_call=True)
        os.makedirs(folder, exist_ok=True)
        if a.should_save:
            try:
                self.create_model_card()  # README.md next to the checkpoints, refreshed at every save
            except Exception:  # a missing template engine must not lose the checkpoint
                pass
        if not a.save_only_model:
            sharded = getattr(self.engine, "per_rank_state", self.engine.sharded)
            if sharded or a.should_save:
                name = f"optimizer_rank{D.rank()}.pt" if sharded else "optimizer.pt"
                torch.save(self.engine.optimizer_state_dict(), os.path.join(folder, name))
            if a.should_save:
                torch.save(self.lr_scheduler.state_dict(), os.path.join(folder, "scheduler.pt"))
            # plain containers and tensors only, so that every file of a checkpoint loads with weights_only=True
            py = random.getstate()
            npst = np.random.get_state()
            rng = {"python": [py[0], list(py[1]), py[2]],
                   "numpy": {"name": npst[0], "keys": torch.from_numpy(npst[1].astype(np.int64)), "pos": int(npst[2]),
                             "has_gauss": int(npst[3]), "cached_gaussian": float(npst[4])},
                   "cpu": torch.get_rng_state()}
            if torch.cuda.is_available() and a.device.type == "cuda":
                rng["cuda"] = torch.cuda.get_rng_state()
            torch.save(rng, os.path.join(folder, f"rng_state_{D.rank()}.pth" if D.world_size() > 1 else "rng_state.pth"))
        if metrics and a.metric_for_best_model:
            k = a.metric_for_best_model if a.metric_for_best_model.startswith("eval_") else f"eval_{a.metric_for_best_model}"
            v = metrics.get(k)
            if v is not None:
                gib = a.greater_is_better if a.greater_is_better is not None else not k.endswith("loss")
                if st.best_metric is None or (v > st.best_metric if gib else v < st.best_metric):
                    st.best_metric, st.best_model_checkpoint, st.best_global_step = v, folder, st.global_step
        if a.should_save:
            st.stateful_callbacks = {type(c).__name__: c.state() for c in self.callback_handler.callbacks
                                     if hasattr(c, "state") and callable(c.state)}
            st.save_to_json(os.path.join(folder, "trainer_state.json"))
            self._rotate_checkpoints()
        D.barrier()

    def _rotate_checkpoints(self):
        lim = self.args.save_total_limit
        if not lim or lim <= 0:
            return
        cks = sorted_checkpoints(self.args.output_dir)
        best = self.state.best_model_checkpoint
        for c in cks[:max(0, len(cks) - lim)]:
            if best and os.path.abspath(c) == os.path.abspath(best):
                continue
            shutil.rmtree(c, ignore_errors=True)

    def _load_from_checkpoint(self, folder: str):
        from ..models.hf_io import load_hf_state_dict, load_state_dict_dir

        if not os.path.isdir(folder):
            raise ValueError(f"Can't find a valid checkpoint at {folder}")
        m = self.model
        if hasattr(m, "load_adapter") and os.path.exists(os.path.join(folder, "adapter_model.safetensors")):
            m.load_adapter(folder)
        elif getattr(m, "_is_native", False) and hasattr(self.engine, "load_weights"):
            self.engine.load_weights(load_state_dict_dir(folder))  # layer weights live as slices inside the engine
        elif getattr(m, "_is_native", False):
            load_hf_state_dict(m, load_state_dict_dir(folder), strict=True)
        sp = os.path.join(folder, "trainer_state.json")
        if os.path.exists(sp):
            old = TrainerState.load_from_json(sp)
            old.is_world_process_zero, old.is_local_process_zero = self.state.is_world_process_zero, self.state.is_local_process_zero
            self.state = old
        per_rank = getattr(self.engine, "per_rank_state", self.engine.sharded)
        op = os.path.join(folder, f"optimizer_rank{D.rank()}.pt" if per_rank else "optimizer.pt")
        saved = sorted(f for f in os.listdir(folder) if re.fullmatch(r"optimizer(_rank\d+)?\.pt", f))
        expect = [f"optimizer_rank{r}.pt" for r in range(D.world_size())] if per_rank else ["optimizer.pt"]
        if saved and sorted(expect) != saved and hasattr(self.engine, "load_optimizer_state_resharded"):
            # elastic resume: the checkpoint was written with another world size or shard mode.  Every rank reads all
            # optimizer files and keeps the slices it owns now.
            shards = [torch.load(os.path.join(folder, f), map_location="cpu", weights_only=True) for f in saved]
            self.engine.load_optimizer_state_resharded(shards)
        elif os.path.exists(op):
            self.engine.load_optimizer_state_dict(torch.load(op, map_location="cpu", weights_only=True))
        elif getattr(m, "_is_native", False):
            self.engine.refresh_master_from_params() if hasattr(self.engine, "refresh_master_from_params") else None
        sc = os.path.join(folder, "scheduler.pt")
        if os.path.exists(sc):
            self.lr_scheduler.load_state_dict(torch.load(sc, weights_only=True))
        for cand in (f"rng_state_{D.rank()}.pth", "rng_state.pth"):
            rp = os.path.join(folder, cand)
            if os.path.exists(rp):
                rng = torch.load(rp, weights_only=True)
                py, npst = rng["python"], rng["numpy"]
                random.setstate((py[0], tuple(py[1]), py[2]))
                np.random.set_state((npst["name"], npst["keys"].numpy().astype(np.uint32), npst["pos"], npst["has_gauss"],
                                     npst["cached_gaussian"]))
                torch.set_rng_state(rng["cpu"])
                if "cuda" in rng and torch.cuda.is_available():
                    torch.cuda.set_rng_state(rng["cuda"])
                break
        self._on_checkpoint_loaded(folder)

    def _on_checkpoint_loaded(self, folder: str):
        pass

    def create_model_card(self, model_name: str | None = None, dataset_name: str | None = None, tags=None):
        """Writes ``README.md`` into ``output_dir`` from the packaged template (trl/trainer/base_trainer.py:127-191)."""
        if not self.is_world_process_zero():
            return
        from ..trainer.utils import generate_model_card

        base = getattr(self.model, "name_or_path", None) or getattr(getattr(self.model, "config", None), "_name_or_path", None)
        if base and os.path.isdir(str(base)):
            base = None
        paper = getattr(self, "_paper", {}) or {}
        text = generate_model_card(base_model=base, model_name=model_name or os.path.basename(self.args.output_dir.rstrip("/")),
                                   dataset_name=dataset_name, tags=list(getattr(self, "_tag_names", [])) + list(tags or []),
                                   trainer_name=getattr(self, "_name", type(self).__name__),
                                   trainer_citation=paper.get("citation"), paper_title=paper.get("title"),
                                   paper_id=paper.get("id"),
                                   template_file=getattr(self, "_template_file", "lm_model_card.md"))
        os.makedirs(self.args.output_dir, exist_ok=True)
        with open(os.path.join(self.args.output_dir, "README.md"), "w") as f:
            f.write(text)

    def push_to_hub(self, *a, **k):
        raise RuntimeError("push_to_hub needs network access, which this build does not assume")


class _AcceleratorShim:
    def __init__(self, trainer):
        self._t = trainer

    num_processes = property(lambda s: D.world_size())
    process_index = property(lambda s: D.rank())
    is_main_process = property(lambda s: D.is_main())
    device = property(lambda s: s._t.args.device)

    def gather(self, t):
        return D.gather(t)

    gather_for_metrics = gather

    def reduce(self, t, reduction="sum"):
        return D.all_reduce(t.clone(), reduction)

    def unwrap_model(self, m, **k):
        return m

    def wait_for_everyone(self):
        D.barrier()

    def pad_across_processes(self, t, dim=0, pad_index=0):
        return D.pad_across_processes(t, dim, pad_index)


def sorted_checkpoints(output_dir: str) -> list[str]:
    if not os.path.isdir(output_dir):
        return []
    out = []
    for d in os.listdir(output_dir):
        m = re.match(rf"^{PREFIX_CHECKPOINT_DIR}-(\d+)$", d)
        if m and os.path.isdir(os.path.join(output_dir, d)):
            out.append((int(m.group(1)), os.path.join(output_dir, d)))
    return [p for _, p in sorted(out)]


def get_last_checkpoint(output_dir: str) -> Optional[str]:
    cks = sorted_checkpoints(output_dir)
    return cks[-1] if cks else None
