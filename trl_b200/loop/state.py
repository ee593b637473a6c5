"""Trainer state, control flags and the callback protocol.

Names and event order follow ``transformers.TrainerCallback`` so callbacks
written for the reference (trl/trainer/callbacks.py) plug in unchanged:
``on_init_end, on_train_begin, on_epoch_begin, on_step_begin,
on_pre_optimizer_step, on_optimizer_step, on_substep_end, on_step_end,
on_evaluate, on_save, on_log, on_prediction_step, on_epoch_end, on_train_end``.
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass
class TrainerState:
    epoch: Optional[float] = None
    global_step: int = 0
    max_steps: int = 0
    logging_steps: int = 500
    eval_steps: int = 500
    save_steps: int = 500
    train_batch_size: Optional[int] = None
    num_train_epochs: int = 0
    num_input_tokens_seen: int = 0
    total_flos: float = 0
    log_history: list = field(default_factory=list)
    best_metric: Optional[float] = None
    best_global_step: Optional[int] = None
    best_model_checkpoint: Optional[str] = None
    is_local_process_zero: bool = True
    is_world_process_zero: bool = True
    is_hyper_param_search: bool = False
    trial_name: Optional[str] = None
    trial_params: Optional[dict] = None
    stateful_callbacks: dict = field(default_factory=dict)

    def save_to_json(self, path: str):
        with open(path, "w", encoding="utf-8") as f:
            f.write(json.dumps(dataclasses.asdict(self), indent=2, sort_keys=True, default=float) + "\n")

    @classmethod
    def load_from_json(cls, path: str) -> "TrainerState":
        with open(path, encoding="utf-8") as f:
            d = json.load(f)
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})


@dataclass
class TrainerControl:
    should_training_stop: bool = False
    should_epoch_stop: bool = False
    should_save: bool = False
    should_evaluate: bool = False
    should_log: bool = False

    def _new_training(self):
        self.should_training_stop = False

    def _new_epoch(self):
        self.should_epoch_stop = False

    def _new_step(self):
        self.should_save = self.should_evaluate = self.should_log = False

    def state(self) -> dict:
        return {"args": dataclasses.asdict(self), "attributes": {}}


class TrainerCallback:
    def on_init_end(self, args, state, control, **kw): ...
    def on_train_begin(self, args, state, control, **kw): ...
    def on_train_end(self, args, state, control, **kw): ...
    def on_epoch_begin(self, args, state, control, **kw): ...
    def on_epoch_end(self, args, state, control, **kw): ...
    def on_step_begin(self, args, state, control, **kw): ...
    def on_pre_optimizer_step(self, args, state, control, **kw): ...
    def on_optimizer_step(self, args, state, control, **kw): ...
    def on_substep_end(self, args, state, control, **kw): ...
    def on_step_end(self, args, state, control, **kw): ...
    def on_evaluate(self, args, state, control, **kw): ...
    def on_predict(self, args, state, control, metrics=None, **kw): ...
    def on_save(self, args, state, control, **kw): ...
    def on_log(self, args, state, control, **kw): ...
    def on_prediction_step(self, args, state, control, **kw): ...


class CallbackHandler:
    def __init__(self, callbacks, model, processing_class, optimizer, lr_scheduler):
        self.callbacks: list[TrainerCallback] = []
        for cb in callbacks or []:
            self.add_callback(cb)
        self.model, self.processing_class = model, processing_class
        self.optimizer, self.lr_scheduler = optimizer, lr_scheduler
        self.train_dataloader = self.eval_dataloader = None

    def add_callback(self, cb):
        cb = cb() if isinstance(cb, type) else cb
        self.callbacks.append(cb)

    def pop_callback(self, cb):
        for c in list(self.callbacks):
            if c is cb or (isinstance(cb, type) and isinstance(c, cb)):
                self.callbacks.remove(c)
                return c
        return None

    def remove_callback(self, cb):
        self.pop_callback(cb)

    def call_event(self, event: str, args, state, control, **kw):
        for cb in self.callbacks:
            res = getattr(cb, event)(
                args, state, control, model=self.model, processing_class=self.processing_class,
                tokenizer=self.processing_class, optimizer=self.optimizer, lr_scheduler=self.lr_scheduler,
                train_dataloader=self.train_dataloader, eval_dataloader=self.eval_dataloader, **kw)
            if res is not None:
                control = res
        return control


class DefaultFlowCallback(TrainerCallback):
    """Decides when to log / evaluate / save from the ``*_strategy`` and ``*_steps`` arguments."""

    def on_step_end(self, args, state, control, **kw):
        gs = state.global_step
        if gs == 1 and args.logging_first_step:
            control.should_log = True
        if args.logging_strategy == "steps" and state.logging_steps and gs % state.logging_steps == 0:
            control.should_log = True
        if args.eval_strategy == "steps" and state.eval_steps and gs % state.eval_steps == 0 and args.eval_delay <= gs:
            control.should_evaluate = True
        if args.save_strategy == "steps" and state.save_steps and gs % state.save_steps == 0:
            control.should_save = True
        if gs >= state.max_steps:
            control.should_training_stop = True
            if args.save_strategy == "steps" and state.save_steps:
                pass
        return control

    def on_epoch_end(self, args, state, control, **kw):
        if args.logging_strategy == "epoch":
            control.should_log = True
        if args.eval_strategy == "epoch" and args.eval_delay <= (state.epoch or 0):
            control.should_evaluate = True
        if args.save_strategy == "epoch":
            control.should_save = True
        return control


class PrinterCallback(TrainerCallback):
    def on_log(self, args, state, control, logs=None, **kw):
        if state.is_world_process_zero and logs is not None:
            logs = dict(logs)
            logs.pop("total_flos", None)
            print(logs, flush=True)


class EarlyStoppingCallback(TrainerCallback):
    def __init__(self, early_stopping_patience: int = 1, early_stopping_threshold: float = 0.0):
        self.patience, self.threshold, self.counter = early_stopping_patience, early_stopping_threshold, 0

    def on_evaluate(self, args, state, control, metrics=None, **kw):
        name = args.metric_for_best_model or "loss"
        name = name if name.startswith("eval_") else f"eval_{name}"
        v = (metrics or {}).get(name)
        if v is None:
            return control
        better = (lambda a, b: a > b + self.threshold) if args.greater_is_better else (lambda a, b: a < b - self.threshold)
        if state.best_metric is None or better(v, state.best_metric):
            self.counter = 0
        else:
            self.counter += 1
        if self.counter >= self.patience:
            control.should_training_stop = True
        return control
