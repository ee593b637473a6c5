"""Trainer callbacks with the behaviour of trl/trainer/callbacks.py:
SyncRefModelCallback (:104-142), RichProgressCallback (:145-253), LogCompletionsCallback
(:256-345), WeaveCallback (:348-575), BEMACallback (:577-762)."""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..loop.state import TrainerCallback
from ..parallel import dist as D


class SyncRefModelCallback(TrainerCallback):
    """``ref <- (1 - alpha) * ref + alpha * policy`` every ``ref_model_sync_steps`` optimizer steps."""

    def __init__(self, ref_model, accelerator=None):
        self.ref_model = ref_model

    @staticmethod
    @torch.no_grad()
    def sync_target_model(model, target_model, alpha: float):
        for tp, p in zip(target_model.parameters(), model.parameters()):
            tp.data.mul_(1.0 - alpha).add_(p.data.to(tp.dtype), alpha=alpha)

    def on_step_end(self, args, state, control, model=None, **kw):
        if self.ref_model is not None and state.global_step % args.ref_model_sync_steps == 0:
            self.sync_target_model(model, self.ref_model, args.ref_model_mixup_alpha)


class RichProgressCallback(TrainerCallback):
    """Progress bars and a live status line rendered with rich (plain prints when rich is absent)."""

    def __init__(self):
        self.progress = self.task = None
        self.current_step = 0

    def on_train_begin(self, args, state, control, **kw):
        if not state.is_world_process_zero:
            return
        try:
            from rich.progress import Progress

            self.progress = Progress()
            self.progress.start()
            self.task = self.progress.add_task("[blue]Training", total=state.max_steps)
        except Exception:
            self.progress = None
        self.current_step = 0

    def on_step_end(self, args, state, control, **kw):
        if self.progress is not None:
            self.progress.update(self.task, advance=state.global_step - self.current_step)
            self.current_step = state.global_step

    def on_log(self, args, state, control, logs=None, **kw):
        if state.is_world_process_zero and self.progress is not None and logs:
            self.progress.console.print({k: v for k, v in logs.items() if k != "total_flos"})

    def on_train_end(self, args, state, control, **kw):
        if self.progress is not None:
            self.progress.stop()
            self.progress = None


class LogCompletionsCallback(TrainerCallback):
    """Every ``freq`` steps, generate completions for eval prompts and log them as a table
    (JSONL under ``output_dir/completions_callback.jsonl``; wandb/trackio are not reachable offline)."""

    def __init__(self, trainer, generation_config=None, num_prompts: Optional[int] = None, freq: Optional[int] = None):
        self.trainer, self.generation_config, self.freq = trainer, generation_config, freq
        self.table, self._last = [], -1
        ds = trainer.eval_dataset
        if ds is None:
            raise ValueError("Trainer must have an evaluation dataset to use the LogCompletionsCallback.")
        self.rows = [ds[i] for i in range(min(len(ds), num_prompts or len(ds)))]

    def on_step_end(self, args, state, control, **kw):
        freq = self.freq or state.eval_steps
        if state.global_step == self._last or not freq or state.global_step % freq != 0:
            return
        from ..data_utils import maybe_apply_chat_template
        from ..rollout.engine import EagerGenerator
        from ..rollout.sampling import SamplingParams

        tok = self.trainer.processing_class
        prompts = [maybe_apply_chat_template({"prompt": r["prompt"]}, tok)["prompt"] for r in self.rows]
        ids = tok(text=prompts)["input_ids"]
        mt = getattr(self.generation_config, "max_new_tokens", None) or 32
        gen = EagerGenerator(self.trainer.model) if self.trainer.args.device.type == "cpu" else self.trainer._get_rollout()
        outs = gen.generate(ids, SamplingParams(max_tokens=mt, eos_token_id=tok.eos_token_id, temperature=1.0))
        texts = tok.batch_decode([o.token_ids for o in outs], skip_special_tokens=True)
        if state.is_world_process_zero:
            import json

            os.makedirs(args.output_dir, exist_ok=True)
            with open(os.path.join(args.output_dir, "completions_callback.jsonl"), "a") as f:
                for p, c in zip(prompts, texts):
                    row = {"step": state.global_step, "prompt": p, "completion": c}
                    self.table.append(row)
                    f.write(json.dumps(row) + "\n")
        self._last = state.global_step


class WeaveCallback(TrainerCallback):
    """Weights & Biases Weave evaluation logging; needs the ``weave`` package and network access."""

    def __init__(self, trainer, project_name=None, scorers=None, generation_config=None, num_prompts=None,
                 dataset_name="eval_dataset", model_name=None):
        try:
            import weave  # noqa: F401
        except ImportError as e:
            raise ImportError("WeaveCallback requires the `weave` package, which is not installed.") from e
        self.trainer = trainer


class BEMACallback(TrainerCallback):
    """Bias-corrected EMA of the weights (Block et al.), saved to ``output_dir/bema`` at the end.

    theta_bema = alpha_t * (theta_t - theta_0) + EMA_t with alpha_t = (rho + gamma*t)^(-eta),
    EMA_t = (1 - beta_t) EMA_{t-1} + beta_t theta_t, beta_t = (rho + gamma*t)^(-ema_power)."""

    def __init__(self, update_freq: int = 400, ema_power: float = 0.5, bias_power: float = 0.2, lag: int = 10,
                 update_after: int = 0, multiplier: float = 1.0, min_ema_multiplier: float = 0.0, device: str = "cpu"):
        self.update_freq, self.ema_power, self.bias_power = update_freq, ema_power, bias_power
        self.lag, self.update_after, self.multiplier, self.min_ema_multiplier = lag, update_after, multiplier, min_ema_multiplier
        self.device = device
        self.theta0, self.ema, self.running, self._model = None, None, None, None

    @torch.no_grad()
    def on_train_begin(self, args, state, control, model=None, **kw):
        self.names = [n for n, p in model.named_parameters() if p.requires_grad]
        self.theta0 = self._snapshot(model)  # theta_0 and the EMA start at the initial weights
        self.ema = [t.clone() for t in self.theta0]
        self.running = [t.clone() for t in self.theta0]

    @torch.no_grad()
    def _snapshot(self, model):
        return [p.detach().to(self.device, torch.float32).clone() for n, p in model.named_parameters() if n in self.names]

    def _ema_beta(self, step: int) -> float:
        """beta_t = (lag + multiplier * t)^(-ema_power), floored at ``min_ema_multiplier``."""
        return max((self.lag + self.multiplier * step) ** (-self.ema_power), self.min_ema_multiplier)

    def _bema_alpha(self, step: int) -> float:
        """alpha_t = (lag + multiplier * t)^(-bias_power)."""
        return (self.lag + self.multiplier * step) ** (-self.bias_power)

    @torch.no_grad()
    def _update_bema_weights(self, step: int):
        beta, alpha = self._ema_beta(step), self._bema_alpha(step)
        for e, r, c, z in zip(self.ema, self.running, self._snapshot(self._model), self.theta0):
            e.mul_(1 - beta).add_(c, alpha=beta)
            r.copy_(e + alpha * (c - z))

    @torch.no_grad()
    def on_step_end(self, args, state, control, model=None, **kw):
        step = state.global_step
        if step < self.update_after:
            return
        self._model = model
        if step == self.update_after:  # restart theta_0 and the EMA from the weights of this step
            self.theta0 = self._snapshot(model)
            self.ema = [t.clone() for t in self.theta0]
        elif (step - self.update_after) % self.update_freq == 0:
            self._update_bema_weights(step)

    @torch.no_grad()
    def on_train_end(self, args, state, control, model=None, **kw):
        if self.running is None or not state.is_world_process_zero:
            return
        backup = self._snapshot(model)
        params = [p for n, p in model.named_parameters() if n in self.names]
        for p, r in zip(params, self.running):
            p.data.copy_(r.to(p.device, p.dtype))
        out = os.path.join(args.output_dir, "bema")
        if hasattr(model, "save_pretrained"):
            model.save_pretrained(out)
        for p, b in zip(params, backup):
            p.data.copy_(b.to(p.device, p.dtype))


class WatchdogCallback(TrainerCallback):
    """Heartbeat files per rank (``utils/watchdog.py``): started with training, peers checked before every optimizer
    step, so a rank that died between steps stops the others with a clear error instead of a collective timeout.
    Added automatically when ``TRL_B200_WATCHDOG_DIR`` is set."""

    def __init__(self, directory: str, interval_s: float = 1.0, stale_after_s: float = 60.0):
        self.directory, self.interval_s, self.stale_after_s = directory, interval_s, stale_after_s
        self.watchdog = None

    def on_train_begin(self, args, state, control, **kw):
        from ..parallel import dist as D
        from ..utils.watchdog import RankWatchdog

        self.watchdog = RankWatchdog(self.directory, D.rank(), D.world_size(), self.interval_s, self.stale_after_s).start()

    def on_step_begin(self, args, state, control, **kw):
        if self.watchdog is not None:
            self.watchdog.check_peers()

    def on_train_end(self, args, state, control, **kw):
        if self.watchdog is not None:
            self.watchdog.stop()
            self.watchdog = None


class JITCheckpointCallback(TrainerCallback):
    """Checkpoint on SIGTERM (``enable_jit_checkpoint=True``): a preempted job saves at the next optimizer-step
    boundary and stops cleanly, so ``resume_from_checkpoint=True`` loses at most one step.  The signal may reach only
    some ranks; every step the ranks agree on the flag with one tiny all-reduce, so that all of them take part in the
    (collective) save.  Same purpose as transformers' ``enable_jit_checkpoint`` training argument."""

    def __init__(self, signals=None):
        import signal

        self.signals = tuple(signals) if signals is not None else (signal.SIGTERM,)
        self.requested = False
        self._previous = {}

    def _handler(self, signum, frame):
        self.requested = True

    def on_train_begin(self, args, state, control, **kw):
        import signal
        import threading

        if threading.current_thread() is threading.main_thread():  # handlers can only be installed there
            for s in self.signals:
                self._previous[s] = signal.signal(s, self._handler)

    def on_step_end(self, args, state, control, **kw):
        import torch

        from ..parallel import dist as D

        flag = torch.tensor([1.0 if self.requested else 0.0], device=args.device)
        if D.world_size() > 1:
            D.all_reduce(flag, "max")
        if float(flag) > 0:
            control.should_save = True
            control.should_training_stop = True
            self.requested = False
        return control

    def on_train_end(self, args, state, control, **kw):
        import signal

        for s, h in self._previous.items():
            signal.signal(s, h)
        self._previous = {}
