"""Teacher maintenance for self-distillation (trl/experimental/sdpo/teacher_sync.py:24-184; shared with SDFT).

``base``: the teacher stays the initial weights.  ``ema``: theta_T <- (1 - rate) theta_T + rate * theta_S every
``teacher_sync_steps`` optimizer steps.  ``student``: the teacher is the live student (no copy, evaluated without
gradient)."""
from __future__ import annotations

import copy

import torch

from ...loop.state import TrainerCallback


class TeacherSyncCallback(TrainerCallback):
    def __init__(self, teacher, rate: float, every: int):
        self.teacher, self.rate, self.every = teacher, rate, max(1, every)

    @torch.no_grad()
    def on_step_end(self, args, state, control, model=None, **kw):
        if state.global_step % self.every:
            return
        t = dict(self.teacher.named_parameters())
        for n, p in model.named_parameters():
            if n in t:
                t[n].mul_(1 - self.rate).add_(p.detach().to(t[n].dtype), alpha=self.rate)


def build_teacher(trainer, kind: str, rate: float, every: int):
    """Returns the teacher module (None = use the student itself) and registers the sync callback when needed."""
    if kind == "student":
        return None
    teacher = copy.deepcopy(trainer.model).eval().requires_grad_(False)
    if kind == "ema":
        trainer.add_callback(TeacherSyncCallback(teacher, rate, every))
    elif kind != "base":
        raise ValueError("teacher_model_kind must be 'base', 'ema' or 'student'")
    return teacher
