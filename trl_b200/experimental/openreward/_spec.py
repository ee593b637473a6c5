"""Spec object for an ORS environment (trl/experimental/openreward/_spec.py: OpenRewardSpec :78-359).

``OpenRewardSpec(env_id)`` needs the ``openreward`` client and a reachable server; it exposes ``dataset`` (one row per
task), ``environment_factory`` and ``reward_funcs`` for GRPOTrainer / AsyncGRPOTrainer.  ``from_session_factory``
builds the same surface from any session factory (used by tests and by custom servers)."""
from __future__ import annotations

from typing import Any, Callable

from .environment import _import_openreward, _spec_to_dict, make_environment_class


def _outcome_only_reward_func(environments=None, **_):
    return [float(e.reward) if e is not None else 0.0 for e in (environments or [])]


class OpenRewardSpec:
    def __init__(self, env_id: str | None = None, *, split: str = "train", num_tasks: int | None = None, base_url=None,
                 _session_factory: Callable[..., Any] | None = None, _tool_specs: list | None = None,
                 _tasks: list[dict] | None = None):
        if _session_factory is None:
            ors = _import_openreward()
            client = ors.Client(base_url=base_url) if base_url else ors.Client()
            env = client.environment(env_id)
            tasks = [dict(t) if isinstance(t, dict) else {"task_id": getattr(t, "id", i), "prompt": getattr(t, "prompt", "")}
                     for i, t in enumerate(env.list_tasks(split=split))]
            _tasks = tasks[:num_tasks] if num_tasks else tasks
            probe = env.session(task=_tasks[0]) if _tasks else None
            _tool_specs = [_spec_to_dict(s) for s in (probe.list_tools() if probe else [])]
            if probe is not None and hasattr(probe, "close"):
                probe.close()
            _session_factory = lambda **row: env.session(task=row)  # noqa: E731
        self._factory, self._tool_specs, self._tasks = _session_factory, _tool_specs or [], _tasks or []
        self._cls = make_environment_class(self._factory, self._tool_specs)

    @classmethod
    def from_session_factory(cls, session_factory, tool_specs, tasks):
        return cls(_session_factory=session_factory, _tool_specs=tool_specs, _tasks=tasks)

    @property
    def dataset(self) -> list[dict]:
        rows = []
        for t in self._tasks:
            p = t.get("prompt", "")
            rows.append({**t, "prompt": p if isinstance(p, list) else [{"role": "user", "content": str(p)}]})
        return rows

    @property
    def environment_factory(self):
        return self._cls

    @property
    def reward_funcs(self):
        return [_outcome_only_reward_func]
