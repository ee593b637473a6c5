"""One object that wires a task suite into a trainer (trl/experimental/harbor/_spec.py: HarborSpec :114-216).

``HarborSpec(path).dataset`` yields rows ``{"prompt": [...], "task_dir": ...}`` for every ``tasks/<name>/`` directory
(``instruction.md``, optional ``task.toml`` metadata, ``environment/``, ``tests/test.sh``); ``environment_factory``
builds the environment class; ``reward_funcs`` reads the verifier outcome from the rollout's environment."""
from __future__ import annotations

import importlib
import importlib.util
import os
from functools import cached_property
from pathlib import Path
from typing import Any

from ._env import AGENTS, HarborBashEnv, HarborEnv


def _outcome_reward_func(environments=None, environment_reward=None, **_) -> list[float]:
    if environment_reward is not None:
        return [float(r) for r in environment_reward]
    return [float(env.reward) if env is not None else 0.0 for env in (environments or [])]


def _resolve_agent(agent) -> type:
    if isinstance(agent, type) and issubclass(agent, HarborEnv):
        return agent
    if isinstance(agent, str) and agent in AGENTS:
        return AGENTS[agent]
    if isinstance(agent, str) and ":" in agent:
        mod, cls = agent.rsplit(":", 1)
        if mod.endswith(".py"):
            spec = importlib.util.spec_from_file_location(Path(mod).stem, mod)
            m = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(m)
        else:
            m = importlib.import_module(mod)
        return getattr(m, cls)
    raise ValueError(f"Unknown agent {agent!r}: use a built-in name ({sorted(AGENTS)}), 'module:Class', 'file.py:Class' "
                     f"or a HarborEnv subclass")


def _read_task_meta(task_dir: Path) -> dict[str, Any]:
    f = task_dir / "task.toml"
    if not f.exists():
        return {}
    import tomllib

    with open(f, "rb") as fh:
        data = tomllib.load(fh)
    return {k: v for k, v in data.get("metadata", data).items() if isinstance(v, (str, int, float, bool))}


class HarborSpec:
    def __init__(self, dataset: str, *, agent="bash", environment_type: str = "docker", num_tasks: int | None = None,
                 indices: list[int] | None = None, include_metadata: bool = True) -> None:
        if num_tasks is not None and indices is not None:
            raise ValueError("Provide num_tasks or indices, not both.")
        self._dataset, self._environment_type = dataset, environment_type
        self._num_tasks, self._indices, self._include_metadata = num_tasks, indices, include_metadata
        self._env_cls = _resolve_agent(agent)

    @cached_property
    def _task_dirs(self) -> list[Path]:
        root = Path(self._dataset)
        if not root.exists():
            raise FileNotFoundError(f"{self._dataset}: not a local task tree (Hub repositories need network access)")
        base = root / "tasks" if (root / "tasks").is_dir() else root
        dirs = sorted(d for d in base.iterdir() if (d / "instruction.md").exists())
        if self._indices is not None:
            dirs = [dirs[i] for i in self._indices]
        elif self._num_tasks is not None:
            dirs = dirs[: self._num_tasks]
        return dirs

    @cached_property
    def dataset(self) -> list[dict]:
        rows = []
        for d in self._task_dirs:
            text = (d / "instruction.md").read_text().strip() + self._env_cls.PROMPT_SUFFIX
            row = {"prompt": [{"role": "user", "content": text}], "task_dir": str(d)}
            if self._include_metadata:
                row.update(_read_task_meta(d))
            rows.append(row)
        return rows

    @property
    def environment_factory(self):
        cls, kind = self._env_cls, self._environment_type
        return lambda: cls(environment_type=kind)

    @property
    def reward_funcs(self):
        return [_outcome_reward_func]
