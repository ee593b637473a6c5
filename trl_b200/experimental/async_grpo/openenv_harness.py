"""Adapter from environment objects to rollout tool calls (trl/experimental/async_grpo/openenv_harness.py:30-391).

An environment exposes ``reset(**row) -> observation text | None`` and public methods that the model may call as
tools; the harness instantiates one environment per rollout, lists its tools and dispatches parsed calls."""
from __future__ import annotations

import inspect
from typing import Any, Callable


class EnvironmentHarness:
    def __init__(self, environment_factory: Callable[[], Any]):
        self.factory = environment_factory

    def open(self, row: dict):
        env = self.factory()
        obs = env.reset(**{k: v for k, v in row.items() if k != "prompt"}) if hasattr(env, "reset") else None
        return env, obs

    @staticmethod
    def tools_of(env) -> dict[str, Callable]:
        return {n: m for n, m in inspect.getmembers(env, predicate=inspect.ismethod)
                if not n.startswith("_") and n not in ("reset", "close")}

    def call(self, env, name: str, arguments: dict) -> str:
        tools = self.tools_of(env)
        if name not in tools:
            return f"error: unknown tool {name!r}"
        try:
            return str(tools[name](**arguments))
        except Exception as e:  # the model sees the failure text and may retry
            return f"error: {e}"
