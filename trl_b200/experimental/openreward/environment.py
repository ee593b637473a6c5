"""Rollout environment over an ORS session (trl/experimental/openreward/environment.py: _RolloutEnvironment :104-303,
tool binding :305-367).

A session object offers ``list_tools()`` and ``call_tool(name, arguments)`` and reports a reward when the episode
ends.  ``make_environment_class`` builds a class whose public methods are the session's tools (with signatures and
docstrings derived from the tool specs, so the chat template can advertise them) and whose ``reward`` is the sum of
the rewards the calls returned."""
from __future__ import annotations

import inspect
from typing import Any, Callable

_PY_TYPES = {"string": str, "integer": int, "number": float, "boolean": bool, "array": list, "object": dict}


def _import_openreward():
    try:
        import openreward

        return openreward
    except ImportError as e:
        raise ImportError("OpenRewardSpec needs the `openreward` client package and network access to an ORS server") from e


def _spec_to_dict(spec: Any) -> dict[str, Any]:
    if isinstance(spec, dict):
        return spec
    return {"name": getattr(spec, "name"), "description": getattr(spec, "description", ""),
            "input_schema": getattr(spec, "input_schema", None) or getattr(spec, "parameters", {}) or {}}


def _join_text_blocks(blocks) -> str:
    if isinstance(blocks, str):
        return blocks
    out = []
    for b in blocks or []:
        out.append(b.get("text", "") if isinstance(b, dict) else str(getattr(b, "text", b)))
    return "\n".join(x for x in out if x)


class _RolloutEnvironment:
    """One episode: opened by ``reset``, driven through tool methods, closed (and scored) at the end."""

    _session_factory: Callable[..., Any] = None
    _tool_specs: list = []

    def __init__(self):
        self._session, self._reward, self._done = None, 0.0, False

    def reset(self, **row) -> str | None:
        self.close()
        self._session = type(self)._session_factory(**row)
        self._reward, self._done = 0.0, False
        first = getattr(self._session, "initial_observation", None)
        return _join_text_blocks(first() if callable(first) else first) or None

    def _call(self, name: str, arguments: dict) -> str:
        if self._done:
            return "error: the episode has ended"
        out = self._session.call_tool(name, arguments)
        r = out.get("reward") if isinstance(out, dict) else getattr(out, "reward", None)
        if r is not None:
            self._reward += float(r)
        fin = out.get("finished") if isinstance(out, dict) else getattr(out, "finished", False)
        self._done = bool(fin)
        blocks = out.get("blocks", out.get("content")) if isinstance(out, dict) else getattr(out, "blocks", None)
        return _join_text_blocks(blocks)

    @property
    def reward(self) -> float:
        return self._reward

    def close(self):
        if self._session is not None and hasattr(self._session, "close"):
            self._session.close()
        self._session = None


def _bind_tool_method(cls: type, spec: dict[str, Any]) -> None:
    name = spec["name"]
    props = (spec.get("input_schema") or {}).get("properties", {})
    required = set((spec.get("input_schema") or {}).get("required", []))
    params = [inspect.Parameter("self", inspect.Parameter.POSITIONAL_OR_KEYWORD)]
    doc = [spec.get("description", "") or name, "", "Args:"]
    for pname, pdef in props.items():
        ann = _PY_TYPES.get(pdef.get("type", "string"), str)
        default = inspect.Parameter.empty if pname in required else pdef.get("default", None)
        params.append(inspect.Parameter(pname, inspect.Parameter.KEYWORD_ONLY if default is not inspect.Parameter.empty
                                        else inspect.Parameter.POSITIONAL_OR_KEYWORD, default=default, annotation=ann))
        doc.append(f"    {pname}: {pdef.get('description', pname)}")
    params.sort(key=lambda p: p.kind)

    def method(self, *args, **kwargs):
        bound = method.__signature__.bind(self, *args, **kwargs)
        arguments = {k: v for k, v in bound.arguments.items() if k != "self" and v is not None}
        return self._call(name, arguments)
    method.__name__, method.__doc__ = name, "\n".join(doc)
    method.__signature__ = inspect.Signature(params, return_annotation=str)
    method.__annotations__ = {p.name: p.annotation for p in params[1:]} | {"return": str}
    setattr(cls, name, method)


def make_environment_class(session_factory: Callable[..., Any], tool_specs: list) -> type:
    cls = type("OpenRewardEnvironment", (_RolloutEnvironment,), {})
    cls._session_factory = staticmethod(session_factory)
    cls._tool_specs = [_spec_to_dict(s) for s in tool_specs]
    for s in cls._tool_specs:
        _bind_tool_method(cls, s)
    return cls
