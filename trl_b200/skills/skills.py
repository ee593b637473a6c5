"""Agent-skill installer (role of trl/skills/skills.py:33-353): copies the packaged ``SKILL.md`` folders into
an agent's skills directory (``.claude/skills``, ``.agents/skills``, ``.cursor/skills`` under a project or
the home directory) and removes them again."""
from __future__ import annotations

import os
import shutil

_ROOT = os.path.dirname(os.path.abspath(__file__))
AGENT_DIRS = {"claude": ".claude/skills", "codex": ".agents/skills", "cursor": ".cursor/skills", "opencode": ".opencode/skills"}


def list_skills() -> list[str]:
    return sorted(d for d in os.listdir(_ROOT) if os.path.isfile(os.path.join(_ROOT, d, "SKILL.md")))


def _target(agent: str | None, target: str | None, scope: str) -> str:
    if target:
        return os.path.abspath(target)
    if agent not in AGENT_DIRS:
        raise ValueError(f"unknown agent {agent!r}; expected one of {sorted(AGENT_DIRS)} or --target")
    base = os.path.expanduser("~") if scope == "global" else os.getcwd()
    return os.path.join(base, AGENT_DIRS[agent])


def install_skill(name: str, agent: str | None = None, target: str | None = None, scope: str = "project",
                  force: bool = False) -> str:
    if name not in list_skills():
        raise ValueError(f"unknown skill {name!r}; available: {list_skills()}")
    dst = os.path.join(_target(agent, target, scope), name)
    if os.path.exists(dst):
        if not force:
            raise FileExistsError(f"{dst} already exists (use --force to overwrite)")
        shutil.rmtree(dst)
    shutil.copytree(os.path.join(_ROOT, name), dst)
    return dst


def uninstall_skill(name: str, agent: str | None = None, target: str | None = None, scope: str = "project") -> bool:
    dst = os.path.join(_target(agent, target, scope), name)
    if os.path.isdir(dst):
        shutil.rmtree(dst)
        return True
    return False
