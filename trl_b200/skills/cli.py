"""``trl skills {list,install,uninstall}`` (role of trl/skills/cli.py:26-199)."""
from __future__ import annotations

import argparse

from .skills import AGENT_DIRS, install_skill, list_skills, uninstall_skill


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trl skills")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("list")
    for name in ("install", "uninstall"):
        p = sub.add_parser(name)
        p.add_argument("skill")
        p.add_argument("--agent", choices=sorted(AGENT_DIRS))
        p.add_argument("--target")
        p.add_argument("--scope", choices=["project", "global"], default="project")
        if name == "install":
            p.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    if a.cmd == "list":
        for s in list_skills():
            print(s)
        return 0
    if a.cmd == "install":
        print(install_skill(a.skill, a.agent, a.target, a.scope, a.force))
        return 0
    print("removed" if uninstall_skill(a.skill, a.agent, a.target, a.scope) else "not installed")
    return 0
