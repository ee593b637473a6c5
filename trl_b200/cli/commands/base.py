"""Command protocol of the CLI (counterpart of trl/cli/commands/base.py:20-62)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class CommandContext:
    argv: list[str] = field(default_factory=list)

    def argv_after(self, token: str) -> list[str]:
        """Arguments that follow the first occurrence of ``token`` (the sub-command name)."""
        return self.argv[self.argv.index(token) + 1:] if token in self.argv else list(self.argv)


class Command:
    name: str = ""
    help: str = ""

    def register(self, subparsers):
        return subparsers.add_parser(self.name, help=self.help, add_help=False)

    def run(self, args, context: CommandContext) -> int:
        raise NotImplementedError
