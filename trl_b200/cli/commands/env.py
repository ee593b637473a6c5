"""``trl env`` (counterpart of trl/cli/commands/env.py)."""
from .base import Command, CommandContext


class EnvCommand(Command):
    name, help = "env", "Print versions of the framework, its dependencies and the GPUs"

    def run(self, args, context: CommandContext) -> int:
        from ...scripts.env import print_env

        print_env()
        return 0
