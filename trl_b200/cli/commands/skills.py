"""``trl skills list|install|uninstall`` (counterpart of trl/cli/commands/skills.py)."""
from .base import Command, CommandContext


class SkillsCommand(Command):
    name, help = "skills", "Manage the agent skills shipped with the package"

    def run(self, args, context: CommandContext) -> int:
        from ...skills.cli import main as skills_main

        return skills_main(context.argv_after(self.name))
