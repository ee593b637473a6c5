"""``trl sft|dpo|grpo|kto|reward|rloo`` (counterpart of trl/cli/commands/training.py:34-72): the script's own arguments plus
``--num_processes`` / ``--accelerate_config``; one process per GPU through ``torch.distributed.run``."""
from __future__ import annotations

from .base import Command, CommandContext


class TrainingCommand(Command):
    def __init__(self, name: str):
        self.name, self.help = name, f"Run the {name.upper()} training script"

    def run(self, args, context: CommandContext) -> int:
        from ..main import run_training

        return run_training(self.name, context.argv_after(self.name))
