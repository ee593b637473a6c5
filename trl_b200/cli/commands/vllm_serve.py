"""``trl vllm-serve`` (counterpart of trl/cli/commands/vllm_serve.py): starts the in-box rollout server."""
from .base import Command, CommandContext


class VllmServeCommand(Command):
    name, help = "vllm-serve", "Serve a model with the rollout engine (generate / chat / weight-update routes)"

    def run(self, args, context: CommandContext) -> int:
        from ...scripts.rollout_serve import main as serve_main

        return serve_main(context.argv_after(self.name))
