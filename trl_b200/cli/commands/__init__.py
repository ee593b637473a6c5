from .base import Command, CommandContext
from .env import EnvCommand
from .skills import SkillsCommand
from .training import TrainingCommand
from .vllm_serve import VllmServeCommand

__all__ = ["Command", "CommandContext", "EnvCommand", "SkillsCommand", "TrainingCommand", "VllmServeCommand"]
