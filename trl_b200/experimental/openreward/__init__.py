"""OpenReward (ORS) environments as rollout environments (trl/experimental/openreward/__init__.py)."""
from ._spec import OpenRewardSpec
from .environment import make_environment_class

__all__ = ["OpenRewardSpec", "make_environment_class"]
