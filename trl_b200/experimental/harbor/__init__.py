"""Harbor task suites as rollout environments (trl/experimental/harbor/__init__.py)."""
from ._env import AGENTS, HarborBashEnv, HarborEnv
from ._spec import HarborSpec

__all__ = ["AGENTS", "HarborBashEnv", "HarborEnv", "HarborSpec"]
