"""Training scripts behind the ``trl`` command line and their shared argument / dataset helpers
(trl/scripts/__init__.py exports the same five names)."""
from .utils import DatasetMixtureConfig, ScriptArguments, TrlParser, get_dataset, init_zero_verbose

__all__ = ["DatasetMixtureConfig", "ScriptArguments", "TrlParser", "get_dataset", "init_zero_verbose"]
