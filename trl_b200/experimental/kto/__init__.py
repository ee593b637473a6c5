"""Former experimental location of KTO (trl/experimental/kto/__init__.py): re-exports the stable classes."""
import warnings

from ...trainer.kto_trainer import KTOConfig, KTOTrainer

warnings.warn("trl_b200.experimental.kto is deprecated: import KTOConfig / KTOTrainer from trl_b200.", FutureWarning,
              stacklevel=2)

__all__ = ["KTOConfig", "KTOTrainer"]
