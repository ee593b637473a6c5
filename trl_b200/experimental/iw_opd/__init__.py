from .iw_opd_config import IWOPDConfig
from .iw_opd_trainer import IWOPDTrainer

__all__ = ["IWOPDConfig", "IWOPDTrainer"]
