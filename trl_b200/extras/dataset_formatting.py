"""Legacy dataset-formatting entry points (trl/extras/dataset_formatting.py): conversion now lives in ``data_utils``
(``maybe_convert_to_chatml``, ``apply_chat_template``); this module only keeps the import path alive."""
from ..data_utils import apply_chat_template, maybe_convert_to_chatml

__all__ = ["apply_chat_template", "maybe_convert_to_chatml"]
