"""Process-wide compatibility settings applied on package import (counterpart of trl/_compat.py:78-164).

The reference patches third-party libraries (vLLM logging level, a transformers cache class for old peft, the
accelerate ParallelismConfig symbol).  This framework owns its engine and generator, so what is left is environment
hygiene: quiet tokenizers fork warnings and a rendezvous address that resolves on machines whose hostname does not."""
from __future__ import annotations

import os


def apply() -> None:
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "ERROR")  # only matters if a user imports vllm next to this package
    if "MASTER_ADDR" in os.environ and os.environ["MASTER_ADDR"] in ("localhost", ""):
        os.environ["MASTER_ADDR"] = "127.0.0.1"
