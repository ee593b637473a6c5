"""Lazy exports for a package ``__init__`` through the module-level ``__getattr__`` / ``__dir__`` hooks (PEP 562).

``import trl_b200`` stays cheap; ``trl_b200.SFTTrainer`` imports only the submodule that defines the class.  The
reference gets the same effect by swapping a ``ModuleType`` subclass into ``sys.modules`` (trl/_lazy_module.py:22-79);
here the package keeps its real module object, so pickling, ``importlib.reload`` and ``__spec__`` need no special care.
"""
from __future__ import annotations

import importlib
from typing import Callable


def lazy_exports(package: str, structure: dict[str, list[str]], namespace: dict) -> tuple[Callable, Callable, list[str]]:
    """Builds ``(__getattr__, __dir__, __all__)`` for ``package``.

    ``structure`` maps a submodule path relative to the package (``"trainer.sft_trainer"``) to the names it exports.
    A resolved attribute is cached in ``namespace`` (the package's ``globals()``), so the hook runs once per name.
    """
    owner = {name: sub for sub, names in structure.items() for name in names}
    exported = sorted(set(owner) | {sub.split(".")[0] for sub in structure})

    def _load(sub: str):
        try:
            return importlib.import_module(f"{package}.{sub}")
        except ModuleNotFoundError as e:
            if e.name is not None and e.name.startswith(package):
                raise AttributeError(f"module {package!r} has no attribute {sub!r}") from None
            raise

    def __getattr__(name: str):
        if name in owner:
            value = getattr(_load(owner[name]), name)
        elif name.startswith("__"):
            raise AttributeError(f"module {package!r} has no attribute {name!r}")
        else:
            value = _load(name)  # a submodule, listed or not
        namespace[name] = value
        return value

    def __dir__():
        return sorted(set(namespace) | set(exported))

    return __getattr__, __dir__, exported
