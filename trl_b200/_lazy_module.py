"""Attribute-triggered submodule import (role of trl/_lazy_module.py:22-79): ``import trl_b200`` stays cheap,
``trl_b200.SFTTrainer`` imports only what that class needs.  Picklable through ``__reduce__``."""
from __future__ import annotations

import importlib
import os
from types import ModuleType


class _LazyModule(ModuleType):
    def __init__(self, name, module_file, import_structure, module_spec=None, extra_objects=None):
        super().__init__(name)
        self._modules = set(import_structure.keys())
        self._class_to_module = {}
        for key, values in import_structure.items():
            for v in values:
                self._class_to_module[v] = key
        self.__all__ = list(import_structure.keys()) + [v for vs in import_structure.values() for v in vs]
        self.__file__ = module_file
        self.__spec__ = module_spec
        self.__path__ = [os.path.dirname(module_file)]
        self._objects = extra_objects or {}
        self._name = name
        self._import_structure = import_structure

    def __dir__(self):
        return sorted(set(super().__dir__()) | set(self.__all__))

    def __getattr__(self, name: str):
        if name in self._objects:
            return self._objects[name]
        if name in self._class_to_module:
            value = getattr(self._get_module(self._class_to_module[name]), name)
        elif name in self._modules:
            value = self._get_module(name)
        else:
            try:
                value = importlib.import_module("." + name, self.__name__)
            except ModuleNotFoundError:
                raise AttributeError(f"module {self.__name__} has no attribute {name}") from None
        setattr(self, name, value)
        return value

    def _get_module(self, module_name: str):
        try:
            return importlib.import_module("." + module_name, self.__name__)
        except Exception as e:
            raise RuntimeError(f"Failed to import {self.__name__}.{module_name} because of the following error "
                               f"(look up to see its traceback):\n{e}") from e

    def __reduce__(self):
        return (self.__class__, (self._name, self.__file__, self._import_structure))
