"""Optional-dependency helpers.  Parity: reference
``src/twinkle/utils/import_utils.py`` (``exists``, ``requires``, ``_LazyModule``)."""
from __future__ import annotations

import importlib
import importlib.util
import sys
from types import ModuleType
from typing import Dict, List


def exists(package: str) -> bool:
    try:
        return importlib.util.find_spec(package) is not None
    except (ImportError, ValueError):
        return False


def requires(package: str, hint: str = '') -> None:
    if not exists(package):
        raise ImportError(f"'{package}' is required for this feature but is not installed. {hint}".strip())


class _LazyModule(ModuleType):
    """Module whose public names are imported on first attribute access."""

    def __init__(self, name: str, module_file: str, import_structure: Dict[str, List[str]], module_spec=None):
        super().__init__(name)
        self._modules = set(import_structure)
        self._class_to_module = {c: m for m, cs in import_structure.items() for c in cs}
        self.__all__ = list(import_structure) + [c for cs in import_structure.values() for c in cs]
        self.__file__ = module_file
        self.__spec__ = module_spec
        self.__path__ = [module_file.rsplit('/', 1)[0]]
        self._name = name

    def __dir__(self):
        return sorted(set(super().__dir__()) | set(self.__all__))

    def __getattr__(self, item: str):
        if item in self._modules:
            value = importlib.import_module('.' + item, self._name)
        elif item in self._class_to_module:
            value = getattr(importlib.import_module('.' + self._class_to_module[item], self._name), item)
        else:
            raise AttributeError(f'module {self._name!r} has no attribute {item!r}')
        setattr(self, item, value)
        return value

    def __reduce__(self):
        return importlib.import_module, (self._name, )
