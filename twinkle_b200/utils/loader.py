"""Resolve ``str | type | instance`` into an instance.

Parity: reference ``src/twinkle/utils/loader.py:16-74`` and ``utils/unsafe.py``:
component selection by string everywhere; ``ms://`` / ``hf://`` plugin ids are
imported from a local directory only when ``TWINKLE_TRUST_REMOTE_CODE=1``.
"""
from __future__ import annotations

import importlib.util
import inspect
import os
import sys
from collections.abc import Mapping
from types import ModuleType
from typing import Any, Optional, Type, Union


def trust_remote_code() -> bool:
    return os.environ.get('TWINKLE_TRUST_REMOTE_CODE', '0').lower() in ('1', 'true', 'yes')


def any_callable(args: Any) -> bool:
    """Whether a (nested) argument structure carries a callable or a class."""
    if isinstance(args, Mapping):
        return any(any_callable(a) for a in args.values())
    if isinstance(args, (tuple, list, set, frozenset)):
        return any(any_callable(a) for a in args)
    return callable(args) or isinstance(args, type)


def check_unsafe(*args, **kwargs) -> None:
    """Safe mode of a served deployment (reference ``utils/unsafe.py:7-23``, applied in ``infra/__init__.py:569, 738``):
    with ``TWINKLE_TRUST_REMOTE_CODE=0`` a call that would ship a callable or a class to a worker is refused — components
    are then named by string only.  Unset (the default for local use) and ``1`` allow them; loading plugin *code* from a
    directory or a hub id additionally needs the explicit ``1`` (:func:`trust_remote_code`)."""
    if os.environ.get('TWINKLE_TRUST_REMOTE_CODE', '').lower() in ('0', 'false', 'no') and (any_callable(args) or any_callable(kwargs)):
        raise ValueError('callables and classes are not accepted as arguments in safe mode (TWINKLE_TRUST_REMOTE_CODE=0): '
                         'name the component by string')


class Plugin:

    @staticmethod
    def load_plugin(plugin_id: str, base: Optional[type] = None) -> type:
        """Import ``__init__.py`` of a plugin directory and return the first
        class deriving from ``base`` that it defines."""
        if not trust_remote_code():
            raise PermissionError('loading plugin code requires TWINKLE_TRUST_REMOTE_CODE=1')
        path = plugin_id
        for prefix in ('ms://', 'hf://'):
            if path.startswith(prefix):
                from ..hub import HubOperation
                path = HubOperation.download_model(plugin_id)
        init = os.path.join(path, '__init__.py')
        if not os.path.isfile(init):
            raise FileNotFoundError(f'plugin {plugin_id!r}: no __init__.py under {path}')
        name = 'twinkle_plugin_' + str(abs(hash(os.path.abspath(path))))
        spec = importlib.util.spec_from_file_location(name, init)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)  # type: ignore[union-attr]
        for _, obj in inspect.getmembers(mod, inspect.isclass):
            if obj.__module__ == name and (base is None or (issubclass(obj, base) and obj is not base)):
                return obj
        raise ImportError(f'plugin {plugin_id!r} defines no subclass of {base}')


def construct_class(spec: Union[str, Type, Any], base: Optional[type], namespace: Union[ModuleType, dict, None], **init_kwargs):
    """``spec`` may be an instance (returned as is), a class (instantiated), a
    name looked up in ``namespace`` (module or dict), or a plugin id."""
    if spec is None:
        return None
    if isinstance(spec, str):
        table = namespace if isinstance(namespace, dict) else (vars(namespace) if namespace is not None else {})
        if spec in table:
            cls = table[spec]
        elif os.path.isdir(spec) or spec.startswith(('ms://', 'hf://')):
            cls = Plugin.load_plugin(spec, base)
        else:
            raise ValueError(f'unknown component {spec!r}; known: {sorted(k for k, v in table.items() if inspect.isclass(v))[:40]}')
        return cls(**init_kwargs) if inspect.isclass(cls) else cls
    if inspect.isclass(spec):
        return spec(**init_kwargs)
    return spec
