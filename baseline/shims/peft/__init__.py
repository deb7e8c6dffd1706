"""Import shim for the third-party ``peft`` package, which is not installed on this image and is not in the
offline wheelhouse.

The reference imports ``peft`` at module scope in its model layer, also on code paths that never build an adapter.
For full-parameter training the names below are only used in ``isinstance`` checks, so empty classes are
enough; anything that would actually build or load an adapter raises.  The shim is put on ``sys.path`` by the
reference arm of ``bench.py`` only — the framework itself never imports it.
"""
from __future__ import annotations

__version__ = '0.0.0+shim'


class PeftConfig:
    """Placeholder: never instantiated on the full-parameter path."""

    def __init__(self, *args, **kwargs):
        raise NotImplementedError('peft is not installed; this shim only satisfies imports')


class LoraConfig(PeftConfig):
    pass


class PeftModel:
    """Placeholder used for ``isinstance(model, PeftModel)`` (always False for real modules)."""

    def __init__(self, *args, **kwargs):
        raise NotImplementedError('peft is not installed; this shim only satisfies imports')


def get_peft_model(*args, **kwargs):
    raise NotImplementedError('peft is not installed; this shim only satisfies imports')


def load_peft_weights(*args, **kwargs):
    raise NotImplementedError('peft is not installed; this shim only satisfies imports')
