"""Reversible model patches.

Parity: reference ``src/twinkle/patch/__init__.py:9-30`` / ``patch/base.py``:
``Patch.__call__(model, **kw)`` applies, ``unpatch`` reverts; ``apply_patch``
resolves a name/class/instance; ``apply_context`` applies for the duration of
a ``with`` block.  Concrete patches here act on the owned decoder:
``FusedCEPatch`` (head → identity so the loss receives hidden states and fuses
the lm_head GEMM with the cross-entropy; reference ``transformers_fused_ce.py:
76-126``), ``EmbeddingPatch`` (switch the task to pooled embeddings;
``transformers_emb.py:56-90``), ``NoSplitModulesPatch`` (no-op marker kept for
API parity).
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Any


class Patch:

    def __call__(self, model, **kwargs):  # pragma: no cover
        raise NotImplementedError

    def unpatch(self, model) -> None:
        pass


class FusedCEPatch(Patch):

    def __call__(self, model, **kwargs):
        self._prev = getattr(model, 'task', None)
        model.task = 'fused_lm_ce'
        return self

    def unpatch(self, model):
        model.task = self._prev


class EmbeddingPatch(Patch):

    def __call__(self, model, **kwargs):
        self._prev = getattr(model, 'task', None)
        model.task = 'embedding'
        return self

    def unpatch(self, model):
        model.task = self._prev


class NoSplitModulesPatch(Patch):

    def __call__(self, model, **kwargs):
        return self


patch_mapping = {'FusedCEPatch': FusedCEPatch, 'TransformersFusedCEPatch': FusedCEPatch, 'EmbeddingPatch': EmbeddingPatch,
                 'TransformersEmbeddingPatch': EmbeddingPatch, 'MegatronEmbeddingPatch': EmbeddingPatch,
                 'NoSplitModulesPatch': NoSplitModulesPatch}


def apply_patch(model, patch_cls, **kwargs) -> Patch:
    if isinstance(patch_cls, str):
        patch_cls = patch_mapping[patch_cls]
    patch = patch_cls() if isinstance(patch_cls, type) else patch_cls
    patch(model, **kwargs)
    return patch


@contextmanager
def apply_context(model, patch_cls, **kwargs):
    p = apply_patch(model, patch_cls, **kwargs)
    try:
        yield p
    finally:
        p.unpatch(model)
