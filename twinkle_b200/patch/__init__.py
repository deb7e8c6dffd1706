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


class Qwen3ChatTemplate(Patch):
    """Repairs the reasoning split of the Qwen3 / Qwen3.5 chat template held by a HF tokenizer (``tokenizer.chat_template``
    is Jinja text). The shipped template takes everything before the LAST ``</think>`` as reasoning even when the content
    never opened a ``<think>`` block, and drops text between several closing tags; a re-rendered conversation then differs
    from the tokens that were sampled, which breaks token-exact multi-turn rollouts. The patched block requires the
    content to start with ``<think>`` and splits at the first closing tag only. Tokenizers whose template does not
    contain the block are left alone (``applied`` tells). Reference: ``patch/qwen3_chat_template.py:62-92``."""

    _BLOCK = None

    @classmethod
    def _pattern(cls):
        import re
        if cls._BLOCK is None:
            cls._BLOCK = re.compile(
                r"(?P<ind>[ \t]*)\{%-\s*if\s+'</think>'\s+in\s+content\s*%\}\s*"
                r"\{%-\s*set\s+reasoning_content\s*=\s*content\.split\('</think>'\)\[0\][^%]*?%\}\s*"
                r"\{%-\s*set\s+content\s*=\s*content\.split\('</think>'\)\[-1\][^%]*?%\}\s*"
                r"\{%-\s*endif\s*%\}")
        return cls._BLOCK

    def __call__(self, tokenizer, **kwargs):
        self._prev, self.applied = getattr(tokenizer, 'chat_template', None), False
        if isinstance(self._prev, str):
            def fixed(m):
                i = m.group('ind')
                return (f"{i}{{%- if content.startswith('<think>') and '</think>' in content %}}\n"
                        f"{i}    {{%- set _parts = content.split('</think>', 1) %}}\n"
                        f"{i}    {{%- set reasoning_content = _parts[0].split('<think>', 1)[1].strip('\\n') %}}\n"
                        f"{i}    {{%- set content = _parts[1].lstrip('\\n') %}}\n"
                        f"{i}{{%- endif %}}")
            new, n = self._pattern().subn(fixed, self._prev)
            if n:
                tokenizer.chat_template, self.applied = new, True
        return self

    def unpatch(self, tokenizer):
        if self.applied:
            tokenizer.chat_template = self._prev


class Qwen3AllowToolTailTemplate(Patch):
    """Lets the Qwen3 chat template render a message list that has no user query before its tool messages (a
    continuation that starts at a tool result): the template's ``raise_exception('No user query found in messages.')``
    becomes a comment. Reference: ``patch/qwen3_chat_template.py:94-124``."""

    def __call__(self, tokenizer, **kwargs):
        import re
        self._prev, self.applied = getattr(tokenizer, 'chat_template', None), False
        if isinstance(self._prev, str):
            new, n = re.subn(r"\{\{-\s*raise_exception\('No user query found in messages\.'\)\s*\}\}",
                             '{#- no user query before the tool messages: allowed -#}', self._prev)
            if n:
                tokenizer.chat_template, self.applied = new, True
        return self

    def unpatch(self, tokenizer):
        if self.applied:
            tokenizer.chat_template = self._prev


patch_mapping = {'FusedCEPatch': FusedCEPatch, 'TransformersFusedCEPatch': FusedCEPatch, 'EmbeddingPatch': EmbeddingPatch,
                 'TransformersEmbeddingPatch': EmbeddingPatch, 'MegatronEmbeddingPatch': EmbeddingPatch,
                 'NoSplitModulesPatch': NoSplitModulesPatch, 'Qwen3ChatTemplate': Qwen3ChatTemplate,
                 'Qwen3AllowToolTailTemplate': Qwen3AllowToolTailTemplate}


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
