"""Kernel registry: swap module classes or functions for registered implementations.

Parity: reference ``src/twinkle/kernel/core.py:20-186`` — ``kernelize(model, mapping)`` where keys are
``nn.Module`` classes (exact type: the instance's ``__class__`` is replaced by a subclass carrying the new
``forward``) or dotted paths (``'pkg.mod.fn'`` / ``'pkg.mod.Class.method'``: the attribute is set), values are
an implementation, a ``{device: impl}`` dict, or a ``HubRef``.  The reference ships Liger (Triton) and Ascend
bundles; the bundle here, ``b200_builtin()``, maps Hugging Face Qwen3 / Llama building blocks onto the
sm_100a kernels of ``twinkle_b200.ops`` so that third-party ``transformers`` models can use them too.
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Union

import torch
import torch.nn as nn


@dataclass(frozen=True)
class HubRef:
    """Reference to a kernel layer in a hub repository, resolved when ``kernelize`` applies it (through the optional
    ``kernels`` package).  Pinned by a ``revision`` (branch / tag / commit) or by a ``version`` number, never by both."""
    repo_id: str
    layer_name: Optional[str] = None
    revision: Optional[str] = None
    version: Optional[int] = None
    backend: Optional[str] = None

    def resolve(self):
        try:
            from kernels import get_kernel  # type: ignore
        except ImportError as e:
            raise ImportError('HubRef needs the `kernels` package, which is not installed') from e
        kw = {k: v for k, v in (('revision', self.revision), ('version', self.version), ('backend', self.backend)) if v is not None}
        mod = get_kernel(self.repo_id, **kw)
        return getattr(mod, self.layer_name) if self.layer_name else mod


def hub(ref: str, layer_name: Optional[str] = None, revision: Optional[str] = None, *, version: Optional[int] = None,
        backend: Optional[str] = None) -> HubRef:
    """``hub('org/repo:LayerName', revision='v1')`` or ``version=2`` (reference ``kernel/core.py:32-49``: exactly one of the
    two pins is required; the part after the last colon names the layer).  ``hub('org/repo', 'LayerName', 'v1')`` is accepted
    as well."""
    if layer_name is None:
        if ':' not in ref:
            raise ValueError(f"a hub kernel is named 'repo_id:LayerName', got {ref!r}")
        ref, layer_name = ref.rsplit(':', 1)
    if (revision is None) == (version is None):
        raise ValueError('exactly one of `revision` and `version` pins a hub kernel')
    return HubRef(ref, layer_name, revision, version, backend)


def resolve_value(value, device: str = 'cuda'):
    if isinstance(value, dict):
        if device in value:
            return resolve_value(value[device], device)
        if 'default' in value:
            return resolve_value(value['default'], device)
        return None
    if isinstance(value, HubRef):
        return value.resolve()
    return value


def _set_dotted(path: str, impl) -> Callable[[], None]:
    parts = path.split('.')
    for i in range(len(parts) - 1, 0, -1):
        try:
            obj = importlib.import_module('.'.join(parts[:i]))
        except ImportError:
            continue
        for p in parts[i:-1]:
            obj = getattr(obj, p)
        old = getattr(obj, parts[-1])
        setattr(obj, parts[-1], impl)
        return lambda: setattr(obj, parts[-1], old)
    raise ImportError(f'cannot resolve {path}')


def kernelize(model: Optional[nn.Module], mapping: Dict[Union[type, str], Any], device: Optional[str] = None):
    """Apply ``mapping``; returns ``(model, undo)`` where ``undo()`` restores everything."""
    device = device or ('cuda' if torch.cuda.is_available() else 'cpu')
    undo = []
    for key, value in mapping.items():
        impl = resolve_value(value, device)
        if impl is None:
            continue
        if isinstance(key, str):
            undo.append(_set_dotted(key, impl))
            continue
        if model is None:
            continue
        for m in model.modules():
            if type(m) is key:
                old_cls = m.__class__
                if isinstance(impl, type):
                    new_cls = type(f'{old_cls.__name__}Kernelized', (impl, old_cls), {}) if not issubclass(impl, old_cls) else impl
                else:
                    new_cls = type(f'{old_cls.__name__}Kernelized', (old_cls, ), {'forward': impl})
                m.__class__ = new_cls
                undo.append(lambda m=m, c=old_cls: setattr(m, '__class__', c))

    def undo_all():
        for u in reversed(undo):
            u()

    return model, undo_all


# ------------------------------------------------------------- built-in bundle
def _rmsnorm_forward(self, hidden_states):
    from .. import ops
    eps = getattr(self, 'variance_epsilon', getattr(self, 'eps', 1e-6))
    return ops.rmsnorm(hidden_states, self.weight, eps, getattr(self, '_kernel_offset', 0.0))


def _gemma_rmsnorm_forward(self, hidden_states):
    from .. import ops
    return ops.rmsnorm(hidden_states, self.weight, getattr(self, 'eps', 1e-6), 1.0)


def _swiglu_mlp_forward(self, x):
    from .. import ops
    g, u = ops.linear(x, self.gate_proj.weight), ops.linear(x, self.up_proj.weight)
    return ops.linear(ops.swiglu(torch.cat([g, u], -1)), self.down_proj.weight)


def _geglu_mlp_forward(self, x):
    from .. import ops
    g, u = ops.linear(x, self.gate_proj.weight), ops.linear(x, self.up_proj.weight)
    return ops.linear(ops.geglu(torch.cat([g, u], -1)), self.down_proj.weight)


def b200_builtin() -> Dict[Any, Any]:
    """HF module classes → sm_100a kernels (only classes importable in this environment are listed)."""
    m: Dict[Any, Any] = {}
    try:
        from transformers.models.qwen3.modeling_qwen3 import Qwen3MLP, Qwen3RMSNorm
        m[Qwen3RMSNorm] = {'cuda': _rmsnorm_forward}
        m[Qwen3MLP] = {'cuda': _swiglu_mlp_forward}
    except Exception:
        pass
    try:
        from transformers.models.llama.modeling_llama import LlamaMLP, LlamaRMSNorm
        m[LlamaRMSNorm] = {'cuda': _rmsnorm_forward}
        m[LlamaMLP] = {'cuda': _swiglu_mlp_forward}
    except Exception:
        pass
    # Gemma family: weight stored as an offset from one ("1 + w"), tanh-GELU gated MLP
    for mod, norm, mlp in (('gemma', 'GemmaRMSNorm', 'GemmaMLP'), ('gemma2', 'Gemma2RMSNorm', 'Gemma2MLP'), ('gemma3', 'Gemma3RMSNorm', 'Gemma3MLP')):
        try:
            pkg = __import__(f'transformers.models.{mod}.modeling_{mod}', fromlist=[norm, mlp])
            m[getattr(pkg, norm)] = {'cuda': _gemma_rmsnorm_forward}
            m[getattr(pkg, mlp)] = {'cuda': _geglu_mlp_forward}
        except Exception:
            pass
    # Qwen3.5 / Qwen3-Next norms use the same "1 + w" form
    for mod, norm in (('qwen3_next', 'Qwen3NextRMSNorm'), ('qwen3_5', 'Qwen3_5RMSNorm')):
        try:
            pkg = __import__(f'transformers.models.{mod}.modeling_{mod}', fromlist=[norm])
            m[getattr(pkg, norm)] = {'cuda': _gemma_rmsnorm_forward}
        except Exception:
            pass
    return m


builtin = liger_builtin = b200_builtin  # the reference's ``liger_builtin()`` slot is filled by our own kernels

__all__ = ['kernelize', 'hub', 'HubRef', 'resolve_value', 'b200_builtin', 'builtin', 'liger_builtin']
