"""Small helpers used across the package: nested attribute lookup, signature-aware calls, pattern file copies, a
host/rank tag for logs, LoRA target discovery on the owned decoder, alignment of ragged per-token values to a label
mask, and loaders for image inputs.

Parity: reference ``src/twinkle/utils/utils.py:10-125``, ``utils/transformers_utils.py:12-47, 76-137, 161-205``,
``utils/vision_tools.py:17-54``."""
from __future__ import annotations

import fnmatch
import inspect
import os
import re
import shutil
from functools import lru_cache
from io import BytesIO
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Union


def deep_getattr(obj: Any, attr: str, default: Any = None) -> Any:
    """``deep_getattr(m, 'a.b.c')``; mappings are indexed, objects read by attribute; a missing link gives ``default``."""
    for name in attr.split('.'):
        if obj is None:
            return default
        obj = obj.get(name, default) if isinstance(obj, dict) else getattr(obj, name, default)
    return obj


@lru_cache(maxsize=None)
def signature_info(fn: Callable):
    """(accepts ``**kwargs``, frozenset of parameter names)."""
    sig = inspect.signature(fn)
    return any(p.kind is inspect.Parameter.VAR_KEYWORD for p in sig.parameters.values()), frozenset(sig.parameters)


def has_signature_parameter(fn: Callable, name: str) -> bool:
    return name in signature_info(fn)[1]


def call_with_supported_kwargs(fn: Callable, *args, **kwargs):
    """Call ``fn`` with the keyword arguments it declares (all of them when it takes ``**kwargs``)."""
    any_kw, names = signature_info(fn)
    if not any_kw:
        kwargs = {k: v for k, v in kwargs.items() if k in names}
    return fn(*args, **kwargs)


def copy_files_by_pattern(source_dir: str, dest_dir: str, patterns: Union[str, Sequence[str]],
                          exclude_patterns: Union[str, Sequence[str], None] = None) -> List[str]:
    """Copy the files under ``source_dir`` whose relative path or base name matches one of ``patterns`` (shell
    wild cards) and none of ``exclude_patterns``, keeping sub-directories. Existing files are left alone. Returns the
    relative paths copied — used to carry tokenizer / config files beside saved weights."""
    pats = [patterns] if isinstance(patterns, str) else list(patterns)
    excl = [exclude_patterns] if isinstance(exclude_patterns, str) else list(exclude_patterns or [])
    copied = []
    for root, _dirs, files in os.walk(source_dir):
        for f in files:
            rel = os.path.relpath(os.path.join(root, f), source_dir)
            hit = lambda ps: any(fnmatch.fnmatch(rel, p) or fnmatch.fnmatch(f, p) for p in ps)  # noqa: E731
            if not hit(pats) or hit(excl):
                continue
            dst = os.path.join(dest_dir, rel)
            if os.path.exists(dst):
                continue
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            shutil.copy2(os.path.join(source_dir, rel), dst)
            copied.append(rel)
    return sorted(copied)


def get_runtime_meta() -> str:
    """``host=… ip=… rank=r/w pid=… python=…`` — prefixed to error notifications so that a report names its source."""
    import platform
    import socket
    host, ip = 'unknown', 'unknown'
    try:
        host = socket.gethostname()
        ip = socket.gethostbyname(host)
    except OSError:
        pass
    return (f"host={host} ip={ip} rank={os.environ.get('RANK', '?')}/{os.environ.get('WORLD_SIZE', '?')} "
            f"local_rank={os.environ.get('LOCAL_RANK', '?')} pid={os.getpid()} python={platform.python_version()}")


# ------------------------------------------------------------------------------------------------- model helpers
def get_llm_model(model: Any):
    """The decoder underneath a wrapper: follows ``.model`` / ``.module`` links until an object with ``layers``."""
    seen = set()
    while model is not None and id(model) not in seen and not hasattr(model, 'layers'):
        seen.add(id(model))
        model = getattr(model, 'model', None) or getattr(model, 'module', None)
    return model


def find_all_linears(model: Any, extra_ignore: Iterable[str] = ()) -> List[str]:
    """Short names (``q_proj``-style suffixes) of every LoRA-targetable projection of the decoder — what
    ``target_modules='all-linear'`` expands to. Fused projections are reported by their parts; the output head, the MoE
    router and classifier / value heads are excluded, as are adapter tensors themselves."""
    ignore = {'lm_head', 'gate', 'score', 'v_head', 'classifier', 'lora_A', 'lora_B', 'base_layer', *extra_ignore}
    dec = get_llm_model(model) or model
    names: set = set()
    mods = dec.lora_modules() if hasattr(dec, 'lora_modules') else [(n, m) for n, m in dec.named_modules() if 'linear' in type(m).__name__.lower()]
    for name, m in mods:
        short = name.rsplit('.', 1)[-1]
        parts = [p[0] for p in getattr(m, 'parts', None) or []] or [short]
        if type(m).__name__ == 'Experts':
            parts = ['gate_up_proj', 'down_proj']
        names.update(p for p in parts if p not in ignore and short not in ignore)
    return sorted(names)


def align_logps_to_mask(ragged: Any, mask, dtype):
    """Per-token values given per sample (ragged lists, scalars, or a tensor) → a dense ``[B, S]`` tensor with the
    values written at the positions where ``mask`` is set, in order, zeros elsewhere. A tensor already of shape
    ``[B, S]`` passes through. Returns ``None`` for inputs that are neither."""
    import torch
    b, s = mask.shape
    if isinstance(ragged, torch.Tensor):
        t = ragged.to(device=mask.device, dtype=dtype)
        if t.shape == (b, s):
            return t
        ragged = [t[i] for i in range(min(b, t.shape[0]))]
    if not isinstance(ragged, (list, tuple)):
        return None
    out = torch.zeros((b, s), dtype=dtype, device=mask.device)
    for i, sample in enumerate(ragged[:b]):
        pos = mask[i].nonzero(as_tuple=True)[0]
        if pos.numel() == 0:
            continue
        if isinstance(sample, (int, float)):
            out[i, pos] = float(sample)
            continue
        vals = torch.as_tensor(sample, dtype=dtype, device=mask.device).flatten()
        n = min(pos.numel(), vals.numel())
        out[i, pos[:n]] = vals[:n]
    return out


# ------------------------------------------------------------------------------------------------- vision inputs
_DATA_URL = re.compile(r'^data:[\w/+.-]+;base64,', re.I)


def load_mm_file(path: Any):
    """Bytes of a multimodal input as a ``BytesIO``: raw bytes, a ``data:`` URL or bare base64 text, an ``http(s)``
    URL (needs network) or a local path. Other objects (already-decoded images, arrays) are returned unchanged."""
    if isinstance(path, bytes):
        return BytesIO(path)
    if not isinstance(path, str):
        return path
    p = path.strip()
    # which kinds of string sources are honoured: a server that takes requests from tenants sets TWINKLE_MM_SOURCES=data so
    # that a request cannot make it read its own files or fetch URLs on the tenant's behalf
    allowed = {x.strip() for x in os.environ.get('TWINKLE_MM_SOURCES', 'data,file,http').split(',') if x.strip()}
    if p.startswith(('http://', 'https://')):
        if 'http' not in allowed:
            raise PermissionError('fetching images from URLs is disabled here (TWINKLE_MM_SOURCES)')
        import requests
        r = requests.get(p, timeout=float(os.environ.get('TWINKLE_MM_TIMEOUT', '20')))
        r.raise_for_status()
        return BytesIO(r.content)
    if len(p) < 4096 and not p.startswith('data:') and os.path.exists(p):
        if 'file' not in allowed:
            raise PermissionError('reading images from local paths is disabled here (TWINKLE_MM_SOURCES)')
        with open(p, 'rb') as f:
            return BytesIO(f.read())
    import base64
    import binascii
    try:
        return BytesIO(base64.b64decode(_DATA_URL.sub('', p), validate=True))
    except (binascii.Error, ValueError):
        raise FileNotFoundError(f'not a file, URL or base64 payload: {p[:80]!r}') from None


def load_image(image: Any):
    """A PIL RGB image from any :func:`load_mm_file` source (or a PIL image, returned in RGB)."""
    from PIL import Image
    src = load_mm_file(image)
    if isinstance(src, BytesIO):
        src = Image.open(src)
    return src.convert('RGB') if getattr(src, 'mode', 'RGB') != 'RGB' else src


def image_to_data_url(image: Any) -> Any:
    """What travels in a JSON request for an image: strings (paths on the server, URLs, base64) pass; bytes, PIL images and
    ``[C, H, W]`` / ``[H, W, C]`` arrays in 0…255 become a PNG ``data:`` URL that :func:`load_mm_file` reads back."""
    import base64
    if isinstance(image, str):
        return image
    if isinstance(image, bytes):
        return 'data:application/octet-stream;base64,' + base64.b64encode(image).decode()
    from PIL import Image
    if not isinstance(image, Image.Image):
        import numpy as np
        arr = image.detach().cpu().numpy() if hasattr(image, 'detach') else np.asarray(image)
        if arr.ndim == 3 and arr.shape[0] in (1, 3) and arr.shape[-1] not in (1, 3):
            arr = arr.transpose(1, 2, 0)
        if arr.ndim == 3 and arr.shape[-1] == 1:
            arr = arr[..., 0]
        image = Image.fromarray(np.clip(np.rint(arr), 0, 255).astype('uint8'))
    buf = BytesIO()
    image.save(buf, format='PNG')
    return 'data:image/png;base64,' + base64.b64encode(buf.getvalue()).decode()
