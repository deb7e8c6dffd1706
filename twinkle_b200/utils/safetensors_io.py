"""Streaming safetensors reader / writer.

Parity: reference ``src/twinkle/utils/safetensors.py:10-169`` —
``SafetensorLazyLoader`` resolves tensor names through
``model.safetensors.index.json`` and materialises one tensor at a time;
``StreamingSafetensorSaver`` writes ≤5 GB shards plus the index as tensors
arrive, or a single ``adapter_model.safetensors`` in PEFT mode.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Iterator, List, Optional, Tuple

import torch
from safetensors import safe_open
from safetensors.torch import save_file


class SafetensorLazyLoader:

    def __init__(self, directory: str):
        self.directory = directory
        self._name_to_file: Dict[str, str] = {}
        index = os.path.join(directory, 'model.safetensors.index.json')
        if os.path.isfile(index):
            with open(index) as f:
                self._name_to_file = dict(json.load(f)['weight_map'])
        else:
            for fn in sorted(os.listdir(directory)):
                if fn.endswith('.safetensors'):
                    with safe_open(os.path.join(directory, fn), 'pt') as f:
                        for k in f.keys():
                            self._name_to_file[k] = fn
        self._open: Dict[str, object] = {}

    def keys(self) -> List[str]:
        return list(self._name_to_file)

    def __contains__(self, name: str) -> bool:
        return name in self._name_to_file

    def _handle(self, fn: str):
        if fn not in self._open:
            self._open[fn] = safe_open(os.path.join(self.directory, fn), 'pt')
        return self._open[fn]

    def get(self, name: str) -> torch.Tensor:
        t = self._handle(self._name_to_file[name]).get_tensor(name)
        if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            # block-quantised checkpoints (DeepSeek-V3 and the like) keep ``<name>_scale_inv`` beside an fp8 weight:
            # expanded to bf16 on the way in, so every consumer of this loader sees ordinary weights
            from .dequantizer import Dequantizer
            t = Dequantizer.maybe_dequantize(name, t, lambda n: self._handle(self._name_to_file[n]).get_tensor(n) if n in self._name_to_file else None)
        return t

    def get_slice(self, name: str):
        return self._handle(self._name_to_file[name]).get_slice(name)

    def items(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for k in self._name_to_file:
            yield k, self.get(k)

    def close(self):
        self._open.clear()


class StreamingSafetensorSaver:

    def __init__(self, directory: str, max_shard_bytes: int = 5 * 10**9, peft: bool = False, is_writer: bool = True):
        self.directory = directory
        self.max_shard_bytes = max_shard_bytes
        self.peft = peft
        self.is_writer = is_writer
        self._pending: Dict[str, torch.Tensor] = {}
        self._pending_bytes = 0
        self._shards: List[Dict[str, int]] = []
        self._total = 0
        if is_writer:
            os.makedirs(directory, exist_ok=True)

    def add(self, name: str, tensor: torch.Tensor) -> None:
        if not self.is_writer:
            return
        t = tensor.detach().to('cpu').contiguous()
        nbytes = t.numel() * t.element_size()
        if not self.peft and self._pending and self._pending_bytes + nbytes > self.max_shard_bytes:
            self._flush()
        self._pending[name] = t
        self._pending_bytes += nbytes
        self._total += nbytes

    def add_many(self, items: Iterable[Tuple[str, torch.Tensor]]) -> None:
        for k, v in items:
            self.add(k, v)

    def _flush(self) -> None:
        if not self._pending:
            return
        tmp = os.path.join(self.directory, f'.shard-{len(self._shards):05d}.tmp')
        save_file(self._pending, tmp, metadata={'format': 'pt'})
        self._shards.append({k: 1 for k in self._pending})
        self._pending, self._pending_bytes = {}, 0

    def finalize(self) -> List[str]:
        if not self.is_writer:
            return []
        if self.peft:
            path = os.path.join(self.directory, 'adapter_model.safetensors')
            save_file(self._pending, path, metadata={'format': 'pt'})
            self._pending = {}
            return [path]
        self._flush()
        n = len(self._shards)
        files, weight_map = [], {}
        for i, names in enumerate(self._shards):
            final = 'model.safetensors' if n == 1 else f'model-{i + 1:05d}-of-{n:05d}.safetensors'
            os.replace(os.path.join(self.directory, f'.shard-{i:05d}.tmp'), os.path.join(self.directory, final))
            files.append(final)
            for k in names:
                weight_map[k] = final
        if n > 1:
            with open(os.path.join(self.directory, 'model.safetensors.index.json'), 'w') as f:
                json.dump({'metadata': {'total_size': self._total}, 'weight_map': weight_map}, f, indent=2)
        return files
