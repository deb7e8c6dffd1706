"""Trainer → sampler weight synchronisation.

Parity: reference ``src/twinkle/checkpoint_engine/{base,manager,mixin,nccl_checkpoint_engine}.py`` —
``CheckpointEngineManager(model, sampler).sync_weights(merge_and_sync)`` orchestrates one sync (first call:
base weights; later calls LoRA-only unless ``merge_and_sync``); an engine implements ``prepare /
build_topology / init_process_group / send_weights / receive_weights / finalize``.

Engines:

* ``PeerCopyCheckpointEngine`` (B200-native): every sampler rank exposes a landing buffer through CUDA IPC;
  the trainer packs ``(name, tensor)`` pairs into it with the peer-copy kernel (``ops/csrc/symm.cu``:
  16-byte stores over NVLink, optional fp32→bf16 cast in flight) — no staging bucket on the trainer, no
  broadcast tree, no second process group.  Control plane (names, shapes, offsets, acks): a ``TCPStore``.
* ``NCCLCheckpointEngine`` (baseline, as in the reference): bucketed ``broadcast`` on a dedicated process
  group with two alternating ``uint8`` buckets.
* ``StoreCheckpointEngine``: host-memory transport for trainer and sampler processes without GPUs (CPU runs, tests):
  buckets of serialised tensors travel through the same ``TCPStore`` that carries the control messages.
* in-process hand-off when trainer and sampler live in one process (tests, colocated mode).

``CheckpointEngineMixin`` gives models and samplers the ``prepare_checkpoint_engine`` / ``send_weights`` /
``receive_weights`` methods the manager drives when the two sides are separate worker groups (reference
``checkpoint_engine/mixin.py:30-34``, ``transformers.py:1507-1616``, ``vllm_sampler.py:439-487``).
"""
from __future__ import annotations

import json
import os
import pickle
import time
from typing import Any, Dict, Iterable, Iterator, List, Optional, Tuple

import torch

from ..utils.logger import get_logger
from ..utils.network import find_free_port

logger = get_logger()
DEFAULT_BUCKET_BYTES = 3072 << 20

_DTYPES = {'bfloat16': torch.bfloat16, 'float32': torch.float32, 'float16': torch.float16, 'int64': torch.int64, 'int32': torch.int32}


class CheckpointEngine:

    def prepare(self) -> Dict[str, Any]:
        return {}

    def build_topology(self, trainer_infos: List[Dict[str, Any]], sampler_infos: List[Dict[str, Any]]) -> None:
        pass

    def init_process_group(self, **kwargs) -> None:
        pass

    def send_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> Dict[str, float]:
        raise NotImplementedError

    def receive_weights(self) -> Iterator[Tuple[str, torch.Tensor]]:
        raise NotImplementedError

    def finalize(self) -> None:
        pass


class PeerCopyCheckpointEngine(CheckpointEngine):
    """``role='send'`` on the trainer's source rank, ``role='recv'`` on every sampler rank."""

    def __init__(self, role: str, store_host: str = '127.0.0.1', store_port: int = 0, n_receivers: int = 1, receiver_index: int = 0,
                 bucket_bytes: int = 512 << 20, device=None, timeout_s: float = 300.0):
        from torch.distributed import TCPStore
        import datetime
        self.role, self.n_recv, self.index, self.bucket_bytes = role, n_receivers, receiver_index, bucket_bytes
        self.device = torch.device(device) if device is not None else torch.device('cuda', torch.cuda.current_device())
        self.port = store_port or find_free_port()
        self.store = TCPStore(store_host, self.port, is_master=(role == 'send'), wait_for_workers=False,
                              timeout=datetime.timedelta(seconds=timeout_s))
        self.timeout_s = timeout_s
        self._landing = None
        self._peer_ptrs: List[int] = []
        self._round = 0

    # ----------------------------------------------------------- set-up
    def prepare(self) -> Dict[str, Any]:
        from .. import ops
        if self.role == 'recv':
            raw, handle, offset = ops.ext().symm_alloc(2 * self.bucket_bytes)
            self._landing = raw
            self.store.set(f'landing/{self.index}', json.dumps({'handle': handle.hex(), 'offset': offset, 'nbytes': raw.numel()}))
        return {'role': self.role, 'port': self.port}

    def init_process_group(self, **kwargs) -> None:
        from .. import ops
        if self.role == 'send' and not self._peer_ptrs:
            for i in range(self.n_recv):
                info = json.loads(self.store.get(f'landing/{i}'))
                self._peer_ptrs.append(ops.ext().symm_open(bytes.fromhex(info['handle'])) + info['offset'])

    # ------------------------------------------------------------- send
    def send_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> Dict[str, float]:
        from .. import ops
        E = ops.ext()
        self.init_process_group()
        t0 = time.time()
        total = 0
        half, meta, used, bucket_id = 0, [], 0, 0
        rnd = self._round

        def flush(last: bool):
            nonlocal half, meta, used, bucket_id
            torch.cuda.synchronize(self.device)  # all pushes of this bucket have been issued and completed
            self.store.set(f'r{rnd}/bucket/{bucket_id}', json.dumps({'half': half, 'tensors': meta, 'last': last}))
            if bucket_id >= 1:  # the half we are about to reuse must have been consumed by every receiver
                for i in range(self.n_recv):
                    self.store.wait([f'r{rnd}/ack/{bucket_id - 1}/{i}'])
            half ^= 1
            meta, used = [], 0
            bucket_id += 1

        for name, t in weights:
            t = t.detach()
            if not t.is_contiguous():
                t = t.contiguous()
            out_bytes = t.numel() * 2 if t.dtype in (torch.float32, torch.bfloat16) else t.numel() * t.element_size()
            aligned = (out_bytes + 255) // 256 * 256
            if aligned > self.bucket_bytes:
                raise ValueError(f'{name}: {aligned} bytes exceed the landing bucket ({self.bucket_bytes})')
            if used + aligned > self.bucket_bytes:
                flush(False)
            if t.dtype not in (torch.float32, torch.bfloat16):
                t = t.float()
            E.peer_copy_cast(t.to(self.device), self._peer_ptrs, half * self.bucket_bytes + used)
            meta.append({'name': name, 'shape': list(t.shape), 'dtype': 'bfloat16', 'offset': used})
            used += aligned
            total += out_bytes
        flush(True)
        for i in range(self.n_recv):
            self.store.wait([f'r{rnd}/ack/{bucket_id - 1}/{i}'])
        self._round += 1
        dt = max(time.time() - t0, 1e-9)
        stats = {'bytes': float(total), 'seconds': dt, 'gb_per_s': total / dt / 1e9}
        logger.info(f'weight sync: {total / 1e6:.1f} MB in {dt:.3f}s, bandwidth={stats["gb_per_s"]:.2f} GB/s')
        return stats

    # ---------------------------------------------------------- receive
    def receive_weights(self) -> Iterator[Tuple[str, torch.Tensor]]:
        rnd, bucket_id = self._round, 0
        while True:
            key = f'r{rnd}/bucket/{bucket_id}'
            self.store.wait([key])
            info = json.loads(self.store.get(key))
            base = info['half'] * self.bucket_bytes
            for m in info['tensors']:
                n = 1
                for s in m['shape']:
                    n *= s
                view = self._landing[base + m['offset']:base + m['offset'] + 2 * n].view(torch.bfloat16).view(m['shape'])
                yield m['name'], view
            torch.cuda.synchronize(self.device)  # consumers copied out of the landing zone
            self.store.set(f'r{rnd}/ack/{bucket_id}/{self.index}', '1')
            bucket_id += 1
            if info['last']:
                break
        self._round += 1

    def finalize(self) -> None:
        from .. import ops
        for p in self._peer_ptrs:
            ops.ext().symm_close(p)
        self._peer_ptrs = []


class StoreCheckpointEngine(CheckpointEngine):
    """Weights through host memory: the sender packs ``(name, dtype, shape, bytes)`` records into buckets stored under
    ``r<round>/bucket/<i>``; every receiver reads a bucket, yields its tensors and acknowledges; the sender deletes a
    bucket once all receivers acknowledged it and never has more than two outstanding."""

    def __init__(self, role: str, store_host: str = '127.0.0.1', store_port: int = 0, n_receivers: int = 1, receiver_index: int = 0,
                 bucket_bytes: int = 32 << 20, timeout_s: float = 300.0, **_):
        from torch.distributed import TCPStore
        import datetime
        self.role, self.n_recv, self.index, self.bucket_bytes = role, n_receivers, receiver_index, bucket_bytes
        self.port = store_port or find_free_port()
        self.store = TCPStore(store_host, self.port, is_master=(role == 'send'), wait_for_workers=False,
                              timeout=datetime.timedelta(seconds=timeout_s))
        self._round = 0

    def prepare(self) -> Dict[str, Any]:
        return {'role': self.role, 'port': self.port, 'engine': 'store'}

    def init_process_group(self, **kwargs) -> None:
        pass

    def _wait_acks(self, rnd: int, bucket_id: int) -> None:
        for i in range(self.n_recv):
            self.store.wait([f'r{rnd}/ack/{bucket_id}/{i}'])
        self.store.delete_key(f'r{rnd}/bucket/{bucket_id}')

    def send_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> Dict[str, float]:
        t0 = time.time()
        rnd, records, used, bucket_id, total = self._round, [], 0, 0, 0

        def flush(last: bool):
            nonlocal records, used, bucket_id
            self.store.set(f'r{rnd}/bucket/{bucket_id}', pickle.dumps({'last': last, 'tensors': records}, protocol=pickle.HIGHEST_PROTOCOL))
            if bucket_id >= 1:
                self._wait_acks(rnd, bucket_id - 1)
            records, used = [], 0
            bucket_id += 1

        for name, t in weights:
            t = t.detach()
            if t.dtype == torch.float32:
                t = t.to(torch.bfloat16)       # the sampler computes in bf16; halves the traffic like the peer-copy cast
            t = t.contiguous().cpu()
            raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b''
            if used and used + len(raw) > self.bucket_bytes:
                flush(False)
            records.append((name, str(t.dtype).replace('torch.', ''), list(t.shape), raw))
            used += len(raw)
            total += len(raw)
        flush(True)
        self._wait_acks(rnd, bucket_id - 1)
        self._round += 1
        dt = max(time.time() - t0, 1e-9)
        return {'bytes': float(total), 'seconds': dt, 'gb_per_s': total / dt / 1e9}

    def receive_weights(self) -> Iterator[Tuple[str, torch.Tensor]]:
        rnd, bucket_id = self._round, 0
        while True:
            key = f'r{rnd}/bucket/{bucket_id}'
            self.store.wait([key])
            info = pickle.loads(self.store.get(key))
            for name, dtype, shape, raw in info['tensors']:
                dt = getattr(torch, dtype)
                t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dt).view(shape) if raw else torch.empty(shape, dtype=dt)
                yield name, t
            self.store.set(f'r{rnd}/ack/{bucket_id}/{self.index}', '1')
            bucket_id += 1
            if info['last']:
                break
        self._round += 1


def make_engine(kind: str, role: str, **kw) -> CheckpointEngine:
    if kind == 'peer':
        return PeerCopyCheckpointEngine(role, **kw)
    if kind == 'store':
        return StoreCheckpointEngine(role, **kw)
    raise ValueError(f'unknown checkpoint engine {kind!r} (peer | store)')


class CheckpointEngineMixin:
    """Remote-callable ends of a weight sync.  A model needs ``weight_iterator``; a sampler needs ``update_weights``."""

    _ckpt_engine: Optional[CheckpointEngine] = None

    def prepare_checkpoint_engine(self, role: str, engine: str = 'store', host: str = '127.0.0.1', port: int = 0, n_receivers: int = 1,
                                  receiver_index: Optional[int] = None, **kwargs) -> Dict[str, Any]:
        """Create (once) this process's end of the engine.  Only the model group's first rank opens a sending end:
        the others take part in ``send_weights`` because gathering sharded parameters is collective."""
        rank = int(os.environ.get('RANK', 0))
        if self._ckpt_engine is None and (role == 'recv' or rank == 0):
            idx = rank if receiver_index is None else receiver_index
            self._ckpt_engine = make_engine(engine, role, store_host=host, store_port=port, n_receivers=n_receivers, receiver_index=idx, **kwargs)
            self._ckpt_engine.prepare()
        return {'role': role, 'rank': rank, 'engine': engine, 'port': port}

    def _send_weights(self, adapter_name: Optional[str] = None, merge_and_sync: bool = False, lora_only: bool = False) -> Dict[str, float]:
        it = self.weight_iterator(adapter_name, merge_and_sync, lora_only)
        if self._ckpt_engine is None:      # not the source rank: only the collectives inside the iterator matter
            for _ in it:
                pass
            return {}
        return self._ckpt_engine.send_weights(it)

    def _receive_weights(self, peft_config: Optional[Dict[str, Any]] = None, **kwargs) -> int:
        if self._ckpt_engine is None:
            raise RuntimeError('prepare_checkpoint_engine(role="recv") must be called before receive_weights')
        n = 0

        def owned():
            # the engine reuses its landing area for the next bucket; update_weights keeps references until the end
            nonlocal n
            for k, v in self._ckpt_engine.receive_weights():
                n += v.numel() * v.element_size()
                yield k, v.clone()

        self.update_weights(owned(), peft_config=peft_config, **kwargs)
        return n

    def finalize_checkpoint_engine(self) -> None:
        if self._ckpt_engine is not None:
            self._ckpt_engine.finalize()
            self._ckpt_engine = None


class NCCLCheckpointEngine(CheckpointEngine):
    """Bucketed broadcast on the given (already created) process group: rank ``src`` sends, all others
    receive.  Metadata travels as a broadcast object list."""

    def __init__(self, group=None, src: int = 0, bucket_bytes: int = DEFAULT_BUCKET_BYTES, device=None):
        import torch.distributed as dist
        self.dist, self.group, self.src, self.bucket_bytes = dist, group, src, bucket_bytes
        self.device = device or (torch.device('cuda', torch.cuda.current_device()) if torch.cuda.is_available() else torch.device('cpu'))
        self.buckets = [torch.empty(bucket_bytes, dtype=torch.uint8, device=self.device) for _ in range(2)]

    def _bcast_meta(self, meta):
        box = [meta]
        self.dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]

    def send_weights(self, weights):
        t0, total, which, used, meta = time.time(), 0, 0, 0, []

        def flush(last):
            nonlocal which, used, meta
            self._bcast_meta({'tensors': meta, 'last': last, 'used': used})
            self.dist.broadcast(self.buckets[which][:max(used, 1)], src=self.src, group=self.group)
            which ^= 1
            used, meta = 0, []

        for name, t in weights:
            b = t.detach().contiguous().view(torch.uint8).reshape(-1) if t.dtype != torch.bfloat16 else t.detach().contiguous().view(torch.uint8).reshape(-1)
            n = b.numel()
            if used + n > self.bucket_bytes:
                flush(False)
            self.buckets[which][used:used + n].copy_(b)
            meta.append({'name': name, 'shape': list(t.shape), 'dtype': str(t.dtype).replace('torch.', ''), 'offset': used, 'nbytes': n})
            used += (n + 255) // 256 * 256
            total += n
        flush(True)
        dt = max(time.time() - t0, 1e-9)
        return {'bytes': float(total), 'seconds': dt, 'gb_per_s': total / dt / 1e9}

    def receive_weights(self):
        which = 0
        while True:
            info = self._bcast_meta(None)
            self.dist.broadcast(self.buckets[which][:max(info['used'], 1)], src=self.src, group=self.group)
            for m in info['tensors']:
                yield m['name'], self.buckets[which][m['offset']:m['offset'] + m['nbytes']].view(_DTYPES[m['dtype']]).view(m['shape'])
            which ^= 1
            if info['last']:
                return


class CheckpointEngineManager:
    """One object per (model, sampler) pair.  When both are plain in-process objects the weights are handed
    over directly; with remote proxies (pool mode) both sides are driven through their ``prepare_checkpoint_engine
    / send_weights / receive_weights`` remote methods."""

    def __init__(self, model, sampler, engine: str = 'auto'):
        self.model, self.sampler, self.engine = model, sampler, engine
        self.base_sync_done = False
        self._prepared = False
        self.last_stats: Dict[str, float] = {}

    def _remote(self) -> bool:
        return getattr(self.model, '_remote_proxy', None) is not None or getattr(self.sampler, '_remote_proxy', None) is not None

    def sync_weights(self, merge_and_sync: bool = False, adapter_name: Optional[str] = None) -> Dict[str, float]:
        t0 = time.time()
        lora_only = self.base_sync_done and not merge_and_sync and adapter_name is not None
        n = 0
        if not self.base_sync_done and adapter_name is not None and not merge_and_sync:
            # first sync: base weights once, then the adapter
            n += self._transfer(None, False, False, None)
            self.base_sync_done = True
            lora_only = True
        peft = self.model.get_peft_config_dict(adapter_name) if (lora_only and adapter_name) else None
        n += self._transfer(adapter_name, merge_and_sync, lora_only, peft)
        self.base_sync_done = True
        if hasattr(self.sampler, 'reset_prefix_cache'):
            self.sampler.reset_prefix_cache()
        self.last_stats = {'seconds': time.time() - t0, 'bytes': float(n), 'gb_per_s': n / max(time.time() - t0, 1e-9) / 1e9}
        return self.last_stats

    def _prepare_remote(self) -> None:
        if self._prepared:
            return
        if getattr(self.model, '_remote_proxy', None) is None or getattr(self.sampler, '_remote_proxy', None) is None:
            raise RuntimeError('weight sync between a worker group and an in-process object is not supported: '
                               'create model and sampler both with remote_group=… or both in this process')
        kind = self.engine
        if kind == 'auto':
            kind = 'peer' if torch.cuda.is_available() else 'store'
        port = find_free_port()
        n_recv = len(self.sampler._remote_proxy.ranks)
        self.model.prepare_checkpoint_engine('send', engine=kind, port=port, n_receivers=n_recv)       # opens the store first
        self.sampler.prepare_checkpoint_engine('recv', engine=kind, port=port, n_receivers=n_recv)
        self._prepared = True

    def _transfer(self, adapter_name, merge_and_sync: bool, lora_only: bool, peft_config) -> int:
        if self._remote():
            from ..infra import LazyCollect
            self._prepare_remote()
            sending = self.model.send_weights(adapter_name=adapter_name, merge_and_sync=merge_and_sync, lora_only=lora_only)   # returns at once
            received = self.sampler.receive_weights(peft_config=peft_config)
            stats = sending() if isinstance(sending, LazyCollect) else sending
            if isinstance(received, (list, tuple)):
                received = received[0] if received else 0
            return int(received or (stats or {}).get('bytes', 0))
        total = 0

        def counted():
            nonlocal total
            for k, v in self.model.weight_iterator(adapter_name, merge_and_sync, lora_only):
                total += v.numel() * v.element_size()
                yield k, v

        self.sampler.update_weights(counted(), peft_config=peft_config)
        return total

    def finalize(self) -> None:
        if self._prepared:
            self.model.finalize_checkpoint_engine()
            self.sampler.finalize_checkpoint_engine()
            self._prepared = False
