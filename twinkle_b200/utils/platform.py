"""Accelerator / rank discovery from the process environment.

Parity: reference ``src/twinkle/utils/platforms/base.py:22-159`` and
``platforms/gpu.py:5-39`` (env-based rank getters, visible-device variable,
collective backend name).  Only two platforms exist here: B200 (``cuda``) and
the CPU used by host-side tests (``gloo``).  Ascend/MPS back ends of the
reference are out of scope for a B200-only build.
"""
from __future__ import annotations

import os
import shutil
from typing import List, Optional


def _env_int(*names: str, default: int = 0) -> int:
    for n in names:
        v = os.environ.get(n)
        if v is not None and v != '':
            try:
                return int(v)
            except ValueError:
                continue
    return default


class Platform:
    """Static helpers; every getter reads ``os.environ`` at call time so that
    tests can monkey-patch the environment (or the getter itself)."""

    @staticmethod
    def device_prefix() -> str:
        try:
            import torch
            if torch.cuda.is_available():
                return 'cuda'
        except Exception:  # pragma: no cover
            pass
        return 'cpu'

    @staticmethod
    def device_backend() -> str:
        return 'nccl' if Platform.device_prefix() == 'cuda' else 'gloo'

    @staticmethod
    def visible_device_env() -> str:
        return 'CUDA_VISIBLE_DEVICES'

    @staticmethod
    def has_nvidia_smi() -> bool:
        return shutil.which('nvidia-smi') is not None

    @staticmethod
    def get_rank() -> int:
        return _env_int('RANK', default=0)

    @staticmethod
    def get_world_size() -> int:
        return max(_env_int('WORLD_SIZE', default=1), 1)

    @staticmethod
    def get_local_rank() -> int:
        return _env_int('LOCAL_RANK', default=0)

    @staticmethod
    def get_local_world_size() -> int:
        return max(_env_int('LOCAL_WORLD_SIZE', default=Platform.get_world_size()), 1)

    @staticmethod
    def get_node_rank() -> int:
        return _env_int('GROUP_RANK', 'NODE_RANK', default=0)

    @staticmethod
    def get_nnodes() -> int:
        lws = Platform.get_local_world_size()
        return max(Platform.get_world_size() // max(lws, 1), 1)

    @staticmethod
    def is_master() -> bool:
        return Platform.get_rank() == 0

    @staticmethod
    def is_local_master() -> bool:
        return Platform.get_local_rank() == 0

    @staticmethod
    def is_last_rank() -> bool:
        return Platform.get_rank() == Platform.get_world_size() - 1

    @staticmethod
    def get_peer_index(target_size: int, rank: Optional[int] = None, world_size: Optional[int] = None) -> List[int]:
        """Which of ``target_size`` peers a worker should talk to when two
        groups of different size are paired (e.g. 6 trainer ranks feeding 2
        sampler ranks).  Balanced contiguous assignment."""
        rank = Platform.get_rank() if rank is None else rank
        world_size = Platform.get_world_size() if world_size is None else world_size
        if target_size >= world_size:
            k, m = divmod(target_size, world_size)
            start = rank * k + min(rank, m)
            return list(range(start, start + k + (1 if rank < m else 0)))
        return [rank * target_size // world_size]

    @staticmethod
    def current_device():
        import torch
        if Platform.device_prefix() == 'cuda':
            return torch.device('cuda', Platform.get_local_rank() % max(torch.cuda.device_count(), 1))
        return torch.device('cpu')

    @staticmethod
    def set_device() -> None:
        import torch
        if Platform.device_prefix() == 'cuda':
            torch.cuda.set_device(Platform.current_device())

    @staticmethod
    def get_rng_state():
        import torch
        state = {'cpu': torch.get_rng_state()}
        if torch.cuda.is_available():
            state['cuda'] = torch.cuda.get_rng_state_all()
        return state

    @staticmethod
    def set_rng_state(state) -> None:
        import torch
        torch.set_rng_state(state['cpu'])
        if 'cuda' in state and torch.cuda.is_available():
            try:
                torch.cuda.set_rng_state_all(state['cuda'])
            except Exception:
                pass


class GPU(Platform):
    """B200 platform constants."""
    SM_COUNT = 148
    HBM_BYTES = 180 * 10**9
    L2_BYTES = 126 * 2**20
    SMEM_PER_CTA = 227 * 1024
    TMEM_COLUMNS = 512
    NVLINK_GBS_PER_DIR = 900.0

    @staticmethod
    def device_prefix() -> str:
        return 'cuda'

    @staticmethod
    def device_backend() -> str:
        return 'nccl'
