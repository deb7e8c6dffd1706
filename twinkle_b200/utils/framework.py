"""Torch-level helpers shared by every layer.

Parity: reference ``src/twinkle/utils/framework.py:37-249`` — seeding with an
optional full-determinism switch, object gather across ranks, DTensor/local
tensor normalisation, device synchronisation.
"""
from __future__ import annotations

import os
import random
from typing import Any, List, Optional

import numpy as np
import torch


class Torch:

    @staticmethod
    def seed_everything(seed: int = 42, full_determinism: bool = False) -> None:
        random.seed(seed)
        np.random.seed(seed % (2**32))
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)
        if full_determinism or os.environ.get('TWINKLE_FULL_DETERMINISM', '0') == '1':
            os.environ.setdefault('CUBLAS_WORKSPACE_CONFIG', ':4096:8')
            os.environ['TWINKLE_B200_DETERMINISTIC'] = '1'  # our kernels: fixed reduction order
            torch.use_deterministic_algorithms(True, warn_only=True)
            torch.backends.cudnn.deterministic = True
            torch.backends.cudnn.benchmark = False

    @staticmethod
    def gather_object(obj: Any, group=None) -> List[Any]:
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()):
            return [obj]
        out: List[Any] = [None] * dist.get_world_size(group)
        dist.all_gather_object(out, obj, group=group)
        return out

    @staticmethod
    def to_local_tensor(t: Any) -> Any:
        """A sharded parameter wrapper or DTensor → the full plain tensor."""
        if hasattr(t, 'full_tensor'):
            return t.full_tensor()
        return t

    @staticmethod
    def synchronize() -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    @staticmethod
    def is_dist() -> bool:
        import torch.distributed as dist
        return dist.is_available() and dist.is_initialized()

    @staticmethod
    def barrier(group=None) -> None:
        import torch.distributed as dist
        if Torch.is_dist():
            dist.barrier(group=group)

    @staticmethod
    def empty_cache() -> None:
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
