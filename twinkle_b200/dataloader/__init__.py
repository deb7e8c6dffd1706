"""Data loading aware of the device mesh.

Parity: reference ``src/twinkle/dataloader/dataloader.py:19-193`` (``DataLoader`` runs on the first worker,
yields global batches that ``slice_dp`` dispatch later cuts per data rank; in local/torchrun mode every rank
iterates and keeps only its own slice), ``retry_sampler.py`` (skip rows that fail, refill from a seeded
permutation), ``device_mesh_sampler.py`` (global batch → this data rank's slice; resume by skipping consumed
samples), ``device_mesh_fetcher.py`` (same for iterable datasets).
"""
from __future__ import annotations

import random
from typing import Any, Callable, Dict, Iterator, List, Optional

import torch
from torch.utils.data import IterableDataset as TorchIterableDataset

from ..infra import get_mode, remote_class, remote_function
from ..utils.device_mesh import DeviceMesh


class RetrySampler:
    """Yields indices of a seeded permutation; ``dataset[idx]`` failures are skipped and replaced by later
    indices so that every epoch still yields ``len(dataset)`` rows when possible."""

    def __init__(self, dataset, shuffle: bool = True, seed: int = 42, max_retries: int = 20):
        self.dataset, self.shuffle, self.seed, self.max_retries = dataset, shuffle, seed, max_retries
        self.epoch = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __len__(self):
        return len(self.dataset)

    def __iter__(self) -> Iterator[int]:
        n = len(self.dataset)
        order = list(range(n))
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(order)
        spare = list(order)
        random.Random(self.seed + self.epoch + 1).shuffle(spare)
        spare_it = iter(spare)
        for idx in order:
            tries = 0
            while True:
                try:
                    self.dataset[idx]
                    yield idx
                    break
                except Exception:
                    tries += 1
                    if tries > self.max_retries:
                        raise
                    idx = next(spare_it, None)
                    if idx is None:
                        return


class DeviceMeshSampler:
    """Groups indices into global batches and keeps this data rank's slice of each."""

    def __init__(self, base_sampler, batch_size: int, device_mesh: Optional[DeviceMesh], drop_last: bool = True,
                 skip_samples: int = 0, slice_for_rank: bool = True, min_batch_size: Optional[int] = None):
        self.base, self.batch_size, self.mesh, self.drop_last = base_sampler, batch_size, device_mesh, drop_last
        self.skip_samples, self.slice_for_rank = skip_samples, slice_for_rank
        self.min_batch_size = min_batch_size or (device_mesh.data_world_size if device_mesh is not None else 1)

    def __iter__(self) -> Iterator[List[int]]:
        batch: List[int] = []
        skipped = 0
        for idx in self.base:
            if skipped < self.skip_samples:
                skipped += 1
                continue
            batch.append(idx)
            if len(batch) == self.batch_size:
                yield self._cut(batch)
                batch = []
        if batch and not self.drop_last and len(batch) >= self.min_batch_size:
            yield self._cut(batch)

    def _cut(self, batch: List[int]) -> List[int]:
        if self.mesh is None or not self.slice_for_rank:
            return batch
        return batch[self.mesh.get_slice(len(batch))]

    def __len__(self):
        n = max(len(self.base) - self.skip_samples, 0)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size


class DeviceMeshIterableFetcher:

    def __init__(self, dataset, batch_size: int, device_mesh: Optional[DeviceMesh], skip_samples: int = 0, slice_for_rank: bool = True):
        self.dataset, self.batch_size, self.mesh, self.skip, self.slice_for_rank = dataset, batch_size, device_mesh, skip_samples, slice_for_rank

    def __iter__(self):
        batch, skipped = [], 0
        for row in self.dataset:
            if skipped < self.skip:
                skipped += 1
                continue
            batch.append(row)
            if len(batch) == self.batch_size:
                yield batch[self.mesh.get_slice(len(batch))] if (self.mesh is not None and self.slice_for_rank) else batch
                batch = []


@remote_class(execute='first')
class DataLoader:
    """Iterates lists of rows (features or trajectories).  ``batch_size`` is the GLOBAL batch size."""

    def __init__(self, dataset, batch_size: int = 8, device_mesh: DeviceMesh = None, shuffle: bool = True, seed: int = 42,
                 drop_last: bool = True, num_workers: int = 0, collate_fn: Optional[Callable] = None, min_batch_size: Optional[int] = None,
                 **kwargs):
        self.dataset, self.batch_size, self.device_mesh = dataset, batch_size, device_mesh
        self.shuffle, self.seed, self.drop_last = shuffle, seed, drop_last
        self.collate_fn = collate_fn
        self.min_batch_size = min_batch_size
        self.consumed_train_samples = 0
        self._skip = 0
        self.epoch = 0
        # under torchrun every rank iterates and keeps its slice; in pool mode the single loader yields
        # global batches and the slice_dp dispatch cuts them
        self._slice_here = get_mode() == 'local'
        if device_mesh is not None and batch_size < device_mesh.data_world_size:
            raise ValueError(f'batch_size {batch_size} is smaller than the data-parallel world size {device_mesh.data_world_size}')

    @remote_function()
    def skip_consumed_samples(self, consumed_train_samples: int) -> None:
        self._skip = consumed_train_samples % max(len(self.dataset), 1) if hasattr(self.dataset, '__len__') else consumed_train_samples
        self.consumed_train_samples = consumed_train_samples

    resume_from_checkpoint = skip_consumed_samples

    @remote_function()
    def set_processor(self, processor_cls, **kwargs) -> None:
        """Collate every batch with an ``InputProcessor`` (a class, its name, an instance, or any callable on a list of rows);
        by default batches stay lists of rows and the model collates (reference ``dataloader/dataloader.py:95-104``)."""
        from .. import processor as processors
        from ..utils.loader import construct_class
        if callable(processor_cls) and not isinstance(processor_cls, (str, type)):
            self.collate_fn = processor_cls
            return
        kwargs.setdefault('device_mesh', self.device_mesh)
        self.collate_fn = construct_class(processor_cls, processors.InputProcessor, processors, **kwargs)

    @remote_function(collect='first')
    def get_state(self) -> Dict[str, Any]:
        return {'consumed_train_samples': self.consumed_train_samples, 'epoch': self.epoch}

    @remote_function(collect='first')
    def __len__(self):
        if isinstance(self.dataset, TorchIterableDataset):
            raise TypeError('iterable dataset has no length')
        return len(self.dataset) // self.batch_size

    def __iter__(self):
        if isinstance(self.dataset, TorchIterableDataset):
            it = DeviceMeshIterableFetcher(self.dataset, self.batch_size, self.device_mesh, self._skip, self._slice_here)
            for batch in it:
                self.consumed_train_samples += self.batch_size
                yield self.collate_fn(batch) if self.collate_fn else batch
        else:
            base = RetrySampler(self.dataset, self.shuffle, self.seed)
            base.set_epoch(self.epoch)
            sampler = DeviceMeshSampler(base, self.batch_size, self.device_mesh, self.drop_last, self._skip, self._slice_here,
                                        self.min_batch_size)
            for idxs in sampler:
                self.consumed_train_samples += self.batch_size
                batch = [self.dataset[i] for i in idxs]
                yield self.collate_fn(batch) if self.collate_fn else batch
            self.epoch += 1
        self._skip = 0
