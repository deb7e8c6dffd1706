"""Sequence packing.

Parity: reference ``src/twinkle/dataset/packing_dataset.py:16-131`` (bin-pack encoded rows to
``template.max_length`` — the reference calls ``binpacking.to_constant_volume``) and
``iterable_packing_dataset.py:15-142`` (streaming, ``packing_interval`` rows per packing round, cyclic).
Packing here is first-fit-decreasing on token counts; each packed row concatenates ``input_ids`` / ``labels``
and restarts ``position_ids`` at every document so attention never crosses documents.
"""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Sequence

from ..infra import remote_class, remote_function
from .base import Dataset, DatasetMeta, IterableDataset


def pack_to_constant_volume(lengths: Sequence[int], capacity: int) -> List[List[int]]:
    """First-fit-decreasing bins of item indices with Σ length ≤ capacity (oversize items get their own bin)."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: List[List[int]] = []
    room: List[int] = []
    for i in order:
        L = lengths[i]
        placed = False
        for b in range(len(bins)):
            if room[b] >= L:
                bins[b].append(i)
                room[b] -= L
                placed = True
                break
        if not placed:
            bins.append([i])
            room.append(max(capacity - L, 0))
    return bins


def concat_features(rows: Sequence[Dict[str, Any]]) -> Dict[str, Any]:
    ids, labels, pos = [], [], []
    for r in rows:
        n = len(r['input_ids'])
        ids += list(r['input_ids'])
        labels += list(r.get('labels', [-100] * n))
        pos += list(range(n))
    out = {'input_ids': ids, 'labels': labels, 'position_ids': pos, 'attention_mask': [1] * len(ids), 'length': len(ids)}
    if any(r.get('pixel_values') is not None for r in rows):
        # documents with images: patches and grids in document order; every document keeps its own (time, height, width)
        # positions (they restart per document like the plain index), text-only documents count up in all three alike
        import torch
        with_img = [r for r in rows if r.get('pixel_values') is not None]
        out['pixel_values'] = torch.cat([torch.as_tensor(r['pixel_values']) for r in with_img], 0)
        out['image_grid_thw'] = [list(map(int, g)) for r in with_img for g in r['image_grid_thw']]
        out['mrope_position_ids'] = torch.cat([torch.as_tensor(r['mrope_position_ids']).long() if r.get('mrope_position_ids') is not None
                                               else torch.arange(len(r['input_ids'])).expand(3, -1) for r in rows], 1)
        out['placeholder_ids'] = sorted({int(t) for r in with_img for t in (r.get('placeholder_ids') or ())})
    return out


@remote_class(execute='first')
class PackingDataset(Dataset):

    @remote_function()
    def pack_dataset(self, max_length: int = None, **kwargs) -> None:
        cap = max_length or (self.template.max_length if self.template is not None else None)
        if not cap:
            raise ValueError('pack_dataset needs max_length (or a template with max_length)')
        rows = [r for r in self._rows() if 'input_ids' in r]
        if len(rows) != len(self._rows()):
            raise ValueError('pack_dataset expects encoded rows; call encode() first')
        bins = pack_to_constant_volume([len(r['input_ids']) for r in rows], cap)
        self._replace([concat_features([rows[i] for i in b]) for b in bins])


@remote_class(execute='first')
class IterablePackingDataset(IterableDataset):

    def __init__(self, dataset_meta: DatasetMeta, packing_interval: int = 128, cyclic: bool = False, max_length: int = None, **kwargs):
        super().__init__(dataset_meta, **kwargs)
        self.packing_interval, self.cyclic, self.max_length = packing_interval, cyclic, max_length

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        cap = self.max_length or (self.template.max_length if self.template is not None else None)
        if not cap:
            raise ValueError('IterablePackingDataset needs max_length')
        while True:
            buf: List[Dict[str, Any]] = []
            for row in super().__iter__():
                buf.append(row)
                if len(buf) >= self.packing_interval:
                    yield from self._emit(buf, cap)
                    buf = []
            if buf:
                yield from self._emit(buf, cap)
            if not self.cyclic:
                return

    @staticmethod
    def _emit(buf, cap):
        for b in pack_to_constant_volume([len(r['input_ids']) for r in buf], cap):
            yield concat_features([buf[i] for i in b])
