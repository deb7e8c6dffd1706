"""Collation: features → model-ready tensors, and model outputs → per-sequence tensors.

Parity: reference ``src/twinkle/processor/base.py`` — padding map
(``labels → −100``, ``position_ids → −1``, ``input_ids → pad``, ``attention_mask
→ 0``), padding-free concatenation to one packed row with sequence boundaries
where ``position_ids == 0``, fixed / variable-length micro-batching, sequence-
parallel splitting, zig-zag context-parallel splitting (chunks ``r`` and
``2cp−1−r`` per packed segment), and the reverse transforms
(``unpack_packed_sequences`` → ``[n_seq, max_len]``).

The owned decoder always consumes packed rows, so ``padding_free`` is the native
form here; the padded form is still produced for consumers that want
``[B, S]`` tensors (losses operate on ``[n_seq, max_len]``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..data_format import InputFeature

PAD_VALUES = {'input_ids': 0, 'attention_mask': 0, 'labels': -100, 'position_ids': -1, 'completion_mask': 0}
_SEQ_KEYS = ('input_ids', 'attention_mask', 'labels', 'position_ids', 'completion_mask')


def _as_long(x) -> torch.Tensor:
    if torch.is_tensor(x):
        return x.reshape(-1).long()
    return torch.as_tensor(np.asarray(x), dtype=torch.long).reshape(-1)


def cu_seqlens_from_position_ids(position_ids: torch.Tensor) -> torch.Tensor:
    """Boundaries of a packed row: a new sequence starts wherever position == 0."""
    starts = (position_ids == 0).nonzero(as_tuple=True)[0]
    if starts.numel() == 0 or starts[0] != 0:
        starts = torch.cat([starts.new_zeros(1), starts])
    return torch.cat([starts, starts.new_tensor([position_ids.numel()])]).to(torch.int32)


def zigzag_indices(length: int, cp: int, rank: int) -> torch.Tensor:
    """Token indices of one sequence (length divisible by 2·cp) owned by ``rank``:
    chunk ``rank`` and chunk ``2cp−1−rank`` — balances causal attention work."""
    c = length // (2 * cp)
    a = torch.arange(rank * c, (rank + 1) * c)
    b = torch.arange((2 * cp - 1 - rank) * c, (2 * cp - rank) * c)
    return torch.cat([a, b])


@dataclass
class MicroBatch:
    """One packed micro-batch.  ``seq_lens`` are the original per-sequence
    lengths (after padding to the parallel multiple) in packed order."""
    input_ids: torch.Tensor
    position_ids: torch.Tensor
    labels: Optional[torch.Tensor]
    cu_seqlens: torch.Tensor
    max_seqlen: int
    seq_lens: List[int]
    local_index: Optional[torch.Tensor] = None  # positions of this rank's tokens inside the full packed row
    extras: Optional[Dict[str, Any]] = None

    def to(self, device) -> 'MicroBatch':
        def mv(t):
            if t is None:
                return None
            if t.device.type == 'cpu' and torch.device(device).type == 'cuda' and not t.is_pinned():
                t = t.pin_memory()  # staged through pinned memory so the copy is asynchronous
            return t.to(device, non_blocking=True)

        return MicroBatch(mv(self.input_ids), mv(self.position_ids), mv(self.labels), mv(self.cu_seqlens), self.max_seqlen,
                          self.seq_lens, mv(self.local_index), self.extras)


class InputProcessor:
    """Stateless apart from its configuration."""

    def __init__(self, device_mesh=None, padding_free: bool = True, padding_side: str = 'right', pad_token_id: int = 0,
                 framework: str = 'native', micro_batch_size: Optional[int] = None, max_tokens_per_micro_batch: Optional[int] = None,
                 sp_size: Optional[int] = None, sp_rank: Optional[int] = None, cp_size: Optional[int] = None, cp_rank: Optional[int] = None,
                 pad_to_multiple_of: int = 1, **kwargs):
        self.device_mesh = device_mesh
        self.padding_free, self.padding_side, self.pad_token_id = padding_free, padding_side, pad_token_id
        self.framework = framework
        self.micro_batch_size = micro_batch_size
        self.max_tokens_per_micro_batch = max_tokens_per_micro_batch
        self.sp_size = sp_size if sp_size is not None else ((device_mesh.ulysses_size or 1) if device_mesh is not None else 1)
        self.sp_rank = sp_rank if sp_rank is not None else (device_mesh.ulysses_rank if device_mesh is not None else 0)
        self.cp_size = cp_size if cp_size is not None else ((device_mesh.cp_world_size or 1) if device_mesh is not None else 1)
        self.cp_rank = cp_rank if cp_rank is not None else ((device_mesh.cp_rank or 0) if device_mesh is not None else 0)
        self.pad_to_multiple_of = pad_to_multiple_of

    # ------------------------------------------------------------- features
    @staticmethod
    def normalize(features: Sequence[InputFeature]) -> List[Dict[str, torch.Tensor]]:
        """Every feature gets 1-D long tensors for input_ids / labels / position_ids."""
        out = []
        for f in features:
            ids = _as_long(f['input_ids'])
            n = ids.numel()
            labels = _as_long(f['labels']) if f.get('labels') is not None else torch.full((n, ), -100, dtype=torch.long)
            pos = _as_long(f['position_ids']) if f.get('position_ids') is not None else torch.arange(n)
            if f.get('attention_mask') is not None:
                am = _as_long(f['attention_mask']).bool()
                if not bool(am.all()):
                    ids, labels = ids[am], labels[am]
                    pos = torch.arange(ids.numel()) if f.get('position_ids') is None else pos[am]
            item = {'input_ids': ids, 'labels': labels, 'position_ids': pos}
            for k in ('routed_experts', 'pixel_values', 'image_grid_thw', 'mrope_position_ids', 'placeholder_ids'):
                if f.get(k) is not None:
                    item[k] = f[k]
            out.append(item)
        return out

    def pad_batch(self, features: Sequence[InputFeature]) -> Dict[str, torch.Tensor]:
        """Padded ``[B, S]`` tensors (reference ``collate_fn`` padded mode)."""
        items = self.normalize(features)
        S = max(i['input_ids'].numel() for i in items)
        m = self.pad_to_multiple_of
        S = (S + m - 1) // m * m
        out: Dict[str, List[torch.Tensor]] = {k: [] for k in ('input_ids', 'labels', 'position_ids', 'attention_mask')}
        for it in items:
            n = it['input_ids'].numel()
            pad = S - n
            for k in ('input_ids', 'labels', 'position_ids'):
                v = it[k]
                fill = self.pad_token_id if k == 'input_ids' else PAD_VALUES[k]
                filler = torch.full((pad, ), fill, dtype=torch.long)
                out[k].append(torch.cat([v, filler]) if self.padding_side == 'right' else torch.cat([filler, v]))
            am = torch.cat([torch.ones(n, dtype=torch.long), torch.zeros(pad, dtype=torch.long)])
            out['attention_mask'].append(am if self.padding_side == 'right' else am.flip(0))
        return {k: torch.stack(v) for k, v in out.items()}

    # -------------------------------------------------------- micro-batches
    def split_micro_batches(self, items: List[Dict[str, torch.Tensor]]) -> List[List[Dict[str, torch.Tensor]]]:
        if self.max_tokens_per_micro_batch:
            groups, cur, tok = [], [], 0
            for it in items:
                n = it['input_ids'].numel()
                if cur and tok + n > self.max_tokens_per_micro_batch:
                    groups.append(cur)
                    cur, tok = [], 0
                cur.append(it)
                tok += n
            if cur:
                groups.append(cur)
            return groups
        mbs = self.micro_batch_size or len(items)
        return [items[i:i + mbs] for i in range(0, len(items), mbs)]

    def _pack(self, items: List[Dict[str, torch.Tensor]], pad_multiple: Optional[int] = None, split: bool = True) -> MicroBatch:
        """Concatenate sequences.  With context parallelism each sequence is
        padded to a multiple of 2·cp (zig-zag halves); with Ulysses the whole
        row is padded to a multiple of sp and each rank keeps one contiguous
        chunk of it."""
        mult = 2 * self.cp_size if self.cp_size > 1 else 1
        ids, labs, poss, lens = [], [], [], []
        for it in items:
            n = it['input_ids'].numel()
            pad = (-n) % mult if mult > 1 else 0
            if pad:
                ids.append(torch.cat([it['input_ids'], torch.full((pad, ), self.pad_token_id, dtype=torch.long)]))
                labs.append(torch.cat([it['labels'], torch.full((pad, ), -100, dtype=torch.long)]))
                last = int(it['position_ids'][-1]) if n else -1
                poss.append(torch.cat([it['position_ids'], torch.arange(last + 1, last + 1 + pad)]))
            else:
                ids.append(it['input_ids'])
                labs.append(it['labels'])
                poss.append(it['position_ids'])
            lens.append(n + pad)
        # the whole row must divide evenly among the sequence-parallel ranks:
        # extend the last sequence with ignored tokens
        total = sum(lens)
        tail = (-total) % max(pad_multiple if pad_multiple is not None else self.sp_size, 1)
        if tail and ids:
            last = int(poss[-1][-1]) if poss[-1].numel() else -1
            ids[-1] = torch.cat([ids[-1], torch.full((tail, ), self.pad_token_id, dtype=torch.long)])
            labs[-1] = torch.cat([labs[-1], torch.full((tail, ), -100, dtype=torch.long)])
            poss[-1] = torch.cat([poss[-1], torch.arange(last + 1, last + 1 + tail)])
            lens[-1] += tail
        input_ids, labels, position_ids = torch.cat(ids), torch.cat(labs), torch.cat(poss)
        # a packed *feature* may itself hold several documents (PackingDataset): boundaries come from position resets
        cu = cu_seqlens_from_position_ids(position_ids)
        seg = (cu[1:] - cu[:-1])
        mb = MicroBatch(input_ids, position_ids, labels, cu, int(seg.max()) if seg.numel() else 0, lens)
        extras = {}
        if any('routed_experts' in it for it in items):
            extras['routed_experts'] = [it.get('routed_experts') for it in items]
        if any('pixel_values' in it for it in items):
            # images travel beside the packed row: all patches in token order, their grids, and (time, height, width)
            # positions for every token (text-only sequences and padding count up in all three components alike)
            mpos = []
            for it, n in zip(items, lens):
                m = torch.as_tensor(it['mrope_position_ids']).long() if 'mrope_position_ids' in it else torch.arange(it['input_ids'].numel()).expand(3, -1)
                extra = n - m.shape[1]
                if extra > 0:
                    start = int(m.max()) + 1 if m.numel() else 0
                    m = torch.cat([m, torch.arange(start, start + extra).expand(3, -1)], 1)
                mpos.append(m)
            extras['mrope_position_ids'] = torch.cat(mpos, 1)
            extras['pixel_values'] = torch.cat([torch.as_tensor(it['pixel_values']) for it in items if 'pixel_values' in it], 0)
            extras['placeholder_ids'] = sorted({int(t) for it in items for t in (it.get('placeholder_ids') or ())})
            extras['image_grid_thw'] = torch.cat([torch.as_tensor(it['image_grid_thw']).long().view(-1, 3) for it in items if 'pixel_values' in it], 0)
        mb.extras = extras or None
        if not split:
            return mb
        out = self._split_parallel(mb)
        if out.local_index is not None and extras.get('pixel_values') is not None:
            # sequence / context parallel: every rank runs the tower on all images (they are small next to the language
            # model) and keeps the features of the placeholder tokens in its share of the row, plus its columns of the positions
            is_ph = torch.zeros(input_ids.numel(), dtype=torch.bool)
            for it_ids in (extras.get('placeholder_ids') or ()):
                is_ph |= input_ids == it_ids
            ordinal = torch.cumsum(is_ph.long(), 0) - 1
            local = out.local_index
            out.extras = dict(extras, mrope_position_ids=extras['mrope_position_ids'][:, local], vision_rows=ordinal[local][is_ph[local]])
        return out

    def _split_parallel(self, mb: MicroBatch) -> MicroBatch:
        """Keep this rank's share of every sequence: contiguous slices for
        Ulysses SP, zig-zag chunk pairs for CP.  ``cu_seqlens`` keeps describing
        the FULL sequences (attention runs on full sequences after the head
        exchange / ring)."""
        if self.sp_size <= 1 and self.cp_size <= 1:
            return mb
        total = int(mb.input_ids.numel())
        if self.cp_size > 1:
            idx, off = [], 0
            for n in mb.seq_lens:
                idx.append(zigzag_indices(n, self.cp_size, self.cp_rank) + off)
                off += n
            index = torch.cat(idx)
        else:
            index = torch.arange(total)
        if self.sp_size > 1:
            c = index.numel() // self.sp_size
            index = index[self.sp_rank * c:(self.sp_rank + 1) * c]
        return MicroBatch(mb.input_ids[index], mb.position_ids[index], mb.labels[index], mb.cu_seqlens, mb.max_seqlen,
                          mb.seq_lens, index, mb.extras)

    def __call__(self, features: Sequence[InputFeature]) -> List[MicroBatch]:
        items = self.normalize(features)
        return [self._pack(g) for g in self.split_micro_batches(items)]

    # -------------------------------------------------------------- outputs
    @staticmethod
    def unpack_packed_sequences(flat: torch.Tensor, seq_lens: Sequence[int], pad_value=0) -> torch.Tensor:
        """``[ΣT, …]`` → ``[n_seq, max_len, …]`` right-padded."""
        n, m = len(seq_lens), max(seq_lens) if seq_lens else 0
        out = flat.new_full((n, m) + tuple(flat.shape[1:]), pad_value)
        off = 0
        for i, L in enumerate(seq_lens):
            out[i, :L] = flat[off:off + L]
            off += L
        return out

    @staticmethod
    def restore_full_order(local: torch.Tensor, gathered: torch.Tensor, indices: Sequence[torch.Tensor]) -> torch.Tensor:
        """Place per-rank pieces (``gathered`` = concat over ranks) back at their
        positions ``indices[r]`` of the full packed row."""
        total = sum(int(i.numel()) for i in indices)
        out = gathered.new_zeros((total, ) + tuple(gathered.shape[1:]))
        off = 0
        for idx in indices:
            n = idx.numel()
            out[idx.to(out.device)] = gathered[off:off + n]
            off += n
        return out
