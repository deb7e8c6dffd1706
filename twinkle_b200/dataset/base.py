"""Datasets: loading, mapping, encoding, mixing, saving.

Parity: reference ``src/twinkle/dataset/base.py:30-642`` (``DatasetMeta``, ``Dataset`` with
``set_template / encode / check / map / filter / add_dataset / mix_dataset / save_as``),
``lazy_dataset.py`` (deferred map/encode applied at ``__getitem__``), ``iterable_dataset.py``.

Rows are plain dicts.  Local files (jsonl / json / csv / parquet / arrow / feather, Lance directories when `pylance` is installed) are read directly, in-memory
lists / dicts / generators are accepted, hub ids go through ``HubOperation.load_dataset`` and become
a list of rows.  ``data_slice`` selects row indices with wrap-around.
"""
from __future__ import annotations

import csv
import fcntl
import itertools
import json
import os
import random
import threading
import uuid
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Union

from torch.utils.data import Dataset as TorchDataset
from torch.utils.data import IterableDataset as TorchIterableDataset

from ..infra import remote_class, remote_function
from ..utils.loader import construct_class


@dataclass
class DatasetMeta:
    dataset_id: str = ''
    subset_name: str = 'default'
    split: str = 'train'
    data_slice: Optional[Iterable] = None
    data: Any = None  # list of rows | dict of columns | generator function

    def __post_init__(self):
        self._uid = uuid.uuid4().hex[:8]
        if self.data_slice is not None and not isinstance(self.data_slice, Iterable):
            raise ValueError('data_slice must be an iterable')
        if not self.dataset_id and self.data is None:
            raise ValueError('Either dataset_id or data must be provided')

    def get_id(self) -> str:
        if self.data is not None:
            return f'__memory_{self._uid}__:{self.subset_name}:{self.split}'
        return self.dataset_id.replace(os.sep, '_').replace('.', '_') + f':{self.subset_name}:{self.split}'


def _read_rows(path: str) -> List[Dict[str, Any]]:
    ext = os.path.splitext(path)[1].lower()
    if ext == '.jsonl':
        with open(path) as f:
            return [json.loads(l) for l in f if l.strip()]
    if ext == '.json':
        with open(path) as f:
            d = json.load(f)
        return d if isinstance(d, list) else [dict(zip(d, vals)) for vals in zip(*d.values())]
    if ext == '.csv':
        with open(path, newline='') as f:
            return [dict(r) for r in csv.DictReader(f)]
    if ext == '.parquet':
        import pyarrow.parquet as pq
        return pq.read_table(path).to_pylist()
    if ext in ('.arrow', '.feather'):
        import pyarrow as pa
        with pa.memory_map(path) as src:
            try:
                return pa.ipc.open_file(src).read_all().to_pylist()
            except pa.ArrowInvalid:          # the streaming layout that `datasets` writes
                src.seek(0)
                return pa.ipc.open_stream(src).read_all().to_pylist()
    if ext == '.lance':                      # a Lance dataset is a directory; the reader is an optional package
        try:
            import lance  # type: ignore
        except ImportError as e:
            raise ImportError(f'{path}: reading Lance datasets needs the `pylance` package') from e
        return lance.dataset(path).to_table().to_pylist()
    raise ValueError(f'unsupported dataset file type: {path}')


def load_rows(meta: DatasetMeta, **kwargs) -> List[Dict[str, Any]]:
    if meta.data is not None:
        d = meta.data
        if callable(d):
            rows = list(d())
        elif isinstance(d, dict):
            rows = [dict(zip(d, vals)) for vals in zip(*d.values())]
        elif hasattr(d, 'to_list'):
            rows = d.to_list()
        else:
            rows = [dict(r) for r in d]
    else:
        path = meta.dataset_id
        for p in ('ms://', 'hf://'):
            if path.startswith(p) and os.path.exists(path[len(p):]):
                path = path[len(p):]
        if os.path.isfile(path) or (os.path.isdir(path) and path.rstrip('/').lower().endswith('.lance')):
            rows = _read_rows(path.rstrip('/'))
        elif os.path.isdir(path):
            rows = []
            for fn in sorted(os.listdir(path)):
                if os.path.splitext(fn)[1].lower() in ('.jsonl', '.json', '.csv', '.parquet', '.arrow', '.feather') and (
                        meta.split in fn or not any(s in fn for s in ('train', 'test', 'valid', 'dev'))):
                    rows += _read_rows(os.path.join(path, fn))
        else:
            from ..hub import HubOperation
            ds = HubOperation.load_dataset(meta.dataset_id, None if meta.subset_name == 'default' else meta.subset_name, meta.split,
                                           **{k: v for k, v in kwargs.items() if k in ('revision', 'streaming')})
            rows = ds.to_list() if hasattr(ds, 'to_list') else list(ds)
    if meta.data_slice is not None:
        n = len(rows)
        rows = [rows[i % n] for i in meta.data_slice] if n else []
    return rows


class _WriteThrough:
    """Background writer with an fcntl lock so several processes can append to one file."""

    def __init__(self, path: str, fmt: str):
        self.path, self.fmt = path, fmt
        self._lock = threading.Lock()
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def write(self, row: Dict[str, Any]) -> None:
        with self._lock, open(self.path, 'a') as f:
            fcntl.flock(f, fcntl.LOCK_EX)
            try:
                if self.fmt == 'jsonl':
                    f.write(json.dumps(row, ensure_ascii=False, default=str) + '\n')
                else:
                    w = csv.DictWriter(f, fieldnames=list(row))
                    if f.tell() == 0:
                        w.writeheader()
                    w.writerow(row)
            finally:
                fcntl.flock(f, fcntl.LOCK_UN)


@remote_class(execute='first')
class Dataset(TorchDataset):

    def __init__(self, dataset_meta: Optional[DatasetMeta] = None, **kwargs):
        self.template = None
        self._mixed = False
        self._writer: Optional[_WriteThrough] = None
        self.datasets: Dict[str, List[Dict[str, Any]]] = {}
        self.dataset: Optional[List[Dict[str, Any]]] = None
        if dataset_meta is not None:
            rows = load_rows(dataset_meta, **kwargs)
            self.datasets = {dataset_meta.get_id(): rows}
            self.dataset = rows

    # ------------------------------------------------------------ template
    @remote_function()
    def set_template(self, template_func, **kwargs) -> None:
        from .. import template as T
        self.template = construct_class(template_func, T.Template, T.template_mapping, **kwargs)

    @remote_function()
    def encode(self, add_generation_prompt: bool = False, **kwargs) -> None:
        if self.template is None:
            raise ValueError('set_template must be called before encode')
        out = []
        for row in self._rows():
            r = self.template.encode(row, add_generation_prompt)
            out.extend(r if isinstance(r, list) else [r])
        self._replace(out)

    @remote_function()
    def check(self, **kwargs) -> None:
        """Drop rows the template cannot encode (too long with strategy ``raise``, malformed…)."""
        if self.template is None:
            raise ValueError('set_template must be called before check')
        good = []
        for row in self._rows():
            try:
                self.template.encode(row)
                good.append(row)
            except Exception:
                continue
        self._replace(good)

    # ------------------------------------------------------------ transforms
    def _rows(self) -> List[Dict[str, Any]]:
        return self.dataset or []

    def _replace(self, rows: List[Dict[str, Any]]) -> None:
        self.dataset = rows
        if len(self.datasets) == 1:
            self.datasets[next(iter(self.datasets))] = rows

    @remote_function()
    def map(self, preprocess_func, dataset_meta: Optional[DatasetMeta] = None, batched: bool = False, **kwargs) -> None:
        """``preprocess_func`` may be a callable row→row (or batch→batch), a ``Preprocessor`` instance/class, or
        the name of a built-in preprocessor."""
        from .. import preprocessor as P
        fn = construct_class(preprocess_func, P.Preprocessor, P.preprocessor_mapping, **kwargs.pop('init_args', {})) \
            if not callable(preprocess_func) or isinstance(preprocess_func, type) else preprocess_func
        key = dataset_meta.get_id() if dataset_meta is not None else None
        targets = [key] if key else list(self.datasets)
        for k in targets:
            rows = self.datasets[k]
            if isinstance(fn, P.Preprocessor):
                new = fn(rows)
            elif batched:
                cols = {c: [r.get(c) for r in rows] for c in (rows[0] if rows else {})}
                res = fn(cols)
                new = [dict(zip(res, vals)) for vals in zip(*res.values())]
            else:
                new = [y for y in (fn(r) for r in rows) if y is not None]
            self.datasets[k] = new
        self._refresh()

    @remote_function()
    def filter(self, filter_func, dataset_meta: Optional[DatasetMeta] = None, **kwargs) -> None:
        key = dataset_meta.get_id() if dataset_meta is not None else None
        for k in ([key] if key else list(self.datasets)):
            self.datasets[k] = [r for r in self.datasets[k] if filter_func(r)]
        self._refresh()

    def _refresh(self) -> None:
        if self._mixed or len(self.datasets) > 1:
            self.mix_dataset(getattr(self, '_interleave', True))
        elif self.datasets:
            self.dataset = next(iter(self.datasets.values()))

    @remote_function()
    def add_dataset(self, dataset_meta: DatasetMeta, **kwargs) -> None:
        self.datasets[dataset_meta.get_id()] = load_rows(dataset_meta, **kwargs)
        if self.dataset is None:
            self.dataset = self.datasets[dataset_meta.get_id()]

    @remote_function()
    def mix_dataset(self, interleave: bool = True) -> None:
        """Interleave round-robin (stopping when the shortest is exhausted) or concatenate."""
        parts = list(self.datasets.values())
        self._interleave = interleave
        if interleave and len(parts) > 1:
            n = min(len(p) for p in parts)
            self.dataset = [p[i] for i in range(n) for p in parts]
        else:
            self.dataset = [r for p in parts for r in p]
        self._mixed = True

    # ------------------------------------------------------------------ save
    @remote_function()
    def save_as(self, path: str, mode: str = 'bulk', **kwargs) -> None:
        """``mode='bulk'`` writes all rows now; ``mode='training'`` appends every row that is read through
        ``__getitem__`` (write-through, process-safe)."""
        fmt = {'.jsonl': 'jsonl', '.csv': 'csv', '.parquet': 'parquet'}.get(os.path.splitext(path)[1].lower(), 'jsonl')
        if mode == 'training':
            if fmt == 'parquet':
                raise ValueError('write-through mode supports jsonl and csv')
            self._writer = _WriteThrough(path, fmt)
            return
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        rows = self._rows()
        if fmt == 'jsonl':
            with open(path, 'w') as f:
                for r in rows:
                    f.write(json.dumps(r, ensure_ascii=False, default=str) + '\n')
        elif fmt == 'csv':
            with open(path, 'w', newline='') as f:
                w = csv.DictWriter(f, fieldnames=list(rows[0]) if rows else [])
                w.writeheader()
                w.writerows(rows)
        else:
            import pyarrow as pa
            import pyarrow.parquet as pq
            pq.write_table(pa.Table.from_pylist(rows), path)

    def flush_save(self) -> None:
        """End the write-through started by ``save_as(mode='training')`` (every row was appended and flushed as it was read,
        so nothing is pending; reference ``dataset/base.py:389-394``)."""
        self._writer = None

    def cast_column(self, column: str, decode: bool = True) -> None:
        """Keep an image column as raw bytes (``decode=False``: ``{'bytes': …}`` per image, cheap to carry through ``map``) or
        as decoded images (``decode=True``) — reference ``dataset/base.py:231-241``."""
        import io

        def one(v):
            if isinstance(v, (list, tuple)):
                return [one(x) for x in v]
            if decode:
                raw = v.get('bytes') if isinstance(v, dict) else (v if isinstance(v, (bytes, bytearray)) else None)
                if raw is None:
                    return v
                from PIL import Image
                return Image.open(io.BytesIO(raw)).convert('RGB')
            if hasattr(v, 'save') and hasattr(v, 'mode'):        # a PIL image
                buf = io.BytesIO()
                v.save(buf, format='PNG')
                return {'bytes': buf.getvalue(), 'path': None}
            return v

        for row in self._rows():
            if column in row:
                row[column] = one(row[column])

    def __getitem__(self, idx):
        row = self._rows()[idx]
        if self._writer is not None:
            self._writer.write(row)
        return row

    def __len__(self):
        return len(self._rows())


@remote_class(execute='first')
class LazyDataset(Dataset):
    """``map`` / ``encode`` are recorded and applied when a row is fetched."""

    def __init__(self, dataset_meta: Optional[DatasetMeta] = None, **kwargs):
        super().__init__(dataset_meta, **kwargs)
        self._ops: List[Callable[[Dict[str, Any]], Any]] = []

    @remote_function()
    def map(self, preprocess_func, dataset_meta=None, **kwargs) -> None:
        from .. import preprocessor as P
        fn = preprocess_func
        if isinstance(fn, (str, type)):
            fn = construct_class(fn, P.Preprocessor, P.preprocessor_mapping)
        self._ops.append((lambda r, f=fn: f([r])[0]) if isinstance(fn, P.Preprocessor) else fn)

    @remote_function()
    def encode(self, add_generation_prompt: bool = False, **kwargs) -> None:
        if self.template is None:
            raise ValueError('set_template must be called before encode')
        self._ops.append(lambda r: self.template.encode(r, add_generation_prompt))

    def __getitem__(self, idx):
        row = self._rows()[idx]
        for op in self._ops:
            row = op(row)
        return row


@remote_class(execute='first')
class IterableDataset(TorchIterableDataset):
    """Streaming rows from a generator function or a jsonl file; ``map``/``filter``/``encode`` compose lazily."""

    def __init__(self, dataset_meta: DatasetMeta, **kwargs):
        self.meta = dataset_meta
        self.template = None
        self._ops: List[Callable] = []

    def _source(self) -> Iterator[Dict[str, Any]]:
        m = self.meta
        if callable(m.data):
            yield from m.data()
        elif m.data is not None:
            yield from m.data
        elif m.dataset_id.endswith('.jsonl') and os.path.isfile(m.dataset_id):
            with open(m.dataset_id) as f:
                for l in f:
                    if l.strip():
                        yield json.loads(l)
        else:
            yield from load_rows(m)

    @remote_function()
    def set_template(self, template_func, **kwargs) -> None:
        from .. import template as T
        self.template = construct_class(template_func, T.Template, T.template_mapping, **kwargs)

    @remote_function()
    def map(self, fn, **kwargs) -> None:
        self._ops.append(('map', fn))

    @remote_function()
    def filter(self, fn, **kwargs) -> None:
        self._ops.append(('filter', fn))

    @remote_function()
    def encode(self, add_generation_prompt: bool = False, **kwargs) -> None:
        self._ops.append(('map', lambda r: self.template.encode(r, add_generation_prompt)))

    def __iter__(self):
        for row in self._source():
            keep = True
            for kind, fn in self._ops:
                if kind == 'map':
                    row = fn(row)
                    if row is None:
                        keep = False
                        break
                elif not fn(row):
                    keep = False
                    break
            if keep:
                if isinstance(row, list):
                    yield from row
                else:
                    yield row
