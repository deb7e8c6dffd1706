"""Runtime: global initialisation and the remote-component decorators.

Parity: reference ``src/twinkle/infra/__init__.py:80-153`` (``initialize``),
``:507-687`` (``remote_class``), ``:690-833`` (``remote_function``),
``:292-467`` (dispatch / collect rules) and ``infra/collectors.py``.

Modes:

* ``local`` — the script itself runs under ``torchrun`` (one process per GPU);
  decorated classes are plain objects, decorated methods are direct calls.
* ``pool`` — what the reference does with Ray actors: a *driver* process owns
  proxies, each decorated class is instantiated once per rank of its
  ``DeviceGroup`` inside a worker process started by ``infra.worker_pool``
  (``multiprocessing`` + pipes; Ray is not a dependency), and method calls
  are dispatched / collected by the rules below.  ``mode='ray'`` is accepted as
  an alias of ``pool``.
"""
from __future__ import annotations

import functools
import inspect
import os
import sys
import traceback
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import numpy as np

from ..utils.device_mesh import DeviceGroup, DeviceMesh
from ..utils.loader import check_unsafe
from ..utils.logger import get_logger
from ..utils.platform import Platform

logger = get_logger()

_STATE: Dict[str, Any] = dict(mode='local', seed=42, mesh=None, groups=[], lazy_collect=False, notifier=None,
                              initialized=False, pool=None, full_determinism=False)


def initialize(mode: str = 'local', nproc_per_node: Optional[int] = None, groups: Optional[List[DeviceGroup]] = None,
               global_device_mesh: Optional[DeviceMesh] = None, lazy_collect: bool = False, seed: int = 42,
               full_determinism: bool = False, notifier=None, **kwargs) -> None:
    """Set the process-wide runtime state.  In ``local`` mode a default
    ``dp``-only mesh over ``WORLD_SIZE`` is built when none is given and the
    mesh size is checked against the launcher's world size."""
    from ..utils.framework import Torch
    mode = os.environ.get('TWINKLE_MODE', mode)
    if mode == 'ray':
        mode = 'pool'
    if mode not in ('local', 'pool'):
        raise ValueError(f'unknown mode {mode!r}')
    seed = int(os.environ.get('TWINKLE_SEED', seed))
    Torch.seed_everything(seed, full_determinism)
    world = Platform.get_world_size()
    if mode == 'local':
        if global_device_mesh is None:
            global_device_mesh = DeviceMesh.from_sizes(dp_size=world)
        if global_device_mesh.world_size != world:
            raise AssertionError(f'device mesh has {global_device_mesh.world_size} ranks but WORLD_SIZE is {world}')
        if not groups:
            groups = [DeviceGroup(name='default', ranks=list(range(world)), device_type=Platform.device_prefix())]
    else:
        from .worker_pool import WorkerPoolManager
        if not groups:
            n = nproc_per_node or (global_device_mesh.world_size if global_device_mesh is not None else 1)
            groups = [DeviceGroup(name='default', ranks=list(range(n)), device_type=Platform.device_prefix())]
        # pool_listen='host:port' + external_groups=[names]: those groups' workers join from other nodes (see infra/agent.py)
        _STATE['pool'] = WorkerPoolManager(groups, seed=seed, listen=kwargs.get('pool_listen'), external_groups=kwargs.get('external_groups'),
                                           join_timeout=float(kwargs.get('join_timeout', 600.0)))
    _STATE.update(mode=mode, seed=seed, mesh=global_device_mesh, groups=groups, lazy_collect=lazy_collect,
                  notifier=notifier, initialized=True, full_determinism=full_determinism)


def is_initialized() -> bool:
    return bool(_STATE['initialized'])


def get_mode() -> str:
    return _STATE['mode']


def get_global_device_mesh() -> Optional[DeviceMesh]:
    return _STATE['mesh']


def get_device_placement(device_group: Optional[Sequence[DeviceGroup]] = None) -> str:
    """Human-readable table: group → ranks → mesh coordinates, of the given device groups or of those ``initialize`` was
    called with (reference ``infra/__init__.py:156-260``)."""
    groups = list(device_group) if device_group is not None else _STATE['groups']
    if not groups:
        return 'No device group provided.'
    lines = []
    for g in groups:
        lines.append(f"group '{g.name}' ({g.device_type}, {g.gpus_per_worker} gpu/worker): ranks {g.rank_list()}")
        for cls_name, mesh in g._device_mesh.items():
            lines.append(f'  {cls_name}: dims {mesh.mesh_dim_names} shape {tuple(mesh.mesh.shape)}')
            for r in mesh.mesh.reshape(-1).tolist():
                lines.append(f'    rank {r}: coord {mesh.coord_of(r)} data_rank {mesh.get_data_rank_from_global_rank(r)}')
    return '\n'.join(lines)


def shutdown() -> None:
    pool = _STATE.get('pool')
    if pool is not None:
        pool.shutdown()
    _STATE.update(pool=None, initialized=False, mode='local')


# ------------------------------------------------------------------ dispatch
def _chunk_bounds(n: int, parts: int, i: int):
    k, m = divmod(n, parts)
    return i * k + min(i, m), (i + 1) * k + min(i + 1, m)


def dispatch_args(dispatch: Union[str, Callable], n_workers: int, args: tuple, kwargs: dict,
                  device_mesh: Optional[DeviceMesh] = None, worker_ranks: Optional[Sequence[int]] = None):
    """Per-worker (args, kwargs) according to the dispatch rule.

    ``all``: identical arguments; ``slice``: every *list* argument is cut into
    ``n`` near-equal contiguous chunks; ``slice_dp``: lists / tensors / arrays
    and (recursively) dict values are cut with the mesh's ``get_slice`` for the
    worker's data rank, so tp/pp/sp peers receive the same slice; scalars are
    replicated.  A batch that would leave some workers empty raises
    ``ValueError('Batch too small…')``.
    """
    if callable(dispatch):
        return dispatch(n_workers, args, kwargs, device_mesh=device_mesh)
    if dispatch == 'all' or n_workers == 1 and dispatch != 'slice_dp':
        return [(args, kwargs) for _ in range(n_workers)]
    import torch

    if dispatch == 'slice':

        def cut(v, i):
            if isinstance(v, list):
                a, b = _chunk_bounds(len(v), n_workers, i)
                return v[a:b]
            return v
    elif dispatch == 'slice_dp':
        if device_mesh is None:
            raise ValueError("dispatch='slice_dp' needs a device mesh")
        ranks = list(worker_ranks) if worker_ranks is not None else list(range(n_workers))
        lengths = []

        def cut(v, i):
            dr = device_mesh.get_data_rank_from_global_rank(ranks[i])
            if isinstance(v, (list, tuple)) and not isinstance(v, str):
                sl = device_mesh.get_slice(len(v), dr)
                lengths.append((len(v), sl.stop - sl.start))
                return type(v)(v[sl]) if isinstance(v, tuple) else v[sl]
            if isinstance(v, (torch.Tensor, np.ndarray)) and v.ndim >= 1:
                sl = device_mesh.get_slice(v.shape[0], dr)
                lengths.append((v.shape[0], sl.stop - sl.start))
                return v[sl]
            if isinstance(v, dict):
                return {k: cut(x, i) for k, x in v.items()}
            return v
    else:
        raise ValueError(f'unknown dispatch {dispatch!r}')
    out = []
    for i in range(n_workers):
        out.append((tuple(cut(a, i) for a in args), {k: cut(v, i) for k, v in kwargs.items()}))
    if dispatch == 'slice_dp':
        if any(total > 0 and got == 0 for total, got in lengths) and any(got > 0 for _, got in lengths):
            raise ValueError('Batch too small: some data-parallel workers would receive no samples '
                             f'(data_world_size={device_mesh.data_world_size}).')
    return out


def collect_results(collect: Union[str, Callable], results: List[Any], device_mesh: Optional[DeviceMesh] = None,
                    worker_ranks: Optional[Sequence[int]] = None):
    """Merge per-worker results.  Tuples are collected element-wise."""
    if callable(collect):
        return collect(results, device_mesh=device_mesh)
    if not results:
        return None
    if isinstance(results[0], tuple) and collect not in ('none', 'first'):
        return tuple(collect_results(collect, [r[i] for r in results], device_mesh, worker_ranks)
                     for i in range(len(results[0])))
    if collect == 'none':
        return results[0] if len(results) == 1 else results
    if collect == 'first':
        return results[0]
    if collect == 'flatten':
        out = []
        for r in results:
            if isinstance(r, (list, tuple)):
                out.extend(r)
            elif r is not None:
                out.append(r)
        return out
    if collect in ('mean', 'avg', 'sum'):
        red = np.mean if collect != 'sum' else np.sum
        if isinstance(results[0], dict):
            out = {}
            for k in results[0]:
                vals = [r[k] for r in results if k in r]
                try:
                    out[k] = float(red([float(v) for v in vals]))
                except (TypeError, ValueError):
                    out[k] = vals
            return out
        return float(red([float(r) for r in results]))
    if collect in ('last_pp', 'last_pp_first'):
        ranks = list(worker_ranks) if worker_ranks is not None else list(range(len(results)))
        last = set((device_mesh.get_pp_last_ranks() or ranks) if device_mesh is not None else ranks)
        kept = [r for r, rk in zip(results, ranks) if rk in last] or results
        return kept[0] if collect == 'last_pp_first' else kept
    raise ValueError(f'unknown collect {collect!r}')


def collect_tensor_dict(results: List[Dict[str, Any]], device_mesh: Optional[DeviceMesh] = None,
                        worker_ranks: Optional[Sequence[int]] = None) -> Dict[str, Any]:
    """Merge model-output dicts of the collect ranks: tensors are padded to a
    common trailing length and concatenated on dim 0, lists extended, nested
    dicts recursed, ``loss`` averaged (reference ``infra/collectors.py:8-55``)."""
    import torch
    if device_mesh is not None and worker_ranks is not None:
        keep = set(device_mesh.get_collect_ranks())
        results = [r for r, rk in zip(results, worker_ranks) if rk in keep] or results
    results = [r for r in results if r is not None]
    if not results:
        return {}
    out: Dict[str, Any] = {}
    for k in results[0]:
        vals = [r[k] for r in results if k in r and r[k] is not None]
        if not vals:
            out[k] = None
        elif k == 'loss':
            out[k] = float(np.mean([float(v) for v in vals]))
        elif isinstance(vals[0], torch.Tensor):
            if vals[0].dim() == 0:
                out[k] = torch.stack([v.cpu() for v in vals])
            else:
                width = max(v.shape[-1] for v in vals) if vals[0].dim() >= 2 else None
                padded = []
                for v in vals:
                    v = v.cpu()
                    if width is not None and v.shape[-1] < width:
                        v = torch.nn.functional.pad(v, (0, width - v.shape[-1]))
                    padded.append(v)
                out[k] = torch.cat(padded, 0)
        elif isinstance(vals[0], list):
            out[k] = [x for v in vals for x in v]
        elif isinstance(vals[0], dict):
            out[k] = collect_tensor_dict(vals)
        elif isinstance(vals[0], (int, float)):
            out[k] = float(np.sum(vals)) if k == 'num_tokens' else float(np.mean(vals))
        else:
            out[k] = vals[0]
    return out


# ---------------------------------------------------------------- decorators
class LazyCollect:
    """Deferred result of a remote call; calling it collects.  Passing it to
    another remote call hands each worker its own un-collected piece."""

    def __init__(self, futures, collect, device_mesh, worker_ranks):
        self.futures, self.collect, self.mesh, self.ranks = futures, collect, device_mesh, worker_ranks
        self._value = None
        self._done = False

    def per_worker(self):
        return [f() if callable(f) else f for f in self.futures]

    def __call__(self):
        if not self._done:
            self._value = collect_results(self.collect, self.per_worker(), self.mesh, self.ranks)
            self._done = True
        return self._value


def _notify(exc: BaseException, where: str) -> None:
    n = _STATE.get('notifier')
    if n is None:
        return
    try:
        n.notify(f'{type(exc).__name__}: {exc}\n at {where}\n{traceback.format_exc()}')
    except Exception:  # a broken notifier must never mask the real error
        pass


def remote_function(dispatch: Union[str, Callable] = 'all', execute: str = 'all', collect: Union[str, Callable] = 'none',
                    sync: bool = False, lazy_collect: Optional[bool] = None, timeout: Optional[float] = None):
    """Method decorator.  ``execute``: ``first`` (only worker 0 runs, gets the
    full arguments), ``peer`` (the worker paired with the caller's rank) or
    ``all``.  In local mode the method is called directly (the launcher already
    runs one process per rank); in pool mode the driver proxy applies
    dispatch → remote call → collect."""

    def deco(fn):
        fn._remote_spec = dict(dispatch=dispatch, execute=execute, collect=collect, sync=sync, lazy_collect=lazy_collect,
                               timeout=timeout)

        @functools.wraps(fn)
        def wrapper(self, *args, **kwargs):
            proxy = getattr(self, '_remote_proxy', None)
            if proxy is not None:
                check_unsafe(*args, **kwargs)       # safe mode: nothing executable travels to a worker
                return proxy.call(fn.__name__, fn._remote_spec, args, kwargs)
            try:
                return fn(self, *args, **kwargs)
            except Exception as e:
                frame = inspect.stack()[1]
                _notify(e, f'{frame.filename}:{frame.lineno}')
                raise

        wrapper._remote_spec = fn._remote_spec
        return wrapper

    return deco


def remote_class(execute: str = 'all'):
    """Class decorator.  Local mode: injects the global mesh into a constructor
    argument annotated ``DeviceMesh`` when the caller passed none.  Pool mode
    (driver side): ``Cls(..., remote_group='name')`` creates one worker object
    per rank of that group and returns a proxy whose decorated methods
    dispatch to them."""

    def deco(cls):
        orig_init = cls.__init__
        sig = inspect.signature(orig_init)
        mesh_arg = None
        for name, p in sig.parameters.items():
            ann = p.annotation
            if ann is DeviceMesh or ann == 'DeviceMesh' or ann == Optional[DeviceMesh] or 'DeviceMesh' in str(ann):
                mesh_arg = name
                break

        @functools.wraps(orig_init)
        def new_init(self, *args, remote_group: Optional[str] = None, **kwargs):
            self._remote_proxy = None
            check_unsafe(*args, **kwargs)
            if _STATE['mode'] == 'pool' and remote_group is not None and not os.environ.get('TWINKLE_WORKER'):
                from .worker_pool import RemoteProxy
                self._remote_proxy = RemoteProxy(_STATE['pool'], cls, remote_group, execute, args, kwargs, mesh_arg)
                return
            if mesh_arg is not None:
                bound = sig.bind_partial(self, *args, **kwargs)
                if bound.arguments.get(mesh_arg) is None and _STATE['mesh'] is not None:
                    kwargs[mesh_arg] = _STATE['mesh']
            orig_init(self, *args, **kwargs)

        cls.__init__ = new_init
        cls._remote_execute = execute
        cls._remote_mesh_arg = mesh_arg
        return cls

    return deco


__all__ = ['initialize', 'is_initialized', 'get_mode', 'get_global_device_mesh', 'get_device_placement', 'shutdown',
           'remote_class', 'remote_function', 'dispatch_args', 'collect_results', 'collect_tensor_dict', 'LazyCollect',
           'DeviceMesh', 'DeviceGroup']
