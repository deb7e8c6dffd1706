"""Logical topology: a named N-d grid of global ranks.

Parity: reference ``src/twinkle/utils/device_mesh.py:11-553`` — same constructor
surface (``DeviceMesh.from_sizes``), same rank arithmetic (``data_rank``,
``data_world_size``, ``get_slice``, ``get_collect_ranks``) and the same
``DeviceGroup`` record.  The implementation keeps one coordinate table
(rank -> coordinate tuple) built once, instead of searching the grid on every
query, and caches one process group per (dim, orthogonal coordinate).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from itertools import product
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np

from .platform import Platform

_VALID_DIMS = ('dp', 'fsdp', 'tp', 'pp', 'cp', 'ep', 'ep_fsdp')


@dataclass
class DeviceMesh:
    """Grid of ranks with named axes.

    Axes: ``dp`` data parallel (replicas), ``fsdp`` sharded data parallel,
    ``tp`` tensor parallel, ``pp`` pipeline, ``cp`` context parallel, ``ep``
    / ``ep_fsdp`` expert-parallel 2-D sub-mesh.  Scalar knobs that do not add
    ranks: ``ulysses_size`` (sequence parallel carved out of dp×fsdp ranks),
    ``ep_size`` / ``ep_fsdp_size`` / ``etp_size``, ``vpp_size`` (virtual
    pipeline chunks per stage), ``sequence_parallel`` (activations sharded on
    the sequence inside a tp group).
    """
    mesh: np.ndarray
    mesh_dim_names: Optional[Tuple[str, ...]]
    ep_size: Optional[int] = None
    etp_size: Optional[int] = None
    ep_fsdp_size: Optional[int] = None
    vpp_size: Optional[int] = None
    ulysses_size: Optional[int] = None
    sequence_parallel: bool = False
    device_type: Optional[str] = None

    def signature(self) -> tuple:
        """Hashable description of the layout.  Caches of process groups are keyed by it: equal meshes share their
        groups, and a key can never be taken over by a different mesh that reuses a freed object's address."""
        m = np.asarray(self.mesh)
        return (m.shape, m.tobytes(), tuple(self.mesh_dim_names or ()), self.ep_size, self.etp_size, self.ep_fsdp_size, self.ulysses_size)

    # ------------------------------------------------------------------ build
    @staticmethod
    def from_sizes(*, world_size: int = 1, dp_size: Optional[int] = 1, fsdp_size: Optional[int] = None,
                   tp_size: Optional[int] = None, pp_size: Optional[int] = None, ulysses_size: Optional[int] = None,
                   cp_size: Optional[int] = None, ep_size: Optional[int] = None, etp_size: int = 1,
                   ep_fsdp_size: Optional[int] = None, vpp_size: Optional[int] = None,
                   device_type: Optional[str] = None, sequence_parallel: bool = False) -> 'DeviceMesh':
        """Axis order is fixed: fsdp, pp, dp, cp, tp (outermost first).  When
        ``world_size`` is left at 1 it is inferred as the product of the given
        sizes; ``dp_size=None`` makes dp the inferred (−1) axis."""
        axes: List[Tuple[str, Optional[int]]] = [('fsdp', fsdp_size), ('pp', pp_size), ('dp', dp_size if dp_size is not None else -1),
                                                 ('cp', cp_size), ('tp', tp_size)]
        names, sizes = [], []
        inferred = world_size
        for name, size in axes:
            if size is None:
                continue
            sizes.append(size)
            if size == -1:
                continue  # unnamed free axis, kept for reshape inference
            names.append(name)
            if world_size == 1:
                inferred *= size
        if ep_size is not None and ep_size > 1 and ep_fsdp_size is None:
            ep_fsdp_size = max(inferred // ep_size, 1)
        grid = np.arange(inferred).reshape(sizes)
        if dp_size is None:
            # the free axis was sized by reshape; name it so ndim matches
            names.insert([n for n, s in axes if s is not None].index('dp'), 'dp')
        return DeviceMesh(mesh=grid, mesh_dim_names=tuple(names), ep_size=ep_size, etp_size=etp_size,
                          ep_fsdp_size=ep_fsdp_size, vpp_size=vpp_size, ulysses_size=ulysses_size,
                          sequence_parallel=sequence_parallel, device_type=device_type)

    def __post_init__(self):
        if self.device_type is None:
            try:
                self.device_type = Platform.device_prefix()
            except Exception:
                self.device_type = 'cuda'
        if not isinstance(self.mesh, np.ndarray):
            self.mesh = np.array(self.mesh)
        if self.mesh_dim_names is not None:
            self.mesh_dim_names = tuple(self.mesh_dim_names)
            if len(self.mesh_dim_names) != self.mesh.ndim:
                raise ValueError(f'mesh_dim_names has {len(self.mesh_dim_names)} entries but mesh has {self.mesh.ndim} axes')
            bad = [n for n in self.mesh_dim_names if n not in _VALID_DIMS]
            if bad:
                raise ValueError(f'unknown mesh axes {bad}; valid: {_VALID_DIMS}')
        self._coord_of: Dict[int, Tuple[int, ...]] = {
            int(self.mesh[idx]): tuple(int(i) for i in idx) for idx in np.ndindex(*self.mesh.shape)
        }
        self._groups: Dict[Tuple[str, ...], Dict[Tuple[int, ...], object]] = {}

    # ---------------------------------------------------------------- lookups
    def _axis(self, name: str) -> Optional[int]:
        if self.mesh_dim_names is None or name not in self.mesh_dim_names:
            return None
        return self.mesh_dim_names.index(name)

    def has_dim(self, dim_name: str) -> bool:
        return self._axis(dim_name) is not None

    _has_dim = has_dim

    def get_dim_size(self, dim_name: str) -> int:
        ax = self._axis(dim_name)
        if ax is None:
            raise ValueError(f"axis '{dim_name}' not in mesh {self.mesh_dim_names}")
        return int(self.mesh.shape[ax])

    def coord_of(self, rank: Optional[int] = None) -> Optional[Tuple[int, ...]]:
        rank = Platform.get_rank() if rank is None else rank
        return self._coord_of.get(int(rank))

    _get_coord_for_rank = coord_of

    def _get_coord(self):
        return self.coord_of(None)

    def _rank_on(self, name: str, rank: Optional[int] = None) -> Optional[int]:
        ax = self._axis(name)
        c = self.coord_of(rank)
        if ax is None or c is None:
            return None
        return c[ax]

    def _size_on(self, name: str) -> Optional[int]:
        ax = self._axis(name)
        return None if ax is None else int(self.mesh.shape[ax])

    def ranks_along(self, dims: Union[str, Sequence[str]], rank: Optional[int] = None) -> List[int]:
        """Global ranks of the sub-grid spanned by ``dims`` through ``rank``."""
        if isinstance(dims, str):
            dims = (dims, )
        c = self.coord_of(rank)
        if c is None:
            return []
        index = tuple(slice(None) if n in dims else c[i] for i, n in enumerate(self.mesh_dim_names))
        return [int(r) for r in np.asarray(self.mesh[index]).reshape(-1)]

    # --------------------------------------------------------- process groups
    def create_process_group(self, dims):
        """Collectively create (on every rank) the groups spanned by ``dims``
        and return the one this rank belongs to."""
        import torch.distributed as dist
        if isinstance(dims, str):
            dims = (dims, )
        key = tuple(n for n in self.mesh_dim_names if n in dims)
        if key not in self._groups:
            other_axes = [i for i, n in enumerate(self.mesh_dim_names) if n not in key]
            table = {}
            for other in product(*[range(self.mesh.shape[i]) for i in other_axes]):
                index = [slice(None)] * self.mesh.ndim
                for ax, v in zip(other_axes, other):
                    index[ax] = v
                ranks = [int(r) for r in np.asarray(self.mesh[tuple(index)]).reshape(-1)]
                table[other] = dist.new_group(ranks=ranks)
            self._groups[key] = table
        c = self.coord_of(dist.get_rank())
        other = tuple(c[i] for i, n in enumerate(self.mesh_dim_names) if n not in key)
        return self._groups[key][other]

    def get_dim_group(self, dims):
        if isinstance(dims, str):
            dims = (dims, )
        for d in dims:
            if not self.has_dim(d):
                raise ValueError(f"axis '{d}' not in mesh {self.mesh_dim_names}")
        return self.create_process_group(dims)

    @property
    def order(self) -> str:
        """Axis nesting used by the tensor/pipeline engine, innermost first."""
        return 'tp-cp-ep-dp-pp'

    def to_torch_device_mesh(self):
        from torch.distributed.device_mesh import DeviceMesh as TorchMesh
        return TorchMesh(self.device_type, self.mesh, mesh_dim_names=self.mesh_dim_names)

    # ------------------------------------------------------------- properties
    @property
    def is_single_process(self) -> bool:
        return self.world_size == 1

    @property
    def world_size(self) -> int:
        return int(self.mesh.size)

    dp_rank = property(lambda self: self._rank_on('dp'))
    fsdp_rank = property(lambda self: self._rank_on('fsdp'))
    tp_rank = property(lambda self: self._rank_on('tp'))
    pp_rank = property(lambda self: self._rank_on('pp'))
    cp_rank = property(lambda self: self._rank_on('cp'))
    dp_world_size = property(lambda self: self._size_on('dp'))
    fsdp_world_size = property(lambda self: self._size_on('fsdp'))
    tp_world_size = property(lambda self: self._size_on('tp'))
    pp_world_size = property(lambda self: self._size_on('pp'))
    cp_world_size = property(lambda self: self._size_on('cp'))

    @property
    def ep_world_size(self) -> Optional[int]:
        return self.ep_size if self.ep_size else self._size_on('ep')

    @property
    def ep_rank(self) -> Optional[int]:
        if self.has_dim('ep'):
            return self._rank_on('ep')
        if self.ep_size and self.ep_size > 1:
            # EP groups are consecutive blocks of the flattened dp×fsdp order.
            return self._flat_data_index(None) % self.ep_size
        return None

    @property
    def ep_fsdp_rank(self) -> Optional[int]:
        if self.has_dim('ep_fsdp'):
            return self._rank_on('ep_fsdp')
        if self.ep_size and self.ep_size > 1:
            return self._flat_data_index(None) // self.ep_size
        return None

    @property
    def etp_world_size(self) -> int:
        if self.etp_size is not None:
            return self.etp_size
        return self.tp_world_size or 1

    @property
    def ulysses_rank(self) -> int:
        return self._flat_data_index(None) % (self.ulysses_size or 1)

    # ------------------------------------------------------------ data ranks
    def _flat_data_index(self, rank: Optional[int]) -> int:
        """Position of ``rank`` in the flattened (dp, fsdp) order before the
        Ulysses division."""
        dp_r, fs_r = self._rank_on('dp', rank), self._rank_on('fsdp', rank)
        fs_ws = self._size_on('fsdp') or 0
        idx = dp_r
        if fs_ws > 1:
            if dp_r is not None and fs_r is not None:
                idx = dp_r * fs_ws + fs_r
            elif fs_r is not None:
                idx = fs_r
        return 0 if idx is None else int(idx)

    @property
    def data_rank(self) -> Optional[int]:
        """Index of the distinct data shard this rank consumes: ranks that
        differ only in tp/pp/cp/ulysses position share a data rank."""
        return self._flat_data_index(None) // (self.ulysses_size or 1)

    def get_data_rank_from_global_rank(self, global_rank: int) -> int:
        if self.coord_of(global_rank) is None:
            return 0
        return self._flat_data_index(global_rank) // (self.ulysses_size or 1)

    def _get_dp_fsdp_world_size(self) -> int:
        dp = self.dp_world_size or 1
        fs = self.fsdp_world_size or 1
        return max(dp, 1) * max(fs, 1)

    @property
    def data_world_size(self) -> int:
        dp, fs = self.dp_world_size, self.fsdp_world_size
        if fs is not None and fs > 1:
            n = fs * (dp if dp is not None else 1)
        else:
            n = dp if dp is not None else 1
        u = self.ulysses_size or 1
        if n % u != 0:
            raise AssertionError(f'data_world_size: {n} cannot be divided by ulysses_size: {u}.')
        return n // u

    def get_slice(self, total_length: int, rank: Optional[int] = None) -> slice:
        """Balanced contiguous split: the first ``total % n`` shards get one
        extra element."""
        n = self.data_world_size
        if n == 1:
            return slice(0, total_length)
        if rank is None:
            rank = self.data_rank
            if rank is None:
                return slice(0, total_length)
        k, m = divmod(total_length, n)
        lo = rank * k + min(rank, m)
        hi = (rank + 1) * k + min(rank + 1, m)
        return slice(lo, hi)

    # ------------------------------------------------------------ tp helpers
    def get_tp_ranks(self) -> List[int]:
        rank = Platform.get_rank()
        if not self.has_dim('tp'):
            return [rank]
        return sorted(self.ranks_along('tp', rank))

    def get_tp_last_ranks(self) -> List[int]:
        if not self.has_dim('tp'):
            return [int(r) for r in self.mesh.reshape(-1)]
        ax = self._axis('tp')
        return sorted(int(r) for r in np.take(self.mesh, self.mesh.shape[ax] - 1, axis=ax).reshape(-1))

    def is_tp_last_rank(self, rank: Optional[int] = None) -> bool:
        if not self.has_dim('tp'):
            return True
        r = self._rank_on('tp', Platform.get_rank() if rank is None else rank)
        return r is not None and r == self.tp_world_size - 1

    # ------------------------------------------------------------ pp helpers
    def get_pp_stage_ranks(self, stage: int) -> Optional[List[int]]:
        ax = self._axis('pp')
        if ax is None:
            if stage == 0:
                return [int(r) for r in self.mesh.reshape(-1)]
            return None
        return sorted(int(r) for r in np.take(self.mesh, stage, axis=ax).reshape(-1))

    def get_pp_first_ranks(self) -> Optional[List[int]]:
        return self.get_pp_stage_ranks(0)

    def get_pp_last_ranks(self) -> Optional[List[int]]:
        return self.get_pp_stage_ranks((self.pp_world_size or 1) - 1)

    def is_pp_first_rank(self) -> bool:
        r = self.get_pp_first_ranks()
        return bool(r) and Platform.get_rank() in r

    def is_pp_last_rank(self) -> bool:
        r = self.get_pp_last_ranks()
        return bool(r) and Platform.get_rank() in r

    def get_collect_ranks(self) -> List[int]:
        """One representative global rank per data rank (lowest rank, taken
        from the last pipeline stage when there is a pp axis): the ranks whose
        outputs are gathered after a ``slice_dp`` dispatch."""
        last = set(self.get_pp_last_ranks() or [])
        chosen: Dict[int, int] = {}
        for r in sorted(self._coord_of):
            d = self.get_data_rank_from_global_rank(r)
            prefer = r in last
            if d not in chosen:
                chosen[d] = r
                continue
            cur = chosen[d]
            if prefer and cur not in last:
                chosen[d] = r
        # second pass: prefer a last-stage rank if any exists for that data rank
        for r in sorted(self._coord_of):
            d = self.get_data_rank_from_global_rank(r)
            if r in last and chosen[d] not in last:
                chosen[d] = r
        return sorted(chosen[d] for d in range(self.data_world_size) if d in chosen)


@dataclass
class DeviceGroup:
    """A named set of ranks (GPUs) that hosts one kind of component — e.g.
    ``model`` on ranks 0-5 and ``sampler`` on ranks 6-7."""
    name: str
    ranks: Union[List[int], int]
    device_type: str = 'cuda'
    gpus_per_worker: int = 1
    visible_devices: Optional[Union[List[str], List[int], str, int]] = None
    _device_mesh: Dict[str, DeviceMesh] = field(default_factory=dict)

    def rank_list(self) -> List[int]:
        return list(range(self.ranks)) if isinstance(self.ranks, int) else list(self.ranks)

    def num_workers(self) -> int:
        return max(len(self.rank_list()) // max(self.gpus_per_worker, 1), 1)


def is_last_rank() -> bool:
    import torch.distributed as dist
    if not dist.is_available() or not dist.is_initialized():
        return True
    return dist.get_rank() == dist.get_world_size() - 1


def is_master() -> bool:
    return Platform.is_master()
