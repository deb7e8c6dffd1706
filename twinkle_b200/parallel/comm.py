"""Collective back ends behind one small interface.

``Communicator`` is what the engines talk to.  Two implementations:

* ``Communicator`` (this file): ``torch.distributed`` calls — NCCL on GPUs,
  gloo on CPU.  This is the baseline path every fused kernel is measured
  against, and the path used for bootstrap, scalars and checkpoints.
* ``parallel.symm.SymmCommunicator``: peer-memory kernels over NVLink
  (all-gather by peer loads, reduce-scatter by peer loads + fp32 accumulate
  fused with the cast/scale), same interface.

Reference call sites covered: FSDP2's all-gather / reduce-scatter
(``strategy/native_fsdp.py:179-205``), grad-norm all-reduce
(``utils/grad_clip.py:208-285``), Ulysses all-to-all
(``sequence_parallel/utils.py:319``), EP all-to-all (``moe/ep_utils.py:32``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class Communicator:

    def __init__(self, group=None, device=None, single: bool = False):
        """``single=True`` forces a one-rank communicator even inside an initialised job (a component
        whose mesh has a single rank must not touch the default process group)."""
        self.group = group
        self.enabled = dist.is_available() and dist.is_initialized() and not single
        self.world_size = dist.get_world_size(group) if self.enabled else 1
        self.rank = dist.get_rank(group) if self.enabled else 0
        self.device = device
        self._stream = None
        self.cuda = bool(device is not None and torch.device(device).type == 'cuda')
        if self.cuda and self.world_size > 1:
            self._stream = torch.cuda.Stream(device=device)

    # ------------------------------------------------------------ all-gather
    def all_gather_async(self, out: torch.Tensor, shard: torch.Tensor):
        """Start gathering ``shard`` from every rank into ``out`` (rank-major).
        Returns a handle for ``wait``.  On GPU the collective runs on a side
        stream so it overlaps the compute stream."""
        if self.world_size == 1:
            if out.data_ptr() != shard.data_ptr():
                out[:shard.numel()].copy_(shard)
            return None
        if self._stream is not None:
            ev_in = torch.cuda.current_stream().record_event()
            with torch.cuda.stream(self._stream):
                self._stream.wait_event(ev_in)
                dist.all_gather_into_tensor(out, shard, group=self.group)
                done = self._stream.record_event()
            out.record_stream(self._stream)
            return done
        return dist.all_gather_into_tensor(out, shard, group=self.group, async_op=True)

    def wait(self, handle) -> None:
        if handle is None:
            return
        if isinstance(handle, torch.cuda.Event):
            torch.cuda.current_stream().wait_event(handle)
        else:
            handle.wait()

    # -------------------------------------------------------- reduce-scatter
    def reduce_scatter_accumulate(self, grad_shard: torch.Tensor, full_grad: torch.Tensor, scale: float = 1.0) -> None:
        """``grad_shard += scale · Σ_ranks full_grad[rank's slice]`` (fp32 accumulate)."""
        if self.world_size == 1:
            grad_shard.add_(full_grad[:grad_shard.numel()], alpha=scale)  # mixed-dtype add: one pass, no fp32 copy first
            return
        n = grad_shard.numel()
        if full_grad.device.type == 'cpu' or full_grad.dtype == torch.float32:
            tmp = torch.empty(n, dtype=full_grad.dtype, device=full_grad.device)
            dist.reduce_scatter_tensor(tmp, full_grad, op=dist.ReduceOp.SUM, group=self.group)
        else:
            tmp = torch.empty(n, dtype=full_grad.dtype, device=full_grad.device)
            dist.reduce_scatter_tensor(tmp, full_grad, op=dist.ReduceOp.SUM, group=self.group)
        grad_shard.add_(tmp, alpha=scale)

    def wait_reduce_scatters(self, all_but: int = 0) -> None:
        """Library reduce-scatters run on the calling stream: nothing is outstanding."""

    # -------------------------------------------------------------- reduce
    def all_reduce(self, t: torch.Tensor, op: str = 'sum') -> torch.Tensor:
        if self.world_size > 1:
            dist.all_reduce(t, op={'sum': dist.ReduceOp.SUM, 'max': dist.ReduceOp.MAX, 'min': dist.ReduceOp.MIN}[op],
                            group=self.group)
        return t

    def all_reduce_scalar(self, v: float, op: str = 'sum') -> float:
        if self.world_size == 1:
            return float(v)
        t = torch.tensor([float(v)], dtype=torch.float64 if not self.cuda else torch.float32,
                         device=self.device if self.cuda else 'cpu')
        self.all_reduce(t, op)
        return float(t.item())

    def all_to_all_single(self, out: torch.Tensor, inp: torch.Tensor, out_splits: Optional[List[int]] = None,
                          in_splits: Optional[List[int]] = None) -> torch.Tensor:
        if self.world_size == 1:
            out.copy_(inp)
            return out
        dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)
        return out

    def all_gather_tensor(self, t: torch.Tensor) -> torch.Tensor:
        """Concatenate equal-shaped ``t`` of every rank along dim 0."""
        if self.world_size == 1:
            return t
        out = torch.empty((self.world_size * t.shape[0], ) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world_size > 1:
            dist.broadcast(t, src=dist.get_global_rank(self.group, src) if self.group is not None else src, group=self.group)
        return t

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier(group=self.group)

    def gather_object(self, obj) -> list:
        if self.world_size == 1:
            return [obj]
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.group)
        return out
