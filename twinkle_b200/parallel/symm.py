"""Peer-memory communicator: collectives as our own kernels over NVLink / NVSwitch.

Every rank of the group allocates *symmetric* buffers (same size on every rank, one ``cudaMalloc`` each),
publishes their CUDA IPC handles through the process group once, and maps the peers' buffers.  Kernels
(``ops/csrc/symm.cu``) then read or write peer memory directly:

* all-gather  = every rank pulls the peers' shards with 16-byte loads (no handshake: parameter shards only
  change in the optimizer step, which is fenced by one cross-GPU barrier per step);
* reduce-scatter = after a flag barrier, every rank pulls its slice of every peer's flat gradient buffer
  and accumulates in fp32 — the bf16→fp32 cast, the ``1/N`` style scale and the accumulation into the
  gradient shard are the same kernel (the reference does an NCCL reduce-scatter followed by separate
  ``grad.div_`` passes, ``utils/grad_clip.py:81-96``);
* Ulysses head↔sequence exchange = each rank pushes its head slices straight into the destination layout.

This replaces NCCL on the FSDP hot path (``strategy/native_fsdp.py:179-205`` in the reference); NCCL stays
for bootstrap and scalars.  Waits inside the kernels are bounded and report through the extension's
error word.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from .comm import Communicator


class SymmBuffer:
    """One symmetric allocation: the local tensor plus the device pointers of every rank's copy."""

    def __init__(self, comm: 'SymmCommunicator', nbytes: int):
        E = ops.ext()
        self.nbytes = (nbytes + 255) // 256 * 256
        self.raw, handle = E.symm_alloc(self.nbytes)
        handles = comm.gather_object(handle)
        self.ptrs: List[int] = []
        for r, h in enumerate(handles):
            self.ptrs.append(self.raw.data_ptr() if r == comm.rank else E.symm_open(h))
        self._comm_rank = comm.rank

    def view(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        t = self.raw[offset_bytes:].view(dtype)
        return t if numel is None else t[:numel]

    def close(self) -> None:
        E = ops.ext()
        for r, p in enumerate(self.ptrs):
            if r != self._comm_rank:
                E.symm_close(p)
        self.ptrs = []


class SymmCommunicator(Communicator):

    def __init__(self, group=None, device=None):
        super().__init__(group, device)
        if not (self.cuda and self.world_size > 1):
            raise RuntimeError('SymmCommunicator needs a multi-GPU CUDA group')
        self.ext = ops.ext()
        self._flags = SymmBuffer(self, 256)
        self._epoch = 0
        self._buffers: List[SymmBuffer] = []
        self._by_ptr: Dict[int, Tuple[SymmBuffer, int]] = {}
        self.copy_blocks = 16  # CTAs per peer stream: enough to fill an NVLink port, few enough to leave SMs to the GEMMs

    # ----------------------------------------------------------- allocation
    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A tensor living in symmetric memory (collective call)."""
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        buf = SymmBuffer(self, nbytes)
        self._buffers.append(buf)
        t = buf.view(dtype, numel)
        self._by_ptr[t.data_ptr()] = (buf, 0)
        return t

    def peer_ptrs(self, t: torch.Tensor) -> Optional[List[int]]:
        hit = self._by_ptr.get(t.data_ptr())
        if hit is None:
            return None
        buf, off = hit
        return [p + off for p in buf.ptrs]

    def barrier_kernel(self) -> None:
        """Cross-GPU barrier on the current stream (flag exchange in peer memory)."""
        self._epoch += 1
        self.ext.symm_barrier(self._flags.ptrs, self.rank, self._epoch)

    # ------------------------------------------------------------ all-gather
    def all_gather_async(self, out: torch.Tensor, shard: torch.Tensor):
        ptrs = self.peer_ptrs(shard)
        if ptrs is None:
            return super().all_gather_async(out, shard)
        nbytes = shard.numel() * shard.element_size()
        ev_in = torch.cuda.current_stream().record_event()
        with torch.cuda.stream(self._stream):
            self._stream.wait_event(ev_in)
            self.ext.peer_all_gather(out, ptrs, nbytes, self.rank, self.copy_blocks)
            done = self._stream.record_event()
        out.record_stream(self._stream)
        return done

    # -------------------------------------------------------- reduce-scatter
    def reduce_scatter_accumulate(self, grad_shard: torch.Tensor, full_grad: torch.Tensor, scale: float = 1.0) -> None:
        ptrs = self.peer_ptrs(full_grad)
        if ptrs is None or grad_shard.dtype != torch.float32 or full_grad.dtype != torch.bfloat16:
            return super().reduce_scatter_accumulate(grad_shard, full_grad, scale)
        # every rank must have finished writing this layer's gradients before anyone reads them
        self.barrier_kernel()
        self.ext.peer_reduce_scatter_acc(grad_shard, ptrs, self.rank, scale, None, 4 * self.copy_blocks)

    def step_barrier(self) -> None:
        """Fences the optimizer step: peers finished reading my shards / gradient buffers."""
        self.barrier_kernel()

    # ---------------------------------------------------------------- Ulysses
    def ulysses_exchange(self, x: torch.Tensor, out: torch.Tensor, seq_to_head: bool, heads_total: int) -> torch.Tensor:
        ptrs = self.peer_ptrs(out)
        assert ptrs is not None, 'destination must be symmetric memory'
        self.barrier_kernel()  # destination buffers are free (previous consumers done)
        self.ext.ulysses_exchange(x, ptrs, self.rank, seq_to_head, heads_total)
        self.barrier_kernel()  # all pushes landed
        return out

    def check(self) -> None:
        code = self.ext.read_and_clear_error()
        if code:
            raise RuntimeError(f'peer-memory kernel gave up waiting (code {code}); a rank is missing or stalled')
