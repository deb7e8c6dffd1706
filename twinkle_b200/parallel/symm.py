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
from ..utils.profiling import PHASES
from .comm import Communicator


class SymmBuffer:
    """One symmetric chunk: the local allocation plus the device pointers of every rank's copy.  Tensors
    are carved out of it with a bump pointer; every rank performs the same sequence of requests, so a
    tensor sits at the same offset on every rank."""

    def __init__(self, comm: 'SymmCommunicator', nbytes: int):
        E = ops.ext()
        self.raw, handle, offset = E.symm_alloc(nbytes)
        self.nbytes = self.raw.numel()
        infos = comm.gather_object((handle, offset, self.nbytes))
        if len({i[2] for i in infos}) != 1:
            raise RuntimeError(f'symmetric allocation sizes differ across ranks: {[i[2] for i in infos]}')
        self.ptrs: List[int] = []
        for r, (h, off, _) in enumerate(infos):
            self.ptrs.append(self.raw.data_ptr() if r == comm.rank else E.symm_open(h) + off)
        self._comm_rank = comm.rank
        self.used = 0

    def carve(self, nbytes: int) -> Optional[int]:
        start = (self.used + 255) // 256 * 256
        if start + nbytes > self.nbytes:
            return None
        self.used = start + nbytes
        return start


class SymmCommunicator(Communicator):

    def __init__(self, group=None, device=None):
        super().__init__(group, device)
        if not (self.cuda and self.world_size > 1):
            raise RuntimeError('SymmCommunicator needs a multi-GPU CUDA group')
        self.ext = ops.ext()
        self.chunk_bytes = 512 << 20
        self._chunks: List[SymmBuffer] = []
        self._by_ptr: Dict[int, Tuple[SymmBuffer, int]] = {}
        self._flags = SymmBuffer(self, 4096)
        self._epoch = 0
        self.copy_blocks = 16  # CTAs per peer stream: enough to fill an NVLink port, few enough to leave SMs to the GEMMs

    # ----------------------------------------------------------- allocation
    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A tensor living in symmetric memory (collective call: every rank of the group must make the
        same request at the same point)."""
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        off = self._chunks[-1].carve(nbytes) if self._chunks else None
        if off is None:
            self._chunks.append(SymmBuffer(self, max(nbytes, self.chunk_bytes)))
            off = self._chunks[-1].carve(nbytes)
        buf = self._chunks[-1]
        t = buf.raw[off:off + nbytes].view(dtype)
        self._by_ptr[t.data_ptr()] = (buf, off)
        return t

    def peer_ptrs(self, t: torch.Tensor) -> Optional[List[int]]:
        hit = self._by_ptr.get(t.data_ptr())
        if hit is None:
            return None
        buf, off = hit
        return [p + off for p in buf.ptrs]

    def sync_all(self) -> None:
        """Host-level rendezvous + device barrier: everything written so far on any rank is visible to all."""
        torch.cuda.synchronize(self.device)
        self.barrier()
        self.barrier_kernel()
        torch.cuda.synchronize(self.device)

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
        with PHASES('fsdp_reduce_scatter'):
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
        with PHASES('ulysses_exchange'):
            self.barrier_kernel()  # destination buffers are free (previous consumers done)
            self.ext.ulysses_exchange(x, ptrs, self.rank, seq_to_head, heads_total)
            self.barrier_kernel()  # all pushes landed
        return out

    def head_scatter_gemm(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows_per_rank: int, q_blocks: int, kv_blocks: int) -> torch.Tensor:
        """``x·wᵀ`` with every 128-column block written into the symmetric ``out`` of the rank that owns its heads."""
        ptrs = self.peer_ptrs(out)
        assert ptrs is not None, 'destination must be symmetric memory'
        self.barrier_kernel()  # every rank is done reading the buffer's previous contents
        self.ext.gemm_head_scatter(x, w, ptrs, self.rank, rows_per_rank, q_blocks, kv_blocks)
        self.barrier_kernel()  # all tiles of all ranks landed
        return out

    def check(self) -> None:
        code = self.ext.read_and_clear_error()
        if code:
            raise RuntimeError(f'peer-memory kernel gave up waiting (code {code}); a rank is missing or stalled')
