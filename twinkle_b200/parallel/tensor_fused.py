"""Tensor-parallel linears whose collective runs inside the GEMM kernel (sequence-parallel activations).

What it replaces: megatron-core / TransformerEngine's column- and row-parallel linears, where an NCCL
all-gather precedes and an NCCL reduce-scatter follows a cuBLAS GEMM (reached by the reference through
``src/twinkle/model/megatron/strategy/megatron.py:37-118``).  Here

* column-parallel forward / row-parallel dgrad = ``ops/csrc/gemm2.cu`` with ``FUSE_AG``: copier CTAs of the GEMM
  launch pull the peers' activation shards over NVLink while the tensor-core CTAs start on the local shard;
* row-parallel forward / column-parallel dgrad = the same kernel with ``FUSE_RS``: finished tiles are stored
  straight into the owner GPU's staging slot from the epilogue, then the owner sums its ``tp`` slots.

Symmetric buffers alternate between two copies per shape.  A copy is overwritten two calls after it was
published; in between this rank has passed a flag barrier that every peer reaches only after the kernels that read
the older copy were issued on its stream, so no separate "buffer free" handshake exists.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .. import ops


class FusedTP:

    def __init__(self, comm, copy_ctas: int = 0):
        self.comm, self.tp, self.rank = comm, comm.world_size, comm.rank
        self.copy_ctas = copy_ctas  # 0: sized per call so that the pulls take about half the GEMM's time
        self.ready = torch.zeros(16, dtype=torch.int32, device=comm.device)
        self.ready_total = 0
        self._bufs: Dict[Tuple, List[torch.Tensor]] = {}
        self._uses: Dict[Tuple, int] = {}

    def _buf(self, key: Tuple, numel: int, dtype) -> torch.Tensor:
        if key not in self._bufs:
            self._bufs[key] = [self.comm.alloc(numel, dtype) for _ in range(2)]
            self._uses[key] = 0
        b = self._bufs[key][self._uses[key] % 2]
        self._uses[key] += 1
        return b

    @staticmethod
    def eligible(rows_per_rank: int, k: int, n: int, dtype) -> bool:
        return dtype == torch.bfloat16 and rows_per_rank % 256 == 0 and k % 8 == 0 and n % 8 == 0

    def ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor, layout: str):
        """(gather(x) · Wᵀ | gather(x) · W, gathered x)."""
        rows, k = x_local.shape
        buf = self._buf(('x', rows, k), rows * k, x_local.dtype).view(rows, k)
        buf.copy_(x_local)
        self.comm.barrier_kernel()  # every rank's shard is in place
        n = w.shape[0] if layout == 'nt' else w.shape[1]
        ctas = self.copy_ctas or self.copier_ctas(rows * self.tp, k, n)
        if self.ready_total + ctas >= (1 << 30):
            self.ready.zero_()
            self.ready_total = 0
        self.ready_total += ctas
        y, gathered = ops.ext().gemm_ag(self.comm.peer_ptrs(buf), rows, w, layout, self.rank, self.ready, self.ready_total, ctas)
        return y, gathered

    def copier_ctas(self, t: int, k: int, n: int) -> int:
        """CTAs of the launch that copy instead of compute: each keeps 160 KB in flight (≈ 50 GB/s over NVLink); enough of
        them that the remote shards arrive in about half the time the tensor cores need for the whole product."""
        remote_bytes = (self.tp - 1) * (t // self.tp) * k * 2
        gemm_s = 2.0 * t * k * n / 1.5e15
        need = remote_bytes / (0.5 * gemm_s * 50e9)
        return int(min(16, max(2, 2 * round(need / 2 + 0.5))))

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, layout: str) -> torch.Tensor:
        """reduce_scatter(a · Wᵀ | a · W) along rows."""
        t = a.shape[0]
        n = w.shape[0] if layout == 'nt' else w.shape[1]
        rows = t // self.tp
        stage = self._buf(('s', rows, n), self.tp * rows * n, a.dtype).view(self.tp, rows, n)
        ops.ext().gemm_rs(a.contiguous(), w, layout, self.comm.peer_ptrs(stage), self.rank)
        self.comm.barrier_kernel()  # every rank's tiles have landed in my slots
        return ops.ext().tp_stage_reduce(stage)


class ColumnLinearFused(torch.autograd.Function):
    """y = gather_tokens(x) · Wᵀ with W the rank's output-row shard; backward reduce-scatters dx from the dgrad epilogue."""

    @staticmethod
    def forward(ctx, x_local, w, fused: FusedTP):
        y, gathered = fused.ag_gemm(x_local.contiguous(), w, 'nt')
        ctx.save_for_backward(gathered, w)
        ctx.fused = fused
        return y

    @staticmethod
    def backward(ctx, gy):
        gathered, w = ctx.saved_tensors
        gy = gy.contiguous()
        gx = ctx.fused.gemm_rs(gy, w, 'nn') if ctx.needs_input_grad[0] else None
        gw = ops.gemm(gy, gathered, 'tn') if ctx.needs_input_grad[1] else None
        return gx, gw, None


class RowLinearFused(torch.autograd.Function):
    """y_local = reduce_scatter_tokens(x · Wᵀ) with W the rank's input-column shard; backward all-gathers dy inside the dgrad."""

    @staticmethod
    def forward(ctx, x, w, fused: FusedTP):
        x = x.contiguous()
        ctx.save_for_backward(x, w)
        ctx.fused = fused
        return fused.gemm_rs(x, w, 'nt')

    @staticmethod
    def backward(ctx, g_local):
        x, w = ctx.saved_tensors
        gx, g_full = ctx.fused.ag_gemm(g_local.contiguous(), w, 'nn')
        gw = ops.gemm(g_full, x, 'tn') if ctx.needs_input_grad[1] else None
        return (gx if ctx.needs_input_grad[0] else None), gw, None
