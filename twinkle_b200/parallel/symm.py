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

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..utils.profiling import PHASES
from .comm import Communicator


def exchange_jobs(shape, elem_size: int, sp: int, me: int, seq_to_head: bool):
    """Copy jobs of rank ``me`` for one tensor of the head ↔ sequence exchange, as byte offsets.

    ``seq_to_head``: every rank stages ``[t, H, D]`` (its tokens, all heads); ``me`` pulls its head slice of every
    peer's tokens into ``[sp·t, H/sp, D]``.  Otherwise every rank stages ``[sp·t, h, D]`` (all tokens, its heads) and
    ``me`` pulls its token chunk of every peer's heads into ``[t, sp·h, D]``.  Returns ``(output shape, [(source rank,
    source offset, source row stride, destination offset, destination row stride, bytes per row, rows)])``; peers are
    visited starting with ``me + 1`` so that no GPU's egress serves every reader at the same moment."""
    jobs = []
    if seq_to_head:
        t, H, D = shape
        if H % sp:
            raise ValueError(f'{H} heads do not divide over {sp} sequence-parallel ranks')
        hl = H // sp
        chunk = hl * D * elem_size
        out_shape = (sp * t, hl, D)
        for k in range(1, sp + 1):
            r = (me + k) % sp
            jobs.append((r, me * chunk, H * D * elem_size, r * t * chunk, chunk, chunk, t))
    else:
        tt, hl, D = shape
        if tt % sp:
            raise ValueError(f'{tt} token rows do not divide over {sp} sequence-parallel ranks')
        t = tt // sp
        chunk = hl * D * elem_size
        out_shape = (t, sp * hl, D)
        for k in range(1, sp + 1):
            r = (me + k) % sp
            jobs.append((r, me * t * chunk, chunk, r * chunk, sp * chunk, chunk, t))
    return out_shape, jobs


def check_jobs(jobs, src_bytes: int, dst_bytes: int) -> None:
    """Debug aid (``TWINKLE_DEBUG_BOUNDS=1``): every byte a job reads lies inside the peers' staged tensor and every
    byte it writes inside the output, rows are multiples of 16 bytes, and no two jobs write the same byte."""
    import numpy as np
    hit = np.zeros(max(dst_bytes // 16, 1), dtype=np.uint8)
    for r, s_off, s_stride, d_off, d_stride, chunk, n in jobs:
        if chunk % 16 or s_off % 16 or d_off % 16 or s_stride % 16 or d_stride % 16:
            raise AssertionError(f'job for rank {r} is not 16-byte aligned: {(s_off, s_stride, d_off, d_stride, chunk)}')
        if n and (s_off < 0 or s_off + (n - 1) * s_stride + chunk > src_bytes):
            raise AssertionError(f'job for rank {r} reads past the staged tensor ({src_bytes} bytes)')
        if n and (d_off < 0 or d_off + (n - 1) * d_stride + chunk > dst_bytes):
            raise AssertionError(f'job for rank {r} writes past the output ({dst_bytes} bytes)')
        if n:
            rows = (d_off // 16 + np.arange(n, dtype=np.int64)[:, None] * (d_stride // 16) + np.arange(chunk // 16, dtype=np.int64)[None, :]).reshape(-1)
            np.add.at(hit, rows, 1)
    if hit.max(initial=0) > 1:
        raise AssertionError('two jobs write the same bytes')
    if dst_bytes >= 16 and hit.min(initial=1) < 1:
        raise AssertionError('the jobs leave part of the output unwritten')


class SymmBuffer:
    """One symmetric chunk: the local allocation plus the device pointers of every rank's copy.  Tensors
    are carved out of it with a bump pointer; every rank performs the same sequence of requests, so a
    tensor sits at the same offset on every rank."""

    def __init__(self, comm: 'SymmCommunicator', nbytes: int):
        E = ops.ext()
        self.raw, handle, offset = E.symm_alloc(nbytes)  # retries once after emptying PyTorch's cache when the driver is out of memory
        self.nbytes = self.raw.numel()
        infos = comm.gather_object((handle, offset, self.nbytes))
        if len({i[2] for i in infos}) != 1:
            raise RuntimeError(f'symmetric allocation sizes differ across ranks: {[i[2] for i in infos]}')
        self.ptrs: List[int] = []
        for r, (h, off, _) in enumerate(infos):
            self.ptrs.append(self.raw.data_ptr() if r == comm.rank else E.symm_open(h) + off)
        self._comm_rank = comm.rank
        self.used = 0

    def carve(self, nbytes: int, guard: int = 0) -> Optional[int]:
        start, end = place_guarded(self.used, nbytes, guard)
        if end > self.nbytes and start + nbytes + guard > self.nbytes:
            return None
        self.used = min(end, self.nbytes)
        return start


GUARD_BYTES = 4096
GUARD_PATTERN = 0xA5


def place_guarded(used: int, nbytes: int, guard: int) -> Tuple[int, int]:
    """Where a tensor of ``nbytes`` goes in a chunk whose first free byte is ``used`` when ``guard`` bytes are kept on
    both sides of it: ``(start of the tensor, first free byte afterwards)``, both 256-byte aligned."""
    start = (used + guard + 255) // 256 * 256
    return start, (start + nbytes + guard + 255) // 256 * 256


def fill_guards(raw: torch.Tensor, start: int, nbytes: int, guard: int) -> None:
    raw[start - guard:start].fill_(GUARD_PATTERN)
    raw[start + nbytes:start + nbytes + guard].fill_(GUARD_PATTERN)


def damaged_guards(raw: torch.Tensor, records) -> List[str]:
    """Names of the tensors whose guard zone (before or after) no longer holds the pattern: something wrote outside a
    neighbouring tensor.  ``records`` = ``[(name, start, nbytes, guard)]``."""
    bad = []
    for name, start, nbytes, guard in records:
        lo_ok = bool((raw[start - guard:start] == GUARD_PATTERN).all())
        hi_ok = bool((raw[start + nbytes:start + nbytes + guard] == GUARD_PATTERN).all())
        if not (lo_ok and hi_ok):
            bad.append(f'{name} ({"below" if not lo_ok else ""}{"+" if not lo_ok and not hi_ok else ""}{"above" if not hi_ok else ""})')
    return bad


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
        # the gradient reduce-scatter runs on a stream of its own with its own flag set: barriers of two streams that
        # shared one epoch counter could pair up differently on different ranks
        self._rs_flags = SymmBuffer(self, 4096)
        self._rs_epoch = 0
        self._rs_stream = torch.cuda.Stream(device=self.device)
        self._rs_events: List[torch.cuda.Event] = []
        # CTAs per peer for side-stream pulls, 64 in total: each keeps 64 KB in flight, which reaches 0.6-0.8 of the link
        # (measured: 2 ranks x 32 CTAs 457 GB/s, 8 ranks x 8 CTAs 633 GB/s) while leaving the SMs to the GEMM it overlaps
        self.copy_blocks = max(8, 64 // max(self.world_size - 1, 1))
        # TWINKLE_SYMM_LEGACY=1 keeps the first-generation kernels (push exchange with two barriers, one load in flight
        # per thread in the all-gather) for A/B measurements
        self.legacy_kernels = os.environ.get('TWINKLE_SYMM_LEGACY', '0') == '1'
        # TWINKLE_SYMM_CANARIES=1 (debug aid; compute-sanitizer cannot follow writes that arrive from a peer GPU): every
        # tensor carved from symmetric memory gets a guard zone on both sides, filled with a pattern that
        # ``check_canaries`` verifies — a peer kernel that writes past a tensor's end is then caught at the next check
        self.guard_bytes = GUARD_BYTES if os.environ.get('TWINKLE_SYMM_CANARIES', '0') == '1' else 0
        self._guards: List[Tuple[SymmBuffer, str, int, int]] = []

    # ----------------------------------------------------------- allocation
    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A tensor living in symmetric memory (collective call: every rank of the group must make the
        same request at the same point)."""
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        g = self.guard_bytes
        off = self._chunks[-1].carve(nbytes, g) if self._chunks else None
        if off is None:
            self._chunks.append(SymmBuffer(self, max(nbytes + 2 * g + 512, self.chunk_bytes)))
            off = self._chunks[-1].carve(nbytes, g)
        buf = self._chunks[-1]
        if g:
            fill_guards(buf.raw, off, nbytes, g)
            self._guards.append((buf, f'tensor #{len(self._guards)} ({numel} x {dtype})', off, nbytes))
        t = buf.raw[off:off + nbytes].view(dtype)
        self._by_ptr[t.data_ptr()] = (buf, off)
        return t

    def check_canaries(self) -> None:
        """Raises if any guard zone of this rank's symmetric tensors was overwritten (a no-op unless the communicator
        was created with ``TWINKLE_SYMM_CANARIES=1``).  Synchronises the device."""
        if not self._guards:
            return
        torch.cuda.synchronize(self.device)
        bad: List[str] = []
        for buf in {id(b): b for b, _, _, _ in self._guards}.values():
            bad += damaged_guards(buf.raw, [(n, o, nb, self.guard_bytes) for b, n, o, nb in self._guards if b is buf])
        if bad:
            raise RuntimeError(f'rank {self.rank}: writes outside symmetric tensors detected next to: ' + '; '.join(bad))

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
            if self.legacy_kernels or nbytes % 16:
                self.ext.peer_all_gather(out, ptrs, nbytes, self.rank, self.copy_blocks)
            else:
                # one job per peer, starting with the next rank so that no GPU's egress serves every reader at once;
                # the own shard is copied too unless the gathered buffer aliases it
                base = out.data_ptr()
                order = [(self.rank + k) % self.world_size for k in range(1, self.world_size + 1)]
                order = [r for r in order if not (r == self.rank and base + r * nbytes == ptrs[r])]
                n = len(order)
                self.ext.peer_pull([ptrs[r] for r in order], [base + r * nbytes for r in order], [nbytes] * n, [nbytes] * n, [nbytes] * n, [1] * n,
                                   self.copy_blocks)
            done = self._stream.record_event()
        out.record_stream(self._stream)
        return done

    # -------------------------------------------------------- reduce-scatter
    def reduce_scatter_accumulate(self, grad_shard: torch.Tensor, full_grad: torch.Tensor, scale: float = 1.0) -> None:
        ptrs = self.peer_ptrs(full_grad)
        if ptrs is None or grad_shard.dtype != torch.float32 or full_grad.dtype != torch.bfloat16:
            return super().reduce_scatter_accumulate(grad_shard, full_grad, scale)
        # Off the compute stream: the barrier (every rank has finished writing this unit's gradients) and the pull
        # overlap the backward pass of the next unit instead of stalling it on the slowest rank.
        ready = torch.cuda.current_stream().record_event()
        with torch.cuda.stream(self._rs_stream):
            self._rs_stream.wait_event(ready)
            with PHASES('fsdp_reduce_scatter'):
                self._rs_epoch += 1
                self.ext.symm_barrier(self._rs_flags.ptrs, self.rank, self._rs_epoch)
                self.ext.peer_reduce_scatter_acc(grad_shard, ptrs, self.rank, scale, None, 64)
            self._rs_events.append(self._rs_stream.record_event())
        grad_shard.record_stream(self._rs_stream)
        full_grad.record_stream(self._rs_stream)
        del self._rs_events[:-4]

    def wait_reduce_scatters(self, all_but: int = 0) -> None:
        """The compute stream waits for the reduce-scatters issued so far, except the newest ``all_but``.  With
        ``all_but=1`` this is the condition for rewriting a gradient buffer of a three-deep ring: once this rank has
        passed the barrier of the reduce-scatter issued after the one that read the buffer, every peer has finished
        pulling from it."""
        evs = self._rs_events[:len(self._rs_events) - all_but] if all_but else self._rs_events
        if evs:
            with PHASES('fsdp_reduce_scatter_wait'):
                torch.cuda.current_stream().wait_event(evs[-1])

    def step_barrier(self) -> None:
        """Fences the optimizer step: peers finished reading my shards / gradient buffers."""
        self.wait_reduce_scatters()
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

    # Receive-side exchange: every rank stages its tensors in symmetric memory, ONE barrier says "staged", then each
    # rank pulls exactly the slices it will own into ordinary (allocator-owned) memory.  The staging buffers rotate in
    # pairs: a buffer is rewritten two exchanges of its kind later, and the barrier of the exchange in between is
    # passed only after every peer has finished pulling from it, so no second barrier is needed.  The results are
    # plain tensors that autograd may keep for as long as it likes.
    def _stage(self, x: torch.Tensor, tag: str) -> torch.Tensor:
        cache = self.__dict__.setdefault('_stage_buffers', {})
        key = (tuple(x.shape), x.dtype, tag)
        ent = cache.get(key)
        if ent is None:
            ent = {'bufs': [self.alloc(x.numel(), x.dtype).view(x.shape) for _ in range(2)], 'next': 0}
            cache[key] = ent
        buf = ent['bufs'][ent['next']]
        ent['next'] ^= 1
        buf.copy_(x)
        return buf

    def exchange_heads(self, xs, seq_to_head: bool):
        """``seq_to_head``: each ``[t, H, D]`` (this rank's tokens, all heads) → ``[sp·t, H/sp, D]`` (all tokens of the
        row, this rank's heads).  Otherwise the inverse: ``[sp·t, h, D]`` → ``[t, sp·h, D]``.  All tensors of ``xs`` go
        through one barrier and one kernel launch."""
        sp, me = self.world_size, self.rank
        with PHASES('ulysses_stage'):
            staged = [self._stage(x if x.is_contiguous() else x.contiguous(), f'x{i}{int(seq_to_head)}') for i, x in enumerate(xs)]
        with PHASES('ulysses_barrier'):
            self.barrier_kernel()
        outs, src, dst, ss, ds, cb, rows = [], [], [], [], [], [], []
        check = os.environ.get('TWINKLE_DEBUG_BOUNDS', '0') == '1'
        for x, st in zip(xs, staged):
            ptrs = self.peer_ptrs(st)
            out_shape, jobs = exchange_jobs(tuple(x.shape), x.element_size(), sp, me, seq_to_head)
            out = torch.empty(out_shape, dtype=x.dtype, device=x.device)
            if check:
                check_jobs(jobs, st.numel() * st.element_size(), out.numel() * out.element_size())
            for r, s_off, s_stride, d_off, d_stride, chunk, n in jobs:
                src.append(ptrs[r] + s_off); ss.append(s_stride)
                dst.append(out.data_ptr() + d_off); ds.append(d_stride)
                cb.append(chunk); rows.append(n)
            outs.append(out)
        with PHASES('ulysses_pull'):
            self.ext.peer_pull(src, dst, ss, ds, cb, rows, max(8, (4 * self.ext.num_sms()) // len(src)))
        return outs

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
