"""Pipeline parallelism: 1F1B and interleaved (virtual stages) schedules over p2p send/recv.

What it replaces: megatron-core's ``get_forward_backward_func()`` schedules used by the reference
(``src/twinkle/model/megatron/megatron.py:480-506``; ``pipeline_model_parallel_size``,
``virtual_pipeline_model_parallel_size``).  Activations cross stage boundaries with ``isend`` / ``irecv``
(NCCL p2p on GPUs, gloo on CPU): sends are asynchronous so the next micro-batch's compute overlaps the
transfer; receives are posted right before they are needed.

Virtual stage ``v = chunk · P + rank`` (P = pipeline size, ``chunk`` < V): layer blocks are dealt round-robin,
so rank r owns chunks r, r+P, r+2P, … of the layer list.  The op order per rank follows the interleaved
1F1B rule: warm-up forwards, steady 1F1B pairs, cool-down backwards, with micro-batches taken in groups of P
per chunk.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Op:
    kind: str  # 'F' | 'B'
    chunk: int
    micro: int


def build_schedule(P: int, V: int, M: int, rank: int) -> List[Op]:
    """Ordered forward/backward ops of one pipeline rank.  V = 1 gives classic 1F1B."""
    if V > 1 and M % P != 0:
        raise ValueError(f'interleaved schedule needs num_microbatches ({M}) to be a multiple of the pipeline size ({P})')
    total = M * V

    def fwd_id(k: int) -> Tuple[int, int]:  # k-th forward of this rank → (chunk, micro)
        group, within = divmod(k, P * V)
        chunk, pos = divmod(within, P)
        return chunk, group * P + pos

    def bwd_id(k: int) -> Tuple[int, int]:
        group, within = divmod(k, P * V)
        chunk, pos = divmod(within, P)
        return V - 1 - chunk, group * P + pos

    if V == 1:
        warm = min(P - rank - 1, M)
    else:
        warm = min((P - rank - 1) * 2 + (V - 1) * P, total)
    ops: List[Op] = []
    f = b = 0
    for _ in range(warm):
        ops.append(Op('F', *fwd_id(f)))
        f += 1
    while f < total:
        ops.append(Op('F', *fwd_id(f)))
        f += 1
        ops.append(Op('B', *bwd_id(b)))
        b += 1
    while b < total:
        ops.append(Op('B', *bwd_id(b)))
        b += 1
    return ops


class PipelineRunner:
    """Executes a schedule for the chunks owned by this rank.

    ``forward_chunk(chunk, micro, hidden_in) -> hidden_out`` runs one chunk; on the last virtual stage it must
    return the scalar loss instead.  ``hidden_shape(micro)`` gives the activation shape exchanged between
    stages (all stages exchange the same shape for a given micro-batch).
    """

    def __init__(self, group, rank: int, size: int, vpp: int, dtype: torch.dtype, device):
        self.group, self.rank, self.P, self.V, self.dtype, self.device = group, rank, size, vpp, dtype, device
        self.prev = (rank - 1) % size
        self.next = (rank + 1) % size
        self._pending: List = []
        self._outbox: List = []
        self._keep: List = []
        assert not (size == 1 and vpp > 1), 'virtual stages need a pipeline of at least 2 ranks'
        self._globals = [dist.get_global_rank(group, r) if group is not None else r for r in range(size)] if size > 1 else [0]

    def is_first(self, chunk: int) -> bool:
        return self.rank == 0 and chunk == 0

    def is_last(self, chunk: int) -> bool:
        return self.rank == self.P - 1 and chunk == self.V - 1

    # Sends are not issued on their own: they wait in an outbox and leave together with the next receive in
    # one ``batch_isend_irecv`` group (the "send forward / receive backward" pairing).  Separate NCCL
    # send and recv kernels to the same neighbour could otherwise wait on each other in a cycle.
    def _send(self, t: torch.Tensor, dst: int, tag: int) -> None:
        self._outbox.append(dist.P2POp(dist.isend, t.contiguous(), self._globals[dst], group=self.group, tag=tag))

    def _flush(self) -> None:
        if self._outbox:
            for w in dist.batch_isend_irecv(self._outbox):
                self._pending.append(w)
            self._keep.append([op.tensor for op in self._outbox])
            self._outbox = []

    def _recv(self, shape, src: int, tag: int) -> torch.Tensor:
        buf = torch.empty(shape, dtype=self.dtype, device=self.device)
        ops_ = self._outbox + [dist.P2POp(dist.irecv, buf, self._globals[src], group=self.group, tag=tag)]
        self._keep.append([op.tensor for op in self._outbox])
        self._outbox = []
        works = dist.batch_isend_irecv(ops_)
        if len(works) == len(ops_):
            # only the receive is awaited here; a send completes whenever the neighbour reaches its matching
            # receive, which may be several ops later in its own schedule
            works[-1].wait()
            self._pending.extend(works[:-1])
        else:  # NCCL coalesces the whole group into one work object
            for w in works:
                w.wait()
        return buf

    @staticmethod
    def _tag(kind: str, vstage: int, micro: int) -> int:
        return (0 if kind == 'F' else 1 << 20) + vstage * 1024 + micro

    def run(self, num_micro: int, forward_chunk: Callable[[int, int, Optional[torch.Tensor]], torch.Tensor],
            hidden_shape: Callable[[int], Sequence[int]], loss_scale: Callable[[int], float] = lambda m: 1.0) -> List[torch.Tensor]:
        """Returns the per-micro-batch losses (on the last stage; empty elsewhere)."""
        P, V = self.P, self.V
        saved: Dict[Tuple[int, int], Tuple[Optional[torch.Tensor], torch.Tensor]] = {}
        losses: List[torch.Tensor] = []
        for op in build_schedule(P, V, num_micro, self.rank):
            vstage = op.chunk * P + self.rank
            if op.kind == 'F':
                x = None
                if not self.is_first(op.chunk):
                    x = self._recv(hidden_shape(op.micro), self.prev, self._tag('F', vstage, op.micro))
                    x.requires_grad_(True)
                else:
                    self._flush()
                y = forward_chunk(op.chunk, op.micro, x)
                saved[(op.chunk, op.micro)] = (x, y)
                if self.is_last(op.chunk):
                    losses.append(y.detach())
                elif P > 1:
                    self._send(y.detach(), self.next, self._tag('F', vstage + 1, op.micro))
            else:
                x, y = saved.pop((op.chunk, op.micro))
                if self.is_last(op.chunk):
                    self._flush()
                    (y * loss_scale(op.micro)).backward()
                else:
                    g = self._recv(y.shape, self.next, self._tag('B', vstage, op.micro))
                    torch.autograd.backward(y, g)
                if not self.is_first(op.chunk) and x is not None:
                    self._send(x.grad, self.prev, self._tag('B', vstage - 1, op.micro))
        self._flush()
        for h in self._pending:
            h.wait()
        self._pending.clear()
        self._keep.clear()
        return losses
