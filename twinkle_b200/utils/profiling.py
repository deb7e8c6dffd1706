"""Device-side timing and profiler ranges.

The reference has no GPU timing beyond wall-clock ``iters/s`` (``src/twinkle/metric/train_metric.py:52-60``).  Here a
step is timed on the device with CUDA events on the launching stream, reduced with MAX over the ranks of a group
(the number every multi-GPU figure in this repository is quoted as), and the fused paths are wrapped in NVTX ranges
so a timeline shows them by name.
"""
from __future__ import annotations

import time
from contextlib import contextmanager
from typing import Dict, List, Optional

import torch


class DeviceTimer:
    """``with timer('fwd'): …`` records one interval; ``summary()`` returns mean milliseconds per name, max over ranks.
    On CPU it falls back to ``time.perf_counter``."""

    def __init__(self, group=None, enabled: bool = True):
        self.group, self.enabled = group, enabled
        self._open: Dict[str, List] = {}
        self._host: Dict[str, List[float]] = {}

    @contextmanager
    def __call__(self, name: str):
        if not self.enabled:
            yield
            return
        cuda = torch.cuda.is_available()
        with nvtx_range(name):
            if cuda:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                yield
                b.record()
                self._open.setdefault(name, []).append((a, b))
            else:
                t0 = time.perf_counter()
                yield
                self._host.setdefault(name, []).append((time.perf_counter() - t0) * 1e3)

    def summary(self, reset: bool = True) -> Dict[str, float]:
        out: Dict[str, float] = {}
        if self._open:
            torch.cuda.synchronize()
        for name, pairs in self._open.items():
            ms = [a.elapsed_time(b) for a, b in pairs]
            out[name] = sum(ms) / len(ms)
        for name, ms in self._host.items():
            out[name] = sum(ms) / len(ms)
        import torch.distributed as dist
        if out and dist.is_available() and dist.is_initialized() and (self.group is not None or dist.get_world_size() > 1):
            names = sorted(out)
            dev = 'cuda' if (torch.cuda.is_available() and dist.get_backend(self.group) == 'nccl') else 'cpu'
            t = torch.tensor([out[n] for n in names], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            out = dict(zip(names, t.tolist()))
        if reset:
            self._open, self._host = {}, {}
        return out


@contextmanager
def nvtx_range(name: str):
    """NVTX range when CUDA is present (visible in Nsight timelines), no-op otherwise."""
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def tokens_per_second(num_tokens: float, ms: float) -> float:
    return num_tokens / (ms / 1e3) if ms > 0 else 0.0


class PhaseClock:
    """Process-wide accumulator of device time per named phase of a training step.

    The engines bracket their communication phases (``with PHASES('ulysses_exchange'): …``); each bracket records a
    pair of CUDA events on the current stream, so the figure is the time the *launching stream* spent between the two
    points — for a phase that only waits on a side stream (``fsdp_gather_wait``) that is exactly the stall.  Off by
    default (one attribute test per bracket); ``bench.py`` switches it on for one extra step after its timed region
    and prints the totals, so the limiter of a multi-GPU step is named by a number.
    """

    def __init__(self):
        self.enabled = False
        self._pairs: Dict[str, List] = {}
        self._counts: Dict[str, int] = {}

    @contextmanager
    def __call__(self, name: str):
        if not self.enabled or not torch.cuda.is_available():
            yield
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.nvtx.range_push(name)  # the same brackets show up by name on a profiler timeline
        a.record()
        try:
            yield
        finally:
            b.record()
            torch.cuda.nvtx.range_pop()
            self._pairs.setdefault(name, []).append((a, b))

    def start(self) -> None:
        self._pairs, self.enabled = {}, True

    def stop(self, group=None) -> Dict[str, Dict[str, float]]:
        """Totals per phase since ``start``: ``{name: {'ms': total, 'ms_min': total, 'n': brackets}}`` — ``ms`` is the
        maximum over the ranks of ``group`` and ``ms_min`` the minimum.  A phase that contains a cross-GPU wait shows the
        skew between ranks as the gap between the two: the rank that arrives last waits for nobody."""
        self.enabled = False
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        names = sorted(self._pairs)
        ms = [sum(a.elapsed_time(b) for a, b in self._pairs[n]) for n in names]
        cnt = [len(self._pairs[n]) for n in names]
        self._pairs = {}
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            # every rank brackets the same phases in the same order, so the name lists agree
            dev = 'cuda' if dist.get_backend(group) == 'nccl' else 'cpu'
            t = torch.tensor(ms, dtype=torch.float64, device=dev)
            lo = t.clone()
            if t.numel():
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
            ms, ms_lo = t.tolist(), lo.tolist()
        else:
            ms_lo = ms
        return {n: {'ms': round(m, 3), 'ms_min': round(l, 3), 'n': c} for n, m, l, c in zip(names, ms, ms_lo, cnt)}


PHASES = PhaseClock()
