"""Server observability.

Parity: reference ``src/twinkle/server/telemetry/*.py`` — request / task / rate-limit / resource metrics, one
span per HTTP request and per queued task with ``twinkle.*`` correlation attributes, host + GPU gauges.  The
reference exports through OpenTelemetry (OTLP); that SDK is not a dependency here: metrics live in an
in-process registry that renders Prometheus text (scraped at ``/metrics``) and spans go to a ring buffer
and, optionally, a JSON-lines file.  ``GpuTimer`` adds what the reference lacks: device-timed step metrics
(CUDA events) for the training loop.
"""
from __future__ import annotations

import collections
import contextlib
import json
import os
import threading
import time
import uuid
from typing import Any, Deque, Dict, Iterator, List, Optional, Tuple

CORRELATION_KEYS = ('session_id', 'model_id', 'replica_id', 'token_id', 'sampling_session_id', 'base_model')


class MetricsRegistry:

    def __init__(self):
        self._lock = threading.Lock()
        self.counters: Dict[Tuple[str, Tuple], float] = collections.defaultdict(float)
        self.gauges: Dict[Tuple[str, Tuple], float] = {}
        self.hist: Dict[Tuple[str, Tuple], List[float]] = collections.defaultdict(list)

    @staticmethod
    def _key(name: str, labels: Optional[Dict[str, Any]]) -> Tuple[str, Tuple]:
        return name, tuple(sorted((labels or {}).items()))

    def inc(self, name: str, value: float = 1.0, **labels) -> None:
        with self._lock:
            self.counters[self._key(name, labels)] += value

    def set_gauge(self, name: str, value: float, **labels) -> None:
        with self._lock:
            self.gauges[self._key(name, labels)] = value

    def observe(self, name: str, value: float, **labels) -> None:
        with self._lock:
            h = self.hist[self._key(name, labels)]
            h.append(value)
            if len(h) > 4096:
                del h[:2048]

    def observe_task(self, exec_s: float, wait_s: float) -> None:
        self.observe('twinkle_task_execution_seconds', exec_s)
        self.observe('twinkle_task_wait_seconds', wait_s)

    def render_prometheus(self) -> str:
        lines = []
        fmt = lambda name, lab: name + ('{' + ','.join(f'{k}="{v}"' for k, v in lab) + '}' if lab else '')
        with self._lock:
            for (n, lab), v in self.counters.items():
                lines.append(f'{fmt(n, lab)} {v}')
            for (n, lab), v in self.gauges.items():
                lines.append(f'{fmt(n, lab)} {v}')
            for (n, lab), vals in self.hist.items():
                if vals:
                    s = sorted(vals)
                    lines.append(f'{fmt(n + "_count", lab)} {len(s)}')
                    lines.append(f'{fmt(n + "_sum", lab)} {sum(s)}')
                    for q in (0.5, 0.9, 0.99):
                        lines.append(f'{fmt(n, lab + (("quantile", q), ))} {s[min(int(q * len(s)), len(s) - 1)]}')
        return '\n'.join(lines) + '\n'


class Tracer:

    def __init__(self, capacity: int = 2048, path: Optional[str] = None):
        self.spans: Deque[Dict[str, Any]] = collections.deque(maxlen=capacity)
        self.path = path
        self._local = threading.local()

    @contextlib.contextmanager
    def span(self, name: str, parent: Optional[str] = None, **attrs) -> Iterator[Dict[str, Any]]:
        s = {'name': name, 'span_id': uuid.uuid4().hex[:16], 'trace_id': parent or getattr(self._local, 'trace', None) or uuid.uuid4().hex,
             'start': time.time(), 'attributes': {f'twinkle.{k}' if k in CORRELATION_KEYS else k: v for k, v in attrs.items()}}
        prev = getattr(self._local, 'trace', None)
        self._local.trace = s['trace_id']
        try:
            yield s
            s['status'] = 'ok'
        except Exception as e:
            s['status'] = 'error'
            s['error'] = f'{type(e).__name__}: {e}'
            raise
        finally:
            s['duration_s'] = time.time() - s['start']
            self._local.trace = prev
            self.spans.append(s)
            if self.path:
                with open(self.path, 'a') as f:
                    f.write(json.dumps(s, default=str) + '\n')


class ResourceMetricsCollector:
    """CPU / memory through psutil, GPU utilisation / memory through NVML (read-only queries)."""

    def __init__(self, registry: MetricsRegistry):
        self.registry = registry

    def collect(self) -> None:
        try:
            import psutil
            self.registry.set_gauge('twinkle_host_cpu_percent', psutil.cpu_percent(interval=None))
            self.registry.set_gauge('twinkle_host_memory_percent', psutil.virtual_memory().percent)
        except Exception:
            pass
        try:
            import pynvml
            pynvml.nvmlInit()
            for i in range(pynvml.nvmlDeviceGetCount()):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                u = pynvml.nvmlDeviceGetUtilizationRates(h)
                m = pynvml.nvmlDeviceGetMemoryInfo(h)
                self.registry.set_gauge('twinkle_gpu_utilization', u.gpu, gpu=i)
                self.registry.set_gauge('twinkle_gpu_memory_used_bytes', m.used, gpu=i)
        except Exception:
            pass


class GpuTimer:
    """Device-side timing of a region with CUDA events; ``max_over_ranks`` reduces across a process group."""

    def __init__(self):
        import torch
        self.torch = torch
        self.start_ev = torch.cuda.Event(enable_timing=True) if torch.cuda.is_available() else None
        self.end_ev = torch.cuda.Event(enable_timing=True) if torch.cuda.is_available() else None
        self._t0 = 0.0

    def __enter__(self):
        if self.start_ev is not None:
            self.start_ev.record()
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.end_ev is not None:
            self.end_ev.record()
            self.torch.cuda.synchronize()
            self.ms = self.start_ev.elapsed_time(self.end_ev)
        else:
            self.ms = (time.perf_counter() - self._t0) * 1e3

    def max_over_ranks(self, group=None) -> float:
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()):
            return self.ms
        t = self.torch.tensor([self.ms], device='cuda' if self.torch.cuda.is_available() else 'cpu')
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t.item())


_REGISTRY = MetricsRegistry()
_TRACER = Tracer(path=os.environ.get('TWINKLE_TELEMETRY_TRACE_FILE'))


def get_registry() -> MetricsRegistry:
    return _REGISTRY


def get_tracer() -> Tracer:
    return _TRACER


def traced_operation(name: str, **attrs):
    return _TRACER.span(name, **attrs)
