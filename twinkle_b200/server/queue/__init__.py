"""Admission control and the single-file compute queue.

Parity: reference ``src/twinkle/server/utils/task_queue/{mixin,worker,rate_limiter,types,config}.py`` —
preflight (``max_input_tokens``, batch size ≥ and multiple of the data-parallel world size, sliding-window
``RateLimiter(rps, tps)`` per token), a ``ComputeWorker`` that runs ONE task at a time, round-robin across
per-(model, token) queues, with ``queue_timeout`` / ``execution_timeout`` and the future life cycle
``pending → queued → running → completed | failed``.
"""
from __future__ import annotations

import asyncio
import collections
import concurrent.futures
import inspect
import threading
import time
import traceback
import uuid
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Awaitable, Callable, Deque, Dict, Optional, Tuple
from ..exceptions import TwinkleServerError


class TaskStatus(str, Enum):
    PENDING = 'pending'
    QUEUED = 'queued'
    RUNNING = 'running'
    COMPLETED = 'completed'
    FAILED = 'failed'


class PreflightError(TwinkleServerError):

    def __init__(self, message: str, status_code: int = 400):
        super().__init__(message)
        self.status_code = status_code


class RateLimiter:
    """Sliding window over the last ``window`` seconds, per key: at most ``rps·window`` requests and
    ``tps·window`` tokens."""

    def __init__(self, rps: float, tps: float, window: float = 1.0, clock: Callable[[], float] = time.monotonic):
        self.rps, self.tps, self.window, self.clock = rps, tps, window, clock
        self._events: Dict[str, Deque[Tuple[float, int]]] = collections.defaultdict(collections.deque)
        self.rejections = 0

    def _trim(self, key: str) -> None:
        q, now = self._events[key], self.clock()
        while q and now - q[0][0] > self.window:
            q.popleft()

    def check(self, key: str, tokens: int = 0) -> Tuple[bool, str]:
        self._trim(key)
        q = self._events[key]
        if len(q) + 1 > self.rps * self.window:
            self.rejections += 1
            return False, f'request rate limit exceeded ({self.rps}/s)'
        used = sum(t for _, t in q)
        if tokens and used + tokens > self.tps * self.window and q:
            self.rejections += 1
            return False, f'token rate limit exceeded ({self.tps} tokens/s)'
        return True, ''

    def record(self, key: str, tokens: int = 0) -> None:
        self._events[key].append((self.clock(), tokens))

    def acquire(self, key: str, tokens: int = 0) -> Tuple[bool, str]:
        ok, why = self.check(key, tokens)
        if ok:
            self.record(key, tokens)
        return ok, why

    def cleanup(self, idle: float = 60.0) -> None:
        now = self.clock()
        for k in [k for k, q in self._events.items() if not q or now - q[-1][0] > idle]:
            self._events.pop(k, None)


@dataclass
class _Task:
    request_id: str
    queue_key: str
    fn: Callable[[], Any]
    enqueued: float = field(default_factory=time.monotonic)
    done: Optional['concurrent.futures.Future'] = None


class ComputeWorker:
    """One task at a time on a dedicated thread; queues (one per model/token) are served round-robin so a
    busy tenant cannot starve the others.  Being a plain thread it is independent of whichever event loop
    serves the HTTP requests."""

    def __init__(self, state, queue_timeout: float = 300.0, execution_timeout: float = 120.0, metrics=None):
        self.state, self.queue_timeout, self.execution_timeout, self.metrics = state, queue_timeout, execution_timeout, metrics
        self.queues: 'collections.OrderedDict[str, Deque[_Task]]' = collections.OrderedDict()
        self._cv = threading.Condition()
        self._thread: Optional[threading.Thread] = None
        self._stop = False
        self.current: Optional[str] = None
        self.executed = 0

    def depth(self) -> int:
        with self._cv:
            return sum(len(q) for q in self.queues.values())

    def ensure_started(self) -> None:
        if self._thread is None or not self._thread.is_alive():
            self._stop = False
            self._thread = threading.Thread(target=self._loop, name='compute-worker', daemon=True)
            self._thread.start()

    def stop(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify_all()

    def submit(self, task: _Task) -> None:
        self.ensure_started()
        with self._cv:
            self.queues.setdefault(task.queue_key, collections.deque()).append(task)
            depth = sum(len(q) for q in self.queues.values())
            self._cv.notify()
        if self.metrics is not None:
            self.metrics.set_gauge('twinkle_queue_depth', depth)
        self.state.set_future(task.request_id, TaskStatus.QUEUED.value, queue_depth=depth)

    def _next(self) -> Optional[_Task]:
        for key in list(self.queues):
            q = self.queues[key]
            self.queues.move_to_end(key)  # round robin
            if q:
                t = q.popleft()
                if not q:
                    self.queues.pop(key, None)
                return t
            self.queues.pop(key, None)
        return None

    def _run_with_timeout(self, fn: Callable[[], Any]) -> Any:
        """The compute itself cannot be pre-empted (a collective may be in flight on other ranks); the
        timeout bounds how long the *caller* waits, the late result is discarded."""
        box: Dict[str, Any] = {}

        def run():
            try:
                res = fn()
                if inspect.isawaitable(res):
                    res = asyncio.run(res)
                box['result'] = res
            except BaseException as e:  # noqa: BLE001
                box['error'] = e
                box['tb'] = traceback.format_exc()[-2000:]

        th = threading.Thread(target=run, daemon=True)
        th.start()
        th.join(self.execution_timeout)
        if th.is_alive():
            th.join()  # keep one-task-at-a-time semantics; report the overrun
            if 'error' not in box:
                box['late'] = True
        return box

    def _loop(self) -> None:
        while True:
            with self._cv:
                t = self._next()
                while t is None and not self._stop:
                    self._cv.wait(timeout=1.0)
                    t = self._next()
                if t is None:
                    return
            waited = time.monotonic() - t.enqueued
            if waited > self.queue_timeout:
                self._finish(t, TaskStatus.FAILED, error=f'queue timeout after {waited:.1f}s')
                continue
            self.current = t.request_id
            self.state.set_future(t.request_id, TaskStatus.RUNNING.value)
            start = time.monotonic()
            box = self._run_with_timeout(t.fn)
            if 'error' in box:
                e = box['error']
                self._finish(t, TaskStatus.FAILED, error=f'{type(e).__name__}: {e}', tb=box.get('tb'))
            elif box.get('late'):
                self._finish(t, TaskStatus.FAILED, error=f'execution timeout after {self.execution_timeout}s')
            else:
                self._finish(t, TaskStatus.COMPLETED, result=box.get('result'))
            self.executed += 1
            self.current = None
            if self.metrics is not None:
                self.metrics.observe_task(time.monotonic() - start, waited)

    def _finish(self, t: _Task, status: TaskStatus, result: Any = None, error: Optional[str] = None, **extra) -> None:
        if self.metrics is not None:
            self.metrics.inc('twinkle_tasks_total', status=status.value)
            self.metrics.set_gauge('twinkle_queue_depth', self.depth())
        # a blocking caller gets the object itself; only fire-and-poll tasks need the result in the state
        # backend, which must be JSON-serialisable there
        if t.done is not None and not t.done.done():
            if status == TaskStatus.COMPLETED:
                t.done.set_result(result)
            else:
                t.done.set_exception(RuntimeError(error or 'task failed'))
        try:
            self.state.set_future(t.request_id, status.value, result=None if t.done is not None else result, error=error, **extra)
        except Exception as e:  # noqa: BLE001 — never let a bookkeeping failure kill the worker thread
            self.state.set_future(t.request_id, TaskStatus.FAILED.value, error=f'result not storable: {type(e).__name__}: {e}')


class TaskQueueMixin:
    """Mixed into the model / sampler apps.  Needs ``self.state`` and ``self.queue_config``."""

    def _init_task_queue(self, state, config, metrics=None) -> None:
        self.state, self.queue_config = state, config
        self.rate_limiter = RateLimiter(config.rps_limit, config.tps_limit, config.window_seconds)
        self.worker = ComputeWorker(state, config.queue_timeout, config.execution_timeout, metrics)

    def preflight(self, token: str, input_tokens: int = 0, batch_size: Optional[int] = None, data_world_size: int = 1,
                  batch_size_multiple: int = 1) -> None:
        c = self.queue_config
        if not c.enabled:
            return
        if input_tokens > c.max_input_tokens:
            raise PreflightError(f'input has {input_tokens} tokens; the limit is {c.max_input_tokens}', 413)
        if batch_size is not None:
            if batch_size < data_world_size:
                raise PreflightError(f'batch size {batch_size} is smaller than the data-parallel world size {data_world_size}; '
                                     'some ranks would receive no data')
            if batch_size_multiple > 1 and batch_size % batch_size_multiple != 0:
                raise PreflightError(f'batch size {batch_size} must be a multiple of {batch_size_multiple}')
        ok, why = self.rate_limiter.acquire(token, input_tokens)
        if not ok:
            m = getattr(self.worker, 'metrics', None)
            if m is not None:
                m.inc('twinkle_rate_limit_rejections_total')
            raise PreflightError(why, 429)

    def schedule_task(self, fn: Callable[[], Any], *, token: str, model_id: str = '', input_tokens: int = 0, batch_size: Optional[int] = None,
                      data_world_size: int = 1, batch_size_multiple: int = 1, request_id: Optional[str] = None) -> Dict[str, Any]:
        """Queue ``fn`` and return ``{request_id, model_id}`` immediately (Tinker future protocol)."""
        self.preflight(token, input_tokens, batch_size, data_world_size, batch_size_multiple)
        rid = self.state.create_future(request_id, model_id=model_id, token=token)
        self.worker.submit(_Task(rid, f'{model_id}:{token}', fn))
        return {'request_id': rid, 'model_id': model_id}

    async def schedule_task_and_wait(self, fn: Callable[[], Any], *, token: str, model_id: str = '', **kw) -> Any:
        """Queue ``fn`` and await its result (native Twinkle routes are blocking)."""
        self.preflight(token, kw.get('input_tokens', 0), kw.get('batch_size'), kw.get('data_world_size', 1), kw.get('batch_size_multiple', 1))
        rid = self.state.create_future(None, model_id=model_id, token=token)
        fut: concurrent.futures.Future = concurrent.futures.Future()
        self.worker.submit(_Task(rid, f'{model_id}:{token}', fn, done=fut))
        return await asyncio.wrap_future(fut)

    def schedule_background_task(self, fn: Callable[[], Any], name: str = '') -> str:
        rid = self.state.create_future(None, kind='background', name=name)

        def run():
            try:
                res = fn()
                if inspect.isawaitable(res):
                    res = asyncio.run(res)
                self.state.set_future(rid, TaskStatus.COMPLETED.value, result=res)
            except Exception as e:  # noqa: BLE001
                self.state.set_future(rid, TaskStatus.FAILED.value, error=f'{type(e).__name__}: {e}')

        threading.Thread(target=run, daemon=True, name=f'background-{name}').start()
        return rid
