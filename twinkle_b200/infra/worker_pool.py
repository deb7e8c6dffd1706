"""Driver / worker process pool: the Ray-free counterpart of the reference's actor mode.

What it replaces: ``ResourceManager`` + per-rank Ray actors created by ``remote_class`` on the driver
(reference ``src/twinkle/infra/_ray/resource_manager.py:12-281``, ``src/twinkle/infra/__init__.py:470-760``).
One OS process per rank of a ``DeviceGroup`` is started with ``multiprocessing`` (spawn) and wired to the
driver by a duplex pipe.  Every group is its own ``torch.distributed`` world: workers receive
``RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT`` (and ``CUDA_VISIBLE_DEVICES`` when the group
pins devices), so a decorated class constructed inside them behaves exactly as under a launcher.

Protocol (pickled with cloudpickle so lambdas and locally defined classes travel):
``('create', oid, cls, args, kwargs)``, ``('call', oid, method, args, kwargs)``, ``('drop', oid)``, ``('stop',)``;
every request carries a sequence number and is answered by ``(seq, ok, payload)``.  A worker executes its
requests in order — collectives issued by the same driver call therefore line up across ranks.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import threading
import traceback
from concurrent.futures import Future
from typing import Any, Dict, List, Optional, Sequence

import cloudpickle

from ..utils.device_mesh import DeviceGroup, DeviceMesh
from ..utils.network import find_free_port


class RemoteError(RuntimeError):
    """An exception raised inside a worker, re-raised on the driver with the remote traceback."""


def _worker_main(conn, env: Dict[str, str]) -> None:
    os.environ.update(env)
    os.environ['TWINKLE_WORKER'] = '1'
    objects: Dict[int, Any] = {}
    while True:
        try:
            raw = conn.recv_bytes()
        except (EOFError, OSError):
            break
        seq, msg = cloudpickle.loads(raw)
        kind = msg[0]
        try:
            if kind == 'stop':
                conn.send_bytes(cloudpickle.dumps((seq, True, None)))
                break
            if kind == 'create':
                _, oid, cls, args, kwargs = msg
                objects[oid] = cls(*args, **kwargs)
                out = None
            elif kind == 'call':
                _, oid, method, args, kwargs = msg
                out = getattr(objects[oid], method)(*args, **kwargs)
            elif kind == 'drop':
                objects.pop(msg[1], None)
                out = None
            else:
                raise ValueError(f'unknown request {kind!r}')
            try:
                payload = cloudpickle.dumps((seq, True, out))
            except Exception as e:  # result cannot travel: say so instead of killing the worker
                payload = cloudpickle.dumps((seq, False, f'result of {msg[:3]} is not picklable: {e}'))
            conn.send_bytes(payload)
        except BaseException as e:  # noqa: BLE001 — the driver decides what to do with it
            conn.send_bytes(cloudpickle.dumps((seq, False, f'{type(e).__name__}: {e}\n{traceback.format_exc()}')))
            if isinstance(e, (KeyboardInterrupt, SystemExit)):
                break
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


class _ExternalProcess:
    """Stands in for ``multiprocessing.Process`` when the worker lives in another process tree (usually on another
    node) and only its connection is known here; it ends when it reads ``stop`` or loses the connection."""
    exitcode = None

    def __init__(self, name: str):
        self.name, self._alive = name, True

    def is_alive(self) -> bool:
        return self._alive

    def join(self, timeout: Optional[float] = None) -> None:
        self._alive = False

    def terminate(self) -> None:
        self._alive = False


class _Worker:

    def __init__(self, ctx, env: Optional[Dict[str, str]], name: str, conn=None):
        if conn is None:
            self.conn, child = ctx.Pipe(duplex=True)
            self.proc = ctx.Process(target=_worker_main, args=(child, env), name=name, daemon=True)
            self.proc.start()
            child.close()
        else:  # a worker that connected over TCP (started by ``python -m twinkle_b200.infra.agent`` somewhere)
            self.conn, self.proc = conn, _ExternalProcess(name)
        self._seq = 0
        self._lock = threading.Lock()
        self._futures: Dict[int, Future] = {}
        self._reader = threading.Thread(target=self._read, name=f'{name}-reader', daemon=True)
        self._reader.start()

    def _read(self) -> None:
        while True:
            try:
                seq, ok, payload = cloudpickle.loads(self.conn.recv_bytes())
            except (EOFError, OSError):
                with self._lock:
                    pending, self._futures = self._futures, {}
                for f in pending.values():
                    f.set_exception(RemoteError(f'worker {self.proc.name} exited (code {self.proc.exitcode}) with calls in flight'))
                return
            with self._lock:
                fut = self._futures.pop(seq, None)
            if fut is None:
                continue
            if ok:
                fut.set_result(payload)
            else:
                fut.set_exception(RemoteError(payload))

    def submit(self, msg: tuple) -> Future:
        fut: Future = Future()
        with self._lock:
            self._seq += 1
            seq = self._seq
            self._futures[seq] = fut
            try:
                self.conn.send_bytes(cloudpickle.dumps((seq, msg)))
            except (OSError, ValueError) as e:
                self._futures.pop(seq, None)
                fut.set_exception(RemoteError(f'worker {self.proc.name} is gone: {e}'))
        return fut

    def stop(self, timeout: float = 10.0) -> None:
        if self.proc.is_alive():
            try:
                self.submit(('stop', )).result(timeout)
            except Exception:
                pass
            self.proc.join(timeout)
        if self.proc.is_alive():
            self.proc.terminate()  # this exact child only
            self.proc.join(5)
        try:
            self.conn.close()
        except OSError:
            pass


class WorkerPoolManager:
    """Owns the worker processes of every ``DeviceGroup``; workers start on first use of their group."""

    def __init__(self, groups: Sequence[DeviceGroup], seed: int = 42, master_addr: str = '127.0.0.1', listen: Optional[str] = None,
                 external_groups: Optional[Sequence[str]] = None, join_timeout: float = 600.0):
        """``listen='host:port'`` opens a TCP listener for workers that are started elsewhere; the groups named in
        ``external_groups`` are then not spawned here but waited for (``join_timeout`` seconds). Connections are
        authenticated with the shared secret in ``TWINKLE_POOL_AUTHKEY`` (HMAC challenge of
        ``multiprocessing.connection``); requests are pickled code, so the listener belongs on a cluster-private network."""
        self.groups = {g.name: g for g in groups}
        self.seed, self.master_addr = seed, master_addr
        self.external = set(external_groups or ())
        self.join_timeout, self._listener = join_timeout, None
        if listen or self.external:
            from multiprocessing.connection import Listener
            key = os.environ.get('TWINKLE_POOL_AUTHKEY')
            if not key:
                raise RuntimeError('TWINKLE_POOL_AUTHKEY must be set (same value on every node) before workers can join over TCP')
            host, _, port = (listen or '0.0.0.0:0').rpartition(':')
            self._listener = Listener((host or '0.0.0.0', int(port or 0)), authkey=key.encode())
            self.listen_address = self._listener.address
        self._ctx = mp.get_context('spawn')
        self._workers: Dict[str, List[_Worker]] = {}
        self._next_oid = 0
        self._lock = threading.Lock()

    def placement(self, group: str) -> List[Dict[str, str]]:
        """Environment of every worker of ``group`` (also what a test can inspect without starting processes).

        ``ranks`` counts devices, as in the reference (``infra/_ray/resource_manager.py:186-201``): a group of
        ``len(ranks)`` devices with ``gpus_per_worker = g`` runs ``len(ranks) // g`` workers, and worker ``i`` owns the
        ``g`` consecutive devices at *position* ``i·g`` of the group — ``visible_devices`` when given, else the rank
        numbers themselves (on one node a rank is a device index).  The worker sees its own devices first (so
        ``LOCAL_RANK`` is 0) followed by the other devices of the group, which keeps CUDA IPC / peer mappings between
        the group's workers possible."""
        g = self.groups[group]
        ranks = g.rank_list()
        port = str(find_free_port())
        envs = []
        per = max(int(g.gpus_per_worker or 1), 1)
        if len(ranks) % per != 0:
            raise ValueError(f"group '{group}': {len(ranks)} ranks do not divide into workers of {per} devices")
        n = len(ranks) // per
        vd = getattr(g, 'visible_devices', None)
        if vd is None:
            visible = None
        elif isinstance(vd, (list, tuple)):
            visible = [str(x) for x in vd]
        else:
            visible = [x for x in str(vd).split(',') if x != '']
        if visible is not None and len(visible) < len(ranks):
            raise ValueError(f"group '{group}': {len(ranks)} ranks but only {len(visible)} visible devices")
        for i in range(n):
            env = {'RANK': str(i), 'LOCAL_RANK': str(i), 'WORLD_SIZE': str(n), 'LOCAL_WORLD_SIZE': str(n),
                   'MASTER_ADDR': self.master_addr, 'MASTER_PORT': port, 'TWINKLE_GROUP': group, 'TWINKLE_GLOBAL_RANK': str(ranks[i * per]),
                   'TWINKLE_SEED': str(self.seed)}
            if g.device_type in ('cuda', 'gpu'):
                pool = visible[:len(ranks)] if visible is not None else [str(r) for r in ranks]
                own = pool[i * per:(i + 1) * per]
                seen = own + [d for d in pool if d not in own]
                for other in self.groups.values():
                    if other is g or other.device_type not in ('cuda', 'gpu'):
                        continue
                    ov = getattr(other, 'visible_devices', None)
                    olist = ([str(x) for x in ov] if isinstance(ov, (list, tuple)) else [x for x in str(ov).split(',') if x != '']) if ov is not None \
                        else [str(r) for r in other.rank_list()]
                    seen += [d for d in olist[:len(other.rank_list())] if d not in seen]
                env['CUDA_VISIBLE_DEVICES'] = ','.join(seen)
                env['TWINKLE_WORKER_DEVICES'] = ','.join(own)
                env['LOCAL_RANK'] = '0'
            elif g.device_type == 'cpu':
                env['CUDA_VISIBLE_DEVICES'] = ''
            envs.append(env)
        return envs

    def workers(self, group: str) -> List[_Worker]:
        with self._lock:
            if group not in self._workers:
                if group not in self.groups:
                    raise KeyError(f'unknown device group {group!r}; known: {sorted(self.groups)}')
                if group in self.external:
                    self._workers[group] = self._accept_external(group)
                else:
                    self._workers[group] = [_Worker(self._ctx, env, f'twinkle-{group}-{i}') for i, env in enumerate(self.placement(group))]
            return self._workers[group]

    def _accept_external(self, group: str) -> List[_Worker]:
        """Waits until every rank of ``group`` has connected. A joining worker says ``('hello', group, rank, address of
        its node, a free port there)``; once all are in, each gets its environment — ``MASTER_ADDR`` / ``MASTER_PORT`` are
        those reported by rank 0, so the group's ``torch.distributed`` rendezvous happens on rank 0's node."""
        import time
        envs = self.placement(group)
        conns: Dict[int, Any] = {}
        hello: Dict[int, tuple] = {}
        deadline = time.monotonic() + self.join_timeout
        sock = self._listener._listener._socket
        while len(conns) < len(envs):
            left = deadline - time.monotonic()
            if left <= 0:
                for c in conns.values():
                    c.close()
                raise TimeoutError(f"group '{group}': {len(conns)} of {len(envs)} workers joined within {self.join_timeout:.0f} s")
            sock.settimeout(min(left, 1.0))
            try:
                c = self._listener.accept()
            except (TimeoutError, OSError):
                continue
            try:
                msg = cloudpickle.loads(c.recv_bytes())
            except (EOFError, OSError):
                continue
            if not (isinstance(msg, tuple) and len(msg) == 5 and msg[0] == 'hello' and msg[1] == group and 0 <= int(msg[2]) < len(envs)
                    and int(msg[2]) not in conns):
                c.send_bytes(cloudpickle.dumps(('refused', f'unexpected hello {msg!r:.80}')))
                c.close()
                continue
            conns[int(msg[2])], hello[int(msg[2])] = c, msg
        addr, port = hello[0][3], hello[0][4]
        workers = []
        for r, env in enumerate(envs):
            env = {k: v for k, v in env.items() if k not in ('CUDA_VISIBLE_DEVICES', 'LOCAL_RANK', 'LOCAL_WORLD_SIZE')}  # the agent pins devices
            env.update(MASTER_ADDR=str(addr), MASTER_PORT=str(port))
            conns[r].send_bytes(cloudpickle.dumps(('welcome', env)))
            workers.append(_Worker(None, None, f'twinkle-{group}-{r}@{hello[r][3]}', conn=conns[r]))
        return workers

    def new_object_id(self) -> int:
        with self._lock:
            self._next_oid += 1
            return self._next_oid

    def shutdown(self) -> None:
        with self._lock:
            all_workers = [w for ws in self._workers.values() for w in ws]
            self._workers = {}
        for w in all_workers:
            w.stop()
        if self._listener is not None:
            self._listener.close()
            self._listener = None


class RemoteProxy:
    """Driver-side stand-in for one decorated class instantiated on every worker of a group."""

    def __init__(self, pool: WorkerPoolManager, cls, group: str, execute: str, args: tuple, kwargs: dict, mesh_arg: Optional[str]):
        from . import _STATE
        self.pool, self.cls, self.group, self.execute = pool, cls, group, execute
        self.oid = pool.new_object_id()
        g = pool.groups[group]
        self.ranks = list(range(len(g.rank_list())))
        mesh = kwargs.get(mesh_arg) if mesh_arg else None
        if mesh_arg and mesh is None:
            mesh = _STATE.get('mesh')
            if mesh is not None and mesh.world_size != len(self.ranks):
                mesh = DeviceMesh.from_sizes(dp_size=len(self.ranks))
            if mesh is not None:
                kwargs = dict(kwargs, **{mesh_arg: mesh})
        self.mesh: Optional[DeviceMesh] = mesh
        if mesh is not None:
            g._device_mesh[cls.__name__] = mesh
        ws = pool.workers(group)
        targets = ws[:1] if execute == 'first' else ws
        self._targets = targets
        futs = [w.submit(('create', self.oid, cls, args, kwargs)) for w in targets]
        for f in futs:
            f.result()

    def call(self, method: str, spec: Dict[str, Any], args: tuple, kwargs: dict):
        from . import _STATE, LazyCollect, collect_results, dispatch_args
        execute = spec.get('execute', 'all')
        targets = self._targets[:1] if execute == 'first' else self._targets
        ranks = self.ranks[:len(targets)]
        n = len(targets)
        # a LazyCollect argument hands every worker its own un-collected piece
        lazy_pos = {i: a.per_worker() for i, a in enumerate(args) if isinstance(a, LazyCollect)}
        lazy_kw = {k: a.per_worker() for k, a in kwargs.items() if isinstance(a, LazyCollect)}
        plain_args = tuple(None if i in lazy_pos else a for i, a in enumerate(args))
        plain_kw = {k: (None if k in lazy_kw else v) for k, v in kwargs.items()}
        dispatch = 'all' if execute == 'first' else spec.get('dispatch', 'all')
        per = dispatch_args(dispatch, n, plain_args, plain_kw, device_mesh=self.mesh, worker_ranks=ranks)
        futs = []
        for i, (w, (a, kw)) in enumerate(zip(targets, per)):
            a = tuple(lazy_pos[j][i] if j in lazy_pos and i < len(lazy_pos[j]) else x for j, x in enumerate(a))
            kw = {k: (lazy_kw[k][i] if k in lazy_kw and i < len(lazy_kw[k]) else v) for k, v in kw.items()}
            futs.append(w.submit(('call', self.oid, method, a, kw)))
        timeout = spec.get('timeout')
        collect = spec.get('collect', 'none')
        lazy = spec.get('lazy_collect')
        if lazy is None:
            lazy = bool(_STATE.get('lazy_collect')) and not spec.get('sync')
        getters = [(lambda f=f: f.result(timeout)) for f in futs]
        if lazy:
            return LazyCollect(getters, collect, self.mesh, ranks)
        return collect_results(collect, [g() for g in getters], self.mesh, ranks)

    def drop(self) -> None:
        for w in self._targets:
            if w.proc.is_alive():
                w.submit(('drop', self.oid))

    def __del__(self):
        try:
            self.drop()
        except Exception:
            pass
