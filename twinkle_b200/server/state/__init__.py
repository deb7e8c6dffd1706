"""Shared server state: key-value backends, resource managers and the cleanup-leader lease.

Parity: reference ``src/twinkle/server/state/server_state.py:38-642``, ``state/backend/base.py:12-99`` and the
``*_manager.py`` files — a process-local facade over a ``StateBackend`` (``set/get/delete/exists/keys/count/
set_nx/update_atomic/mget``); back ends: in-process memory, fcntl-locked JSON file, Redis (optional package);
managers for sessions (heartbeats), models (per-token limit, replica capacity), sampling sessions, futures
and config; one replica holds a TTL lease (``LEASE_TTL`` 30 s, renewed every 10 s) and is the only one that
sweeps expired resources and publishes gauges.
"""
from __future__ import annotations

import fcntl
import json
import os
import threading
import time
import uuid
from typing import Any, Callable, Dict, Iterable, List, Optional
from ..exceptions import ConcurrencyError, ResourceExhaustedError, StateBackendError

LEASE_TTL = 30.0
LEASE_RENEW = 10.0


class StateBackend:

    def set(self, key: str, value: Any, ttl: Optional[float] = None) -> None: raise NotImplementedError
    def get(self, key: str, default: Any = None) -> Any: raise NotImplementedError
    def delete(self, key: str) -> bool: raise NotImplementedError
    def keys(self, prefix: str = '') -> List[str]: raise NotImplementedError
    def update_atomic(self, key: str, fn: Callable[[Any], Any], default: Any = None) -> Any: raise NotImplementedError

    def exists(self, key: str) -> bool:
        return self.get(key, _MISSING) is not _MISSING

    def count(self, prefix: str = '') -> int:
        return len(self.keys(prefix))

    def mget(self, keys: Iterable[str]) -> List[Any]:
        return [self.get(k) for k in keys]

    def set_nx(self, key: str, value: Any, ttl: Optional[float] = None) -> bool:
        won = {'v': False}

        def fn(cur):
            if cur is None:
                won['v'] = True
                return value
            return cur

        self.update_atomic(key, fn)
        if won['v'] and ttl:
            self.set(key, value, ttl)
        return won['v']


_MISSING = object()


class MemoryBackend(StateBackend):

    def __init__(self):
        self._d: Dict[str, Any] = {}
        self._exp: Dict[str, float] = {}
        self._lock = threading.RLock()

    def _alive(self, key: str) -> bool:
        e = self._exp.get(key)
        if e is not None and time.time() > e:
            self._d.pop(key, None)
            self._exp.pop(key, None)
            return False
        return key in self._d

    def set(self, key, value, ttl=None):
        with self._lock:
            self._d[key] = value
            if ttl:
                self._exp[key] = time.time() + ttl
            else:
                self._exp.pop(key, None)

    def get(self, key, default=None):
        with self._lock:
            return self._d[key] if self._alive(key) else default

    def delete(self, key):
        with self._lock:
            self._exp.pop(key, None)
            return self._d.pop(key, _MISSING) is not _MISSING

    def keys(self, prefix=''):
        with self._lock:
            return [k for k in list(self._d) if k.startswith(prefix) and self._alive(k)]

    def update_atomic(self, key, fn, default=None):
        with self._lock:
            cur = self._d[key] if self._alive(key) else default
            new = fn(cur)
            if new is None:
                self._d.pop(key, None)
            else:
                self._d[key] = new
            return new


class FileBackend(StateBackend):
    """One JSON document guarded by ``flock``; survives restarts and is shared by processes on a host."""

    def __init__(self, path: str):
        self.path = path
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        if not os.path.exists(path):
            with open(path, 'w') as f:
                json.dump({'data': {}, 'exp': {}}, f)

    def _txn(self, fn):
        with open(self.path, 'r+') as f:
            fcntl.flock(f, fcntl.LOCK_EX)
            try:
                try:
                    doc = json.load(f)
                except json.JSONDecodeError:
                    doc = {'data': {}, 'exp': {}}
                now = time.time()
                for k in [k for k, e in doc['exp'].items() if e < now]:
                    doc['data'].pop(k, None)
                    doc['exp'].pop(k, None)
                out, dirty = fn(doc)
                if dirty:
                    f.seek(0)
                    f.truncate()
                    json.dump(doc, f)
                    f.flush()  # the data must be in the file before the lock is released
                return out
            finally:
                fcntl.flock(f, fcntl.LOCK_UN)

    def set(self, key, value, ttl=None):
        def fn(doc):
            doc['data'][key] = value
            if ttl:
                doc['exp'][key] = time.time() + ttl
            else:
                doc['exp'].pop(key, None)
            return None, True
        self._txn(fn)

    def get(self, key, default=None):
        return self._txn(lambda doc: (doc['data'].get(key, default), False))

    def delete(self, key):
        def fn(doc):
            doc['exp'].pop(key, None)
            return (doc['data'].pop(key, _MISSING) is not _MISSING), True
        return self._txn(fn)

    def keys(self, prefix=''):
        return self._txn(lambda doc: ([k for k in doc['data'] if k.startswith(prefix)], False))

    def update_atomic(self, key, fn, default=None):
        def t(doc):
            new = fn(doc['data'].get(key, default))
            if new is None:
                doc['data'].pop(key, None)
            else:
                doc['data'][key] = new
            return new, True
        return self._txn(t)

    def clear(self):
        self._txn(lambda doc: (doc.update(data={}, exp={}), True))


class RedisBackend(StateBackend):
    MAX_RETRIES = 64

    def __init__(self, url: str, prefix: str = 'twinkle'):
        import redis  # type: ignore
        self.r = redis.Redis.from_url(url)
        self.prefix = prefix + ':'

    def set(self, key, value, ttl=None):
        self.r.set(self.prefix + key, json.dumps(value), ex=int(ttl) if ttl else None)

    def get(self, key, default=None):
        v = self.r.get(self.prefix + key)
        return default if v is None else json.loads(v)

    def delete(self, key):
        return bool(self.r.delete(self.prefix + key))

    def keys(self, prefix=''):
        return [k.decode()[len(self.prefix):] for k in self.r.scan_iter(self.prefix + prefix + '*')]

    def update_atomic(self, key, fn, default=None):
        import redis  # type: ignore
        k = self.prefix + key
        with self.r.pipeline() as p:
            for _attempt in range(self.MAX_RETRIES):
                try:
                    p.watch(k)
                    cur = p.get(k)
                    new = fn(default if cur is None else json.loads(cur))
                    p.multi()
                    if new is None:
                        p.delete(k)
                    else:
                        p.set(k, json.dumps(new))
                    p.execute()
                    return new
                except redis.WatchError:
                    continue
                except redis.RedisError as e:
                    raise StateBackendError(f'redis update of {key!r} failed: {e}') from e
        raise ConcurrencyError(f'update of {key!r} lost {self.MAX_RETRIES} races in a row')


def build_backend(cfg) -> StateBackend:
    mode = getattr(cfg, 'mode', 'memory')
    if mode == 'file':
        return FileBackend(cfg.file_path)
    if mode == 'redis':
        return RedisBackend(cfg.redis_url, cfg.key_prefix)
    return MemoryBackend()


class ServerState:
    """Facade used by every app.  Keys: ``session:<id>``, ``model:<id>``, ``sampling:<id>``, ``future:<id>``,
    ``replica:<id>``, ``config:<k>``, ``lease:cleanup``."""

    def __init__(self, backend: Optional[StateBackend] = None, replica_id: Optional[str] = None, per_token_model_limit: int = 30):
        self.backend = backend or MemoryBackend()
        self.replica_id = replica_id or uuid.uuid4().hex[:12]
        self.per_token_model_limit = per_token_model_limit
        self._last_renew = 0.0

    # ------------------------------------------------------------ sessions
    def create_session(self, token: str, metadata: Optional[Dict[str, Any]] = None, session_id: Optional[str] = None) -> str:
        sid = session_id or uuid.uuid4().hex
        self.backend.set(f'session:{sid}', {'token': token, 'created': time.time(), 'heartbeat': time.time(), 'metadata': metadata or {}})
        return sid

    def heartbeat(self, session_id: str) -> bool:
        hit = {'v': False}

        def fn(cur):
            if cur is None:
                return None
            hit['v'] = True
            cur['heartbeat'] = time.time()
            return cur

        self.backend.update_atomic(f'session:{session_id}', fn)
        return hit['v']

    def get_session(self, session_id: str) -> Optional[Dict[str, Any]]:
        return self.backend.get(f'session:{session_id}')

    def session_age(self, session_id: str) -> Optional[float]:
        s = self.get_session(session_id)
        return None if s is None else time.time() - s['heartbeat']

    # -------------------------------------------------------------- models
    def register_model(self, model_id: str, token: str, base_model: str, session_id: Optional[str], replica_id: Optional[str] = None,
                       info: Optional[Dict[str, Any]] = None) -> None:
        n = sum(1 for k in self.backend.keys('model:') if (self.backend.get(k) or {}).get('token') == token)
        if n >= self.per_token_model_limit:
            raise ResourceExhaustedError(f'model limit reached for this token ({self.per_token_model_limit})')
        self.backend.set(f'model:{model_id}', {'token': token, 'base_model': base_model, 'session_id': session_id,
                                               'replica_id': replica_id or self.replica_id, 'created': time.time(), **(info or {})})

    def get_model(self, model_id: str) -> Optional[Dict[str, Any]]:
        return self.backend.get(f'model:{model_id}')

    def unregister_model(self, model_id: str) -> bool:
        return self.backend.delete(f'model:{model_id}')

    def list_models(self, token: Optional[str] = None) -> Dict[str, Dict[str, Any]]:
        out = {}
        for k in self.backend.keys('model:'):
            v = self.backend.get(k)
            if v and (token is None or v.get('token') == token):
                out[k[len('model:'):]] = v
        return out

    def register_replica(self, replica_id: str, base_model: str, max_loras: int, used: int = 0) -> None:
        self.backend.set(f'replica:{replica_id}', {'base_model': base_model, 'max_loras': max_loras, 'used': used, 'seen': time.time()},
                         ttl=3 * LEASE_TTL)

    def replica_capacity(self) -> Dict[str, Dict[str, Any]]:
        return {k[len('replica:'):]: self.backend.get(k) for k in self.backend.keys('replica:')}

    # --------------------------------------------------- sampling sessions
    def create_sampling_session(self, token: str, base_model: str, model_path: Optional[str], session_id: Optional[str]) -> str:
        sid = uuid.uuid4().hex
        self.backend.set(f'sampling:{sid}', {'token': token, 'base_model': base_model, 'model_path': model_path, 'session_id': session_id,
                                             'created': time.time()})
        return sid

    def get_sampling_session(self, sid: str) -> Optional[Dict[str, Any]]:
        return self.backend.get(f'sampling:{sid}')

    # -------------------------------------------------------------- futures
    def create_future(self, request_id: Optional[str] = None, **meta) -> str:
        rid = request_id or uuid.uuid4().hex
        self.backend.set(f'future:{rid}', {'status': 'pending', 'created': time.time(), **meta}, ttl=3600)
        return rid

    def set_future(self, rid: str, status: str, result: Any = None, error: Optional[str] = None, **extra) -> None:
        def fn(cur):
            cur = cur or {'created': time.time()}
            cur.update(status=status, updated=time.time(), **extra)
            if result is not None:
                cur['result'] = result
            if error is not None:
                cur['error'] = error
            return cur
        self.backend.update_atomic(f'future:{rid}', fn)

    def get_future(self, rid: str) -> Optional[Dict[str, Any]]:
        return self.backend.get(f'future:{rid}')

    # --------------------------------------------------------------- config
    def set_config(self, key: str, value: Any) -> None:
        self.backend.set(f'config:{key}', value)

    def get_config(self, key: str, default: Any = None) -> Any:
        return self.backend.get(f'config:{key}', default)

    # ---------------------------------------------------------------- lease
    def try_acquire_leadership(self, now: Optional[float] = None) -> bool:
        """True while this replica holds (or just took) the cleanup lease."""
        now = time.time() if now is None else now
        me = self.replica_id
        res = {'leader': False}

        def fn(cur):
            if cur is None or cur.get('expires', 0) < now or cur.get('owner') == me:
                res['leader'] = True
                return {'owner': me, 'expires': now + LEASE_TTL}
            return cur

        try:
            self.backend.update_atomic('lease:cleanup', fn)
        except Exception:
            return False
        return res['leader']

    def is_leader(self) -> bool:
        cur = self.backend.get('lease:cleanup')
        return bool(cur and cur.get('owner') == self.replica_id and cur.get('expires', 0) >= time.time())

    def release_leadership(self) -> None:
        def fn(cur):
            return None if cur and cur.get('owner') == self.replica_id else cur
        self.backend.update_atomic('lease:cleanup', fn)

    # -------------------------------------------------------------- cleanup
    def sweep(self, session_timeout: float, max_lifetime: float = float('inf')) -> Dict[str, List[str]]:
        """Leader only: expire sessions without heartbeat and everything that hangs off them."""
        removed: Dict[str, List[str]] = {'sessions': [], 'models': [], 'sampling': []}
        if not self.try_acquire_leadership():
            return removed
        now = time.time()
        dead = set()
        for k in self.backend.keys('session:'):
            s = self.backend.get(k)
            if s and (now - s['heartbeat'] > session_timeout or now - s['created'] > max_lifetime):
                dead.add(k[len('session:'):])
                self.backend.delete(k)
                removed['sessions'].append(k[len('session:'):])
        for prefix, name in (('model:', 'models'), ('sampling:', 'sampling')):
            for k in self.backend.keys(prefix):
                v = self.backend.get(k)
                if v and v.get('session_id') in dead:
                    self.backend.delete(k)
                    removed[name].append(k[len(prefix):])
        return removed

    def gauges(self) -> Dict[str, int]:
        return {'sessions': self.backend.count('session:'), 'models': self.backend.count('model:'),
                'sampling_sessions': self.backend.count('sampling:'), 'futures': self.backend.count('future:')}
