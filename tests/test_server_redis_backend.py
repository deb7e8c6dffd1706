"""The Redis state backend against an in-memory stand-in for the ``redis`` package: JSON round trip, key listing under
the prefix, optimistic ``update_atomic`` (retry on a lost race, give up after ``MAX_RETRIES``, library errors mapped to the
server's own exception), expiry passed through, and the ``ServerState`` facade on top of it."""
import sys
import types

import pytest


def _fake_redis(fail_watches=0, broken=False):
    mod = types.ModuleType('redis')

    class RedisError(Exception):
        pass

    class WatchError(RedisError):
        pass

    store, ttls, state = {}, {}, {'fail': fail_watches}

    class Pipeline:

        def __init__(self):
            self.queued, self.watched = [], None

        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

        def watch(self, k):
            self.watched = k

        def get(self, k):
            if broken:
                raise RedisError('connection lost')
            return store.get(k)

        def multi(self):
            self.queued = []

        def set(self, k, v):
            self.queued.append(('set', k, v))

        def delete(self, k):
            self.queued.append(('del', k, None))

        def execute(self):
            if state['fail'] > 0:              # somebody else wrote the watched key between WATCH and EXEC
                state['fail'] -= 1
                raise WatchError()
            for op, k, v in self.queued:
                if op == 'set':
                    store[k] = v.encode()
                else:
                    store.pop(k, None)

    class Redis:

        @classmethod
        def from_url(cls, url):
            assert url.startswith('redis://')
            return cls()

        def set(self, k, v, ex=None):
            store[k] = v.encode()
            ttls[k] = ex

        def get(self, k):
            return store.get(k)

        def delete(self, k):
            return 1 if store.pop(k, None) is not None else 0

        def scan_iter(self, pattern):
            assert pattern.endswith('*')
            return [k.encode() for k in sorted(store) if k.startswith(pattern[:-1])]

        def pipeline(self):
            return Pipeline()

    mod.Redis, mod.RedisError, mod.WatchError = Redis, RedisError, WatchError
    mod._store, mod._ttls = store, ttls
    return mod


def test_redis_backend_round_trip_listing_and_expiry(monkeypatch):
    fake = _fake_redis()
    monkeypatch.setitem(sys.modules, 'redis', fake)
    from twinkle_b200.server.state import RedisBackend, ServerState
    b = RedisBackend('redis://h:6379/0', prefix='tw')
    b.set('session:a', {'x': 1}, ttl=30)
    b.set('model:m', [1, 2])
    assert fake._ttls['tw:session:a'] == 30 and 'tw:model:m' in fake._store
    assert b.get('session:a') == {'x': 1} and b.get('nope', 'dflt') == 'dflt'
    assert b.keys('session:') == ['session:a'] and sorted(b.keys()) == ['model:m', 'session:a']
    assert b.exists('model:m') and b.count('model:') == 1 and b.mget(['model:m', 'zz']) == [[1, 2], None]
    assert b.update_atomic('counter', lambda c: (c or 0) + 1) == 1 and b.update_atomic('counter', lambda c: c + 1) == 2
    assert b.update_atomic('counter', lambda c: None) is None and not b.exists('counter')
    assert b.set_nx('lease', 'me') and not b.set_nx('lease', 'you') and b.get('lease') == 'me'
    assert b.delete('model:m') and not b.delete('model:m')
    st = ServerState(b)
    sid = st.create_session('tok', {'who': 'x'})
    assert st.heartbeat(sid) and st.get_session(sid)['token'] == 'tok' and not st.heartbeat('missing')


def test_redis_update_retries_lost_races_then_gives_up(monkeypatch):
    fake = _fake_redis(fail_watches=3)
    monkeypatch.setitem(sys.modules, 'redis', fake)
    from twinkle_b200.server.exceptions import ConcurrencyError, StateBackendError
    from twinkle_b200.server.state import RedisBackend
    b = RedisBackend('redis://h/0')
    calls = []
    assert b.update_atomic('k', lambda c: calls.append(c) or (c or 0) + 5) == 5
    assert len(calls) == 4                                   # three lost races, then the write went through
    monkeypatch.setattr(RedisBackend, 'MAX_RETRIES', 2)
    monkeypatch.setitem(sys.modules, 'redis', _fake_redis(fail_watches=10))
    with pytest.raises(ConcurrencyError):
        RedisBackend('redis://h/0').update_atomic('k', lambda c: 1)
    monkeypatch.setitem(sys.modules, 'redis', _fake_redis(broken=True))
    with pytest.raises(StateBackendError):
        RedisBackend('redis://h/0').update_atomic('k', lambda c: 1)
