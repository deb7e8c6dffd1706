"""Pool mode: one worker process per rank of a device group, dispatch / execute / collect rules on the driver."""
import pytest

from twinkle_b200 import infra
from twinkle_b200.utils.device_mesh import DeviceGroup, DeviceMesh


@pytest.fixture()
def pool():
    infra.initialize(mode='pool', groups=[DeviceGroup(name='model', ranks=2, device_type='cpu')],
                     global_device_mesh=DeviceMesh.from_sizes(dp_size=2))
    yield
    infra.shutdown()


def test_pool_dispatch_collect(pool):
    from tests.pool_components import Adder
    a = Adder(5, remote_group='model')
    assert a.whoami() == [(0, 2, '1'), (1, 2, '1')]
    assert a.add([1, 2, 3, 4, 5]) == [6, 7, 8, 9, 10]
    assert a.tag(['a', 'b', 'c', 'd']) == [(0, 'a'), (0, 'b'), (1, 'c'), (1, 'd')]
    assert a.loss() == {'loss': 0.5, 'n': 1.0}
    assert a.only_first([1, 2, 3]) == (0, 3)
    assert a.allreduce() == 6.0  # both workers joined one gloo world: (1+2) on each, summed by collect
    lazy = a.produce()
    assert isinstance(lazy, infra.LazyCollect)
    assert a.consume(lazy) == [0, 1, 1010, 1011]  # each worker got its own piece back
    assert lazy() == [[0, 1], [10, 11]]
    with pytest.raises(Exception, match='bad thing on rank'):
        a.boom()
    assert a.add([1, 2]) == [6, 7]  # workers survive a remote exception


def test_local_instances_are_plain_objects():
    from tests.pool_components import Adder
    a = Adder(1)
    assert a.add([1, 2]) == [2, 3]


def test_workers_join_over_tcp_from_an_agent(monkeypatch):
    """The group's workers are not spawned by the driver: an agent (here in a thread, on another node in practice)
    starts them and they connect to the driver's listener; dispatch, collectives and shutdown work as for local ones."""
    import threading
    from tests.pool_components import Adder
    from twinkle_b200.infra.agent import launch, parse_ranks
    assert parse_ranks('0-2, 5,7-8') == [0, 1, 2, 5, 7, 8]
    monkeypatch.setenv('TWINKLE_POOL_AUTHKEY', 'test-secret')
    infra.initialize(mode='pool', groups=[DeviceGroup(name='far', ranks=2, device_type='cpu')], global_device_mesh=DeviceMesh.from_sizes(dp_size=2),
                     pool_listen='127.0.0.1:0', external_groups=['far'], join_timeout=120)
    try:
        host, port = infra._STATE['pool'].listen_address
        procs = []
        t = threading.Thread(target=lambda: procs.extend(launch(f'{host}:{port}', 'far', [0, 1], wait=False)), daemon=True)
        t.start()
        a = Adder(3, remote_group='far')         # blocks until both ranks have joined
        t.join()
        assert a.whoami() == [(0, 2, '1'), (1, 2, '1')]
        assert a.add([1, 2, 3, 4]) == [4, 5, 6, 7]
        assert a.allreduce() == 6.0              # MASTER_ADDR / MASTER_PORT came from rank 0's hello
        with pytest.raises(Exception, match='bad thing on rank'):
            a.boom()
    finally:
        infra.shutdown()
    for p in procs:
        p.join(30)
        assert not p.is_alive()


def test_tcp_pool_needs_a_shared_secret(monkeypatch):
    from twinkle_b200.infra.worker_pool import WorkerPoolManager
    monkeypatch.delenv('TWINKLE_POOL_AUTHKEY', raising=False)
    with pytest.raises(RuntimeError, match='TWINKLE_POOL_AUTHKEY'):
        WorkerPoolManager([DeviceGroup(name='far', ranks=1, device_type='cpu')], listen='127.0.0.1:0', external_groups=['far'])
    monkeypatch.setenv('TWINKLE_POOL_AUTHKEY', 'k')
    m = WorkerPoolManager([DeviceGroup(name='far', ranks=1, device_type='cpu')], listen='127.0.0.1:0', external_groups=['far'], join_timeout=1.5)
    try:
        with pytest.raises(TimeoutError, match='0 of 1 workers joined'):
            m.workers('far')
    finally:
        m.shutdown()
