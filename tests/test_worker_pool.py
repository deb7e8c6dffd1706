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


def test_placement_counts_devices_not_workers():
    """``ranks`` counts devices: 8 ranks with 2 devices per worker are 4 workers, each owning two consecutive devices by
    *position* in the group; a group whose ranks do not start at 0 still gets its own devices."""
    from twinkle_b200.infra.worker_pool import WorkerPoolManager
    groups = [DeviceGroup(name='wide', ranks=8, device_type='cuda', gpus_per_worker=2),
              DeviceGroup(name='tail', ranks=[4, 5, 6, 7], device_type='cuda', visible_devices=['4', '5', '6', '7']),
              DeviceGroup(name='plain', ranks=[6, 7], device_type='cuda'),
              DeviceGroup(name='host', ranks=2, device_type='cpu')]
    mgr = WorkerPoolManager(groups)
    wide = mgr.placement('wide')
    assert len(wide) == 4 == groups[0].num_workers()
    assert [e['RANK'] for e in wide] == ['0', '1', '2', '3'] and all(e['WORLD_SIZE'] == '4' for e in wide)
    assert [e['TWINKLE_WORKER_DEVICES'] for e in wide] == ['0,1', '2,3', '4,5', '6,7']
    assert [e['TWINKLE_GLOBAL_RANK'] for e in wide] == ['0', '2', '4', '6']
    # a worker sees its own devices first (LOCAL_RANK 0), then the rest of its group
    assert wide[1]['CUDA_VISIBLE_DEVICES'].split(',')[:2] == ['2', '3'] and sorted(set(wide[1]['CUDA_VISIBLE_DEVICES'].split(','))) == [str(i) for i in range(8)]
    assert all(e['LOCAL_RANK'] == '0' for e in wide)
    tail = mgr.placement('tail')
    assert [e['TWINKLE_WORKER_DEVICES'] for e in tail] == ['4', '5', '6', '7']
    assert [e['TWINKLE_GLOBAL_RANK'] for e in tail] == ['4', '5', '6', '7'] and all(e['WORLD_SIZE'] == '4' for e in tail)
    plain = mgr.placement('plain')
    assert [e['TWINKLE_WORKER_DEVICES'] for e in plain] == ['6', '7']          # never devices 0 and 1 of another group
    # devices of the other GPU groups come last: visible for peer copies across groups, never device 0 of this worker
    vis = plain[0]['CUDA_VISIBLE_DEVICES'].split(',')
    assert vis[:2] == ['6', '7'] and set(vis) >= {'0', '1', '2', '3', '4', '5'} and len(vis) == len(set(vis))
    host = mgr.placement('host')
    assert all(e['CUDA_VISIBLE_DEVICES'] == '' for e in host) and [e['LOCAL_RANK'] for e in host] == ['0', '1']
    with pytest.raises(ValueError):
        WorkerPoolManager([DeviceGroup(name='odd', ranks=3, device_type='cuda', gpus_per_worker=2)]).placement('odd')
