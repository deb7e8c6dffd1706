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
