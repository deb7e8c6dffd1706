"""Decorated components instantiated inside pool workers by ``test_worker_pool.py``."""
import os

import torch

from twinkle_b200.infra import remote_class, remote_function
from twinkle_b200.utils.device_mesh import DeviceMesh


@remote_class()
class Adder:

    def __init__(self, base: int, device_mesh: DeviceMesh = None):
        self.base = base
        self.mesh = device_mesh
        self.rank = int(os.environ.get('RANK', 0))

    @remote_function(dispatch='all', collect='none')
    def whoami(self):
        return (self.rank, int(os.environ['WORLD_SIZE']), os.environ.get('TWINKLE_WORKER'))

    @remote_function(dispatch='slice', collect='flatten')
    def add(self, xs):
        return [x + self.base for x in xs]

    @remote_function(dispatch='slice_dp', collect='flatten')
    def tag(self, xs):
        return [(self.rank, x) for x in xs]

    @remote_function(dispatch='all', collect='mean')
    def loss(self):
        return {'loss': float(self.rank), 'n': 1}

    @remote_function(dispatch='all', execute='first', collect='first')
    def only_first(self, xs):
        return (self.rank, len(xs))

    @remote_function(dispatch='all', collect='sum')
    def allreduce(self):
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group('gloo')
        t = torch.tensor([float(self.rank + 1)])
        dist.all_reduce(t)
        return float(t)

    @remote_function(dispatch='all', collect='none', lazy_collect=True)
    def produce(self):
        return [self.rank * 10, self.rank * 10 + 1]

    @remote_function(dispatch='all', collect='flatten')
    def consume(self, piece):
        return [p + 1000 * self.rank for p in piece]

    @remote_function()
    def boom(self):
        raise ValueError(f'bad thing on rank {self.rank}')
