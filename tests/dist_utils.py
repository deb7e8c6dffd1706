"""Helpers to run a function on N CPU ranks (gloo) inside a test."""
import io
import os
import socket
import sys
import traceback

import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn, args, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world),
                      MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    torch.set_num_threads(2)
    try:
        import torch.distributed as dist
        dist.init_process_group('gloo', rank=rank, world_size=world, init_method=f'tcp://127.0.0.1:{port}')
        out = fn(rank, world, *args)
        # by value: tensors put on a queue travel as file descriptors fetched from this process, which may be gone by the
        # time the parent unpickles them
        buf = io.BytesIO()
        torch.save(out, buf)
        q.put((rank, 'ok', buf.getvalue()))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        q.put((rank, 'err', traceback.format_exc()))


def run_ranks(fn, world: int, *args, timeout: float = 300.0):
    """Returns the list of per-rank results (rank order); raises on any failure."""
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=timeout)
            if status != 'ok':
                raise RuntimeError(f'rank {rank} failed:\n{payload}')
            results[rank] = torch.load(io.BytesIO(payload), weights_only=False)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
