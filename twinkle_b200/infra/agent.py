"""Starts the workers of one device group on this node and connects them to a driver on another node:

    TWINKLE_POOL_AUTHKEY=… python -m twinkle_b200.infra.agent --driver 10.0.0.1:29400 --group model --ranks 8-15 --gpus 0,1,2,3,4,5,6,7

One process per rank is spawned; rank ``r`` gets ``gpus[i]`` (or ``gpus_per_worker`` consecutive ones) as its only visible
device. Each connects to the driver's listener (``WorkerPoolManager(listen=…, external_groups=[…])``), receives its
``RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT`` and then serves the same request loop as a locally spawned worker. This
is the counterpart of the reference's Ray placement across nodes (``infra/_ray/resource_manager.py:12-281``) without Ray."""
from __future__ import annotations

import argparse
import multiprocessing as mp
import os
import socket
from typing import Dict, List, Optional

import cloudpickle


def parse_ranks(spec: str) -> List[int]:
    """``"0-3,6,8-9"`` → ``[0, 1, 2, 3, 6, 8, 9]``."""
    out: List[int] = []
    for part in spec.split(','):
        part = part.strip()
        if not part:
            continue
        if '-' in part:
            a, b = part.split('-', 1)
            out.extend(range(int(a), int(b) + 1))
        else:
            out.append(int(part))
    return out


def node_address(driver_host: str, driver_port: int) -> str:
    """The address of this node as the driver's side of the network sees it (the source address of a route to it)."""
    try:
        s = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        try:
            s.connect((driver_host, driver_port))
            return s.getsockname()[0]
        finally:
            s.close()
    except OSError:
        return '127.0.0.1'


def external_worker_main(driver: str, authkey: str, group: str, rank: int, env: Dict[str, str]) -> None:
    from multiprocessing.connection import Client

    from ..utils.network import find_free_port
    from .worker_pool import _worker_main
    os.environ.update(env)
    host, _, port = driver.rpartition(':')
    conn = Client((host, int(port)), authkey=authkey.encode())
    conn.send_bytes(cloudpickle.dumps(('hello', group, rank, node_address(host, int(port)), find_free_port())))
    kind, payload = cloudpickle.loads(conn.recv_bytes())
    if kind != 'welcome':
        raise RuntimeError(f'driver refused worker {group}:{rank}: {payload}')
    _worker_main(conn, payload)


def launch(driver: str, group: str, ranks: List[int], gpus: Optional[List[str]] = None, gpus_per_worker: int = 1, wait: bool = True):
    key = os.environ.get('TWINKLE_POOL_AUTHKEY')
    if not key:
        raise RuntimeError('TWINKLE_POOL_AUTHKEY must be set to the driver\'s value')
    ctx = mp.get_context('spawn')
    procs = []
    for i, r in enumerate(ranks):
        env = {'LOCAL_RANK': '0' if gpus else str(i), 'LOCAL_WORLD_SIZE': str(len(ranks))}
        if gpus is not None:
            env['CUDA_VISIBLE_DEVICES'] = ','.join(gpus[i * gpus_per_worker:(i + 1) * gpus_per_worker])
        p = ctx.Process(target=external_worker_main, args=(driver, key, group, r, env), name=f'twinkle-{group}-{r}', daemon=False)
        p.start()
        procs.append(p)
    if wait:
        for p in procs:
            p.join()
    return procs


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split('\n')[0])
    ap.add_argument('--driver', required=True, help='host:port of the driver\'s listener')
    ap.add_argument('--group', required=True)
    ap.add_argument('--ranks', required=True, help='ranks of the group that run on this node, e.g. 8-15')
    ap.add_argument('--gpus', default=None, help='comma-separated device ids to hand out in rank order (omit for CPU workers)')
    ap.add_argument('--gpus-per-worker', type=int, default=1)
    a = ap.parse_args(argv)
    launch(a.driver, a.group, parse_ranks(a.ranks), a.gpus.split(',') if a.gpus else None, a.gpus_per_worker)


if __name__ == '__main__':
    main()
