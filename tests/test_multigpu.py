"""2-GPU parity: peer-memory collectives vs NCCL, sharded and sequence-parallel training vs one GPU."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def test_two_gpu_checks():
    import torch
    n = min(torch.cuda.device_count(), 2)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    r = subprocess.run([sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={n}', '--master-addr', '127.0.0.1',
                        '--master-port', '29631', os.path.join(root, 'tests', 'mgpu_worker.py')], capture_output=True, text=True,
                       timeout=900, env=env)
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith('{')]
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert lines and all(l['ok'] for l in lines), lines
