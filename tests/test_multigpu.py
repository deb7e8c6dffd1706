"""Multi-GPU parity checks, one short torchrun per group (2 ranks): fused tensor-parallel GEMM+collective kernels vs
NCCL + library GEMM, expert parallel (NCCL and peer-memory modes) vs one GPU, tensor x pipeline parallel vs one GPU,
the peer all-gather / reduce-scatter / Ulysses exchange kernels vs NCCL, and FSDP / FSDP + Ulysses training in both
communication modes vs the single-GPU loss curve.  Everything runs wherever at least two GPUs are visible."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _run(only: str, port: int, timeout: int):
    import torch
    n = min(torch.cuda.device_count(), 2)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE='0', TK_MGPU_ONLY=only)
    r = subprocess.run([sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={n}', '--master-addr', '127.0.0.1',
                        '--master-port', str(port), os.path.join(root, 'tests', 'mgpu_worker.py')], capture_output=True, text=True,
                       timeout=timeout, env=env)
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith('{')]
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert lines and all(l['ok'] for l in lines), lines
    return lines


def test_fused_tensor_parallel_kernels():
    _run('tp_fused', 29631, 240)


def test_expert_parallel_matches_single_gpu():
    _run('ep', 29632, 240)


def test_tensor_pipeline_parallel_matches_single_gpu():
    _run('megatron', 29633, 240)


def test_ulysses_projection_with_fused_head_scatter():
    _run('ulysses_fused', 29635, 240)


def test_peer_collective_kernels_match_nccl():
    _run('peer', 29634, 300)


def test_fsdp_and_ulysses_training_match_single_gpu():
    _run('fsdp', 29636, 600)
