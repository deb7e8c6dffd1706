import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a B200 (run with -m gpu on the GPU box)')
    config.addinivalue_line('markers', 'multigpu: needs 2+ GPUs')


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
        n_gpu = torch.cuda.device_count() if has_gpu else 0
    except Exception:
        has_gpu, n_gpu = False, 0
    for item in items:
        if 'gpu' in item.keywords and not has_gpu:
            item.add_marker(pytest.mark.skip(reason='no GPU in this process'))
        if 'multigpu' in item.keywords and n_gpu < 2:
            item.add_marker(pytest.mark.skip(reason='needs >= 2 GPUs'))
