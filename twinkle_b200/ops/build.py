"""Builds / loads the in-tree sm_100a extension.

``build_extension()`` compiles every ``csrc/*.cu`` with
``-gencode arch=compute_100a,code=sm_100a`` into ``ops/_C.so`` next to this
file (nvcc cross-compiles without a GPU).  ``load_extension()`` imports the
built module; when a GPU is present and the module is missing it is built on
the spot, and any failure raises — there is no silent fallback on a GPU box.
"""
from __future__ import annotations

import glob
import hashlib
import importlib.util
import os
import subprocess
import sys
import sysconfig
from typing import List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, 'csrc')
_SO = os.path.join(_HERE, '_C.so')
_STAMP = os.path.join(_HERE, '_C.stamp')
_MOD = None

NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17', '--use_fast_math',
              '-Xcompiler', '-fPIC', '--expt-relaxed-constexpr', '--expt-extended-lambda', '-DNDEBUG',
              '-U__CUDA_NO_HALF_OPERATORS__', '-U__CUDA_NO_BFLOAT16_CONVERSIONS__', '-U__CUDA_NO_HALF_CONVERSIONS__']


def _sources() -> List[str]:
    return sorted(glob.glob(os.path.join(_CSRC, '*.cu')) + glob.glob(os.path.join(_CSRC, '*.cpp')))


def _local_includes(path: str, seen=None) -> List[str]:
    """In-tree headers reachable from ``path`` through ``#include "…"`` lines (sorted, each once)."""
    import re
    seen = set() if seen is None else seen
    with open(path, errors='replace') as f:
        for name in re.findall(r'^\s*#\s*include\s*"([^"]+)"', f.read(), flags=re.M):
            hdr = os.path.join(_CSRC, name)
            if os.path.isfile(hdr) and hdr not in seen:
                seen.add(hdr)
                _local_includes(hdr, seen)
    return sorted(seen)


def _digest() -> str:
    h = hashlib.sha1()
    for f in _sources() + sorted(glob.glob(os.path.join(_CSRC, '*.cuh')) + glob.glob(os.path.join(_CSRC, '*.h'))):
        with open(f, 'rb') as fh:
            h.update(fh.read())
    h.update(' '.join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_built() -> bool:
    if not os.path.isfile(_SO) or not os.path.isfile(_STAMP):
        return False
    with open(_STAMP) as f:
        return f.read().strip() == _digest()


def build_extension(verbose: bool = False, jobs: Optional[int] = None) -> str:
    """Compile each source to an object (in parallel) and link ``_C.so``.  Processes that arrive together (the ranks
    of one job) take a file lock in turn: the first builds, the others find the stamp current and return."""
    if is_built():
        return _SO
    import fcntl
    lock = open(os.path.join(_HERE, '.build.lock'), 'w')
    fcntl.flock(lock, fcntl.LOCK_EX)
    try:
        if is_built():
            return _SO
        return _build_locked(verbose, jobs)
    finally:
        fcntl.flock(lock, fcntl.LOCK_UN)
        lock.close()


def _build_locked(verbose: bool, jobs: Optional[int]) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    from concurrent.futures import ThreadPoolExecutor
    cuda_home = os.environ.get('CUDA_HOME', '/usr/local/cuda')
    nvcc = os.path.join(cuda_home, 'bin', 'nvcc')
    inc = ['-I' + p for p in ce.include_paths(device_type='cuda')] + ['-I' + sysconfig.get_paths()['include'], '-I' + _CSRC]
    abi = getattr(torch._C, '_GLIBCXX_USE_CXX11_ABI', True)
    defs = ['-DTORCH_EXTENSION_NAME=_C', '-DTORCH_API_INCLUDE_EXTENSION_H', f'-D_GLIBCXX_USE_CXX11_ABI={int(abi)}']
    build_dir = os.path.join(_HERE, 'build')
    os.makedirs(build_dir, exist_ok=True)
    objs = []

    def compile_one(src: str) -> str:
        obj = os.path.join(build_dir, os.path.basename(src) + '.o')
        dep_stamp = obj + '.sha'
        h = hashlib.sha1(open(src, 'rb').read())
        for hdr in _local_includes(src):  # only the headers this source pulls in: touching one header rebuilds its users
            h.update(open(hdr, 'rb').read())
        h.update(' '.join(NVCC_FLAGS).encode())
        if os.path.isfile(obj) and os.path.isfile(dep_stamp) and open(dep_stamp).read() == h.hexdigest():
            return obj
        cmd = [nvcc, '-c', src, '-o', obj] + NVCC_FLAGS + inc + defs
        if verbose:
            cmd += ['-Xptxas', '-v']
            print(' '.join(cmd), file=sys.stderr)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f'nvcc failed for {src}:\n{r.stdout}\n{r.stderr}')
        if verbose:
            print(r.stderr, file=sys.stderr)
        with open(dep_stamp, 'w') as f:
            f.write(h.hexdigest())
        return obj

    with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 4)) as pool:
        objs = list(pool.map(compile_one, _sources()))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), 'lib')
    link = ['g++', '-shared', '-o', _SO] + objs + [
        '-L' + torch_lib, '-L' + os.path.join(cuda_home, 'lib64'), '-lc10', '-lc10_cuda', '-ltorch_cpu', '-ltorch_cuda',
        '-ltorch', '-ltorch_python', '-lcudart', '-Wl,-rpath,' + torch_lib, '-Wl,-rpath,' + os.path.join(cuda_home, 'lib64')]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f'link failed:\n{r.stdout}\n{r.stderr}')
    with open(_STAMP, 'w') as f:
        f.write(_digest())
    return _SO


def load_extension():
    global _MOD
    if _MOD is not None:
        return _MOD
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    if not is_built():
        if not torch.cuda.is_available() and os.environ.get('TWINKLE_B200_BUILD', '0') != '1' and not os.path.isfile(_SO):
            raise ImportError('twinkle_b200.ops._C is not built (run `python -c "import __graft_entry__ as g; g.build()"`)')
        if not os.path.isfile(_SO) or os.environ.get('TWINKLE_B200_BUILD', '0') == '1' or torch.cuda.is_available():
            # a binary whose stamp does not match the sources is never loaded in place of a failed rebuild: the
            # numbers and tests of a run must come from the code in the tree
            build_extension()
    spec = importlib.util.spec_from_file_location('twinkle_b200.ops._C', _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)  # type: ignore[union-attr]
    sys.modules['twinkle_b200.ops._C'] = mod
    _MOD = mod
    return mod
