"""Cross-process coordination through the file system.

Parity: reference ``src/twinkle/utils/parallel.py:42-169`` — fcntl file locks,
a ``processing_lock`` context, and a single-winner claim used so that only one
rank fires a notification.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import tempfile
import time
from contextlib import contextmanager
from typing import Iterator, Optional

_LOCK_DIR = os.path.join(tempfile.gettempdir(), 'twinkle_b200_locks')


def _lock_path(key: str) -> str:
    os.makedirs(_LOCK_DIR, exist_ok=True)
    return os.path.join(_LOCK_DIR, hashlib.sha1(key.encode()).hexdigest() + '.lock')


@contextmanager
def file_lock(key: str, shared: bool = False, timeout: Optional[float] = None) -> Iterator[None]:
    """Exclusive (or shared) advisory lock named by ``key``."""
    path = _lock_path(key)
    fd = os.open(path, os.O_CREAT | os.O_RDWR, 0o666)
    mode = fcntl.LOCK_SH if shared else fcntl.LOCK_EX
    try:
        if timeout is None:
            fcntl.flock(fd, mode)
        else:
            deadline = time.monotonic() + timeout
            while True:
                try:
                    fcntl.flock(fd, mode | fcntl.LOCK_NB)
                    break
                except BlockingIOError:
                    if time.monotonic() > deadline:
                        raise TimeoutError(f'lock {key!r} not acquired within {timeout}s')
                    time.sleep(0.01)
        yield
    finally:
        try:
            fcntl.flock(fd, fcntl.LOCK_UN)
        finally:
            os.close(fd)


processing_lock = file_lock


def claim_once(key: str, ttl: float = 60.0) -> bool:
    """True for exactly one caller per ``key`` within ``ttl`` seconds — used to
    elect the single rank that reports an exception."""
    marker = _lock_path('claim:' + key) + '.claim'
    with file_lock('claim:' + key):
        now = time.time()
        try:
            if now - os.path.getmtime(marker) < ttl:
                return False
        except OSError:
            pass
        with open(marker, 'w') as f:
            f.write(str(os.getpid()))
        return True
