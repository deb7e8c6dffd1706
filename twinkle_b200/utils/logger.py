"""Rank-aware logging.

Parity: reference ``src/twinkle/utils/logger.py:36-217`` — ``get_logger()``
returns a process-wide logger whose ``info``/``warning`` accept ``ranks=``
('all', 'master', 'local_master' or a list of ranks) and which has
``info_once`` / ``warning_once``.  Level from ``LOG_LEVEL``.
"""
from __future__ import annotations

import logging
import os
import sys
from typing import Iterable, Optional, Union

from .platform import Platform

_LOGGER: Optional['RankLogger'] = None


class RankLogger(logging.Logger):

    def __init__(self, name: str):
        super().__init__(name)
        self._seen = set()

    def _emit_here(self, ranks: Union[str, Iterable[int], None]) -> bool:
        if ranks is None or ranks == 'local_master':
            return Platform.is_local_master()
        if ranks == 'all':
            return True
        if ranks == 'master':
            return Platform.is_master()
        return Platform.get_rank() in set(ranks)

    def _log_ranked(self, level, msg, args, ranks=None, once=False, **kw):
        if not self._emit_here(ranks):
            return
        if once:
            key = (level, str(msg))
            if key in self._seen:
                return
            self._seen.add(key)
        if self.isEnabledFor(level):
            self._log(level, msg, args, **kw)

    def info(self, msg, *args, ranks=None, **kw):  # type: ignore[override]
        self._log_ranked(logging.INFO, msg, args, ranks, **kw)

    def warning(self, msg, *args, ranks=None, **kw):  # type: ignore[override]
        self._log_ranked(logging.WARNING, msg, args, ranks, **kw)

    def debug(self, msg, *args, ranks=None, **kw):  # type: ignore[override]
        self._log_ranked(logging.DEBUG, msg, args, ranks, **kw)

    def error(self, msg, *args, ranks='all', **kw):  # type: ignore[override]
        self._log_ranked(logging.ERROR, msg, args, ranks, **kw)

    def info_once(self, msg, *args, ranks=None, **kw):
        self._log_ranked(logging.INFO, msg, args, ranks, once=True, **kw)

    def warning_once(self, msg, *args, ranks=None, **kw):
        self._log_ranked(logging.WARNING, msg, args, ranks, once=True, **kw)


def get_logger(name: str = 'twinkle_b200', log_file: Optional[str] = None) -> RankLogger:
    global _LOGGER
    if _LOGGER is not None and log_file is None:
        return _LOGGER
    logger = RankLogger(name)
    level = getattr(logging, os.environ.get('LOG_LEVEL', 'INFO').upper(), logging.INFO)
    logger.setLevel(level)
    fmt = logging.Formatter('[%(asctime)s rank' + str(Platform.get_rank()) + ' %(levelname)s] %(message)s', '%H:%M:%S')
    handler = logging.StreamHandler(sys.stderr)
    handler.setFormatter(fmt)
    logger.addHandler(handler)
    if log_file:
        fh = logging.FileHandler(log_file)
        fh.setFormatter(fmt)
        logger.addHandler(fh)
    logger.propagate = False
    _LOGGER = logger
    return logger
