"""Library logger: ``logging.getLogger("deep_ep")`` with a rank prefix and per-message rate limiting.

The reference prints to stderr from Python and C++ (e.g. deep_ep/buffer.py:262, 1942; csrc/deep_ep.cpp:2889) and
logs every iteration from its worker thread; here messages go through the standard ``logging`` module, are prefixed
with the rank, and repeat at most once per ``min_interval_s``. Level from env ``DEEPEP_LOG_LEVEL`` (default WARNING).
"""
from __future__ import annotations

import logging
import os
import time
from typing import Dict

_LOGGER = logging.getLogger("deep_ep")
if not _LOGGER.handlers:
    _h = logging.StreamHandler()
    _h.setFormatter(logging.Formatter("[deep_ep %(levelname)s] %(message)s"))
    _LOGGER.addHandler(_h)
    _LOGGER.setLevel(os.environ.get("DEEPEP_LOG_LEVEL", "WARNING").upper())
    _LOGGER.propagate = False

_last: Dict[str, float] = {}


def get_logger() -> logging.Logger:
    return _LOGGER


def log(level: int, rank: int, msg: str, key: str = "", min_interval_s: float = 0.0) -> bool:
    """Emit ``[rN] msg`` unless the same ``key`` was logged less than ``min_interval_s`` ago. Returns whether it was emitted."""
    if min_interval_s > 0:
        k = key or msg
        now = time.monotonic()
        if now - _last.get(k, -1e18) < min_interval_s:
            return False
        _last[k] = now
    _LOGGER.log(level, "[r%d] %s", rank, msg)
    return True
