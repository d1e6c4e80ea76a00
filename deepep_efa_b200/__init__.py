"""deepep_efa_b200: Blackwell-native expert-parallel (EP) communication for Mixture-of-Experts models.

Public surface (same names as the reference's ``deep_ep`` package, deep_ep/__init__.py:3-7):
``Buffer``, ``EventOverlap``, ``Config``, ``topk_idx_t``.
"""
import torch

from .utils.event import EventHandle, EventOverlap  # noqa: F401
from .config import Config, LowLatencyLayout  # noqa: F401
from .buffer import Buffer, EPTimeoutError, topk_idx_t  # noqa: F401

__version__ = "0.1.0"


def install_as_deep_ep() -> None:
    """Register this package under the module name ``deep_ep`` so that code written against the reference
    (``import deep_ep; deep_ep.Buffer(...)``) runs unchanged."""
    import sys
    sys.modules.setdefault("deep_ep", sys.modules[__name__])
