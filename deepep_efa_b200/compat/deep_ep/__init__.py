"""Drop-in import path: put ``deepep_efa_b200/compat`` on ``PYTHONPATH`` and ``import deep_ep`` resolves to this
library with the reference's module surface (deep_ep/__init__.py:1-7: Buffer, EventOverlap, Config, topk_idx_t)."""
import torch

from deepep_efa_b200 import Buffer, Config, EventOverlap, topk_idx_t  # noqa: F401
from deepep_efa_b200.utils.event import EventHandle  # noqa: F401

__all__ = ["Buffer", "EventOverlap", "Config", "topk_idx_t"]
