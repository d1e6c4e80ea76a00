"""``Config`` and buffer-size hints.

``Config`` is the native class (csrc/host/config.hpp) with the reference's five-field signature
(csrc/config.hpp:23-50). The recommended-config tables are re-tuned for B200: the only field that
selects anything here is ``num_sms`` (grid size of the normal-mode kernels); the chunk sizes of the
reference's ring queues (deep_ep/buffer.py:361-419) are carried for signature compatibility.
"""
from __future__ import annotations

from . import _ext

_C = _ext.load()
Config = _C.Config
LowLatencyLayout = _C.LowLatencyLayout

# num_ranks -> (num_sms, nvl_send, nvl_recv, rdma_send, rdma_recv)
DISPATCH_CONFIGS = {
    1: (32, 6, 256, 6, 128),
    2: (32, 6, 256, 6, 128),
    4: (32, 6, 256, 6, 128),
    8: (32, 6, 256, 6, 128),
    # several NVLink domains: the config drives the node-level NVLink kernels of the two-level path
    16: (32, 6, 256, 6, 128), 24: (32, 6, 256, 6, 128), 32: (32, 6, 256, 6, 128), 48: (32, 6, 256, 6, 128), 64: (32, 6, 256, 6, 128),
}
COMBINE_CONFIGS = {
    1: (32, 4, 256, 6, 128),
    2: (32, 4, 256, 6, 128),
    4: (32, 4, 256, 6, 128),
    8: (32, 4, 256, 6, 128),
    16: (32, 4, 256, 6, 128), 24: (32, 4, 256, 6, 128), 32: (32, 4, 256, 6, 128), 48: (32, 4, 256, 6, 128), 64: (32, 4, 256, 6, 128),
}


def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int, num_experts: int) -> int:
    """Bytes of symmetric memory the low-latency region needs (two parities of count matrix, landing zone,
    scales, source info, combine stage and zero-copy combine input). Reference: csrc/config.hpp:190-193."""
    return int(_C.get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank, hidden, num_ranks, num_experts))
