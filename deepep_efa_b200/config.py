"""``Config`` and buffer-size hints.

``Config`` is the native class (csrc/host/config.hpp) with the reference's five-field signature
(csrc/config.hpp:23-50). The only field that selects anything here is ``num_sms`` (grid size of the
normal-mode kernels); the chunk sizes of the reference's ring queues (deep_ep/buffer.py:361-419) are
carried for signature compatibility.

The per-rank-count tables come from ``bench_normal_sweep.py`` (4096 tokens per rank, hidden 7168, top-8 of
256 experts, grid sizes 16 / 24 / 32 / 48 / 64, GB/s with the reference's byte definition). At 8 ranks
dispatch peaks at 48 CTAs (FP8 674-681, BF16 745 GB/s; 32 CTAs: 642-671 / 726) and combine still gains up
to 64 CTAs (679 GB/s; 32 CTAs: 620). With fewer ranks fewer peers share the work of one warp (a warp stores a
token to at most R destinations, combine reads at most R rows), so more warps are needed for the same bytes in
flight: the smaller groups keep at least the 8-rank grid. The reference sweeps its NVL chunk size at a
fixed 24 SMs (tests/test_intranode.py:194-262); this library has no chunking, its knob is the grid.
"""
from __future__ import annotations

from . import _ext

_C = _ext.load()
Config = _C.Config
LowLatencyLayout = _C.LowLatencyLayout

# num_ranks -> (num_sms, nvl_send, nvl_recv, rdma_send, rdma_recv)
DISPATCH_CONFIGS = {
    1: (32, 6, 256, 6, 128),
    2: (48, 6, 256, 6, 128),
    4: (48, 6, 256, 6, 128),
    8: (48, 6, 256, 6, 128),
    # several NVLink domains: the config drives the node-level NVLink kernels of the two-level path
    16: (32, 6, 256, 6, 128), 24: (32, 6, 256, 6, 128), 32: (32, 6, 256, 6, 128), 48: (32, 6, 256, 6, 128), 64: (32, 6, 256, 6, 128),
}
COMBINE_CONFIGS = {
    1: (32, 4, 256, 6, 128),
    2: (64, 4, 256, 6, 128),
    4: (64, 4, 256, 6, 128),
    8: (64, 4, 256, 6, 128),
    16: (32, 4, 256, 6, 128), 24: (32, 4, 256, 6, 128), 32: (32, 4, 256, 6, 128), 48: (32, 4, 256, 6, 128), 64: (32, 4, 256, 6, 128),
}


def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int, num_experts: int) -> int:
    """Bytes of symmetric memory the low-latency region needs (two parities of count matrix, landing zone,
    scales, source info, combine stage and zero-copy combine input). Reference: csrc/config.hpp:190-193."""
    return int(_C.get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank, hidden, num_ranks, num_experts))
