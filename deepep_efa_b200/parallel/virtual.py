"""Single-GPU emulation of a multi-rank expert-parallel job.

``VirtualCluster(R)`` owns R :class:`~deepep_efa_b200.Buffer` objects on ONE GPU whose "peers" are each
other's symmetric buffers. Every collective is issued for all R ranks at once and runs as ONE cooperative
launch with ``gridDim.y = R``: ranks that wait on each other are then guaranteed to be co-resident, which
separate launches (streams, threads or processes) on one GPU are not. The kernels are the same
instantiations that a real 8-GPU job runs; only the peer pointers differ.

Uses: correctness tests of the cross-rank protocol at R = 2/4/8 on a single GPU, and bring-up without
a multi-GPU box. The reference has no counterpart (its tests need one GPU per rank,
tests/test_intranode.py:310-311).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import _ext
from ..buffer import (Buffer, _DispatchReq, _combine_many, _dispatch_many, _ll_combine_many, _ll_dispatch_many)
from ..config import Config


class VirtualCluster:
    def __init__(self, num_ranks: int, num_nvl_bytes: int = 0, num_rdma_bytes: int = 0, timeout_ms: Optional[float] = None,
                 enable_shrink: bool = False) -> None:
        assert 1 <= num_ranks <= 8
        self.num_ranks = num_ranks
        self.buffers: List[Buffer] = [
            Buffer(None, num_nvl_bytes, num_rdma_bytes, low_latency_mode=num_rdma_bytes > 0, explicitly_destroy=True,
                   enable_shrink=enable_shrink, timeout_ms=timeout_ms, _virtual=(r, num_ranks)) for r in range(num_ranks)
        ]
        C = _ext.load()
        C.set_local_peers([b.runtime for b in self.buffers])
        torch.cuda.synchronize()

    def destroy(self) -> None:
        torch.cuda.synchronize()
        for b in self.buffers:
            b._ll_cache.clear()
            b._destroyed = True
            b.runtime.release()

    # ---- normal mode -------------------------------------------------------------------------------
    def get_dispatch_layout(self, topk_idxs: Sequence[torch.Tensor], num_experts: int):
        return [b.get_dispatch_layout(t, num_experts) for b, t in zip(self.buffers, topk_idxs)]

    def dispatch(self, xs, *, handles=None, layouts=None, topk_idxs=None, topk_weights=None, expert_alignment: int = 1,
                 num_worst_tokens: int = 0, config: Optional[Config] = None, quantize_fp8: bool = False, round_scale: bool = False):
        """``layouts[r]`` is the tuple returned by ``get_dispatch_layout`` of rank r."""
        R = self.num_ranks
        reqs = []
        for r in range(R):
            if handles is not None:
                reqs.append(_DispatchReq(xs[r], handles[r], None, None, None, None, None, expert_alignment, num_worst_tokens,
                                         quantize_fp8, round_scale))
            else:
                per_rank, _, per_expert, in_rank, _ = layouts[r]
                reqs.append(_DispatchReq(xs[r], None, per_rank, in_rank, per_expert, topk_idxs[r] if topk_idxs else None,
                                         topk_weights[r] if topk_weights else None, expert_alignment, num_worst_tokens,
                                         quantize_fp8, round_scale))
        config = config or Buffer.get_dispatch_config(R)
        return _dispatch_many(self.buffers, reqs, config, None, False, False)

    def combine(self, xs, handles, topk_weights=None, biases=None, config: Optional[Config] = None):
        R = self.num_ranks
        calls = [(xs[r], handles[r], topk_weights[r] if topk_weights else None, biases[r] if biases else None) for r in range(R)]
        config = config or Buffer.get_combine_config(R)
        return _combine_many(self.buffers, calls, config, None, False, False)

    # ---- low latency -------------------------------------------------------------------------------
    def low_latency_dispatch(self, xs, topk_idxs, num_max_tokens: int, num_experts: int, use_fp8: bool = True,
                             round_scale: bool = False, use_ue8m0: bool = False, return_recv_hook: bool = False,
                             cumulative_stats=None):
        calls = [(xs[r], topk_idxs[r], cumulative_stats[r] if cumulative_stats else None, None) for r in range(self.num_ranks)]
        return _ll_dispatch_many(self.buffers, calls, num_max_tokens, num_experts, use_fp8, round_scale, use_ue8m0, False,
                                 return_recv_hook)

    def low_latency_combine(self, xs, topk_idxs, topk_weights, handles, zero_copy: bool = False, return_recv_hook: bool = False,
                            outs=None):
        calls = [(xs[r], topk_idxs[r], topk_weights[r], handles[r], outs[r] if outs else None, None) for r in range(self.num_ranks)]
        return _ll_combine_many(self.buffers, calls, zero_copy, False, return_recv_hook)

    def barrier(self) -> None:
        _ext.load().barrier([b.runtime for b in self.buffers])
