"""CPU backend of ``Buffer`` for process groups without GPUs (gloo).

Every collective all-gathers the participating ranks' inputs over the group, evaluates the pure-PyTorch
semantics of :mod:`deepep_efa_b200.reference.oracle` and keeps this rank's share. That is deliberately
simple: the backend exists to run the API, the handle formats and the model code on machines without
a GPU and to serve as the oracle for the CUDA kernels, not to be fast.

The reference has no CPU path at all (its tests need 8 GPUs, tests/test_intranode.py:310-311).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..reference import oracle
from ..utils.event import EventOverlap


class _F8:
    """An 8-bit float tensor as bytes: object collectives pickle tensors, and pickling knows no float8 storage."""

    def __init__(self, t: torch.Tensor) -> None:
        self.dtype, self.data = t.dtype, t.view(torch.uint8)


def _encode(obj):
    if isinstance(obj, torch.Tensor):
        return _F8(obj) if obj.element_size() == 1 and obj.is_floating_point() else obj
    if isinstance(obj, (tuple, list)):
        return type(obj)(_encode(o) for o in obj)
    return obj


def _decode(obj):
    if isinstance(obj, _F8):
        return obj.data.view(obj.dtype)
    if isinstance(obj, (tuple, list)):
        return type(obj)(_decode(o) for o in obj)
    return obj


class GlooBackend:
    def __init__(self, rank: int, num_ranks: int, group) -> None:
        self.rank, self.num_ranks, self.group = rank, num_ranks, group
        self.mask = torch.zeros(num_ranks, dtype=torch.int32)
        self._combine_buffers = {}

    # -- helpers ---------------------------------------------------------------------------------
    def _gather(self, obj) -> List:
        if self.num_ranks == 1:
            return [obj]
        out = [None] * self.num_ranks
        dist.all_gather_object(out, _encode(obj), self.group)
        return [_decode(o) for o in out]

    def _masked(self):
        return tuple(int(i) for i in self.mask.nonzero().flatten().tolist())

    # -- normal mode ---------------------------------------------------------------------------------
    def get_dispatch_layout(self, topk_idx, num_experts):
        return oracle.get_dispatch_layout(topk_idx, num_experts, self.num_ranks)

    def dispatch(self, x, handle, num_tokens_per_rank, is_token_in_rank, num_tokens_per_expert, topk_idx, topk_weights,
                 expert_alignment, num_worst_tokens):
        x, x_scales = x if isinstance(x, tuple) else (x, None)
        cached = handle is not None
        if cached:
            is_token_in_rank = handle[4]
            num_experts = self.num_ranks
        else:
            num_experts = num_tokens_per_expert.numel()
        everyone = self._gather((x, x_scales, topk_idx, topk_weights, is_token_in_rank))
        outs = oracle.dispatch([e[0] for e in everyone], [e[2] for e in everyone], [e[3] for e in everyone], num_experts,
                               x_scales=[e[1] for e in everyone], expert_alignment=expert_alignment,
                               is_token_in_rank=[e[4] for e in everyone])
        o = outs[self.rank]
        recv_x, recv_scales = o["recv_x"], o["recv_x_scales"]
        recv_idx, recv_w = o["recv_topk_idx"], o["recv_topk_weights"]
        per_expert = o["num_recv_tokens_per_expert_list"]
        if num_worst_tokens > 0:
            pad = num_worst_tokens - recv_x.size(0)
            assert pad >= 0, "num_worst_tokens is smaller than the number of received tokens"
            recv_x = torch.cat([recv_x, recv_x.new_zeros(pad, recv_x.size(1))])
            if recv_scales is not None:
                recv_scales = torch.cat([recv_scales, recv_scales.new_zeros(pad, recv_scales.size(1))])
            if recv_idx is not None:
                recv_idx = torch.cat([recv_idx, recv_idx.new_full((pad, recv_idx.size(1)), -1)])
            if recv_w is not None:
                recv_w = torch.cat([recv_w, recv_w.new_zeros(pad, recv_w.size(1))])
            per_expert = []
        rx = (recv_x, recv_scales) if recv_scales is not None else recv_x
        if cached:
            return rx, None, None, None, None, EventOverlap()
        R = self.num_ranks
        C = 1
        rpm = o["rank_prefix_matrix"]
        cpm = rpm.new_zeros(R, C)
        cpm[:, 0] = o["send_head"].ge(0).sum(dim=0).to(torch.int32)
        rcpm = rpm.new_zeros(R, C)
        col = rpm[:, self.rank]
        rcpm[:, 0] = col - torch.cat([col.new_zeros(1), col[:-1]])
        src_idx = o["recv_src_idx"]
        if num_worst_tokens > 0:
            src_idx = torch.cat([src_idx, src_idx.new_zeros(num_worst_tokens - src_idx.numel())])
        h = (rpm, cpm, rcpm, src_idx, o["is_token_in_rank"], o["send_head"])
        return rx, recv_idx, recv_w, per_expert, h, EventOverlap()

    def combine(self, x, handle, topk_weights, bias):
        rpm, _, _, _, _, send_head = handle
        b0, b1 = None, None
        if isinstance(bias, torch.Tensor):
            b0 = bias
        elif isinstance(bias, tuple):
            b0, b1 = bias
        everyone = self._gather((x, topk_weights, send_head, (b0, b1)))
        outs, outs_w = oracle.combine([e[0] for e in everyone], [e[2] for e in everyone], rpm,
                                      topk_weights=[e[1] for e in everyone], biases=[e[3] for e in everyone])
        return outs[self.rank], outs_w[self.rank], EventOverlap()

    # -- low latency -----------------------------------------------------------------------------
    def low_latency_dispatch(self, x, topk_idx, num_max_tokens, num_experts, use_fp8, round_scale, use_ue8m0, cumulative_stats,
                             return_recv_hook):
        everyone = self._gather((x, topk_idx))
        outs = oracle.low_latency_dispatch([e[0] for e in everyone], [e[1] for e in everyone], num_max_tokens, num_experts,
                                           use_fp8, round_scale, use_ue8m0, masked_ranks=self._masked())
        o = outs[self.rank]
        if cumulative_stats is not None:
            cumulative_stats += o["packed_recv_count"]
        handle = (o["src_info"], o["layout_range"], num_max_tokens, x.size(1), num_experts)
        rx = (o["packed_recv_x"], o["packed_recv_x_scales"]) if use_fp8 else o["packed_recv_x"]
        return rx, o["packed_recv_count"], handle, EventOverlap(), ((lambda: None) if return_recv_hook else None)

    def low_latency_combine(self, x, topk_idx, topk_weights, handle, out, return_recv_hook):
        src_info, layout_range, _, _, num_experts = handle
        everyone = self._gather((x, topk_idx, topk_weights, src_info, layout_range))
        outs = oracle.low_latency_combine([e[0] for e in everyone], [e[1] for e in everyone], [e[2] for e in everyone],
                                          [e[3] for e in everyone], [e[4] for e in everyone], num_experts,
                                          masked_ranks=self._masked())
        res = outs[self.rank]
        if out is not None:
            out.copy_(res)
            res = out
        return res, EventOverlap(), ((lambda: None) if return_recv_hook else None)

    def get_next_low_latency_combine_buffer(self, handle):
        src_info, _, num_max_tokens, hidden, num_experts = handle
        key = (num_max_tokens, hidden, num_experts)
        if key not in self._combine_buffers:
            L = num_experts // self.num_ranks
            self._combine_buffers[key] = torch.zeros(L, self.num_ranks * num_max_tokens, hidden, dtype=torch.bfloat16)
        return self._combine_buffers[key]

    def update_mask(self, rank_to_mask, mask):
        self.mask[rank_to_mask] = 1 if mask else 0

    def query_mask(self, mask_status):
        mask_status.copy_(self.mask)

    def clean_mask(self):
        self.mask.zero_()
