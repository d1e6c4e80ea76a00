"""Pure-PyTorch reference semantics of every collective of this library.

Each function takes the inputs of ALL ranks as Python lists (index = rank) and returns the outputs
of all ranks, so a whole expert-parallel job can be evaluated in one process on the CPU. The GPU
kernels and the gloo backend are tested against these functions, and they double as executable
documentation of the tensor formats.

Formats follow the reference: layout outputs (``csrc/deep_ep.cpp:540-545``), normal-mode receive order
= (source rank, source token order) (``csrc/kernels/intranode.cu:410-426``), local expert ids or -1 and
zeroed weights for foreign experts (``intranode.cu:367-379``), un-weighted fp32 combine with optional
biases (``intranode.cu:942-1019``), low-latency ``[L, N, hidden]`` packing with
``layout_range = begin << 32 | count`` (``csrc/kernels/efa_kernels.cu:1038-1043``) and weighted
low-latency combine (``csrc/kernels/coop_combine_recv.cuh:184-203``). FP8 math restates
``tests/utils.py:50-74`` and ``deep_ep/buffer.py:1590-1621``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

FP8_MAX = 448.0
FP8_AMAX_FLOOR = 1e-4


# --------------------------------------------------------------------------------------------
# metrics used by the tests
# --------------------------------------------------------------------------------------------
def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - cosine-like similarity on x+1, y+1 in fp64 (the reference's error metric, tests/utils.py:39-43)."""
    x, y = x.double() + 1, y.double() + 1
    denom = (x * x + y * y).sum()
    return float(1 - 2 * (x * y).sum() / denom)


def hash_tensor(t: torch.Tensor) -> int:
    """Order-independent integer hash of a tensor's bytes (tests/utils.py:274-275)."""
    return int(t.contiguous().view(torch.uint8).to(torch.int64).sum().item())


# --------------------------------------------------------------------------------------------
# FP8 block scaling
# --------------------------------------------------------------------------------------------
def per_token_cast_to_fp8(x: torch.Tensor, round_scale: bool = False, use_ue8m0: bool = False):
    """bf16/fp32 [M, H] -> (e4m3 [M, H], scales). Scales are fp32 [M, H/128], or int32 [M, H/512] holding
    four UE8M0 exponent bytes when ``use_ue8m0`` (power-of-two scales)."""
    assert x.dim() == 2 and x.size(1) % 128 == 0
    m, n = x.shape
    g = x.float().view(m, -1, 128)
    amax = g.abs().amax(dim=2).clamp(min=FP8_AMAX_FLOOR)
    if round_scale or use_ue8m0:
        scales = torch.exp2(torch.ceil(torch.log2(amax / FP8_MAX)))
        inv = 1.0 / scales
    else:
        scales = amax / FP8_MAX
        inv = FP8_MAX / amax
    q = (g * inv.unsqueeze(2)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(m, n)
    if use_ue8m0:
        assert (n // 128) % 4 == 0
        ex = ((scales.contiguous().view(torch.int32) >> 23) & 0xFF).view(m, -1, 4)
        packed = ex[:, :, 0] | (ex[:, :, 1] << 8) | (ex[:, :, 2] << 16) | (ex[:, :, 3] << 24)
        return q, packed.to(torch.int32)
    return q, scales


def per_token_cast_back(x_fp8: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`per_token_cast_to_fp8`; returns bf16."""
    if x_fp8.numel() == 0:
        return x_fp8.to(torch.bfloat16)
    m, n = x_fp8.shape
    if scales.dtype == torch.int32:
        ex = scales.contiguous().view(torch.uint8).to(torch.int32) << 23
        scales = ex.view(torch.float32)
    g = x_fp8.float().view(m, -1, 128)
    return (g * scales.reshape(m, -1, 1)).view(m, n).to(torch.bfloat16)


# --------------------------------------------------------------------------------------------
# layout
# --------------------------------------------------------------------------------------------
def get_dispatch_layout(topk_idx: torch.Tensor, num_experts: int, num_ranks: int):
    """Returns (num_tokens_per_rank[R] i32, num_tokens_per_expert[E] i32, is_token_in_rank[T,R] bool)."""
    t, _ = topk_idx.shape
    per_local = num_experts // num_ranks
    valid = (topk_idx >= 0) & (topk_idx < num_experts)
    flat = topk_idx[valid].long()
    per_expert = torch.bincount(flat, minlength=num_experts).to(torch.int32)
    in_rank = torch.zeros(t, num_ranks, dtype=torch.bool, device=topk_idx.device)
    rank_of = torch.where(valid, topk_idx // per_local, torch.zeros_like(topk_idx))
    for r in range(num_ranks):
        in_rank[:, r] = ((rank_of == r) & valid).any(dim=1)
    per_rank = in_rank.sum(dim=0).to(torch.int32)
    return per_rank, per_expert, in_rank


# --------------------------------------------------------------------------------------------
# normal mode
# --------------------------------------------------------------------------------------------
def dispatch(xs: Sequence[torch.Tensor], topk_idxs: Sequence[Optional[torch.Tensor]],
             topk_weights: Sequence[Optional[torch.Tensor]], num_experts: int,
             x_scales: Optional[Sequence[Optional[torch.Tensor]]] = None, expert_alignment: int = 1,
             is_token_in_rank: Optional[Sequence[torch.Tensor]] = None):
    """All-rank normal dispatch.

    Returns a list (index = destination rank) of dicts with ``recv_x``, ``recv_x_scales``,
    ``recv_topk_idx`` (local ids or -1), ``recv_topk_weights`` (0 where -1), ``recv_src_idx``,
    ``num_recv_tokens_per_expert_list`` and the handle pieces ``rank_prefix_matrix`` [R,R] and per
    SOURCE rank ``send_head`` [T,R] (position inside the (src -> dst) stream or -1).
    """
    R = len(xs)
    L = num_experts // R
    if is_token_in_rank is None:
        is_token_in_rank = [get_dispatch_layout(topk_idxs[r], num_experts, R)[2] for r in range(R)]
    counts = torch.stack([m.sum(dim=0) for m in is_token_in_rank]).to(torch.int32)  # [src, dst]
    rank_prefix_matrix = counts.cumsum(dim=0).to(torch.int32)
    send_heads = []
    for s in range(R):
        m = is_token_in_rank[s]
        pos = m.to(torch.int32).cumsum(dim=0) - 1
        send_heads.append(torch.where(m, pos, torch.full_like(pos, -1)).to(torch.int32))
    outs = []
    for d in range(R):
        rows_x, rows_s, rows_i, rows_w, rows_src = [], [], [], [], []
        for s in range(R):
            sel = is_token_in_rank[s][:, d].nonzero(as_tuple=True)[0]
            rows_x.append(xs[s][sel])
            if x_scales is not None and x_scales[s] is not None:
                rows_s.append(x_scales[s][sel])
            if topk_idxs[s] is not None:
                idx = topk_idxs[s][sel]
                mine = (idx >= d * L) & (idx < (d + 1) * L)
                rows_i.append(torch.where(mine, idx - d * L, torch.full_like(idx, -1)))
                if topk_weights[s] is not None:
                    rows_w.append(torch.where(mine, topk_weights[s][sel], torch.zeros_like(topk_weights[s][sel])))
            rows_src.append(sel.to(torch.int32))
        recv_idx = torch.cat(rows_i) if rows_i else None
        per_expert = []
        if recv_idx is not None:
            for e in range(L):
                n = int((recv_idx == e).sum())
                per_expert.append((n + expert_alignment - 1) // expert_alignment * expert_alignment)
        outs.append(dict(
            recv_x=torch.cat(rows_x), recv_x_scales=torch.cat(rows_s) if rows_s else None,
            recv_topk_idx=recv_idx, recv_topk_weights=torch.cat(rows_w) if rows_w else None,
            recv_src_idx=torch.cat(rows_src), num_recv_tokens_per_expert_list=per_expert,
            rank_prefix_matrix=rank_prefix_matrix, send_head=send_heads[d], is_token_in_rank=is_token_in_rank[d]))
    return outs


def combine(xs: Sequence[torch.Tensor], send_heads: Sequence[torch.Tensor], rank_prefix_matrix: torch.Tensor,
            topk_weights: Optional[Sequence[Optional[torch.Tensor]]] = None,
            biases: Optional[Sequence[Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]]] = None):
    """All-rank normal combine: ``out[h][t] = sum over ranks r that hold token t of xs[r][row] (+ biases)``,
    accumulated in fp32 and cast to bf16. ``xs[r]`` are the expert outputs in receive order."""
    R = len(xs)
    outs, outs_w = [], []
    for h in range(R):
        head = send_heads[h]
        T = head.size(0)
        H = xs[0].size(1)
        acc = torch.zeros(T, H, dtype=torch.float32, device=xs[0].device)
        acc_w = None
        if topk_weights is not None and topk_weights[0] is not None:
            acc_w = torch.zeros(T, topk_weights[0].size(1), dtype=torch.float32, device=xs[0].device)
        for r in range(R):
            base = int(rank_prefix_matrix[h - 1, r]) if h > 0 else 0
            sel = (head[:, r] >= 0).nonzero(as_tuple=True)[0]
            rows = base + head[sel, r].long()
            acc[sel] += xs[r][rows].float()
            if acc_w is not None:
                acc_w[sel] += topk_weights[r][rows]
        if biases is not None and biases[h] is not None:
            for b in biases[h]:
                if b is not None:
                    acc += b.float()
        outs.append(acc.to(torch.bfloat16))
        outs_w.append(acc_w)
    return outs, outs_w


# --------------------------------------------------------------------------------------------
# low-latency mode
# --------------------------------------------------------------------------------------------
def low_latency_dispatch(xs: Sequence[torch.Tensor], topk_idxs: Sequence[torch.Tensor], num_max_tokens: int,
                         num_experts: int, use_fp8: bool = True, round_scale: bool = False, use_ue8m0: bool = False,
                         masked_ranks: Sequence[int] = ()):
    """All-rank low-latency dispatch.

    Returns per destination rank a dict with ``packed_recv_x`` [L, N, H] (e4m3 or bf16),
    ``packed_recv_x_scales`` ([L, N, H/128] f32 or [L, N, H/512] i32, None for bf16),
    ``packed_recv_count`` [L] i32, ``src_info`` [L, N] i32 and ``layout_range`` [L, R] i64.
    Rows of one expert are ordered by source rank, then by (token, k) order at the source.
    """
    R = len(xs)
    L = num_experts // R
    N = R * num_max_tokens
    H = xs[0].size(1)
    dev = xs[0].device
    outs = []
    for d in range(R):
        if use_fp8:
            px = torch.zeros(L, N, H, dtype=torch.float8_e4m3fn, device=dev)
            ps = torch.zeros(L, N, H // 512, dtype=torch.int32, device=dev) if use_ue8m0 else \
                torch.zeros(L, N, H // 128, dtype=torch.float32, device=dev)
        else:
            px = torch.zeros(L, N, H, dtype=torch.bfloat16, device=dev)
            ps = None
        outs.append(dict(packed_recv_x=px, packed_recv_x_scales=ps,
                         packed_recv_count=torch.zeros(L, dtype=torch.int32, device=dev),
                         src_info=torch.zeros(L, N, dtype=torch.int32, device=dev),
                         layout_range=torch.zeros(L, R, dtype=torch.int64, device=dev)))
    fill = [[0] * L for _ in range(R)]
    for d in range(R):
        if d in masked_ranks:
            continue
        for le in range(L):
            e = d * L + le
            for s in range(R):
                if s in masked_ranks:
                    outs[d]['layout_range'][le, s] = fill[d][le] << 32  # empty segment
                    continue
                hits = (topk_idxs[s] == e).nonzero()  # row-major order = (token, k) order
                toks = hits[:, 0]
                n = toks.numel()
                begin = fill[d][le]
                outs[d]['layout_range'][le, s] = (begin << 32) | n
                if n:
                    if use_fp8:
                        q, sc = per_token_cast_to_fp8(xs[s][toks], round_scale, use_ue8m0)
                        outs[d]['packed_recv_x'][le, begin:begin + n] = q
                        outs[d]['packed_recv_x_scales'][le, begin:begin + n] = sc
                    else:
                        outs[d]['packed_recv_x'][le, begin:begin + n] = xs[s][toks]
                    outs[d]['src_info'][le, begin:begin + n] = toks.to(torch.int32)
                fill[d][le] = begin + n
            outs[d]['packed_recv_count'][le] = fill[d][le]
    return outs


def low_latency_combine(ys: Sequence[torch.Tensor], topk_idxs: Sequence[torch.Tensor], topk_weights: Sequence[torch.Tensor],
                        src_infos: Sequence[torch.Tensor], layout_ranges: Sequence[torch.Tensor], num_experts: int,
                        masked_ranks: Sequence[int] = ()):
    """All-rank low-latency combine: ``out[h][t] = sum_k w[t,k] * ys[rank(e)][e_local, slot(h,t,e)]`` in fp32 -> bf16,
    where e = topk_idx[t,k] >= 0."""
    R = len(ys)
    L = num_experts // R
    H = ys[0].size(2)
    outs = []
    for h in range(R):
        T, K = topk_idxs[h].shape
        acc = torch.zeros(T, H, dtype=torch.float32, device=ys[0].device)
        for d in range(R):
            if d in masked_ranks:
                continue
            for le in range(L):
                e = d * L + le
                lr = int(layout_ranges[d][le, h])
                begin, n = lr >> 32, lr & 0xFFFFFFFF
                if n == 0:
                    continue
                toks = src_infos[d][le, begin:begin + n].long()
                rows = ys[d][le, begin:begin + n].float()
                w = torch.zeros(n, dtype=torch.float32, device=acc.device)
                hit = (topk_idxs[h][toks] == e)
                w = (topk_weights[h][toks] * hit).sum(dim=1)
                acc.index_add_(0, toks, rows * w.unsqueeze(1))
        outs.append(acc.to(torch.bfloat16))
    return outs
