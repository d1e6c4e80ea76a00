"""Expert-major permutation of dispatch results for the grouped GEMM, and its weighted inverse.

After a normal dispatch, ``recv_x`` is ordered by source rank and each row carries up to K local expert ids.
The grouped GEMM wants rows grouped by expert with every group starting on a multiple of 128 rows. The plan
built here needs no host synchronisation: group sizes come from the per-expert counts that
``Buffer.dispatch(..., expert_alignment=128)`` already returned to the host.

    pos[n, k]   row of selection (n, k) in the expert-major layout, -1 if unselected
    src_row[m]  receive row feeding expert-major row m, -1 for padding
    src_k[m]    which of the K selections of that receive row it is

``permute`` and ``unpermute_weighted`` are autograd functions backed by the gather kernels of
csrc/kernels/permute.cu (on CPU tensors they fall back to PyTorch indexing so the layer runs under gloo).

The reference has no counterpart (its users permute with framework ops between dispatch and their GEMMs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import _ext


@dataclass
class ExpertPlan:
    pos: torch.Tensor        # [N, K] int32
    src_row: torch.Tensor    # [M_pad] int32
    src_k: torch.Tensor      # [M_pad] int32 (0 where padding)
    m_offsets: torch.Tensor  # [L+1] int32
    num_rows: int            # M_pad


def build_expert_plan(recv_topk_idx: torch.Tensor, aligned_counts: List[int]) -> ExpertPlan:
    """``recv_topk_idx`` [N, K] holds local expert ids or -1; ``aligned_counts[e]`` >= rows of expert e."""
    dev = recv_topk_idx.device
    N, K = recv_topk_idx.shape
    L = len(aligned_counts)
    offs_host = [0]
    for c in aligned_counts:
        offs_host.append(offs_host[-1] + int(c))
    m_pad = offs_host[-1]
    m_offsets = torch.tensor(offs_host, dtype=torch.int32).to(dev, non_blocking=True)
    if recv_topk_idx.is_cuda:
        pos, src_row, src_k = _ext.load().build_plan(recv_topk_idx.contiguous(), m_offsets, m_pad)
        return ExpertPlan(pos, src_row, src_k, m_offsets, m_pad)
    flat = recv_topk_idx.reshape(-1)
    valid = flat >= 0
    safe = flat.clamp(min=0)
    onehot = (safe.unsqueeze(1) == torch.arange(L, device=dev).unsqueeze(0)) & valid.unsqueeze(1)
    rank = onehot.to(torch.int32).cumsum(dim=0).gather(1, safe.unsqueeze(1)).squeeze(1) - 1
    pos = torch.where(valid, m_offsets[:-1].long()[safe] + rank.long(), torch.full_like(safe, -1))
    src_row = torch.full((m_pad + 1,), -1, dtype=torch.int32, device=dev)
    src_k = torch.zeros((m_pad + 1,), dtype=torch.int32, device=dev)
    tgt = torch.where(valid, pos, torch.full_like(pos, m_pad))
    ids = torch.arange(N * K, device=dev)
    src_row.scatter_(0, tgt, (ids // K).to(torch.int32))
    src_k.scatter_(0, tgt, (ids % K).to(torch.int32))
    src_row[m_pad] = -1
    return ExpertPlan(pos.to(torch.int32).view(N, K).contiguous(), src_row[:m_pad].contiguous(), src_k[:m_pad].contiguous(), m_offsets, m_pad)


# ---- raw ops with a CPU fallback -------------------------------------------------------------------
def gather_rows(src: torch.Tensor, src_row: torch.Tensor, scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
    if src.is_cuda:
        return _ext.load().gather_rows(src.contiguous(), src_row, scale, out)
    sel = src.index_select(0, src_row.clamp(min=0).long())
    if scale is not None:
        sel = (sel.float() * scale.unsqueeze(1)).to(src.dtype)
    sel = torch.where((src_row >= 0).unsqueeze(1), sel, torch.zeros_like(sel))
    if out is not None:
        out.copy_(sel)
        return out
    return sel


def gather_reduce_rows(src: torch.Tensor, pos: torch.Tensor, w: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
    if src.is_cuda:
        return _ext.load().gather_reduce_rows(src.contiguous(), pos, w, out)
    N, K = pos.shape
    acc = torch.zeros(N, src.size(1), dtype=torch.float32)
    for k in range(K):
        p = pos[:, k]
        rows = src.index_select(0, p.clamp(min=0).long()).float()
        wk = w[:, k] if w is not None else torch.ones(N)
        acc += torch.where((p >= 0).unsqueeze(1), rows * wk.unsqueeze(1), torch.zeros_like(rows))
    res = acc.to(src.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


# ---- autograd ------------------------------------------------------------------------------------------
class _Permute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, recv_x, plan: ExpertPlan):
        ctx.plan = plan
        return gather_rows(recv_x, plan.src_row)

    @staticmethod
    def backward(ctx, grad):
        return gather_reduce_rows(grad.contiguous(), ctx.plan.pos), None


class _UnpermuteWeighted(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_perm, weights, plan: ExpertPlan, out):
        ctx.plan = plan
        ctx.save_for_backward(y_perm, weights)
        return gather_reduce_rows(y_perm, plan.pos, weights, out)

    @staticmethod
    def backward(ctx, grad):
        y_perm, weights = ctx.saved_tensors
        plan = ctx.plan
        grad = grad.contiguous()
        # d y_perm[m] = w[src_row[m], src_k[m]] * grad[src_row[m]]
        w_flat = weights.reshape(-1)
        K = weights.size(1)
        idx = (plan.src_row.clamp(min=0).long() * K + plan.src_k.long())
        row_scale = torch.where(plan.src_row >= 0, w_flat[idx], torch.zeros_like(w_flat[idx])).float().contiguous()
        d_y_perm = gather_rows(grad, plan.src_row, row_scale)
        # d w[n, k] = <y_perm[pos[n, k]], grad[n]>
        if grad.is_cuda and grad.dtype == torch.bfloat16 and y_perm.dtype == torch.bfloat16:
            return d_y_perm, _ext.load().rowdot(y_perm, grad, plan.pos).to(weights.dtype), None, None
        d_w = torch.zeros_like(weights)
        for k in range(K):
            p = plan.pos[:, k]
            rows = y_perm.index_select(0, p.clamp(min=0).long())
            d_w[:, k] = torch.where(p >= 0, (rows.float() * grad.float()).sum(dim=1), torch.zeros_like(d_w[:, k]))
        return d_y_perm, d_w, None, None


def permute(recv_x: torch.Tensor, plan: ExpertPlan) -> torch.Tensor:
    """Expert-major copy of ``recv_x`` ([M_pad, H], zero rows as padding)."""
    return _Permute.apply(recv_x, plan)


def unpermute_weighted(y_perm: torch.Tensor, weights: torch.Tensor, plan: ExpertPlan, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y[n] = sum_k weights[n, k] * y_perm[pos[n, k]]`` in receive order (fp32 accumulation)."""
    return _UnpermuteWeighted.apply(y_perm, weights, plan, out)
