"""Bookkeeping ops of the two-level (NVLink domain x rail) path: CUDA kernels of csrc/kernels/hier.cu with a
pure-PyTorch fallback for CPU tensors (gloo ranks), which also serves as their oracle in the tests.

Reference counterparts: ``deep_ep_cpp.moe_routing_sort`` / ``topk_remap`` / ``build_recv_src_meta`` /
``efa_permute`` (csrc/kernels/efa_kernels.cu:1591-1751) and the layout's ``num_tokens_per_rdma_rank``
(csrc/kernels/layout.cu:54-119).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _ext


def layout_hier(topk_idx: torch.Tensor, num_experts: int, num_ranks: int, ranks_per_node: int):
    """``(num_tokens_per_rank [R], num_tokens_per_node [R/P], num_tokens_per_expert [E], is_token_in_rank [T,R])``."""
    if topk_idx.is_cuda:
        return _ext.load().layout_hier(topk_idx.contiguous(), num_experts, num_ranks, ranks_per_node)
    T, _ = topk_idx.shape
    L = num_experts // num_ranks
    valid = (topk_idx >= 0) & (topk_idx < num_experts)
    safe = topk_idx.clamp(min=0, max=num_experts - 1)
    per_expert = torch.bincount(safe[valid].reshape(-1), minlength=num_experts).to(torch.int32)
    in_rank = torch.zeros(T, num_ranks, dtype=torch.int32).scatter_add_(1, safe // L, valid.to(torch.int32)) > 0
    per_rank = in_rank.sum(0).to(torch.int32)
    per_node = in_rank.view(T, num_ranks // ranks_per_node, ranks_per_node).any(2).sum(0).to(torch.int32)
    return per_rank, per_node, per_expert, in_rank


def routing_sort(member: torch.Tensor, ranks_per_group: int = 1):
    """Stable counting sort of (token, group) pairs by group. ``member`` is bool ``[T, G*ranks_per_group]``.

    Returns ``(sorted_ids int32 [>= S], counts int32 [G], prefix int32 [G+1], pos int32 [T, G])`` where the first
    ``S = prefix[G]`` entries of ``sorted_ids`` are token ids ordered by (group, token) and ``pos[t, g]`` is the slot
    of the pair in that list or -1."""
    if member.is_cuda:
        return _ext.load().routing_sort(member.contiguous(), ranks_per_group)
    T = member.size(0)
    G = member.size(1) // ranks_per_group
    grp = member.view(T, G, ranks_per_group).any(2)  # [T, G]
    flat = grp.t().contiguous().view(-1)             # group-major
    idx = flat.nonzero().flatten()
    sorted_ids = (idx % T).to(torch.int32)
    counts = grp.sum(0).to(torch.int32)
    prefix = torch.cat([torch.zeros(1, dtype=torch.int32), counts.cumsum(0).to(torch.int32)])
    pos_gm = torch.full((G * T,), -1, dtype=torch.int32)
    pos_gm[idx] = torch.arange(idx.numel(), dtype=torch.int32)
    return sorted_ids, counts, prefix, pos_gm.view(G, T).t().contiguous()


def topk_remap_pack(topk_idx: torch.Tensor, topk_weights: Optional[torch.Tensor], sorted_ids: torch.Tensor, prefix: torch.Tensor,
                    num_entries: int, experts_per_group: int) -> torch.Tensor:
    """One packed row ``[K x int64 | K x f32]`` per send entry: expert ids relative to the destination group (-1 when the
    expert lives elsewhere) and the weights (0 there)."""
    if topk_idx.is_cuda:
        w = topk_weights.float().contiguous() if topk_weights is not None else None
        return _ext.load().topk_remap_pack(topk_idx.contiguous(), w, sorted_ids, prefix, num_entries, experts_per_group)
    K = topk_idx.size(1)
    ids = sorted_ids[:num_entries].long()
    grp = torch.searchsorted(prefix[1:].long().contiguous(), torch.arange(num_entries), right=True)
    lo = (grp * experts_per_group).unsqueeze(1)
    e = topk_idx[ids]
    mine = (e >= lo) & (e < lo + experts_per_group)
    out_idx = torch.where(mine, e - lo, torch.full_like(e, -1))
    w = topk_weights[ids].float() if topk_weights is not None else torch.zeros(num_entries, K)
    out_w = torch.where(mine, w, torch.zeros_like(w))
    return torch.cat([out_idx.contiguous().view(torch.uint8).view(num_entries, K * 8),
                      out_w.contiguous().view(torch.uint8).view(num_entries, K * 4)], dim=1)


def unpack_topk(packed: torch.Tensor, num_topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    n, K = packed.size(0), num_topk
    idx = packed[:, :K * 8].contiguous().view(torch.int64).view(n, K)
    w = packed[:, K * 8:].contiguous().view(torch.float32).view(n, K)
    return idx, w


def recv_src_meta(recv_prefix: torch.Tensor, is_row_in_local_rank: Optional[torch.Tensor], num_rows: int) -> torch.Tensor:
    """int32 ``[n, 2]`` = (source group of the row, bitmask of the local ranks the row is forwarded to); the 8-byte
    SourceMeta of the reference (csrc/kernels/internode_efa.cu:31-49)."""
    if recv_prefix.is_cuda:
        return _ext.load().recv_src_meta(recv_prefix, is_row_in_local_rank, num_rows)
    grp = torch.searchsorted(recv_prefix[1:].long().contiguous(), torch.arange(num_rows), right=True).to(torch.int32)
    bits = torch.zeros(num_rows, dtype=torch.int32)
    if is_row_in_local_rank is not None:
        for j in range(is_row_in_local_rank.size(1)):
            bits |= is_row_in_local_rank[:num_rows, j].to(torch.int32) << j
    return torch.stack([grp, bits], dim=1)


def segmented_copy(src: torch.Tensor, dst: torch.Tensor, segments: torch.Tensor) -> None:
    """Copy ``segments[i] = (src byte offset, dst byte offset, bytes)`` from ``src`` to ``dst`` (both contiguous)."""
    if src.is_cuda:
        _ext.load().segmented_copy(src, dst, segments.contiguous())
        return
    s8, d8 = src.view(-1).view(torch.uint8), dst.view(-1).view(torch.uint8)
    for so, do, n in segments.tolist():
        d8[do:do + n] = s8[so:so + n]


def take_rows(src: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """``src[ids]`` for a 2-D tensor: the byte-generic gather kernel when rows are 16-byte multiples, else index_select."""
    if src.is_cuda and src.dim() == 2 and (src.size(1) * src.element_size()) % 16 == 0 and ids.numel() > 0:
        return _ext.load().gather_rows(src.contiguous(), ids.to(torch.int32).contiguous(), None, None)
    return src.index_select(0, ids.long())
