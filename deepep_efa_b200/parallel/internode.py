"""Two-level expert parallelism for groups that span several NVLink domains (more than one NVSwitch).

A group of ``W = nodes x P`` ranks is split into NVLink domains of ``P`` consecutive ranks and into rails (the
ranks with the same local index in every domain). A token crosses the inter-domain network ONCE per destination
domain and is fanned out inside that domain over NVLink:

    dispatch   rail hop   one copy of the token (row, scales, domain-relative top-k) to the rank with my local index
                          in every domain that owns one of its experts          (all-to-all among the rail)
               NVLink hop the receiving rank dispatches what it got inside its domain with the peer-memory
                          dispatch kernel of the node-level ``Buffer``

    combine    NVLink hop the node-level combine reduces the expert outputs of a domain back onto the forwarded rows
               rail hop   partial sums return to the token's home rank, which adds the (at most ``nodes``) partials

So the expensive links carry ``tokens x destination domains`` rows instead of ``tokens x destination ranks``, and the
fan-out / reduction inside a domain runs at NVLink speed with the kernels this library is about.

Reference counterpart: ``Buffer.internode_dispatch`` / ``internode_combine`` / ``_efa_do_dispatch_data`` /
``_efa_transfer`` (deep_ep/buffer.py:582-1560), which send one copy per destination RANK through NCCL + libfabric and
keep per-call state on the buffer object (``self._efa_dispatch_info``); here everything a combine or a cached
dispatch needs is inside the returned handle. The low-latency pair below has the structure of the reference's
single-node NCCL fallback (deep_ep/buffer.py:2265-2303, 2722-2741): count exchange, packed rows, one all-to-all per
direction, scatter into ``[L, N, hidden]``; it is the inter-domain fallback here, the NVLink kernels being the real
low-latency path inside a domain.

Everything in this module is backend-agnostic: CUDA tensors use the kernels of csrc/kernels/hier.cu and permute.cu
and NCCL, CPU tensors use PyTorch ops and gloo, which is how the path is tested without several NVSwitch domains.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import hier as H
from ..ops.permute import gather_reduce_rows
from ..utils.event import EventOverlap
from .transport import CollectiveTransport, Transport, make_subgroups


class HierarchicalEP:
    """Owner of the node-level buffer and the rail transport of one rank."""

    def __init__(self, group: dist.ProcessGroup, ranks_per_node: int, node_buffer_factory, rail: Optional[Transport] = None) -> None:
        self.group = group
        self.num_ranks, self.rank = group.size(), group.rank()
        self.P = int(ranks_per_node)
        assert self.num_ranks % self.P == 0 and self.num_ranks > self.P
        self.num_nodes = self.num_ranks // self.P
        assert self.num_ranks <= 64, "at most 64 ranks (8 NVLink domains of 8)"
        self.node, self.local = divmod(self.rank, self.P)
        self.node_group, rail_group = make_subgroups(group, self.P)
        self.rail = rail if rail is not None else CollectiveTransport(rail_group)
        self.flat = CollectiveTransport(group)
        self.node_buf = node_buffer_factory(self.node_group)

    def destroy(self) -> None:
        self.node_buf.destroy()

    # ------------------------------------------------------------------------------------------
    # layout
    # ------------------------------------------------------------------------------------------
    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int):
        per_rank, per_node, per_expert, in_rank = H.layout_hier(topk_idx, num_experts, self.num_ranks, self.P)
        return per_rank, per_node, per_expert, in_rank, EventOverlap()

    # ------------------------------------------------------------------------------------------
    # normal mode
    # ------------------------------------------------------------------------------------------
    def dispatch(self, x, handle, num_tokens_per_rank, num_tokens_per_rdma_rank, is_token_in_rank, num_tokens_per_expert, topk_idx,
                 topk_weights, expert_alignment, num_worst_tokens, config, quantize_fp8=False, round_scale=False):
        """Same return tuple as the single-domain dispatch. Received rows are ordered by the local index of the rail
        peer that forwarded them, then by source domain, then by token order at the source.

        The handle is a 10-tuple like the reference's (deep_ep/buffer.py:851-855) but self-contained:
        ``(is_token_in_rank, rail_token_ids, rail_pos [T, nodes], rail_send_splits, rail_recv_splits,
        recv_rdma_rank_prefix_sum [nodes] i32, recv_gbl_rank_prefix_sum [W] i32 or None, recv_src_meta [F, 2] i32,
        node_handle, (num_tokens, num_topk))``."""
        x_data, x_scales = x if isinstance(x, tuple) else (x, None)
        if quantize_fp8 and x_scales is None and x_data.is_cuda:
            from .. import _ext
            x_data, x_scales = _ext.load().per_token_cast_to_fp8(x_data.contiguous(), round_scale, False)[:2]
        cached = handle is not None
        if cached:
            assert topk_idx is None and topk_weights is None
            (is_token_in_rank, ids, pos, send_splits, recv_splits, _, _, _, node_handle, _) = handle
        else:
            assert is_token_in_rank is not None and num_tokens_per_expert is not None
            if topk_idx is None:
                raise NotImplementedError("a fresh dispatch across NVLink domains needs topk_idx (the second hop routes by it)")
            num_experts = num_tokens_per_expert.numel()
            experts_per_node = num_experts // self.num_nodes
            sorted_ids, counts, prefix, pos = H.routing_sort(is_token_in_rank, self.P)
            recv_counts = self.rail.all_to_all_equal(counts)
            host = torch.cat([counts, recv_counts]).tolist()  # the one host synchronisation of the rail hop
            send_splits, recv_splits = host[:self.num_nodes], host[self.num_nodes:]
            S = sum(send_splits)
            ids = sorted_ids[:S]
            packed = H.topk_remap_pack(topk_idx, topk_weights, ids, prefix, S, experts_per_node)
            fwd_idx, fwd_w = H.unpack_topk(self.rail.all_to_all_rows(packed, send_splits, recv_splits), topk_idx.size(1))
            if topk_weights is None:
                fwd_w = None
        # rail hop of the payload
        fwd_x = self.rail.all_to_all_rows(H.take_rows(x_data, ids), send_splits, recv_splits)
        fwd = fwd_x
        if x_scales is not None:
            fwd_s = self.rail.all_to_all_rows(H.take_rows(x_scales.contiguous(), ids), send_splits, recv_splits)
            fwd = (fwd_x, fwd_s)
        nb = self.node_buf
        if cached:
            recv_x, _, _, _, _, ev = nb.dispatch(fwd, handle=node_handle, config=config)
            return recv_x, None, None, None, None, ev
        # NVLink hop
        per_rank, _, per_expert, in_rank, _ = nb.get_dispatch_layout(fwd_idx, experts_per_node)
        recv_x, recv_idx, recv_w, per_expert_list, node_handle, ev = nb.dispatch(
            fwd, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert, topk_idx=fwd_idx,
            topk_weights=fwd_w, expert_alignment=expert_alignment, num_worst_tokens=num_worst_tokens, config=config)
        dev = x_data.device
        F = sum(recv_splits)
        recv_node_prefix = torch.tensor([0] + recv_splits, dtype=torch.int64).cumsum(0).to(torch.int32).to(dev)
        meta = H.recv_src_meta(recv_node_prefix, in_rank, F)
        gbl_prefix = None
        if num_tokens_per_rank is not None:
            gbl_prefix = self.flat.all_to_all_equal(num_tokens_per_rank.to(torch.int32)).cumsum(0).to(torch.int32)
        handle = (is_token_in_rank, ids, pos, send_splits, recv_splits, recv_node_prefix[1:], gbl_prefix, meta, node_handle,
                  (x_data.size(0), topk_idx.size(1)))
        return recv_x, recv_idx, recv_w, per_expert_list, handle, ev

    def combine(self, x: torch.Tensor, handle: Tuple, topk_weights: Optional[torch.Tensor], bias, config):
        """Un-weighted sum of every copy of a token, bf16 out: NVLink reduction per domain, then one partial per domain
        returns over the rail and the home rank adds them in fp32."""
        (_, ids, pos, send_splits, recv_splits, _, _, _, node_handle, (T, K)) = handle
        part, part_w, _ = self.node_buf.combine(x, node_handle, topk_weights=topk_weights, config=config)
        back = self.rail.all_to_all_rows(part, recv_splits, send_splits)
        out = gather_reduce_rows(back, pos)
        b0, b1 = _unpack_bias(bias)
        if b0 is not None or b1 is not None:
            acc = out.float()
            for b in (b0, b1):
                if b is not None:
                    acc = acc + b.float()
            out = acc.to(out.dtype)
        out_w = None
        if topk_weights is not None:
            back_w = self.rail.all_to_all_rows(part_w.float().contiguous(), recv_splits, send_splits)
            out_w = torch.zeros(T, back_w.size(1), dtype=torch.float32, device=back_w.device).index_add_(0, ids.long(), back_w)
        return out, out_w, EventOverlap()

    # ------------------------------------------------------------------------------------------
    # low-latency mode across domains (collective fallback)
    # ------------------------------------------------------------------------------------------
    def low_latency_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, num_max_tokens: int, num_experts: int, use_fp8: bool,
                             round_scale: bool, use_ue8m0: bool, cumulative_stats: Optional[torch.Tensor]):
        """Same outputs as the single-domain call; the handle carries a sixth entry (the send/receive plan)."""
        W, T, K, Hd = self.num_ranks, x.size(0), topk_idx.size(1), x.size(1)
        L, N = num_experts // W, W * num_max_tokens
        dev = x.device
        assert T <= num_max_tokens
        e = topk_idx.reshape(-1)
        valid = (e >= 0) & (e < num_experts)
        key = torch.where(valid, e, torch.full_like(e, num_experts))
        order = torch.sort(key, stable=True).indices          # selections ordered by (destination rank, expert, token)
        cnt = torch.bincount(key, minlength=num_experts + 1)[:num_experts].to(torch.int32)
        recv_cnt = self.flat.all_to_all_equal(cnt).view(W, L)  # [source, local expert]
        host = torch.cat([cnt.view(W, L).sum(1), recv_cnt.sum(1)]).tolist()
        send_splits, recv_splits = host[:W], host[W:]
        S, n_recv = sum(send_splits), sum(recv_splits)
        sel = order[:S]
        tok = (sel // K).to(torch.int32)
        # payload rows: [data | scales | token id], padded to 16 bytes
        if use_fp8:
            q, s = _cast_fp8(x, round_scale, use_ue8m0)
            parts = [H.take_rows(q.view(torch.uint8), tok), H.take_rows(s.contiguous().view(torch.uint8).view(T, -1), tok)]
        else:
            parts = [H.take_rows(x.contiguous().view(torch.uint8).view(T, -1), tok)]
        parts.append(tok.view(torch.uint8).view(S, 4))
        row = torch.cat(parts, dim=1)
        got = self.flat.all_to_all_rows(row, send_splits, recv_splits)
        # destination slot of every received row
        flat_cnt = recv_cnt.reshape(-1).long()                 # source-major, expert-minor: the order rows arrive in
        cum = flat_cnt.cumsum(0)
        seg = torch.searchsorted(cum, torch.arange(n_recv, device=dev), right=True)
        src_rank, exp = seg // L, seg % L
        begin = recv_cnt.long().cumsum(0) - recv_cnt.long()    # [source, expert]: rows of earlier sources for that expert
        within = torch.arange(n_recv, device=dev) - (cum - flat_cnt)[seg]
        dst = exp * N + begin.reshape(-1)[seg] + within
        data_bytes = Hd if use_fp8 else Hd * 2
        if use_fp8:
            recv_x = torch.empty(L * N, Hd, dtype=torch.float8_e4m3fn, device=dev)
            recv_x.view(torch.uint8).index_copy_(0, dst, got[:, :Hd].contiguous())
            sc_bytes = got.size(1) - Hd - 4
            sc_dtype = torch.int32 if use_ue8m0 else torch.float32
            recv_s = torch.empty(L * N, sc_bytes // 4, dtype=sc_dtype, device=dev)
            recv_s.view(torch.uint8).view(L * N, sc_bytes).index_copy_(0, dst, got[:, Hd:Hd + sc_bytes].contiguous())
            packed = (recv_x.view(L, N, Hd), recv_s.view(L, N, -1))
        else:
            recv_x = torch.empty(L * N, Hd, dtype=torch.bfloat16, device=dev)
            recv_x.view(torch.uint8).view(L * N, Hd * 2).index_copy_(0, dst, got[:, :data_bytes].contiguous())
            packed = recv_x.view(L, N, Hd)
        src_info = torch.zeros(L * N, dtype=torch.int32, device=dev)
        src_info.index_copy_(0, dst, got[:, -4:].contiguous().view(torch.int32).view(-1))
        layout_range = ((begin << 32) | recv_cnt.long()).t().contiguous()       # [L, W]
        count = recv_cnt.sum(0).to(torch.int32)
        if cumulative_stats is not None:
            cumulative_stats += count.to(cumulative_stats.dtype)
        inv = torch.full((T * K,), -1, dtype=torch.int32, device=dev)
        inv[sel] = torch.arange(S, dtype=torch.int32, device=dev)
        plan = {"dst": dst.to(torch.int32), "send_splits": send_splits, "recv_splits": recv_splits, "pos": inv.view(T, K)}
        handle = (src_info.view(L, N), layout_range, num_max_tokens, Hd, num_experts, plan)
        return packed, count, handle, EventOverlap(), None

    def low_latency_combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, handle: tuple,
                            out: Optional[torch.Tensor]):
        plan = handle[5]
        L, N, Hd = x.shape
        rows = H.take_rows(x.reshape(L * N, Hd), plan["dst"])
        back = self.flat.all_to_all_rows(rows, plan["recv_splits"], plan["send_splits"])
        res = gather_reduce_rows(back, plan["pos"], topk_weights.float().contiguous(), out)
        return res, EventOverlap(), None


def _unpack_bias(bias):
    if isinstance(bias, torch.Tensor):
        return bias, None
    if isinstance(bias, tuple):
        assert len(bias) == 2
        return bias
    return None, None


def _cast_fp8(x: torch.Tensor, round_scale: bool, use_ue8m0: bool):
    if x.is_cuda:
        from .. import _ext
        q, s = _ext.load().per_token_cast_to_fp8(x.contiguous(), round_scale or use_ue8m0, use_ue8m0)[:2]
        return q, s
    from ..reference import oracle
    return oracle.per_token_cast_to_fp8(x, round_scale=round_scale or use_ue8m0, use_ue8m0=use_ue8m0)
