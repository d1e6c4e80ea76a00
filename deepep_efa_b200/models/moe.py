"""Expert-parallel MoE layer on top of ``Buffer``: gate -> layout -> dispatch -> grouped expert GEMMs (SwiGLU FFN)
-> weighted un-permute -> combine, with autograd.

Two execution paths share the structure:

* **training (BF16)**: every stage is an autograd function. The backward of dispatch is a combine and the backward
  of combine is a cached-handle dispatch (deep_ep/buffer.py:512-519 documents that contract for the reference); the
  expert GEMMs use the grouped tcgen05 kernel for forward, input gradients (transposed weights) and weight
  gradients (K-grouped mode).
* **inference (FP8)**: ``forward_fp8`` quantises inside the dispatch kernel, runs block-scaled FP8 grouped GEMMs
  with the SwiGLU fused into the first GEMM's epilogue, and combines in BF16 (DeepSeek-V3-shaped experts).
* **fused inference (FP8)**: ``forward_fused`` is the overlapped form of the same computation. The dispatch kernel
  quantises AND places every (token, expert) row at its final expert-major, 128-row-aligned position in the expert's
  rank (no permutation pass, no host synchronisation); the first grouped GEMM runs concurrently on the compute stream
  and starts on an expert as soon as that expert's arrival counter reaches the expected total; the second grouped
  GEMM's epilogue stores every output row straight into the stage of the token's home rank over NVLink, so the
  combine that remains is a cross-rank flag exchange and a local weighted sum.

The reference is a communication library only and has no model code; this module is the model-side user of the
API that the benchmark configurations (fused MoE forward, MoE training step) call for.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import grouped_gemm as gg
from ..ops.permute import build_expert_plan, gather_rows, permute, unpermute_weighted

EXPERT_ALIGNMENT = 128


@dataclass
class MoEConfig:
    hidden: int
    intermediate: int
    num_experts: int
    num_topk: int
    init_std: float = 0.02
    router_dtype: torch.dtype = torch.float32


# ---------------------------------------------------------------------------------------------------------
# communication autograd functions
# ---------------------------------------------------------------------------------------------------------
class _Dispatch(torch.autograd.Function):
    """x [T,H], topk_weights [T,K] -> recv_x [N,H], recv_topk_weights [N,K]; routing outputs ride on ``ctx_out``."""

    @staticmethod
    def forward(ctx, x, topk_weights, topk_idx, buffer, num_experts, ctx_out):
        per_rank, _, per_expert, in_rank, _ = buffer.get_dispatch_layout(topk_idx, num_experts)
        recv_x, recv_idx, recv_w, counts, handle, _ = buffer.dispatch(
            x, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert, topk_idx=topk_idx,
            topk_weights=topk_weights, expert_alignment=EXPERT_ALIGNMENT)
        ctx.buffer, ctx.handle = buffer, handle
        ctx_out["recv_topk_idx"], ctx_out["counts"], ctx_out["handle"] = recv_idx, counts, handle
        ctx.mark_non_differentiable(recv_idx)
        return recv_x, recv_w

    @staticmethod
    def backward(ctx, grad_recv_x, grad_recv_w):
        gx, gw, _ = ctx.buffer.combine(grad_recv_x.contiguous(), ctx.handle,
                                       topk_weights=None if grad_recv_w is None else grad_recv_w.contiguous())
        return gx, gw, None, None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_recv, buffer, handle):
        ctx.buffer, ctx.handle = buffer, handle
        out, _, _ = buffer.combine(y_recv, handle)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        g, *_ = ctx.buffer.dispatch(grad_out.contiguous(), handle=ctx.handle)
        return g, None, None


class _GroupedLinear(torch.autograd.Function):
    """y[m] = x[m] @ w[g].T for the rows m of expert g (w: [G, N, K])."""

    @staticmethod
    def forward(ctx, x, w, m_offsets):
        ctx.save_for_backward(x, w, m_offsets)
        if x.is_cuda:
            return gg.grouped_gemm(x, w, m_offsets)
        return gg.reference_grouped_gemm(x, w, m_offsets).to(x.dtype)

    @staticmethod
    def backward(ctx, grad):
        x, w, m_offsets = ctx.saved_tensors
        grad = grad.contiguous()
        if x.is_cuda and x.size(1) % 128 == 0 and w.size(1) % 128 == 0:
            # weight, gradient and activation are read in place as MN-major operands: no transposed copies
            dx = gg.grouped_gemm_dgrad(grad, w, m_offsets)
            dw = gg.grouped_gemm_wgrad_inplace(grad, x, m_offsets)
        elif x.is_cuda:
            dx = gg.grouped_gemm(grad, gg.transpose_last2(w), m_offsets)
            dw = gg.grouped_gemm_wgrad(gg.transpose_last2(grad), gg.transpose_last2(x), m_offsets)
        else:
            dx = gg.reference_grouped_gemm(grad, w.transpose(1, 2).contiguous(), m_offsets).to(x.dtype)
            offs = m_offsets.tolist()
            dw = torch.stack([grad[offs[g]:offs[g + 1]].float().t() @ x[offs[g]:offs[g + 1]].float() for g in range(w.size(0))]).to(w.dtype)
        return dx, dw, None


def grouped_linear(x, w, m_offsets):
    return _GroupedLinear.apply(x, w, m_offsets)


# ---------------------------------------------------------------------------------------------------------
# the layer
# ---------------------------------------------------------------------------------------------------------
class MoELayer(nn.Module):
    """Top-k routed SwiGLU experts, block-partitioned over the ranks of ``buffer`` (expert e lives on rank e // (E/R))."""

    def __init__(self, cfg: MoEConfig, buffer, device: Optional[torch.device] = None, seed: int = 0) -> None:
        super().__init__()
        self.cfg, self.buffer = cfg, buffer
        R = buffer.group_size
        assert cfg.num_experts % R == 0
        self.num_local_experts = L = cfg.num_experts // R
        dev = device if device is not None else (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        # weights are drawn on the target device (an expert-parallel shard of a large model does not fit a host pass)
        g = torch.Generator(device=dev).manual_seed(seed)
        self.gate = nn.Parameter((torch.randn(cfg.num_experts, cfg.hidden, generator=g, device=dev) * cfg.init_std).to(cfg.router_dtype))
        ge = torch.Generator(device=dev).manual_seed(seed + 1 + buffer.rank)
        w13 = torch.empty(L, 2 * cfg.intermediate, cfg.hidden, dtype=torch.bfloat16, device=dev)
        w2 = torch.empty(L, cfg.hidden, cfg.intermediate, dtype=torch.bfloat16, device=dev)
        for e in range(L):  # per expert, so the fp32 temporary stays small
            w13[e] = (torch.randn(2 * cfg.intermediate, cfg.hidden, generator=ge, device=dev) * cfg.init_std).to(torch.bfloat16)
            w2[e] = (torch.randn(cfg.hidden, cfg.intermediate, generator=ge, device=dev) * cfg.init_std).to(torch.bfloat16)
        self.w13, self.w2 = nn.Parameter(w13), nn.Parameter(w2)
        self._fp8 = None

    # -- routing ------------------------------------------------------------------------------------------
    def route(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        logits = x.to(self.gate.dtype) @ self.gate.t()
        topk_logits, topk_idx = logits.topk(self.cfg.num_topk, dim=-1)
        return topk_idx.to(torch.int64), torch.softmax(topk_logits.float(), dim=-1)

    # -- BF16 path with autograd ----------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        if topk_idx is None:
            topk_idx, topk_weights = self.route(x)
        routing = {}
        recv_x, recv_w = _Dispatch.apply(x, topk_weights, topk_idx, self.buffer, self.cfg.num_experts, routing)
        plan = build_expert_plan(routing["recv_topk_idx"], routing["counts"])
        x_perm = permute(recv_x, plan)
        h13 = grouped_linear(x_perm, self.w13, plan.m_offsets)
        h = gg.swiglu(h13)
        y_perm = grouped_linear(h, self.w2, plan.m_offsets)
        out_buf = self._symmetric_like(recv_x)
        y_recv = unpermute_weighted(y_perm, recv_w, plan, out_buf)
        return _Combine.apply(y_recv, self.buffer, routing["handle"])

    def _symmetric_like(self, recv_x: torch.Tensor) -> Optional[torch.Tensor]:
        """Combine reads its input in place when it lives in the symmetric arena."""
        if recv_x.is_cuda and getattr(self.buffer, "runtime", None) is not None:
            return self.buffer.empty_symmetric(list(recv_x.shape), torch.bfloat16)
        return None

    # -- FP8 inference path -------------------------------------------------------------------------------------
    def prepare_fp8(self, native_block_scaling: bool = True) -> None:
        """Quantise the expert weights to e4m3 with one scale per 128x128 block (done once).

        ``native_block_scaling=True`` (the default on this hardware: the expert GEMMs run about 1.6x faster) rounds every scale
        up to a power of two and builds the UE8M0 scale atoms the tensor core reads directly (``tcgen05.mma
        kind::mxf8f6f4.block_scale``); the forward paths then quantise activations with power-of-two scales as well and the
        GEMMs accumulate a whole tile in TMEM. ``False`` keeps arbitrary fp32 scales (the recipe DeepSeek-V3 was published
        with), which the GEMM applies by promoting every K block on the CUDA cores."""
        self._mx = None

        def q(w):
            G, N, K = w.shape
            out = torch.empty(G, N, K, dtype=torch.float8_e4m3fn, device=w.device)
            scales = torch.empty(G, N // 128, K // 128, dtype=torch.float32, device=w.device)
            for e in range(G):  # per expert: bounded fp32 temporaries
                wb = w[e].detach().float().view(N // 128, 128, K // 128, 128)
                s = (wb.abs().amax(dim=(1, 3)).clamp(min=1e-4) / 448.0)
                if native_block_scaling:
                    s = torch.exp2(torch.ceil(torch.log2(s)))
                out[e] = (wb / s.view(N // 128, 1, K // 128, 1)).view(N, K).to(torch.float8_e4m3fn)
                scales[e] = s
            return out, scales
        self._fp8 = (q(self.w13), q(self.w2))
        if native_block_scaling:
            (_, s13), (_, s2) = self._fp8
            n13 = self.w13.size(1)
            # (first GEMM wide tiles for large groups, second GEMM narrow, first GEMM narrow for small groups / decode, second GEMM wide)
            n2 = self.w2.size(1)
            self._mx = (gg.build_sf_atoms_b(s13, n13, swiglu=True, wide=True), gg.build_sf_atoms_b(s2, n2, wide=False),
                        gg.build_sf_atoms_b(s13, n13, swiglu=True, wide=False),
                        gg.build_sf_atoms_b(s2, n2, wide=True) if n2 % 256 == 0 else gg.build_sf_atoms_b(s2, n2, wide=False))

    @torch.no_grad()
    def forward_fp8(self, x: torch.Tensor, topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Forward only: FP8 on the wire and in both expert GEMMs, SwiGLU fused into the first GEMM, BF16 combine."""
        from .. import _ext
        C = _ext.load()
        if self._fp8 is None:
            self.prepare_fp8()
        (w13, s13), (w2, s2) = self._fp8
        if topk_idx is None:
            topk_idx, topk_weights = self.route(x)
        buf = self.buffer
        mx = getattr(self, "_mx", None)
        per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(topk_idx, self.cfg.num_experts)
        (rx, rs), recv_idx, recv_w, counts, handle, _ = buf.dispatch(
            x, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert, topk_idx=topk_idx,
            topk_weights=topk_weights, expert_alignment=EXPERT_ALIGNMENT, quantize_fp8=True, round_scale=mx is not None)
        plan = build_expert_plan(recv_idx, counts)
        a = gather_rows(rx, plan.src_row)
        a_s = gather_rows(rs, plan.src_row) if rs.size(1) % 4 == 0 else rs.index_select(0, plan.src_row.clamp(min=0).long())
        if mx is not None:
            # padding rows of the plan carry all-zero data; whatever exponent their zero scale maps to does not matter
            wide = plan.num_rows >= WIDE_TILE_MIN_ROWS_PER_EXPERT * self.num_local_experts
            h = gg.grouped_gemm(a, w13, plan.m_offsets, swiglu=True, sfa_atoms=gg.build_sf_atoms_a(a_s), sfb_atoms=mx[0 if wide else 2])
            hq, hs = C.per_token_cast_to_fp8(h, True, False)
            y_perm = gg.grouped_gemm(hq, w2, plan.m_offsets, sfa_atoms=gg.build_sf_atoms_a(hs), sfb_atoms=mx[3 if wide else 1])
        else:
            h = gg.grouped_gemm(a, w13, plan.m_offsets, swiglu=True, a_scales=a_s, b_scales=s13)
            hq, hs = C.per_token_cast_to_fp8(h, False, False)
            y_perm = gg.grouped_gemm(hq, w2, plan.m_offsets, a_scales=hs, b_scales=s2)
        y_recv = unpermute_weighted(y_perm, recv_w, plan, buf.empty_symmetric([rx.size(0), self.cfg.hidden], torch.bfloat16))
        out, _, _ = buf.combine(y_recv, handle)
        return out


    # -- fused FP8 inference path -----------------------------------------------------------------------------------
    @staticmethod
    def _C():
        from .. import _ext
        return _ext.load()

    def fused_workspace(self, num_tokens: int, capacity_rows: Optional[int] = None) -> "_FusedWorkspace":
        cache = self.__dict__.setdefault("_fused_ws", {})
        native = getattr(self, "_mx", None) is not None
        key = (num_tokens, native)
        if key not in cache:
            cache[key] = _FusedWorkspace(self, num_tokens, native, capacity_rows)
        return cache[key]

    @torch.no_grad()
    def forward_fused(self, x: torch.Tensor, topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None,
                      overlap: bool = True) -> torch.Tensor:
        """Forward only, same arithmetic as :meth:`forward_fp8`, as one overlapped pipeline (see the module docstring).
        Collective: every rank of the buffer calls it with the same number of tokens. The first call with a new token
        count allocates the workspace (symmetric memory sized for the worst case)."""
        if topk_idx is None:
            topk_idx, topk_weights = self.route(x)
        return fused_forward_many([self], [x.contiguous()], [topk_idx.contiguous()], [topk_weights.contiguous()], overlap=overlap)[0]

    # -- low-latency (decode) path ------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_low_latency(self, x: torch.Tensor, topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None,
                            num_max_tokens: Optional[int] = None) -> torch.Tensor:
        """Decode-sized forward: low-latency dispatch (FP8 on the wire) -> masked grouped FP8 GEMMs over the
        ``[L, N, hidden]`` landing zone (only the ``packed_recv_count[e]`` valid rows of every expert are computed) ->
        the second GEMM writes straight into the zero-copy combine buffer -> low-latency combine. No host
        synchronisation anywhere, so the whole layer can be captured in a CUDA graph."""
        from .. import _ext
        C = _ext.load()
        if self._fp8 is None:
            self.prepare_fp8()
        (w13, s13), (w2, s2) = self._fp8
        if topk_idx is None:
            topk_idx, topk_weights = self.route(x)
        buf, cfg = self.buffer, self.cfg
        R, L = buf.group_size, self.num_local_experts
        M = num_max_tokens or x.size(0)
        N, H, I = R * M, cfg.hidden, cfg.intermediate
        mx = getattr(self, "_mx", None) if N % 128 == 0 else None  # scale atoms cover whole 128-row tiles
        (px, ps), cnt, handle, _, _ = buf.low_latency_dispatch(x, topk_idx, M, cfg.num_experts, use_fp8=True, round_scale=mx is not None)
        ws = self.__dict__.setdefault("_ll_ws", {})
        key = (M, x.device)
        if key not in ws:
            dev = x.device
            ws[key] = dict(starts=(torch.arange(L + 1, device=dev, dtype=torch.int32) * N).contiguous(),
                           h=torch.empty(L * N, I, dtype=torch.bfloat16, device=dev),
                           hq=torch.empty(L * N, I, dtype=torch.float8_e4m3fn, device=dev),
                           hs=torch.empty(L * N, I // 128, dtype=torch.float32, device=dev))
        w_ = ws[key]
        ends = w_["starts"][:L] + cnt
        a, a_s = px.view(L * N, H), ps.view(L * N, H // 128)
        y = buf.get_next_low_latency_combine_buffer(handle)
        if mx is not None:
            wd = DECODE_WIDE_TILES
            gg.grouped_gemm(a, w13, w_["starts"], swiglu=True, out=w_["h"], m_ends=ends, sfa_atoms=gg.build_sf_atoms_a(a_s), sfb_atoms=mx[0 if wd else 2])
            C.per_token_cast_to_fp8(w_["h"], True, False, cnt, N, w_["hq"], w_["hs"])
            gg.grouped_gemm(w_["hq"], w2, w_["starts"], out=y.view(L * N, H), m_ends=ends, sfa_atoms=gg.build_sf_atoms_a(w_["hs"]),
                            sfb_atoms=mx[3 if wd else 1])
        else:
            gg.grouped_gemm(a, w13, w_["starts"], swiglu=True, a_scales=a_s, b_scales=s13, out=w_["h"], m_ends=ends)
            C.per_token_cast_to_fp8(w_["h"], False, False, cnt, N, w_["hq"], w_["hs"])
            gg.grouped_gemm(w_["hq"], w2, w_["starts"], a_scales=w_["hs"], b_scales=s2, out=y.view(L * N, H), m_ends=ends)
        out, _, _ = buf.low_latency_combine(y, topk_idx, topk_weights, handle, zero_copy=True)
        return out


# ---------------------------------------------------------------------------------------------------------
# fused forward: expert-major dispatch -> arrival-gated GEMM1 -> cast -> GEMM2 with scatter epilogue -> local reduce
# ---------------------------------------------------------------------------------------------------------
DECODE_WIDE_TILES = True  # masked low-latency layout (a handful of valid rows per expert): 128x256 tiles stream the weights faster (1 rank, 256 experts: 1.96 vs 2.25 ms per step)
UNIT_ROWS = 8  # rows of one expert a dispatch warp sends between two arrival-counter updates
# SMs the arrival-gated GEMM leaves to the dispatch kernel while the two overlap. Sharing SMs cannot be relied on: a CTA of
# the promotion kernel (10 warps of 160 registers) leaves no room for a dispatch warp in a scheduler partition's quarter of
# the register file, and next to the natively block-scaled kernel the dispatch was measured several times slower than on
# SMs of its own. A GEMM that got every SM before the dispatch CTAs were placed would wait for rows that nobody can send.
FUSE_CAST_INTO_GEMM1 = True  # wide natively block-scaled tiles: GEMM1's epilogue emits e4m3 + scale atoms itself
# Natively block-scaled GEMMs: average rows per expert from which the 128x256 tiles are used instead of the 128x128 ones. Since the
# wide tiles drain their accumulator in two halves they win from the smallest sizes measured on (8 experts x 4096 rows down to 256
# experts x 128 rows: +22 % to +54 %); below one tile of rows per expert the narrow tiles stay (fewer wasted columns per padded tile).
WIDE_TILE_MIN_ROWS_PER_EXPERT = 64
RESERVED_SMS = 16
# The gated GEMM runs as two launches when it overlaps the dispatch: the first part of the experts (arrival order = expert
# order) on the SMs the dispatch does not use, the rest on all SMs once the dispatch is about done.
SPLIT_FRACTION = 0.5
PREQUANTIZE = True  # cast every token to e4m3 once before the dispatch, which then only copies rows (8 selections share a cast)
GEMM_TIMEOUT_MS = 2000.0  # bound of every wait inside the gated GEMMs (pipeline barriers and arrival counters)


class _FusedWorkspace:
    """Buffers of one layer for ``num_tokens`` tokens per rank, allocated once: the receive side is sized for the worst
    case (every selection of every rank lands here), so no step ever needs a host round trip to size anything."""

    def __init__(self, layer: "MoELayer", num_tokens: int, native: bool, capacity_rows: Optional[int] = None) -> None:
        buf, cfg = layer.buffer, layer.cfg
        R, L, E, K, H, I = buf.group_size, layer.num_local_experts, cfg.num_experts, cfg.num_topk, cfg.hidden, cfg.intermediate
        T = num_tokens
        dev = buf.device
        worst = R * T * min(K, L) + L * 127
        rows = worst if capacity_rows is None else capacity_rows
        self.rows = rows = (rows + 127) // 128 * 128
        self.num_tokens, self.native = T, native
        sym = buf.empty_symmetric
        self.recv_x = sym([rows, H], torch.float8_e4m3fn)
        # fp32 scales [rows, H/128] or UE8M0 scale atoms [rows/128, H/128, 512]: the same number of bytes
        self.recv_scales_raw = sym([rows * (H // 128) * 4], torch.uint8)
        self.recv_scales = (self.recv_scales_raw.view(rows // 128, H // 128, 512) if native
                            else self.recv_scales_raw.view(torch.float32).view(rows, H // 128))
        self.recv_info = sym([rows], torch.int32)
        self.stage = sym([T * K, H], torch.bfloat16)
        i32 = dict(dtype=torch.int32, device=dev)
        self.my_counts = torch.zeros(E, **i32)
        self.sel_list = torch.zeros(E * T, **i32)
        self.send_base = torch.zeros(E, **i32)
        self.unit_start = torch.zeros(E + 2, **i32)  # prefix of work units [E + 1] and the hand-out counter
        self.m_offsets = torch.zeros(L + 1, **i32)
        self.m_ends = torch.zeros(L, **i32)
        self.peer_bases = torch.zeros(4 * R, dtype=torch.int64, device=dev)
        self.h = torch.empty(rows, I, dtype=torch.bfloat16, device=dev)
        self.hq = torch.empty(rows, I, dtype=torch.float8_e4m3fn, device=dev)
        self.hs = (torch.empty(rows // 128, I // 128, 512, dtype=torch.uint8, device=dev) if native
                   else torch.empty(rows, I // 128, dtype=torch.float32, device=dev))
        self.xq = torch.empty(T, H, dtype=torch.float8_e4m3fn, device=dev)
        self.xs = torch.empty(T, H // 128, dtype=torch.float32, device=dev)
        C = layer._C()
        arrived, expected = C.em_gate_words(buf.runtime)
        self.arrived, self.expected = arrived[:L], expected[:L]
        self.trace = None

    def enable_trace(self) -> None:
        """[dispatch first start, dispatch last end, GEMM1 first tile load, GEMM1 last epilogue end] in ns of the GPU's
        global timer (min / max over the CTAs), for the overlap evidence; [4] = the first bounded wait of GEMM1 that gave up
        (role, tile, K block, slot), [5] = what GEMM1's loader was doing then."""
        self.trace = torch.zeros(6, dtype=torch.int64, device=self.h.device)

    def reset_trace(self) -> None:
        big = torch.iinfo(torch.int64).max
        self.trace.copy_(torch.tensor([big, 0, big, 0, 0, 0], dtype=torch.int64))


def fused_forward_many(layers, xs, idxs, ws, overlap: bool = True, num_dispatch_sms: int = 0):
    """Fused FP8 forward of one MoE layer on every given rank (one entry per rank: a single entry in a real job, one per
    emulated rank on a single GPU, where the collectives run as one cooperative launch each and nothing overlaps).

    Streams: the count exchange and the dispatch run on the buffer's communication stream; the expert GEMMs run on the
    caller's stream as soon as the exchange is done, concurrently with the dispatch, and gate every expert on its arrival
    counter. The dispatch kernel is launched first and never waits for the GEMM, so the pair cannot deadlock; its small
    CTAs share the SMs with the GEMM's persistent CTAs."""
    V = len(layers)
    l0 = layers[0]
    C = l0._C()
    cfg = l0.cfg
    bufs = [l.buffer for l in layers]
    rts = [b.runtime for b in bufs]
    E, K = cfg.num_experts, cfg.num_topk
    for b in bufs:
        b.check_status()
    wss = []
    for l, x in zip(layers, xs):
        if l._fp8 is None:
            l.prepare_fp8()
        wss.append(l.fused_workspace(x.size(0)))
    native = wss[0].native
    cur = torch.cuda.current_stream()
    comm = bufs[0].comm_stream if (V == 1 and overlap) else cur
    if comm is not cur:
        comm.wait_stream(cur)
    # the quantisation of x (caller's stream) and the count exchange (communication stream) do not depend on each other: side by side
    quantised = None
    if PREQUANTIZE:
        for x, w in zip(xs, wss):
            C.per_token_cast_to_fp8(x, native, False, None, 1, w.xq, w.xs)
        if comm is not cur:
            quantised = torch.cuda.Event()
            quantised.record(cur)
    with torch.cuda.stream(comm):
        C.em_notify(rts, [(i, w.recv_x, w.recv_scales_raw, w.recv_info, w.stage, w.my_counts, w.sel_list, w.send_base, w.unit_start,
                           w.m_offsets, w.m_ends, w.peer_bases) for i, w in zip(idxs, wss)], E, UNIT_ROWS)
        planned = torch.cuda.Event()
        planned.record(comm)
        if quantised is not None:
            comm.wait_event(quantised)
        sms = num_dispatch_sms or (148 if V == 1 else max(1, 148 // V - 1))
        C.em_dispatch(rts, [(w.xq if PREQUANTIZE else x, w.my_counts, w.sel_list, w.send_base, w.unit_start, w.peer_bases, None,
                             None if w.trace is None else w.trace[0:2], w.xs if PREQUANTIZE else None) for x, w in zip(xs, wss)],
                      E, K, UNIT_ROWS, native, native, sms)
    if comm is not cur:
        cur.wait_event(planned)
    outs = []
    for l, w in zip(layers, wss):
        (w13, s13), (w2, s2) = l._fp8
        R_, L = l.buffer.group_size, l.num_local_experts
        overlapped = comm is not cur
        ga = min(L, max(1, int(round(L * SPLIT_FRACTION)))) if overlapped else L
        if native:
            wide = R_ * w.num_tokens * K >= WIDE_TILE_MIN_ROWS_PER_EXPERT * E
            sfb = l._mx[0 if wide else 2]
            fuse_cast = wide and FUSE_CAST_INTO_GEMM1
        # (first group, number of groups, SMs): the early experts next to the dispatch, the rest on the whole GPU
        parts = [(0, ga, 148 - RESERVED_SMS), (ga, L - ga, 0)] if (overlapped and ga < L) else [(0, L, (148 - RESERVED_SMS) if overlapped else 0)]
        for pi, (g0, ng, sms1) in enumerate(parts):
            tr = None if (w.trace is None or pi > 0) else w.trace[2:6]
            gate = dict(ready=w.arrived[g0:g0 + ng], expected=w.expected[g0:g0 + ng], trace=tr)
            mo, me_ = w.m_offsets[g0:g0 + ng + 1], w.m_ends[g0:g0 + ng]
            if native:
                if fuse_cast:
                    # a wide tile holds one whole scale block of the intermediate per row: the epilogue writes e4m3 + scale atoms itself
                    C.grouped_gemm(w.recv_x, w13[g0:g0 + ng], mo, 0, True, None, None, None, sms1, GEMM_TIMEOUT_MS, me_, w.recv_scales, sfb[g0:g0 + ng],
                                   out_fp8=w.hq, out_atoms=w.hs, **gate)
                else:
                    C.grouped_gemm(w.recv_x, w13[g0:g0 + ng], mo, 0, True, None, None, w.h, sms1, GEMM_TIMEOUT_MS, me_, w.recv_scales, sfb[g0:g0 + ng], **gate)
            else:
                C.grouped_gemm(w.recv_x, w13[g0:g0 + ng], mo, 0, True, w.recv_scales, s13[g0:g0 + ng], w.h, sms1, GEMM_TIMEOUT_MS, me_, None, None, **gate)
        if native:
            if not fuse_cast:
                C.per_token_cast_to_fp8(w.h, True, False, None, 1, w.hq, w.hs, w.m_offsets[L:], True)
            C.grouped_gemm(w.hq, w2, w.m_offsets, 0, False, None, None, None, 0, GEMM_TIMEOUT_MS, w.m_ends, w.hs, l._mx[3 if wide else 1],
                           row_info=w.recv_info, scatter_bases=w.peer_bases[3 * R_:])
        else:
            C.per_token_cast_to_fp8(w.h, False, False, None, 1, w.hq, w.hs, w.m_offsets[L:], False)
            C.grouped_gemm(w.hq, w2, w.m_offsets, 0, False, w.hs, s2, None, 0, GEMM_TIMEOUT_MS, w.m_ends, None, None,
                           row_info=w.recv_info, scatter_bases=w.peer_bases[3 * R_:])
    # every rank's second GEMM has finished scattering before anybody sums its stage
    C.barrier(rts)
    for l, x, i, wt, w in zip(layers, xs, idxs, ws, wss):
        out = torch.empty(x.size(0), cfg.hidden, dtype=torch.bfloat16, device=x.device)
        C.stage_reduce(w.stage, out, i, wt, E)
        outs.append(out)
    if comm is not cur:
        cur.wait_stream(comm)  # the dispatch kernel has read x before the caller may reuse it
    return outs


def dense_reference(x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, w13_all: torch.Tensor, w2_all: torch.Tensor) -> torch.Tensor:
    """Single-process fp32 loop over all experts (w13_all [E, 2I, H], w2_all [E, H, I]); the oracle for the layer."""
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    inter = w2_all.size(2)
    for e in range(w13_all.size(0)):
        rows, ks = (topk_idx == e).nonzero(as_tuple=True)
        if rows.numel() == 0:
            continue
        h = x[rows].float() @ w13_all[e].float().t()
        h = F.silu(h[:, :inter]) * h[:, inter:]
        y = h.to(torch.bfloat16).float() @ w2_all[e].float().t()
        out.index_add_(0, rows, y * topk_weights[rows, ks].unsqueeze(1))
    return out
