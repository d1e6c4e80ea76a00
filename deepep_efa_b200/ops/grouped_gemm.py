"""Grouped expert GEMM (tcgen05 / TMEM / TMA kernel in csrc/kernels/grouped_gemm.cu) and its autograd wrapper.

``grouped_gemm(a, b, m_offsets)`` computes ``c[m] = a[m] @ b[g].T`` for the rows m of expert g, where the rows of
expert g are ``[m_offsets[g], m_offsets[g+1])`` (any boundaries: a tile never writes past its group's end; the
K-grouped weight-gradient mode needs boundaries on multiples of 128). With ``m_ends`` only the rows
``[m_offsets[g], m_ends[g])`` of every group are computed, which is how the low-latency ``[L, N, hidden]`` landing
zone with its per-expert counts is consumed without compaction. Operands are bf16, or
e4m3 with DeepSeek-style fp32 scales (1x128 on ``a``, 128x128 on ``b``). ``swiglu=True`` treats ``b`` as
``[G, 2*I, K]`` = [gate; up] and returns ``silu(a @ gate.T) * (a @ up.T)``.

The reference library ships no GEMM (its users run the expert FFN themselves); this exists for the fused MoE
layer and the training path.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _ext


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, m_offsets: torch.Tensor, *, swiglu: bool = False,
                 a_scales: Optional[torch.Tensor] = None, b_scales: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, num_sms: int = 0, m_ends: Optional[torch.Tensor] = None,
                 sfa_atoms: Optional[torch.Tensor] = None, sfb_atoms: Optional[torch.Tensor] = None) -> torch.Tensor:
    """M-grouped GEMM; see the module docstring. Returns bf16 ``[M, N]`` (``[M, N/2]`` with ``swiglu``).

    ``m_ends`` (int32 ``[G]``, optional) makes group g cover rows ``[m_offsets[g], m_ends[g])``: the "masked" form for the
    low-latency layout ``[L, N, hidden]``, where every expert starts at ``g * N`` and only ``packed_recv_count[g]`` rows
    are valid; rows past ``m_ends[g]`` are never written.

    ``sfa_atoms`` / ``sfb_atoms`` (from :func:`build_sf_atoms_a` / :func:`build_sf_atoms_b`) select the natively block-scaled
    FP8 kernel: power-of-two scales are applied by the tensor core (``kind::mxf8f6f4.block_scale``) and a whole tile
    accumulates in TMEM. Every group must then start on a multiple of 128 rows."""
    return _ext.load().grouped_gemm(a, b, m_offsets, 0, swiglu, a_scales, b_scales, out, num_sms, 2000.0, m_ends, sfa_atoms, sfb_atoms)


def build_sf_atoms_a(a_scales: torch.Tensor) -> torch.Tensor:
    """UE8M0 scale atoms of the activations for the natively block-scaled FP8 GEMM (``a_scales`` f32 ``[M, K/128]``, powers
    of two, e.g. from a cast with ``round_scale=True``)."""
    return _ext.load().build_sf_atoms_a(a_scales.contiguous())


def build_sf_atoms_b(b_scales: torch.Tensor, n: int, swiglu: bool = False, wide: Optional[bool] = None) -> torch.Tensor:
    """UE8M0 scale atoms of the weights (``b_scales`` f32 ``[G, N/128, K/128]``, powers of two); built once per weight.

    The atoms also fix the tile width of the GEMM that consumes them: ``wide=True`` is the 256-column tile with one
    accumulator window (fastest for several hundred rows per expert and more; without ``swiglu`` it needs ``N % 256 == 0``),
    ``wide=False`` the 128-column tile with two windows (better for small groups and for the masked low-latency layout).
    Default: wide with ``swiglu``, narrow without."""
    if wide is None:
        wide = swiglu
    return _ext.load().build_sf_atoms_b(b_scales.contiguous(), n, swiglu, bool(wide))


def grouped_gemm_wgrad(a_t: torch.Tensor, b_t: torch.Tensor, m_offsets: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                       num_sms: int = 0) -> torch.Tensor:
    """K-grouped GEMM for weight gradients: ``c[g] = a_t[:, rows of g] @ b_t[:, rows of g].T`` with
    ``a_t`` ``[N_out, M]`` and ``b_t`` ``[K_out, M]`` (both bf16, M contiguous). Returns bf16 ``[G, N_out, K_out]``."""
    return _ext.load().grouped_gemm(a_t, b_t, m_offsets, 1, False, None, None, out, num_sms)


def grouped_gemm_dgrad(grad: torch.Tensor, w: torch.Tensor, m_offsets: torch.Tensor, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Input gradient of ``y = grouped_gemm(x, w)``: ``dx[m] = grad[m] @ w[g]`` for the rows of expert g, with ``w``
    ``[G, N, K]`` read in place as an MN-major operand (no transposed copy of the weight). bf16; ``grad`` is ``[M, N]``."""
    return _ext.load().grouped_gemm(grad, w, m_offsets, 0, False, None, None, out, 0, 2000.0, mn_major=True)


def grouped_gemm_wgrad_inplace(grad: torch.Tensor, x: torch.Tensor, m_offsets: torch.Tensor, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Weight gradient ``dw[g] = grad[rows of g].T @ x[rows of g]`` with ``grad`` ``[M, N_out]`` and ``x`` ``[M, K_out]`` read in
    place as MN-major operands (no transposed copies). Group boundaries on multiples of 64 rows. Returns bf16 ``[G, N_out, K_out]``."""
    return _ext.load().grouped_gemm(grad, x, m_offsets, 1, False, None, None, out, 0, 2000.0, mn_major=True)


def reference_grouped_gemm(a: torch.Tensor, b: torch.Tensor, m_offsets: torch.Tensor, swiglu: bool = False,
                           a_scales: Optional[torch.Tensor] = None, b_scales: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Plain PyTorch fp32 reference of :func:`grouped_gemm` (used by the tests)."""
    G = m_offsets.numel() - 1
    offs = m_offsets.tolist()
    af = a.float()
    if a_scales is not None:
        af = (af.view(a.size(0), -1, 128) * a_scales.unsqueeze(-1)).view(a.shape)
    K = a.size(1)
    bf = b.float().view(G, -1, K)
    if b_scales is not None:
        N = bf.size(1)
        bf = (bf.view(G, N // 128, 128, K // 128, 128) * b_scales.view(G, N // 128, 1, K // 128, 1)).view(G, N, K)
    N = bf.size(1)
    out = torch.zeros(a.size(0), N // 2 if swiglu else N, dtype=torch.float32, device=a.device)
    for g in range(G):
        r = slice(offs[g], offs[g + 1])
        y = af[r] @ bf[g].t()
        if swiglu:
            gate, up = y[:, :N // 2], y[:, N // 2:]
            y = torch.nn.functional.silu(gate) * up
        out[r] = y
    return out


def transpose_last2(x: torch.Tensor) -> torch.Tensor:
    """Contiguous ``x.transpose(-1, -2)`` for a 2-D or 3-D tensor (tiled kernel for bf16 on the GPU)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.dim() in (2, 3) and x.size(-1) % 8 == 0 and x.size(-2) % 8 == 0:
        return _ext.load().transpose_bf16(x.contiguous())
    return x.transpose(-1, -2).contiguous()


class _SwiGLU(torch.autograd.Function):
    """``h = silu(h13[:, :I]) * h13[:, I:]`` with fp32 math and bf16 storage, one kernel per direction."""

    @staticmethod
    def forward(ctx, h13):
        ctx.save_for_backward(h13)
        if h13.is_cuda and h13.dtype == torch.bfloat16 and h13.size(1) % 16 == 0:
            return _ext.load().swiglu_fwd(h13.contiguous())
        inter = h13.size(1) // 2
        return (torch.nn.functional.silu(h13[:, :inter].float()) * h13[:, inter:].float()).to(h13.dtype)

    @staticmethod
    def backward(ctx, dh):
        (h13,) = ctx.saved_tensors
        if h13.is_cuda and h13.dtype == torch.bfloat16 and h13.size(1) % 16 == 0:
            return _ext.load().swiglu_bwd(h13.contiguous(), dh.contiguous().to(torch.bfloat16))
        inter = h13.size(1) // 2
        g, u, d = h13[:, :inter].float(), h13[:, inter:].float(), dh.float()
        sig = torch.sigmoid(g)
        return torch.cat([d * u * sig * (1 + g * (1 - sig)), d * g * sig], dim=1).to(h13.dtype)


def swiglu(h13: torch.Tensor) -> torch.Tensor:
    return _SwiGLU.apply(h13)
