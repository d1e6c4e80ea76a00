"""Grouped tcgen05 GEMM against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _offsets(rows, device="cuda"):
    o = [0]
    for r in rows:
        o.append(o[-1] + r)
    return torch.tensor(o, dtype=torch.int32, device=device)


def _rel_err(x, ref):
    return ((x.float() - ref).norm() / ref.norm().clamp(min=1e-12)).item()


@pytest.mark.parametrize("rows,K,N", [([128], 64, 128), ([128, 256, 0, 384], 512, 256), ([256, 128], 1024, 384), ([128] * 5, 192, 512)])
def test_bf16_mgrouped(rows, K, N):
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.ops.grouped_gemm import grouped_gemm, reference_grouped_gemm
    C = _ext.load()
    C.gemm_clear_error(0)
    torch.manual_seed(0)
    G, M = len(rows), sum(rows)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(G, N, K, device="cuda") * 0.1).to(torch.bfloat16)
    offs = _offsets(rows)
    c = grouped_gemm(a, b, offs)
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0
    ref = reference_grouped_gemm(a, b, offs)
    assert _rel_err(c, ref) < 1e-2, _rel_err(c, ref)
    # a second launch on a smaller persistent grid walks several tiles per CTA
    c2 = grouped_gemm(a, b, offs, num_sms=3)
    assert torch.equal(c, c2)


def test_unaligned_and_masked_groups():
    """Group boundaries anywhere, and m_ends: only the first rows of every group are computed, the rest stay untouched."""
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.ops.grouped_gemm import grouped_gemm, reference_grouped_gemm
    C = _ext.load()
    C.gemm_clear_error(0)
    torch.manual_seed(5)
    rows, K, N = [40, 200, 0, 77, 3], 256, 256
    G, M = len(rows), sum(rows)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(G, N, K, device="cuda") * 0.1).to(torch.bfloat16)
    offs = _offsets(rows)
    c = grouped_gemm(a, b, offs)
    ref = reference_grouped_gemm(a, b, offs)
    assert _rel_err(c, ref) < 1e-2, _rel_err(c, ref)
    # masked: fixed stride 64 per group (tiles of 128 rows overlap the next group), counts 0..64
    stride, counts = 64, [64, 0, 17, 33, 1]
    starts = torch.arange(G + 1, device="cuda", dtype=torch.int32) * stride
    ends = starts[:G] + torch.tensor(counts, device="cuda", dtype=torch.int32)
    a = torch.randn(G * stride, K, device="cuda").to(torch.bfloat16)
    out = torch.full((G * stride, N), 7.0, device="cuda", dtype=torch.bfloat16)
    grouped_gemm(a, b, starts, out=out, m_ends=ends)
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0
    full = reference_grouped_gemm(a, b, starts)
    for g, n in enumerate(counts):
        lo = g * stride
        if n:
            assert _rel_err(out[lo:lo + n], full[lo:lo + n]) < 1e-2
        assert (out[lo + n:lo + stride] == 7.0).all()
    sw = torch.full((G * stride, N // 2), 7.0, device="cuda", dtype=torch.bfloat16)
    grouped_gemm(a, b, starts, swiglu=True, out=sw, m_ends=ends)
    fsw = reference_grouped_gemm(a, b, starts, swiglu=True)
    for g, n in enumerate(counts):
        lo = g * stride
        if n:
            assert _rel_err(sw[lo:lo + n], fsw[lo:lo + n]) < 1.5e-2
        assert (sw[lo + n:lo + stride] == 7.0).all()


@pytest.mark.parametrize("rows,K,I", [([128, 256], 256, 128), ([128, 128, 384], 512, 192)])
def test_bf16_swiglu(rows, K, I):
    from deepep_efa_b200.ops.grouped_gemm import grouped_gemm, reference_grouped_gemm
    torch.manual_seed(1)
    G, M = len(rows), sum(rows)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(G, 2 * I, K, device="cuda") * 0.1).to(torch.bfloat16)
    offs = _offsets(rows)
    c = grouped_gemm(a, b, offs, swiglu=True)
    assert c.shape == (M, I)
    ref = reference_grouped_gemm(a, b, offs, swiglu=True)
    assert _rel_err(c, ref) < 1.5e-2, _rel_err(c, ref)


@pytest.mark.parametrize("swiglu", [False, True])
def test_fp8_blockscaled(swiglu):
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.ops.grouped_gemm import grouped_gemm, reference_grouped_gemm
    from deepep_efa_b200.reference import oracle
    C = _ext.load()
    torch.manual_seed(2)
    rows, K, N = [128, 256, 128], 512, 256
    G, M = len(rows), sum(rows)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    a, a_s = C.per_token_cast_to_fp8(x, False, False)
    w = torch.randn(G, N, K, device="cuda") * 0.05
    wb = w.view(G, N // 128, 128, K // 128, 128)
    b_s = (wb.abs().amax(dim=(2, 4)).clamp(min=1e-4) / 448.0).contiguous()
    b = (wb / b_s.view(G, N // 128, 1, K // 128, 1)).view(G, N, K).to(torch.float8_e4m3fn)
    offs = _offsets(rows)
    c = grouped_gemm(a, b, offs, swiglu=swiglu, a_scales=a_s, b_scales=b_s)
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0
    ref = reference_grouped_gemm(a, b, offs, swiglu=swiglu, a_scales=a_s, b_scales=b_s)
    assert _rel_err(c, ref) < 1e-2, _rel_err(c, ref)


def test_bf16_wgrad_kgrouped():
    from deepep_efa_b200.ops.grouped_gemm import grouped_gemm_wgrad
    torch.manual_seed(3)
    rows, n_out, k_out = [128, 0, 256], 256, 128
    M = sum(rows)
    dy = torch.randn(M, n_out, device="cuda").to(torch.bfloat16)
    x = torch.randn(M, k_out, device="cuda").to(torch.bfloat16)
    offs = _offsets(rows)
    dw = grouped_gemm_wgrad(dy.t().contiguous(), x.t().contiguous(), offs)
    assert dw.shape == (3, n_out, k_out)
    o = offs.tolist()
    for g in range(3):
        ref = dy[o[g]:o[g + 1]].float().t() @ x[o[g]:o[g + 1]].float()
        if rows[g] == 0:
            assert dw[g].float().abs().max().item() == 0
        else:
            assert _rel_err(dw[g], ref) < 1e-2


@pytest.mark.parametrize("shape", [(64, 64), (200, 72), (3, 136, 4096), (2, 1408, 264)])
def test_transpose_kernel(shape):
    from deepep_efa_b200.ops.grouped_gemm import transpose_last2
    torch.manual_seed(7)
    x = torch.randn(*shape, device="cuda").to(torch.bfloat16)
    assert torch.equal(transpose_last2(x), x.transpose(-1, -2).contiguous())


def test_swiglu_kernels_match_autograd():
    from deepep_efa_b200.ops.grouped_gemm import swiglu
    torch.manual_seed(8)
    M, I = 300, 1408
    h13 = torch.randn(M, 2 * I, device="cuda").to(torch.bfloat16).requires_grad_(True)
    dh = torch.randn(M, I, device="cuda").to(torch.bfloat16)
    h = swiglu(h13)
    h.backward(dh)
    ref_in = h13.detach().float().requires_grad_(True)
    ref = torch.nn.functional.silu(ref_in[:, :I]) * ref_in[:, I:]
    ref.backward(dh.float())
    assert _rel_err(h, ref.detach()) < 4e-3
    assert _rel_err(h13.grad, ref_in.grad) < 4e-3


def test_rowdot_kernel():
    from deepep_efa_b200 import _ext
    torch.manual_seed(9)
    Mp, N, K, H = 500, 120, 6, 4096
    a = torch.randn(Mp, H, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, H, device="cuda").to(torch.bfloat16)
    pos = torch.randint(-1, Mp, (N, K), device="cuda", dtype=torch.int32)
    got = _ext.load().rowdot(a, b, pos)
    want = torch.where(pos >= 0, (a[pos.clamp(min=0).long()].float() * b.float().unsqueeze(1)).sum(-1), torch.zeros(N, K, device="cuda"))
    assert torch.allclose(got, want, rtol=1e-3, atol=1e-2)


@pytest.mark.parametrize("swiglu,wide", [(False, True), (False, False), (True, True), (True, False)])
def test_fp8_native_block_scaling(swiglu, wide):
    """tcgen05 block-scaled MMA with UE8M0 scale atoms against the dequantised fp32 reference; the row scales differ by
    powers of two from row to row so that a wrong row-to-scale mapping cannot pass."""
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.ops.grouped_gemm import build_sf_atoms_a, build_sf_atoms_b, grouped_gemm, reference_grouped_gemm
    C = _ext.load()
    C.gemm_clear_error(0)
    torch.manual_seed(11)
    rows, K = [128, 256, 0, 384], 512
    N = 512
    G, M = len(rows), sum(rows)
    x = torch.randn(M, K, device="cuda") * torch.pow(2.0, (torch.arange(M, device="cuda") % 7).float()).unsqueeze(1)
    x = x * torch.pow(2.0, (torch.arange(K, device="cuda") // 128 % 3).float()).unsqueeze(0)
    a, a_s = C.per_token_cast_to_fp8(x.to(torch.bfloat16), True, False)  # power-of-two scales
    w = torch.randn(G, N, K, device="cuda") * 0.1 * torch.pow(2.0, (torch.arange(N, device="cuda") // 128 % 4).float()).view(1, N, 1)
    wb = w.view(G, N // 128, 128, K // 128, 128)
    b_s = torch.exp2(torch.ceil(torch.log2(wb.abs().amax(dim=(2, 4)).clamp(min=1e-4) / 448.0))).contiguous()
    b = (wb / b_s.view(G, N // 128, 1, K // 128, 1)).view(G, N, K).to(torch.float8_e4m3fn).contiguous()
    offs = _offsets(rows)
    c = grouped_gemm(a, b, offs, swiglu=swiglu, sfa_atoms=build_sf_atoms_a(a_s), sfb_atoms=build_sf_atoms_b(b_s, N, swiglu, wide))
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0
    ref = reference_grouped_gemm(a, b, offs, swiglu=swiglu, a_scales=a_s, b_scales=b_s)
    assert _rel_err(c, ref) < (1.5e-2 if swiglu else 1e-2), _rel_err(c, ref)


@pytest.mark.parametrize("rows,N_w,K_w", [([128, 256, 0, 384], 256, 512), ([40, 200, 77], 384, 128), ([256] * 3, 1408, 4096)])
def test_bf16_dgrad_reads_weight_in_place(rows, N_w, K_w):
    """dx = grad @ w[g] with the forward weight [G, N, K] consumed as an MN-major operand: no transposed copy."""
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.ops.grouped_gemm import grouped_gemm_dgrad
    C = _ext.load()
    C.gemm_clear_error(0)
    torch.manual_seed(11)
    G, M = len(rows), sum(rows)
    grad = torch.randn(M, N_w, device="cuda").to(torch.bfloat16)
    w = (torch.randn(G, N_w, K_w, device="cuda") * 0.1).to(torch.bfloat16)
    offs = _offsets(rows)
    dx = grouped_gemm_dgrad(grad, w, offs)
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0 and dx.shape == (M, K_w)
    o = offs.tolist()
    for g in range(G):
        if rows[g]:
            ref = grad[o[g]:o[g + 1]].float() @ w[g].float()
            assert _rel_err(dx[o[g]:o[g + 1]], ref) < 1e-2, (g, _rel_err(dx[o[g]:o[g + 1]], ref))


@pytest.mark.parametrize("rows,n_out,k_out", [([128, 0, 256], 256, 128), ([64, 192, 128], 384, 256), ([512, 256], 1408, 4096)])
def test_bf16_wgrad_reads_gradient_and_activation_in_place(rows, n_out, k_out):
    """dw[g] = grad[rows of g].T @ x[rows of g] with both operands MN-major: no transposed copies."""
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.ops.grouped_gemm import grouped_gemm_wgrad_inplace
    C = _ext.load()
    C.gemm_clear_error(0)
    torch.manual_seed(12)
    M = sum(rows)
    dy = torch.randn(M, n_out, device="cuda").to(torch.bfloat16)
    x = torch.randn(M, k_out, device="cuda").to(torch.bfloat16)
    offs = _offsets(rows)
    dw = grouped_gemm_wgrad_inplace(dy, x, offs)
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0 and dw.shape == (len(rows), n_out, k_out)
    o = offs.tolist()
    for g in range(len(rows)):
        ref = dy[o[g]:o[g + 1]].float().t() @ x[o[g]:o[g + 1]].float()
        if rows[g] == 0:
            assert dw[g].float().abs().max().item() == 0
        else:
            assert _rel_err(dw[g], ref) < 1e-2, (g, _rel_err(dw[g], ref))


def test_fp8_native_wide_swiglu_writes_quantised_output():
    """The wide natively block-scaled SwiGLU kernel can emit e4m3 rows plus UE8M0 scale atoms itself; both must equal what
    the standalone cast makes of the kernel's BF16 output, bit for bit (valid rows only; masked groups stay untouched)."""
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.ops.grouped_gemm import build_sf_atoms_a, build_sf_atoms_b
    C = _ext.load()
    C.gemm_clear_error(0)
    torch.manual_seed(21)
    rows, K, N = [128, 200, 0, 384], 512, 1024  # N/2 = 512 outputs = 4 scale blocks per row
    G = len(rows)
    starts = [0]
    for r in rows:
        starts.append(starts[-1] + (r + 127) // 128 * 128)
    M = starts[-1]
    offs = torch.tensor(starts, dtype=torch.int32, device="cuda")
    ends = torch.tensor([starts[g] + rows[g] for g in range(G)], dtype=torch.int32, device="cuda")
    x = torch.randn(M, K, device="cuda") * torch.pow(2.0, (torch.arange(M, device="cuda") % 5).float()).unsqueeze(1)
    a, a_s = C.per_token_cast_to_fp8(x.to(torch.bfloat16), True, False)
    w = torch.randn(G, N, K, device="cuda") * 0.1
    wb = w.view(G, N // 128, 128, K // 128, 128)
    b_s = torch.exp2(torch.ceil(torch.log2(wb.abs().amax(dim=(2, 4)).clamp(min=1e-4) / 448.0))).contiguous()
    b = (wb / b_s.view(G, N // 128, 1, K // 128, 1)).view(G, N, K).to(torch.float8_e4m3fn).contiguous()
    sfa, sfb = build_sf_atoms_a(a_s), build_sf_atoms_b(b_s, N, True, True)
    h = torch.zeros(M, N // 2, dtype=torch.bfloat16, device="cuda")
    C.grouped_gemm(a, b, offs, 0, True, None, None, h, 0, 2000.0, ends, sfa, sfb)
    hq_ref, atoms_ref = C.per_token_cast_to_fp8(h, True, False, None, 1, None, None, None, True)
    hq = torch.full((M, N // 2), 0x55, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    atoms = torch.full(((M + 127) // 128, N // 2 // 128, 512), 0x55, dtype=torch.uint8, device="cuda")
    C.grouped_gemm(a, b, offs, 0, True, None, None, None, 0, 2000.0, ends, sfa, sfb, out_fp8=hq, out_atoms=atoms)
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0
    rr = torch.arange(M, device="cuda")
    for g in range(G):
        lo, hi = starts[g], starts[g] + rows[g]
        assert torch.equal(hq.view(torch.uint8)[lo:hi], hq_ref.view(torch.uint8)[lo:hi]), g
        assert (hq.view(torch.uint8)[hi:starts[g + 1]] == 0x55).all()
        r = rr[lo:hi]
        for kb in range(N // 2 // 128):
            idx = (r % 32) * 16 + ((r // 32) % 4) * 4
            assert torch.equal(atoms[r // 128, kb, idx], atoms_ref[r // 128, kb, idx]), (g, kb)


def test_fp8_native_wide_swiglu_cta_pairs(monkeypatch):
    """The wide natively block-scaled SwiGLU tile on CTA pairs (one 256-row MMA per pair, each CTA staging its own rows of A,
    half of the B tile and its own copy of the scale atoms) gives the same numbers as the single-CTA kernel; rows carry
    different power-of-two scales, so scale atoms that reached the wrong CTA's TMEM cannot pass."""
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.ops.grouped_gemm import build_sf_atoms_a, build_sf_atoms_b, grouped_gemm, reference_grouped_gemm
    C = _ext.load()
    C.gemm_clear_error(0)
    torch.manual_seed(31)
    rows, K, N = [256, 512, 0, 384, 128], 1024, 1024
    G = len(rows)
    starts = [0]
    for r in rows:
        starts.append(starts[-1] + (r + 127) // 128 * 128)
    M = starts[-1]
    offs = torch.tensor(starts, dtype=torch.int32, device="cuda")
    x = torch.randn(M, K, device="cuda") * torch.pow(2.0, (torch.arange(M, device="cuda") % 7).float()).unsqueeze(1)
    x = x * torch.pow(2.0, (torch.arange(K, device="cuda") // 128 % 3).float()).unsqueeze(0)
    a, a_s = C.per_token_cast_to_fp8(x.to(torch.bfloat16), True, False)
    w = torch.randn(G, N, K, device="cuda") * 0.1 * torch.pow(2.0, (torch.arange(N, device="cuda") // 128 % 4).float()).view(1, N, 1)
    wb = w.view(G, N // 128, 128, K // 128, 128)
    b_s = torch.exp2(torch.ceil(torch.log2(wb.abs().amax(dim=(2, 4)).clamp(min=1e-4) / 448.0))).contiguous()
    b = (wb / b_s.view(G, N // 128, 1, K // 128, 1)).view(G, N, K).to(torch.float8_e4m3fn).contiguous()
    sfa, sfb = build_sf_atoms_a(a_s), build_sf_atoms_b(b_s, N, True, True)
    monkeypatch.setenv("DEEPEP_GEMM_PAIR", "0")
    single = grouped_gemm(a, b, offs, swiglu=True, sfa_atoms=sfa, sfb_atoms=sfb)
    monkeypatch.setenv("DEEPEP_GEMM_PAIR", "1")
    paired = grouped_gemm(a, b, offs, swiglu=True, sfa_atoms=sfa, sfb_atoms=sfb)
    paired_small_grid = grouped_gemm(a, b, offs, swiglu=True, sfa_atoms=sfa, sfb_atoms=sfb, num_sms=6)
    torch.cuda.synchronize()
    assert C.gemm_error(0) == 0
    ref = reference_grouped_gemm(a, b, offs, swiglu=True, a_scales=a_s, b_scales=b_s)
    assert _rel_err(single, ref) < 1.5e-2
    assert _rel_err(paired, ref) < 1.5e-2, _rel_err(paired, ref)
    assert torch.equal(paired, single) and torch.equal(paired_small_grid, single)
