"""MoE layer on the GPU (one rank): tcgen05 grouped GEMMs, gather kernels and the dispatch/combine kernels, forward
and backward against a dense fp32 loop over all experts; plus the FP8 forward path."""
import pytest
import torch

from helpers import make_routing, make_tokens

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


def test_permute_kernels_match_indexing():
    from deepep_efa_b200.ops.permute import build_expert_plan, gather_reduce_rows, gather_rows
    torch.manual_seed(0)
    N, K, L, H = 300, 4, 5, 256
    idx = torch.randint(-1, L, (N, K), device="cuda")
    counts = [int(((idx == e).sum().item() + 127) // 128 * 128) for e in range(L)]
    plan = build_expert_plan(idx, counts)
    x = torch.randn(N, H, device="cuda").to(torch.bfloat16)
    xp = gather_rows(x, plan.src_row)
    o = plan.m_offsets.tolist()
    for e in range(L):
        rows, ks = (idx == e).nonzero(as_tuple=True)
        n = rows.numel()
        seg_rows, seg_k = plan.src_row[o[e]:o[e] + n].long(), plan.src_k[o[e]:o[e] + n].long()
        # the selections of an expert fill its segment in some order: same multiset of (row, k), payload follows src_row
        assert torch.equal(torch.sort(seg_rows * K + seg_k).values, torch.sort(rows * K + ks).values)
        assert torch.equal(xp[o[e]:o[e] + n], x[seg_rows])
        assert (plan.src_row[o[e] + n:o[e + 1]] == -1).all() and xp[o[e] + n:o[e + 1]].abs().sum().item() == 0
        assert torch.equal(plan.pos[seg_rows, seg_k].long(), torch.arange(o[e], o[e] + n, device="cuda"))
    w = torch.rand(N, K, device="cuda")
    y = gather_reduce_rows(xp, plan.pos, w)
    ref = x.float() * (w * (idx >= 0)).sum(1, keepdim=True)
    assert _rel(y, ref) < 1e-2
    # fp8 rows and fp32 scale rows go through the same byte-row gather
    q = x.to(torch.float8_e4m3fn)
    assert torch.equal(gather_rows(q, plan.src_row).view(torch.uint8)[o[1]:o[1] + 3], q.view(torch.uint8)[plan.src_row[o[1]:o[1] + 3].long()])


def test_moe_layer_forward_backward_gpu():
    import deepep_efa_b200 as ep
    from deepep_efa_b200.models.moe import MoEConfig, MoELayer, dense_reference
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    T, H, I, E, K = 256, 512, 256, 8, 2
    vc = VirtualCluster(1, num_nvl_bytes=128 << 20)
    try:
        buf = vc.buffers[0]
        cfg = MoEConfig(hidden=H, intermediate=I, num_experts=E, num_topk=K, init_std=0.05)
        layer = MoELayer(cfg, buf)
        x = make_tokens(T, H, "cuda", seed=3).requires_grad_(True)
        idx, w = make_routing(T, E, K, "cuda", seed=3)
        w = w.requires_grad_(True)
        y = layer(x, idx, w)
        (y.float() ** 2).mean().backward()
        torch.cuda.synchronize()
        buf.check_status()
        assert ep._ext.load().gemm_error(0) == 0
        w13 = layer.w13.detach().float().requires_grad_(True)
        w2 = layer.w2.detach().float().requires_grad_(True)
        xr, wr = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
        ref = dense_reference(xr, idx, wr, w13, w2)
        (ref ** 2).mean().backward()
        assert _rel(y, ref) < 3e-2, _rel(y, ref)
        assert _rel(x.grad, xr.grad) < 6e-2, _rel(x.grad, xr.grad)
        assert _rel(w.grad, wr.grad) < 6e-2, _rel(w.grad, wr.grad)
        assert _rel(layer.w13.grad, w13.grad) < 6e-2, _rel(layer.w13.grad, w13.grad)
        assert _rel(layer.w2.grad, w2.grad) < 6e-2, _rel(layer.w2.grad, w2.grad)
        # routing through the layer's own gate
        y2 = layer(x.detach())
        assert y2.shape == (T, H) and torch.isfinite(y2.float()).all()
        # FP8 forward path with arbitrary fp32 block scales (promoted on the CUDA cores)
        layer.prepare_fp8(native_block_scaling=False)
        y8 = layer.forward_fp8(x.detach(), idx, w.detach())
        torch.cuda.synchronize()
        buf.check_status()
        assert _rel(y8, ref.detach()) < 8e-2, _rel(y8, ref.detach())
        # the same path with power-of-two scales consumed by the tensor core itself (UE8M0 block scaling)
        layer.prepare_fp8(native_block_scaling=True)
        y8n = layer.forward_fp8(x.detach(), idx, w.detach())
        torch.cuda.synchronize()
        buf.check_status()
        assert ep._ext.load().gemm_error(0) == 0
        assert _rel(y8n, ref.detach()) < 8e-2, _rel(y8n, ref.detach())
    finally:
        vc.destroy()


def test_moe_low_latency_decode_path():
    import deepep_efa_b200 as ep
    from deepep_efa_b200.models.moe import MoEConfig, MoELayer, dense_reference
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    T, H, I, E, K = 48, 512, 256, 8, 2
    vc = VirtualCluster(1, num_nvl_bytes=8 << 20, num_rdma_bytes=ep.Buffer.get_low_latency_rdma_size_hint(128, H, 1, E))
    try:
        buf = vc.buffers[0]
        layer = MoELayer(MoEConfig(hidden=H, intermediate=I, num_experts=E, num_topk=K, init_std=0.05), buf)
        x = make_tokens(T, H, "cuda", seed=5)
        idx, w = make_routing(T, E, K, "cuda", seed=5, masked_fraction=0.1)
        ref = dense_reference(x, idx, w.masked_fill(idx == -1, 0), layer.w13.detach().float(), layer.w2.detach().float())
        layer.prepare_fp8(native_block_scaling=False)
        for _ in range(3):  # both parities, workspace reuse
            y = layer.forward_low_latency(x, idx, w, num_max_tokens=64)
            torch.cuda.synchronize()
            buf.check_status()
            assert ep._ext.load().gemm_error(0) == 0
            assert _rel(y, ref) < 8e-2, _rel(y, ref)
        # tile-aligned landing zone (N = 128): power-of-two scales applied by the tensor core itself
        layer.prepare_fp8(native_block_scaling=True)
        for _ in range(2):
            y = layer.forward_low_latency(x, idx, w, num_max_tokens=128)
            torch.cuda.synchronize()
            buf.check_status()
            assert ep._ext.load().gemm_error(0) == 0
            assert _rel(y, ref) < 8e-2, _rel(y, ref)
    finally:
        vc.destroy()
