"""Low-latency kernels against the oracle; sweeps follow the reference's tests/test_low_latency.py
(:92-95 hook x fp8 x round_scale x ue8m0, :113-147 per-expert checks, :181-184 tolerances, -1 masks)."""
import pytest
import torch

from helpers import make_routing, make_tokens

pytestmark = pytest.mark.gpu


def _cluster(R, T, H, E, **kw):
    from deepep_efa_b200 import Buffer
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    return VirtualCluster(R, num_nvl_bytes=2 << 20, num_rdma_bytes=Buffer.get_low_latency_rdma_size_hint(T, H, R, E),
                          timeout_ms=2000, **kw)


@pytest.mark.parametrize("R,T,H,E,K", [(1, 16, 512, 8, 4), (2, 33, 1024, 16, 8), (4, 24, 7168, 32, 8), (8, 16, 2048, 64, 8)])
@pytest.mark.parametrize("use_fp8,round_scale,ue8m0", [(False, False, False), (True, False, False), (True, True, False), (True, True, True)])
@pytest.mark.parametrize("hook", [False, True])
def test_ll_dispatch_combine(R, T, H, E, K, use_fp8, round_scale, ue8m0, hook):
    from deepep_efa_b200.reference import oracle
    vc = _cluster(R, T, H, E)
    try:
        L = E // R
        xs, idxs, ws = [], [], []
        for r in range(R):
            i, w = make_routing(T, E, K, "cuda", seed=20 + r, masked_fraction=0.05)
            idxs.append(i), ws.append(w), xs.append(make_tokens(T, H, "cuda", seed=r))
        for rep in range(3):  # exercises both parities and buffer reuse
            stats = [torch.zeros(L, dtype=torch.int32, device="cuda") for _ in range(R)]
            res = vc.low_latency_dispatch(xs, idxs, T, E, use_fp8=use_fp8, round_scale=round_scale, use_ue8m0=ue8m0,
                                          return_recv_hook=hook, cumulative_stats=stats)
            if hook:
                res[0][4]()
            torch.cuda.synchronize()
            for b in vc.buffers:
                b.check_status()
            ref = oracle.low_latency_dispatch([x.cpu() for x in xs], [i.cpu() for i in idxs], T, E, use_fp8, round_scale, ue8m0)
            ys = []
            for r in range(R):
                rx, cnt, handle, _, _ = res[r]
                o = ref[r]
                assert torch.equal(cnt.cpu(), o["packed_recv_count"]) and torch.equal(stats[r].cpu(), o["packed_recv_count"])
                assert torch.equal(handle[1].cpu(), o["layout_range"])
                assert handle[2:] == (T, H, E)
                for le in range(L):
                    n = int(cnt[le])
                    assert torch.equal(handle[0][le, :n].cpu(), o["src_info"][le, :n])
                    if use_fp8:
                        assert torch.equal(rx[0][le, :n].cpu().view(torch.uint8), o["packed_recv_x"][le, :n].view(torch.uint8))
                        assert torch.equal(rx[1][le, :n].cpu(), o["packed_recv_x_scales"][le, :n])
                    else:
                        assert torch.equal(rx[le, :n].cpu(), o["packed_recv_x"][le, :n])
                if use_fp8:
                    ys.append(oracle.per_token_cast_back(rx[0].view(-1, H).cpu(), rx[1].view(L * R * T, -1).cpu()).view(L, R * T, H).cuda())
                else:
                    ys.append(rx.clone())
            handles = [r[2] for r in res]
            zero_copy = rep == 1
            if zero_copy:
                for r in range(R):
                    vc.buffers[r].get_next_low_latency_combine_buffer(handles[r]).copy_(ys[r])
            comb = vc.low_latency_combine(ys, idxs, ws, handles, zero_copy=zero_copy, return_recv_hook=hook)
            if hook:
                comb[0][2]()
            torch.cuda.synchronize()
            for b in vc.buffers:
                b.check_status()
            for r in range(R):
                want = xs[r].float() * ws[r].masked_fill(idxs[r] == -1, 0).sum(dim=1, keepdim=True)
                out = comb[r][0]
                assert torch.isnan(out.float()).sum().item() == 0
                d = oracle.calc_diff(want, out.float())
                if not round_scale:
                    assert d < (9e-4 if use_fp8 else 1e-5), d
                else:
                    assert d < 5e-3, d
    finally:
        vc.destroy()


def test_ll_masked_rank_is_skipped():
    from deepep_efa_b200.reference import oracle
    R, T, H, E, K = 4, 16, 512, 16, 4
    vc = _cluster(R, T, H, E, enable_shrink=True)
    try:
        xs, idxs, ws = [], [], []
        for r in range(R):
            i, w = make_routing(T, E, K, "cuda", seed=r)
            idxs.append(i), ws.append(w), xs.append(make_tokens(T, H, "cuda", seed=r))
        # rank 2 plays dead: it selects nothing and is cut off from the others in both directions
        idxs[2] = torch.full_like(idxs[2], -1)
        for r, b in enumerate(vc.buffers):
            if r == 2:
                for other in (0, 1, 3):
                    b.low_latency_update_mask_buffer(other, True)
            else:
                b.low_latency_update_mask_buffer(2, True)
        st = torch.zeros(R, dtype=torch.int32, device="cuda")
        vc.buffers[0].low_latency_query_mask_buffer(st)
        assert st.tolist() == [0, 0, 1, 0]
        res = vc.low_latency_dispatch(xs, idxs, T, E, use_fp8=False)
        torch.cuda.synchronize()
        ref = oracle.low_latency_dispatch([x.cpu() for x in xs], [i.cpu() for i in idxs], T, E, False, masked_ranks=(2,))
        for r in (0, 1, 3):
            assert torch.equal(res[r][1].cpu(), ref[r]["packed_recv_count"])
            assert torch.equal(res[r][2][1].cpu(), ref[r]["layout_range"])
        comb = vc.low_latency_combine([r[0].clone() for r in res], idxs, ws, [r[2] for r in res])
        torch.cuda.synchronize()
        L = E // R
        for r in (0, 1, 3):
            keep = (idxs[r] >= 0) & (idxs[r] // L != 2)
            want = xs[r].float() * (ws[r] * keep).sum(dim=1, keepdim=True)
            assert oracle.calc_diff(want, comb[r][0].float()) < 1e-5
        for b in vc.buffers:
            b.low_latency_clean_mask_buffer()
        vc.buffers[0].low_latency_query_mask_buffer(st)
        assert st.tolist() == [0, 0, 0, 0]
    finally:
        vc.destroy()


@pytest.mark.parametrize("R,T,H,E,K,num_sms", [(2, 300, 512, 16, 8, 9), (4, 40, 1024, 32, 6, None), (1, 128, 7168, 16, 8, 24)])
def test_ll_pull_equals_push_host_out_and_sm_knob(R, T, H, E, K, num_sms):
    """The pull form of combine (expert outputs in symmetric memory: zero-copy buffer or arena tensor) gives bit-identical
    results to the staged push form; the result may land in pinned host memory; a bounded grid (several tokens per CTA,
    which exercises the running per-expert slot count of dispatch) changes nothing."""
    from deepep_efa_b200 import Buffer
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    from deepep_efa_b200.reference import oracle
    vc = VirtualCluster(R, num_nvl_bytes=(2 << 20) + 2 * (E // R) * R * T * H * 2,
                        num_rdma_bytes=Buffer.get_low_latency_rdma_size_hint(T, H, R, E), timeout_ms=2000)
    Buffer.set_low_latency_num_sms(num_sms)
    try:
        L = E // R
        xs, idxs, ws = [], [], []
        for r in range(R):
            i, w = make_routing(T, E, K, "cuda", seed=70 + r, masked_fraction=0.1)
            idxs.append(i), ws.append(w), xs.append(make_tokens(T, H, "cuda", seed=40 + r))
        res = vc.low_latency_dispatch(xs, idxs, T, E, use_fp8=False)
        torch.cuda.synchronize()
        ref = oracle.low_latency_dispatch([x.cpu() for x in xs], [i.cpu() for i in idxs], T, E, False)
        for r in range(R):
            assert torch.equal(res[r][1].cpu(), ref[r]["packed_recv_count"])
            for le in range(L):
                n = int(res[r][1][le])
                assert torch.equal(res[r][2][0][le, :n].cpu(), ref[r]["src_info"][le, :n])
                assert torch.equal(res[r][0][le, :n].cpu(), ref[r]["packed_recv_x"][le, :n])
        handles = [r_[2] for r_ in res]
        ys = [(r_[0].float() * 0.5).to(torch.bfloat16) for r_ in res]            # ordinary device tensors -> push
        push = [o[0].clone() for o in vc.low_latency_combine(ys, idxs, ws, handles)]
        sym = []
        for r in range(R):                                                       # arena tensors -> pull + closing barrier
            t = vc.buffers[r].empty_symmetric(list(ys[r].shape), torch.bfloat16)
            t.copy_(ys[r])
            sym.append(t)
        pull = [o[0].clone() for o in vc.low_latency_combine(sym, idxs, ws, handles)]
        for r in range(R):                                                       # zero-copy buffer -> pull, result to host
            vc.buffers[r].get_next_low_latency_combine_buffer(handles[r]).copy_(ys[r])
        host = [torch.zeros(T, H, dtype=torch.bfloat16).pin_memory() for _ in range(R)]
        vc.low_latency_combine(ys, idxs, ws, handles, zero_copy=True, outs=host)
        torch.cuda.synchronize()
        for b in vc.buffers:
            b.check_status()
        for r in range(R):
            want = xs[r].float() * 0.5 * ws[r].masked_fill(idxs[r] == -1, 0).sum(dim=1, keepdim=True)
            assert oracle.calc_diff(want, push[r].float()) < 2e-5
            assert torch.equal(push[r], pull[r])
            assert torch.equal(push[r].cpu(), host[r])
        # activations in pinned host memory: the dispatch kernel reads the rows over PCIe itself, same bits
        first = [((r_[0][0].clone(), r_[0][1].clone()), r_[1].clone(), r_[2][0].clone()) for r_ in vc.low_latency_dispatch(xs, idxs, T, E, use_fp8=True)]
        pinned = [x.cpu().pin_memory() for x in xs]
        again = vc.low_latency_dispatch(pinned, idxs, T, E, use_fp8=True)
        torch.cuda.synchronize()
        for b in vc.buffers:
            b.check_status()
        for r in range(R):
            assert torch.equal(first[r][1], again[r][1])
            for le in range(L):
                n = int(first[r][1][le])
                assert torch.equal(first[r][2][le, :n], again[r][2][0][le, :n])
                assert torch.equal(first[r][0][0][le, :n].view(torch.uint8), again[r][0][0][le, :n].view(torch.uint8))
                assert torch.equal(first[r][0][1][le, :n], again[r][0][1][le, :n])
    finally:
        Buffer.set_low_latency_num_sms(None)
        vc.destroy()
