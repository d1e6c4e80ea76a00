"""Normal-mode kernels against the pure-PyTorch oracle. R > 1 runs all ranks on one GPU as one cooperative
launch (deepep_efa_b200.parallel.virtual); the kernels are the ones a real multi-GPU job runs.

Mirrors the checks of the reference's tests/test_intranode.py: layout vs brute force (:40-66), payload per
source-rank segment (:80-86), local expert id range and per-expert counts (:127-131), num_worst_tokens
(:141-154), cached handle (:157-165), combine round trip (:168-183)."""
import pytest
import torch

from helpers import make_routing, make_tokens

pytestmark = pytest.mark.gpu


def _cluster(R, nvl=256 << 20, ll=0, **kw):
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    return VirtualCluster(R, num_nvl_bytes=nvl, num_rdma_bytes=ll, timeout_ms=2000, **kw)


def _inputs(R, T, H, E, K, masked=0.0, seed=0):
    xs, idxs, ws = [], [], []
    for r in range(R):
        i, w = make_routing(T, E, K, "cuda", seed=seed + r, masked_fraction=masked)
        idxs.append(i), ws.append(w), xs.append(make_tokens(T, H, "cuda", seed=seed + r))
    return xs, idxs, ws


@pytest.mark.parametrize("R", [1, 2, 4, 8])
def test_layout_matches_oracle(R):
    from deepep_efa_b200.reference import oracle
    vc = _cluster(R)
    try:
        E, K, T = 8 * R, 4, 333
        _, idxs, _ = _inputs(R, T, 128, E, K, masked=0.1)
        lay = vc.get_dispatch_layout(idxs, E)
        for r in range(R):
            per_rank, none, per_expert, in_rank, _ = lay[r]
            a, b, c = oracle.get_dispatch_layout(idxs[r].cpu(), E, R)
            assert none is None
            assert torch.equal(per_rank.cpu(), a) and torch.equal(per_expert.cpu(), b) and torch.equal(in_rank.cpu(), c)
        # a second call reuses the scratch (ticket must have been reset)
        lay2 = vc.get_dispatch_layout(idxs, E)
        assert torch.equal(lay2[0][2], lay[0][2])
    finally:
        vc.destroy()


@pytest.mark.parametrize("R,T,H", [(1, 200, 1024), (2, 257, 7168), (4, 96, 2048), (8, 130, 1024)])
@pytest.mark.parametrize("mode", ["bf16", "fp8_pair", "fp8_fused"])
def test_dispatch_combine_vs_oracle(R, T, H, mode):
    from deepep_efa_b200.reference import oracle
    vc = _cluster(R)
    try:
        E, K = 4 * R, min(4, 4 * R)
        xs, idxs, ws = _inputs(R, T, H, E, K, masked=0.05, seed=7)
        lay = vc.get_dispatch_layout(idxs, E)
        if mode == "fp8_pair":
            pairs = [oracle.per_token_cast_to_fp8(x.cpu()) for x in xs]
            send = [(q.cuda(), s.cuda()) for q, s in pairs]
        else:
            send = xs
        res = vc.dispatch(send, layouts=lay, topk_idxs=idxs, topk_weights=ws, expert_alignment=4,
                          quantize_fp8=(mode == "fp8_fused"))
        torch.cuda.synchronize()
        for b in vc.buffers:
            b.check_status()
        if mode == "bf16":
            ref = oracle.dispatch([x.cpu() for x in xs], [i.cpu() for i in idxs], [w.cpu() for w in ws], E, expert_alignment=4)
        else:
            pairs = [oracle.per_token_cast_to_fp8(x.cpu()) for x in xs]
            ref = oracle.dispatch([p[0] for p in pairs], [i.cpu() for i in idxs], [w.cpu() for w in ws], E,
                                  x_scales=[p[1] for p in pairs], expert_alignment=4)
        for r in range(R):
            recv_x, recv_idx, recv_w, per_expert, handle, _ = res[r]
            o = ref[r]
            if mode == "bf16":
                assert torch.equal(recv_x.cpu(), o["recv_x"])
            else:
                q, s = recv_x
                assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float32
                assert torch.equal(s.cpu(), o["recv_x_scales"]), (s.cpu() - o["recv_x_scales"]).abs().max()
                assert torch.equal(q.cpu().view(torch.uint8), o["recv_x"].view(torch.uint8))
            assert torch.equal(recv_idx.cpu(), o["recv_topk_idx"])
            assert torch.equal(recv_w.cpu(), o["recv_topk_weights"])
            assert per_expert == o["num_recv_tokens_per_expert_list"]
            assert torch.equal(handle[0].cpu(), o["rank_prefix_matrix"])
            assert torch.equal(handle[3].cpu(), o["recv_src_idx"])
            assert torch.equal(handle[5].cpu(), o["send_head"])
            # channel prefix matrices: last column = tokens per destination / per source
            assert torch.equal(handle[1][:, -1].cpu(), o["send_head"].ge(0).sum(0).to(torch.int32))
            col = o["rank_prefix_matrix"][:, r]
            assert torch.equal(handle[2][:, -1].cpu(), col - torch.cat([col.new_zeros(1), col[:-1]]))
        # combine: the "expert" returns what it received (bf16), combine sums over the ranks hit
        if mode == "bf16":
            ys = [res[r][0] for r in range(R)]
        else:
            ys = [oracle.per_token_cast_back(res[r][0][0].cpu(), res[r][0][1].cpu()).cuda() for r in range(R)]
        handles = [res[r][4] for r in range(R)]
        bias = [(make_tokens(T, H, "cuda", seed=90 + r), None) for r in range(R)]
        comb = vc.combine(ys, handles, topk_weights=[res[r][2] for r in range(R)], biases=bias)
        torch.cuda.synchronize()
        for b in vc.buffers:
            b.check_status()
        ref_c, ref_w = oracle.combine([y.cpu() for y in ys], [o["send_head"] for o in ref], ref[0]["rank_prefix_matrix"],
                                      topk_weights=[o["recv_topk_weights"] for o in ref],
                                      biases=[(b[0].cpu(), None) for b in bias])
        for r in range(R):
            out, out_w, _ = comb[r]
            assert oracle.calc_diff(out.float().cpu(), ref_c[r].float()) < 5e-6
            assert (out_w.cpu() - ref_w[r]).abs().max() < 1e-6
            hits = res[r][4][4].sum(dim=1, keepdim=True)
            assert (out_w.cpu() - ws[r].cpu().masked_fill(idxs[r].cpu() == -1, 0)).abs().max() < 1e-6
    finally:
        vc.destroy()


@pytest.mark.parametrize("R", [2, 8])
def test_cached_handle_and_worst_tokens(R):
    from deepep_efa_b200.reference import oracle
    vc = _cluster(R)
    try:
        T, H, E, K = 120, 1024, 4 * R, 4
        xs, idxs, ws = _inputs(R, T, H, E, K, seed=3)
        lay = vc.get_dispatch_layout(idxs, E)
        res = vc.dispatch(xs, layouts=lay, topk_idxs=idxs, topk_weights=ws)
        handles = [r[4] for r in res]
        # cached: only x travels, same rows
        xs2 = [make_tokens(T, H, "cuda", seed=50 + r) for r in range(R)]
        res2 = vc.dispatch(xs2, handles=handles)
        ref2 = oracle.dispatch([x.cpu() for x in xs2], [i.cpu() for i in idxs], [w.cpu() for w in ws], E)
        for r in range(R):
            rx, a, b, c, d, _ = res2[r]
            assert a is None and b is None and c is None and d is None
            assert torch.equal(rx.cpu(), ref2[r]["recv_x"])
        # worst-case sizing: no host sync, -1 tail
        worst = T * R
        res3 = vc.dispatch(xs, layouts=lay, topk_idxs=idxs, topk_weights=ws, num_worst_tokens=worst)
        torch.cuda.synchronize()
        for r in range(R):
            rx, ridx, rw, per_expert, h, _ = res3[r]
            n = res[r][0].size(0)
            assert rx.size(0) == worst and per_expert == []
            assert torch.equal(rx[:n], res[r][0]) and torch.equal(ridx[:n], res[r][1])
            assert (ridx[n:] == -1).all()
        # combine through a cached-handle result (the backward of dispatch)
        comb = vc.combine([r[0] for r in res2], handles)
        ref_c, _ = oracle.combine([o["recv_x"] for o in ref2], [o["send_head"] for o in ref2], ref2[0]["rank_prefix_matrix"])
        for r in range(R):
            assert oracle.calc_diff(comb[r][0].float().cpu(), ref_c[r].float()) < 5e-6
        for b in vc.buffers:
            b.check_status(sync=True)
    finally:
        vc.destroy()


def test_combine_stages_non_symmetric_input():
    from deepep_efa_b200.reference import oracle
    R = 4
    vc = _cluster(R)
    try:
        T, H, E, K = 64, 512, 16, 4
        xs, idxs, ws = _inputs(R, T, H, E, K, seed=11)
        lay = vc.get_dispatch_layout(idxs, E)
        res = vc.dispatch(xs, layouts=lay, topk_idxs=idxs, topk_weights=ws)
        ys = [(r[0].float() * 2).to(torch.bfloat16) for r in res]  # ordinary torch tensors, not in the arena
        assert all(vc.buffers[r].runtime.symmetric_offset(ys[r]) < 0 for r in range(R))
        comb = vc.combine(ys, [r[4] for r in res])
        for r in range(R):
            hits = res[r][4][4].sum(dim=1, keepdim=True).float()
            assert oracle.calc_diff(comb[r][0].float(), xs[r].float() * 2 * hits) < 5e-6
    finally:
        vc.destroy()


def test_repeated_runs_hash_identical():
    from deepep_efa_b200.reference import oracle
    R = 4
    vc = _cluster(R)
    try:
        T, H, E, K = 100, 1024, 16, 4
        xs, idxs, ws = _inputs(R, T, H, E, K, seed=5)
        ref_hash = None
        for _ in range(5):
            lay = vc.get_dispatch_layout(idxs, E)
            res = vc.dispatch(xs, layouts=lay, topk_idxs=idxs, topk_weights=ws, quantize_fp8=True)
            comb = vc.combine([oracle.per_token_cast_back(r[0][0].cpu(), r[0][1].cpu()).cuda() for r in res], [r[4] for r in res])
            h = 0
            for r in range(R):
                h ^= oracle.hash_tensor(res[r][0][0]) ^ oracle.hash_tensor(res[r][0][1]) ^ oracle.hash_tensor(comb[r][0])
            assert ref_hash is None or h == ref_hash
            ref_hash = h
    finally:
        vc.destroy()


def test_arena_memory_returns():
    vc = _cluster(2, nvl=64 << 20)
    try:
        T, H, E, K = 256, 2048, 8, 4
        xs, idxs, ws = _inputs(2, T, H, E, K)
        for _ in range(40):  # would exhaust 64 MiB many times over if blocks never came back
            lay = vc.get_dispatch_layout(idxs, E)
            res = vc.dispatch(xs, layouts=lay, topk_idxs=idxs, topk_weights=ws)
            del res
        torch.cuda.synchronize()
        assert vc.buffers[0].runtime.arena_in_use() <= vc.buffers[0].runtime.arena_capacity()
    finally:
        vc.destroy()


def test_handle_validation_catches_foreign_and_corrupt_handles():
    from deepep_efa_b200.buffer import validate_handle
    R = 4
    vc = _cluster(R)
    try:
        T, H, E, K = 64, 512, 16, 4
        xs, idxs, ws = _inputs(R, T, H, E, K, seed=2)
        lay = vc.get_dispatch_layout(idxs, E)
        res = vc.dispatch(xs, layouts=lay, topk_idxs=idxs, topk_weights=ws)
        for r in range(R):
            validate_handle(res[r][4], r, R)
        with pytest.raises(AssertionError):
            validate_handle(res[1][4], 2, R)  # another rank's handle
        h = list(res[0][4])
        bad = h[5].clone()
        bad[bad >= 0] += 1  # positions no longer start at zero
        h[5] = bad
        with pytest.raises(AssertionError):
            validate_handle(tuple(h), 0, R)
    finally:
        vc.destroy()
