"""Single-process checks of the pure-PyTorch semantics (no GPU, no process group)."""
import torch

from deepep_efa_b200.reference import oracle
from helpers import make_routing, make_tokens


def test_fp8_roundtrip_and_formats():
    x = make_tokens(16, 512, "cpu")
    q, s = oracle.per_token_cast_to_fp8(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (16, 4) and s.dtype == torch.float32
    back = oracle.per_token_cast_back(q, s)
    assert oracle.calc_diff(x, back) < 1e-3
    q2, s2 = oracle.per_token_cast_to_fp8(x, round_scale=True, use_ue8m0=True)
    assert s2.dtype == torch.int32 and s2.shape == (16, 1)
    back2 = oracle.per_token_cast_back(q2, s2)
    assert oracle.calc_diff(x, back2) < 2e-3
    # power-of-two scales are >= the exact ones
    _, s3 = oracle.per_token_cast_to_fp8(x, round_scale=True)
    assert torch.all(s3 >= s - 1e-12) and torch.all(torch.log2(s3) == torch.log2(s3).round())


def test_layout_counts_bruteforce():
    E, R, K, T = 64, 4, 8, 100
    idx, _ = make_routing(T, E, K, "cpu", seed=3, masked_fraction=0.1)
    per_rank, per_expert, in_rank = oracle.get_dispatch_layout(idx, E, R)
    for e in range(E):
        assert per_expert[e].item() == (idx == e).sum().item()
    for r in range(R):
        hit = ((idx >= r * 16) & (idx < (r + 1) * 16)).any(dim=1)
        assert torch.equal(hit, in_rank[:, r]) and per_rank[r].item() == hit.sum().item()


def test_dispatch_combine_identity():
    E, R, K, T, H = 32, 4, 4, 50, 256
    xs, idxs, ws = [], [], []
    for r in range(R):
        i, w = make_routing(T, E, K, "cpu", seed=r)
        idxs.append(i), ws.append(w), xs.append(make_tokens(T, H, "cpu", seed=r))
    outs = oracle.dispatch(xs, idxs, ws, E)
    # every received row is the source row, local ids are in range, per-expert counts add up
    for d, o in enumerate(outs):
        rpm = o["rank_prefix_matrix"]
        start = 0
        for s in range(R):
            end = int(rpm[s, d])
            src = o["recv_src_idx"][start:end].long()
            assert torch.equal(o["recv_x"][start:end], xs[s][src])
            start = end
        li = o["recv_topk_idx"]
        assert ((li == -1) | ((li >= 0) & (li < E // R))).all()
        for e in range(E // R):
            assert o["num_recv_tokens_per_expert_list"][e] == sum(int((idxs[s] == d * (E // R) + e).sum()) for s in range(R))
    comb, comb_w = oracle.combine([o["recv_x"] for o in outs], [o["send_head"] for o in outs], outs[0]["rank_prefix_matrix"],
                                  topk_weights=[o["recv_topk_weights"] for o in outs])
    for r in range(R):
        hits = outs[r]["is_token_in_rank"].sum(dim=1, keepdim=True).float()
        assert oracle.calc_diff(comb[r].float(), xs[r].float() * hits) < 5e-6
        assert (comb_w[r] - ws[r]).abs().max() < 1e-6


def test_low_latency_roundtrip():
    E, R, K, T, H = 16, 2, 4, 12, 512
    xs, idxs, ws = [], [], []
    for r in range(R):
        i, w = make_routing(T, E, K, "cpu", seed=10 + r, masked_fraction=0.05)
        idxs.append(i), ws.append(w), xs.append(make_tokens(T, H, "cpu", seed=r))
    for use_fp8 in (False, True):
        outs = oracle.low_latency_dispatch(xs, idxs, T, E, use_fp8=use_fp8)
        ys = []
        for o in outs:
            if use_fp8:
                L, N, _ = o["packed_recv_x"].shape
                ys.append(oracle.per_token_cast_back(o["packed_recv_x"].view(-1, H), o["packed_recv_x_scales"].view(-1, H // 128)).view(L, N, H))
            else:
                ys.append(o["packed_recv_x"])
        for d, o in enumerate(outs):
            for le in range(E // R):
                assert o["packed_recv_count"][le].item() == sum(int((idxs[s] == d * (E // R) + le).sum()) for s in range(R))
                assert int((o["layout_range"][le] & 0xFFFFFFFF).sum()) == o["packed_recv_count"][le].item()
        comb = oracle.low_latency_combine(ys, idxs, ws, [o["src_info"] for o in outs], [o["layout_range"] for o in outs], E)
        for r in range(R):
            ref = xs[r].float() * ws[r].masked_fill(idxs[r] == -1, 0).sum(dim=1, keepdim=True)
            assert oracle.calc_diff(ref, comb[r].float()) < (9e-4 if use_fp8 else 1e-5)
