"""Bookkeeping kernels of the two-level path (csrc/kernels/hier.cu) against their PyTorch restatement on CPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,G,P", [(1, 2, 1), (37, 3, 2), (5000, 8, 8), (1024, 4, 4)])
def test_routing_sort_and_remap(T, G, P):
    from deepep_efa_b200.ops import hier as H
    torch.manual_seed(T)
    member = torch.rand(T, G * P) < (0.5 / P)
    ids_c, counts_c, prefix_c, pos_c = H.routing_sort(member, P)
    ids_g, counts_g, prefix_g, pos_g = H.routing_sort(member.cuda(), P)
    S = int(prefix_c[-1])
    assert torch.equal(counts_g.cpu(), counts_c) and torch.equal(prefix_g.cpu(), prefix_c)
    assert torch.equal(ids_g[:S].cpu(), ids_c[:S]) and torch.equal(pos_g.cpu(), pos_c)
    K, Eg = 6, 5
    topk = torch.randint(-1, G * Eg, (T, K))
    w = torch.rand(T, K)
    pk_c = H.topk_remap_pack(topk, w, ids_c, prefix_c, S, Eg)
    pk_g = H.topk_remap_pack(topk.cuda(), w.cuda(), ids_g, prefix_g, S, Eg)
    assert torch.equal(pk_g.cpu(), pk_c)
    pk_n = H.topk_remap_pack(topk.cuda(), None, ids_g, prefix_g, S, Eg)
    assert torch.equal(H.unpack_topk(pk_n.cpu(), K)[0], H.unpack_topk(pk_c, K)[0]) and (H.unpack_topk(pk_n.cpu(), K)[1] == 0).all()
    local = torch.rand(S, P) < 0.5
    assert torch.equal(H.recv_src_meta(prefix_g, local.cuda(), S).cpu(), H.recv_src_meta(prefix_c, local, S))
    assert torch.equal(H.recv_src_meta(prefix_g, None, S).cpu()[:, 0], H.recv_src_meta(prefix_c, None, S)[:, 0])


@pytest.mark.parametrize("T,E,R,P", [(300, 64, 16, 8), (4096, 256, 32, 8), (7, 8, 4, 2), (0, 16, 16, 4)])
def test_layout_with_domains(T, E, R, P):
    from deepep_efa_b200.ops import hier as H
    from helpers import make_routing
    idx, _ = make_routing(max(T, 1), E, 4, "cpu", seed=T + R, masked_fraction=0.1)
    idx = idx[:T]
    want = H.layout_hier(idx, E, R, P)
    got = H.layout_hier(idx.cuda(), E, R, P)
    for a, b in zip(got, want):
        assert torch.equal(a.cpu(), b)


def test_segmented_copy():
    from deepep_efa_b200.ops import hier as H
    torch.manual_seed(3)
    src = torch.randint(0, 255, (1 << 20,), dtype=torch.uint8)
    # short and empty segments, an unaligned one, and two that span several 32 KiB chunks (one aligned, one not, ragged tails)
    segs = torch.tensor([[0, 16, 4096], [5000, 9001, 333], [8192, 32768, 16384], [7, 60000, 1], [100, 61000, 0],
                         [65536, 131072, 200000 + 48], [300001, 400003, 100001]])
    want = torch.zeros(1 << 20, dtype=torch.uint8)
    H.segmented_copy(src, want, segs)
    got = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    H.segmented_copy(src.cuda(), got, segs.cuda())
    assert torch.equal(got.cpu(), want)
