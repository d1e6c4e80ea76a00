"""Public-API behaviour on one real rank (R = 1 goes through the same peer-store kernels with itself as the peer):
stream/event contract (previous_event x async_finish x allocate_on_comm_stream, as swept by the reference's
tests/test_intranode.py:88-91), CUDA-graph capture of the low-latency pair, int32 expert ids, accessors, stress hash."""
import pytest
import torch

from helpers import make_routing, make_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture()
def buf():
    import deepep_efa_b200 as ep
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    T, H, E = 128, 1024, 16
    vc = VirtualCluster(1, num_nvl_bytes=64 << 20, num_rdma_bytes=ep.Buffer.get_low_latency_rdma_size_hint(T, H, 1, E))
    yield vc.buffers[0]
    vc.destroy()


@pytest.mark.parametrize("use_prev", [False, True])
@pytest.mark.parametrize("async_finish", [False, True])
def test_stream_event_contract(buf, use_prev, async_finish):
    from deepep_efa_b200 import Buffer
    from deepep_efa_b200.reference import oracle
    T, H, E, K = 128, 1024, 16, 4
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        x = make_tokens(T, H, "cuda", seed=1)
        idx, w = make_routing(T, E, K, "cuda", seed=1)
        prev = Buffer.capture() if use_prev else None
        alloc_on_comm = use_prev and async_finish
        per_rank, _, per_expert, in_rank, ev = buf.get_dispatch_layout(idx, E, previous_event=prev, async_finish=async_finish,
                                                                        allocate_on_comm_stream=alloc_on_comm)
        ev.current_stream_wait()
        recv_x, recv_idx, recv_w, counts, handle, ev = buf.dispatch(
            x, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert, topk_idx=idx, topk_weights=w,
            previous_event=Buffer.capture() if use_prev else None, async_finish=async_finish, allocate_on_comm_stream=alloc_on_comm)
        with ev:  # the context manager waits on exit; work issued inside overlaps the communication
            filler = torch.ones(1024, device="cuda").sum()
        out, out_w, ev = buf.combine(recv_x, handle, topk_weights=recv_w, previous_event=Buffer.capture() if use_prev else None,
                                     async_finish=async_finish, allocate_on_comm_stream=alloc_on_comm)
        ev.current_stream_wait()
    side.synchronize()
    buf.check_status()
    assert filler.item() == 1024
    assert sum(counts) == int((idx >= 0).sum())
    assert oracle.calc_diff(out.float(), x.float()) < 5e-6  # one rank: every token comes back once
    assert (out_w - w).abs().max() < 1e-6
    if not (use_prev and async_finish):
        with pytest.raises(AssertionError):
            buf.get_dispatch_layout(idx, E, allocate_on_comm_stream=True)


def test_low_latency_pair_in_a_cuda_graph(buf):
    """No per-call value travels in the launch arguments (sequence numbers live on the device), so a captured
    dispatch + combine can be replayed."""
    from deepep_efa_b200.reference import oracle
    T, H, E, K = 128, 1024, 16, 4
    x = make_tokens(T, H, "cuda", seed=2)
    idx, w = make_routing(T, E, K, "cuda", seed=2, masked_fraction=0.05)
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        def step():
            rx, cnt, h, _, _ = buf.low_latency_dispatch(x, idx, T, E, use_fp8=False)
            buf.low_latency_combine(rx, idx, w, h, out=out)
        step()
        step()  # both parities seen before capture
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            step()
            step()
    torch.cuda.current_stream().wait_stream(s)
    want = x.float() * w.masked_fill(idx == -1, 0).sum(dim=1, keepdim=True)
    for _ in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        buf.check_status()
        assert oracle.calc_diff(want, out.float()) < 1e-5


def test_int32_expert_ids_and_accessors(buf):
    T, E, K = 64, 16, 4
    idx, _ = make_routing(T, E, K, "cuda", seed=3)
    a = buf.get_dispatch_layout(idx, E)
    b = buf.get_dispatch_layout(idx.to(torch.int32), E)
    assert torch.equal(a[0], b[0]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])
    assert buf.is_available() and buf.get_num_rdma_ranks() == 1 and buf.get_rdma_rank() == 0
    assert buf.get_local_device_id() == torch.cuda.current_device()
    assert len(buf.get_local_ipc_handle()) == 64
    assert buf.get_comm_stream() is buf.comm_stream
    with pytest.raises(NotImplementedError):  # a single NVLink domain has no cross-domain path
        buf.internode_dispatch(torch.empty(0))
    with pytest.raises(NotImplementedError):
        buf.internode_combine(torch.empty(0), ())


def test_low_latency_repeated_runs_hash_identical(buf):
    """Stress in the spirit of the reference's --pressure-test (tests/test_low_latency.py:305-329): identical inputs give
    byte-identical outputs over many repeats, across both buffer parities."""
    from deepep_efa_b200.reference import oracle
    T, H, E, K = 128, 1024, 16, 4
    x = make_tokens(T, H, "cuda", seed=4)
    idx, w = make_routing(T, E, K, "cuda", seed=4, masked_fraction=0.05)
    ref = None
    for _ in range(20):
        (px, ps), cnt, h, _, _ = buf.low_latency_dispatch(x, idx, T, E, use_fp8=True)
        sim = oracle.per_token_cast_back(px.view(-1, H), ps.view(-1, H // 128)).view(px.shape)
        out, _, _ = buf.low_latency_combine(sim, idx, w, h)
        hv = oracle.hash_tensor(out) ^ oracle.hash_tensor(cnt)
        for le in range(E):
            n = int(cnt[le])
            hv ^= oracle.hash_tensor(px[le, :n]) ^ oracle.hash_tensor(ps[le, :n])
        assert ref is None or hv == ref
        ref = hv
    buf.check_status(sync=True)
