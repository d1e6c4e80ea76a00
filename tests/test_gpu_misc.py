"""FP8 cast kernel, bounded waits, buffer housekeeping."""
import pytest
import torch

from helpers import make_tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("H", [128, 512, 7168])
@pytest.mark.parametrize("round_scale,ue8m0", [(False, False), (True, False), (True, True)])
def test_fp8_cast_kernel(H, round_scale, ue8m0):
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.reference import oracle
    if ue8m0 and H % 512:
        pytest.skip("UE8M0 packs four scales per word")
    C = _ext.load()
    x = make_tokens(77, H, "cuda", seed=1) * 3
    x[0] = 0  # amax floor path
    q, s = C.per_token_cast_to_fp8(x, round_scale, ue8m0)
    qr, sr = oracle.per_token_cast_to_fp8(x.cpu(), round_scale, ue8m0)
    assert torch.equal(s.cpu(), sr)
    assert torch.equal(q.cpu().view(torch.uint8), qr.view(torch.uint8))
    back = oracle.per_token_cast_back(q.cpu(), s.cpu())
    assert oracle.calc_diff(x.float().cpu(), back.float()) < 2e-3


def test_timed_out_wait_reports_status_and_context_survives():
    """A wait on a flag nothing sets must end by itself, set the status word, and leave the context usable."""
    from deepep_efa_b200 import EPTimeoutError
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    vc = VirtualCluster(1, num_nvl_bytes=8 << 20, timeout_ms=50)
    try:
        b = vc.buffers[0]
        b.check_status(sync=True)
        b._timeout_probe()
        with pytest.raises(EPTimeoutError) as ei:
            b.check_status(sync=True)
        assert "timeout probe" in str(ei.value)
        # the context still works and the buffer recovers
        b.recover()
        b.check_status(sync=True)
        t = torch.ones(4, device="cuda") * 2
        assert t.sum().item() == 8
    finally:
        vc.destroy()


def test_debug_range_check_turns_a_bad_row_into_a_status():
    """With the debug range checks on, a cached handle whose send position points far outside the symmetric buffer
    makes the kernel skip that row and report a status code; everything else of the call still happens."""
    from deepep_efa_b200 import EPTimeoutError
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    from helpers import make_routing, make_tokens
    vc = VirtualCluster(1, num_nvl_bytes=32 << 20)
    try:
        b = vc.buffers[0]
        b.runtime.set_debug_checks(True)
        T, H, E, K = 64, 512, 8, 2
        x = make_tokens(T, H, "cuda", seed=1)
        idx, w = make_routing(T, E, K, "cuda", seed=1)
        per_rank, _, per_expert, in_rank, _ = b.get_dispatch_layout(idx, E)
        recv_x, _, _, _, handle, _ = b.dispatch(x, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank,
                                                num_tokens_per_expert=per_expert, topk_idx=idx, topk_weights=w)
        b.check_status(sync=True)  # the checks do not fire on a healthy call
        assert torch.equal(recv_x, x)
        # The checked extent is made smaller than the real allocation and the bad row lies between the two: if the check
        # ever regressed, the stray store would land in this rank's own (free) arena memory instead of somewhere wild.
        b.runtime.set_debug_extent(4 << 20)
        bad_head = handle[5].clone()
        bad_head[5, 0] = 8192  # 8 MiB past recv_x with 1 KiB rows: outside the 4 MiB extent, inside the 32 MiB buffer
        bad = handle[:5] + (bad_head,)
        rx2, *_ = b.dispatch(x, handle=bad)
        with pytest.raises(EPTimeoutError) as ei:
            b.check_status(sync=True)
        assert "bounds check" in str(ei.value)
        keep = torch.arange(T, device="cuda") != 5
        assert torch.equal(rx2[keep], x[keep])
        b.recover()
        b.runtime.set_debug_extent(0)
        rx3, *_ = b.dispatch(x, handle=handle)
        b.check_status(sync=True)
        assert torch.equal(rx3, x)
    finally:
        vc.destroy()


def test_symmetric_alloc_and_views():
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    vc = VirtualCluster(1, num_nvl_bytes=16 << 20)
    try:
        b = vc.buffers[0]
        t = b.empty_symmetric([128, 64], torch.bfloat16)
        assert b.runtime.symmetric_offset(t) >= 0 and t.shape == (128, 64)
        t.fill_(3)
        assert t.float().sum().item() == 3 * 128 * 64
        used = b.runtime.arena_in_use()
        del t
        torch.cuda.synchronize()
        u = b.empty_symmetric([16], torch.int32)  # triggers reclamation of finished blocks
        assert b.runtime.arena_in_use() <= used
        raw = b.get_local_buffer_tensor(torch.int32)
        assert raw.numel() > 0
        with pytest.raises(RuntimeError):
            b.empty_symmetric([1 << 30], torch.float32)
    finally:
        vc.destroy()
