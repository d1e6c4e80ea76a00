"""Failure detection without touching a GPU: a rank that never joins a collective, a fake NVML that reports a missing
NVLink, and the rate-limited logger. (Device-side bounded waits are tested on the GPU in test_gpu_misc.py with a flag
that nothing sets.)"""
import datetime
import logging
import os
import socket
import types

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_fn(rank, world, port, q):
    import traceback
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
        import deepep_efa_b200 as ep
        from helpers import make_routing, make_tokens
        buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=1 << 20)
        x = make_tokens(16, 128, "cpu", seed=rank)
        idx, w = make_routing(16, 8, 2, "cpu", seed=rank)
        per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(idx, 8)
        if rank == 1:
            # this rank "fails" between steps: it simply never calls dispatch and leaves
            q.put((rank, "left"))
            return
        try:
            buf.dispatch(x, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert,
                         topk_idx=idx, topk_weights=w)
            q.put((rank, "dispatch returned although a peer never joined"))
        except Exception as e:  # the process-group timeout ends the collective with an error
            q.put((rank, "detected:" + type(e).__name__))
    except Exception:
        q.put((rank, traceback.format_exc()))


def test_rank_that_never_joins_is_detected_by_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_fn, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(30)
        if p.is_alive():
            p.terminate()
    assert res[1] == "left"
    assert res[0].startswith("detected:"), res[0]


def _fake_nvml(ok_pairs):
    m = types.SimpleNamespace()
    m.NVML_P2P_CAPS_INDEX_NVLINK, m.NVML_P2P_STATUS_OK = 1, 0
    m.calls = []
    m.nvmlInit = lambda: m.calls.append("init")
    m.nvmlShutdown = lambda: m.calls.append("shutdown")
    m.nvmlDeviceGetHandleByIndex = lambda i: i
    m.nvmlDeviceGetP2PStatus = lambda a, b, idx: 0 if (a, b) in ok_pairs or (b, a) in ok_pairs else 5
    return m


def test_nvlink_pair_check_with_fake_nvml():
    from deepep_efa_b200.utils.nvlink import check_pairs
    good = _fake_nvml({(0, 1)})
    check_pairs([0, 1], good)
    assert good.calls == ["init", "shutdown"]
    bad = _fake_nvml(set())
    with pytest.raises(AssertionError, match="not connected via NVLink"):
        check_pairs([0, 1], bad)
    assert bad.calls[-1] == "shutdown"  # NVML is shut down on the error path too


def test_logger_prefix_and_rate_limit(caplog):
    from deepep_efa_b200.utils.logging import get_logger, log
    lg = get_logger()
    lg.propagate = True
    try:
        with caplog.at_level(logging.WARNING, logger="deep_ep"):
            assert log(logging.WARNING, 3, "peer slow", key="k1", min_interval_s=60)
            assert not log(logging.WARNING, 3, "peer slow", key="k1", min_interval_s=60)
            assert log(logging.WARNING, 3, "other", key="k2", min_interval_s=60)
        msgs = list(dict.fromkeys(r.getMessage() for r in caplog.records))  # a record may be seen by more than one handler
        assert msgs == ["[r3] peer slow", "[r3] other"]
    finally:
        lg.propagate = False


def test_phase_profiler_accumulates_without_cuda():
    from deepep_efa_b200.utils.profiler import PhaseProfiler
    p = PhaseProfiler("T", 0, interval=2, warmup=0)
    for _ in range(3):
        p.mark("a")
        p.mark("b")
        p.finish_iter()
    assert p.iters == 3  # without CUDA no events are recorded, but the bookkeeping must not fail


def test_transport_stubs_and_domain_limits():
    """The libfabric/EFA transport is a declared stub; a single-domain buffer refuses the cross-domain entry points."""
    import deepep_efa_b200 as ep
    from deepep_efa_b200.parallel.transport import EfaTransport
    with pytest.raises(NotImplementedError, match="libfabric"):
        EfaTransport()
    fake_group = types.SimpleNamespace(rank=lambda: 0, size=lambda: 16)
    with pytest.raises(AssertionError, match="at most 8"):
        ep.Buffer(fake_group, num_nvl_ranks=16)
    assert ep.Buffer.get_dispatch_config(16) is not None and ep.Buffer.get_combine_config(64) is not None


def test_clock_sampler_reads_a_fake_nvml(monkeypatch):
    """The benchmark's clock record comes from NVML reads only; a fake NVML shows median, maximum and reasons."""
    import sys
    import time
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.calls = []
    fake.nvmlInit = lambda: fake.calls.append("init")
    fake.nvmlShutdown = lambda: fake.calls.append("shutdown")
    fake.nvmlDeviceGetCount = lambda: 8
    fake.nvmlDeviceGetHandleByIndex = lambda i: i
    fake.nvmlDeviceGetClockInfo = lambda h, k: 1900 + h
    fake.nvmlDeviceGetMaxClockInfo = lambda h, k: 1965
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0x4 if h == 3 else 0
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    s = bench.ClockSampler(period_ms=5, gpus={0, 3})
    s.start()
    time.sleep(0.05)
    rec = s.stop()
    assert rec["samples"] >= 4 and rec["sm_max_mhz"] == 1965 and 1900 <= rec["sm_mhz"] <= 1903
    assert rec["reasons"] == ["sw_power_cap"]
    assert fake.calls == ["init", "shutdown"]  # nothing but reads in between
