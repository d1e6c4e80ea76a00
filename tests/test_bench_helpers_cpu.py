"""Host-side helpers of bench.py that run before any GPU work: GPU index mapping and CPU pinning (against a fake NVML)."""
import os
import sys
import types

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_physical_gpu_index_follows_cuda_visible_devices(monkeypatch):
    import bench
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    assert bench.physical_gpu_index(3) == 3
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "4,6,7")
    assert bench.physical_gpu_index(1) == 6
    assert bench.physical_gpu_index(5) == 5          # out of range: falls back to the local rank
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "GPU-abc,GPU-def")
    assert bench.physical_gpu_index(1) == 1          # UUIDs: falls back to the local rank


def test_bind_to_gpu_local_cpus_uses_nvml_mask_and_respects_the_cpuset(monkeypatch):
    import bench
    allowed = sorted(os.sched_getaffinity(0))
    if len(allowed) < 2:
        pytest.skip("needs at least two CPUs in the cpuset")
    want = set(allowed[:2])
    words = [0] * ((max(allowed) // 64) + 1)
    for c in want | {4095}:                          # a CPU outside the cpuset must be dropped
        if c // 64 < len(words):
            words[c // 64] |= 1 << (c % 64)
    seen = {}
    fake = types.SimpleNamespace(
        nvmlInit=lambda: None,
        nvmlDeviceGetHandleByIndex=lambda i: seen.setdefault("index", i) or "h",
        nvmlDeviceGetCpuAffinity=lambda h, n: words + [0] * max(0, n - len(words)))
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "2,5")
    before = os.sched_getaffinity(0)
    try:
        n = bench.bind_to_gpu_local_cpus(1)
        assert n == len(want) and os.sched_getaffinity(0) == want
        assert seen["index"] == 5                    # NVML is asked about the physical GPU of this local rank
    finally:
        os.sched_setaffinity(0, before)


def test_bind_to_gpu_local_cpus_is_best_effort(monkeypatch):
    import bench
    before = os.sched_getaffinity(0)

    def boom():
        raise RuntimeError("no NVML here")
    monkeypatch.setitem(sys.modules, "pynvml", types.SimpleNamespace(nvmlInit=boom))
    assert bench.bind_to_gpu_local_cpus(0) is None and os.sched_getaffinity(0) == before
    # a mask that shares no CPU with the cpuset changes nothing either
    fake = types.SimpleNamespace(nvmlInit=lambda: None, nvmlDeviceGetHandleByIndex=lambda i: "h",
                                 nvmlDeviceGetCpuAffinity=lambda h, n: [0] * n)
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    assert bench.bind_to_gpu_local_cpus(0) is None and os.sched_getaffinity(0) == before
