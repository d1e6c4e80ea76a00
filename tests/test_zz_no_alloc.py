"""The allocation-free layout entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory at the point where they need a dispatch layout
(a plugin that only received raw pointers, a serving loop that bans cudaMalloc after start-up). For them the
library exports ``dx_get_dispatch_layout_noalloc``, which writes into caller-owned buffers and keeps its
scratch in a fixed array inside the library. This test calls it with ctypes, twice in a row on different
problems (the second reuses the scratch the first one dirtied), and compares every output exactly with the
regular allocating entry point. It lives in a file that pytest collects last so that a failure here cannot
hide the results of the other tests in a stop-at-first-failure run; it passes both alone in a fresh process
and after all other tests.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from deepep_efa_b200 import _ext
    _ext.load()  # makes sure the in-tree library is built and libtorch is loaded before dlopen
    lib = ctypes.CDLL(str(_ext.so_path()))
    fn = lib.dx_get_dispatch_layout_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p]
    lib.dx_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _reference(topk_idx, E, R):
    """The existing entry point (allocates its outputs and scratch through PyTorch)."""
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    vc = VirtualCluster(R, num_nvl_bytes=2 << 20)
    try:
        per_rank, _, per_expert, in_rank, _ = vc.buffers[0].get_dispatch_layout(topk_idx, E)
        torch.cuda.synchronize()
        return per_rank.clone(), per_expert.clone(), in_rank.clone()
    finally:
        vc.destroy()


def test_noalloc_layout_matches_regular_entry_point_twice():
    lib, fn = _lib()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    cases = [(3000, 8, 256, 8, 1), (517, 6, 64, 4, 2)]  # (T, K, E, R, seed); second is smaller: stale partials must not leak
    for T, K, E, R, seed in cases:
        g = torch.Generator(device="cpu").manual_seed(seed)
        topk_idx = torch.rand(T, E, generator=g).topk(K, dim=-1).indices.to(torch.int64)
        topk_idx[torch.rand(T, K, generator=g) < 0.05] = -1
        topk_idx = topk_idx.cuda()
        per_rank = torch.full((R,), -7, dtype=torch.int32, device="cuda")
        per_expert = torch.full((E,), -7, dtype=torch.int32, device="cuda")
        in_rank = torch.zeros((T, R), dtype=torch.bool, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(topk_idx.data_ptr(), T, K, E, R, per_rank.data_ptr(), per_expert.data_ptr(), in_rank.data_ptr(), stream)
        assert rc == 0, lib.dx_noalloc_last_error().decode()
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        ref_rank, ref_expert, ref_in = _reference(topk_idx, E, R)
        assert torch.equal(per_rank, ref_rank)
        assert torch.equal(per_expert, ref_expert)
        assert torch.equal(in_rank, ref_in)


def test_noalloc_rejects_oversized_and_bad_arguments():
    lib, fn = _lib()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    buf = torch.zeros(16, dtype=torch.int64, device="cuda")
    p = buf.data_ptr()
    rc = fn(p, 10_000_000, 8, 256, 8, p, p, p, stream)  # far beyond the built-in scratch
    assert rc == -2 and b"scratch" in lib.dx_noalloc_last_error()
    rc = fn(p, 16, 8, 250, 8, p, p, p, stream)  # experts not divisible by ranks
    assert rc == -1
    rc = fn(None, 16, 8, 256, 8, p, p, p, stream)
    assert rc == -1
    # 8 ranks: a membership output that is not 8-byte aligned is refused on the host, nothing is launched
    rc = fn(p, 2, 8, 256, 8, p, p, p + 1, stream)
    assert rc == -1 and b"aligned" in lib.dx_noalloc_last_error()
    # the shared-memory bound is the launcher's (experts + 2 * ranks bins): 12280 + 16 bins exceed 48 KiB
    rc = fn(p, 16, 8, 12280, 8, p, p, p, stream)
    assert rc == -2 and b"shared-memory" in lib.dx_noalloc_last_error()
    torch.cuda.synchronize()
