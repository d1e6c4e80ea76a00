"""Reference arm of bench.py: runs the reference (pbelevich/deepep_efa) through ITS OWN public API on the same
metric, config and timing protocol as our arm.

The reference is built by ``baseline/build_reference.py`` into ``baseline/_ref`` from unmodified sources (its stock
``setup.py`` cannot build here: libfabric and GDRCopy are absent). On one node the reference runs

* low-latency mode through its NCCL fallback (deep_ep/buffer.py:2265-2303, 2722-2741): FP8 cast + route/pack kernels +
  two ``all_to_all_single`` + unpack kernels for dispatch, gather + one ``all_to_all_single`` + atomic-add reduce for
  combine — this is the stock code path of ``Buffer.low_latency_dispatch / low_latency_combine`` whenever EFA was not
  initialised, i.e. whenever there is a single node;
* normal mode through its NVLink kernels (csrc/kernels/intranode.cu), which support 2, 4 or 8 ranks.

If ``baseline/_ref`` is missing the arm prints ``{"impl": "reference", "unavailable": ...}`` and exits 0.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def _unavailable(reason: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        import bench as B
        B.emit({"impl": "reference", "unavailable": reason})


def _import_reference():
    sys.path.insert(0, REF_DIR)
    import deep_ep_cpp  # noqa: F401  built from csrc/deep_ep.cpp + runtime.cu + layout.cu + intranode.cu
    import deep_ep_ll_shim
    for name in dir(deep_ep_ll_shim):
        if not name.startswith("_") and not hasattr(deep_ep_cpp, name):
            setattr(deep_ep_cpp, name, getattr(deep_ep_ll_shim, name))
    import deep_ep
    return deep_ep


def main(args) -> None:
    if not (os.path.isfile(os.path.join(REF_DIR, "deep_ep_cpp.so")) and os.path.isdir(os.path.join(REF_DIR, "deep_ep"))):
        _unavailable("reference not installed: its setup.py needs libfabric (rdma/fabric.h) and GDRCopy, absent from this image; "
                     "run baseline/build_reference.py to build its single-node code paths")
        return
    import bench as B  # the shared protocol helpers
    try:
        rank, world, local_rank = B.init_dist(args.gpus)
        deep_ep = _import_reference()
    except Exception as e:  # pragma: no cover
        _unavailable(f"reference failed to import: {type(e).__name__}: {str(e)[:200]}")
        return
    group = dist.group.WORLD
    steps, warmup = args.steps, max(args.warmup, 3)
    flush = torch.empty(256 << 20, dtype=torch.int8, device="cuda")
    T, H, E, K = B.LL_TOKENS, B.HIDDEN, B.NUM_EXPERTS, B.TOPK

    # The reference sizes normal-mode ring queues from num_nvl_bytes; its own tests use 2 GB (tests/test_intranode.py:273-274).
    nvl_bytes = int(2e9) if world >= 2 else 0
    try:
        buf = deep_ep.Buffer(group, nvl_bytes, 0, low_latency_mode=False, explicitly_destroy=True)
    except Exception as e:
        _unavailable(f"reference Buffer() failed: {type(e).__name__}: {str(e)[:200]}")
        return

    x_h, idx_h, w_h = B.make_inputs(rank, T)
    x, topk_idx, topk_w = x_h.cuda(), idx_h.cuda().to(deep_ep.topk_idx_t), w_h.cuda()
    L = E // world
    sim = torch.randn(L, world * T, H, device="cuda").to(torch.bfloat16) * 0.1
    result = {"impl": "reference", "metric": "ll_dispatch_combine_us", "unit": "us", "n_gpus": world, "steps": steps, "warmup": warmup,
              "higher_is_better": False, "scaling": "weak", "dtype": "fp8_e4m3 dispatch / bf16 combine",
              "data": "synthetic: N(0,1) bf16 activations, uniform top-8 of 256 experts without replacement, softmax weights",
              "config": {"model": "low-latency EP dispatch+combine", "tokens_per_rank": T, "global_batch": T * world, "seq_len": 1,
                         "hidden": H, "num_experts": E, "topk": K, "parallelism": f"ep{world}", "l2": "256 MB flush between timed iterations",
                         "timing": "CUDA events per iteration, max over ranks"},
              "path": "reference low_latency_dispatch/combine, single-node NCCL fallback (deep_ep/buffer.py:2265-2303)"}

    def ll_step():
        _, _, handle, _, _ = buf.low_latency_dispatch(x, topk_idx, T, E, use_fp8=True, topk_weights=topk_w)
        buf.low_latency_combine(sim, topk_idx, topk_w, handle)

    try:
        B.ramp_clocks(local_rank)
        sampler = B.ClockSampler(gpus={B.physical_gpu_index(r) for r in range(world)}) if rank == 0 else None
        if sampler is not None:
            sampler.start()
        for _ in range(warmup):
            ll_step()
        ll_us = B.max_over_ranks(B.timed_loop(ll_step, steps, flush) * 1e3)
        clocks = sampler.stop({B.physical_gpu_index(r) for r in range(world)}) if sampler is not None else \
            {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        result.update(value=round(ll_us, 3), ms_per_step=round(ll_us / 1e3, 6), vs_baseline=round(ll_us / B.PUBLISHED_LL_US, 5),
                      clocks={"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                              "samples": clocks["samples"]})
    except Exception as e:
        result.update(value=None, ll_error=f"{type(e).__name__}: {str(e)[:300]}")

    # end to end (same definition as our arm)
    try:
        x_p, idx_p, w_p = x_h.pin_memory(), idx_h.pin_memory(), w_h.pin_memory()
        out_p = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
        x_d, idx_d, w_d = torch.empty_like(x), torch.empty_like(topk_idx), torch.empty_like(topk_w)

        def e2e_step():
            x_d.copy_(x_p, non_blocking=True)
            idx_d.copy_(idx_p, non_blocking=True)
            w_d.copy_(w_p, non_blocking=True)
            _, _, h, _, _ = buf.low_latency_dispatch(x_d, idx_d, T, E, use_fp8=True, topk_weights=w_d)
            o, _, _ = buf.low_latency_combine(sim, idx_d, w_d, h)
            out_p.copy_(o, non_blocking=True)

        for _ in range(warmup):
            e2e_step()
        e2e_us = B.max_over_ranks(B.timed_loop(e2e_step, steps, flush) * 1e3)
        result["e2e"] = {"value": round(e2e_us, 3), "unit": "us", "h2d_bytes_per_step": x_p.numel() * 2 + idx_p.numel() * 8 + w_p.numel() * 4,
                         "d2h_bytes_per_step": out_p.numel() * 2, "process_pinned_to_gpu_local_cpus": B.BOUND_CPUS}
    except Exception as e:
        result["e2e"] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}

    # normal mode (reference supports 2/4/8 ranks): its tests' protocol with 24 SMs and a tuned chunk size
    if world in (2, 4, 8) and not args.skip_normal:
        try:
            result["normal"] = _bench_normal(deep_ep, buf, rank, world, flush, max(10, min(steps, 50)), warmup, B)
        except Exception as e:
            result["normal"] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
    try:
        buf.destroy()
    except Exception:
        pass
    if not getattr(args, "skip_moe", False):
        try:
            import bench_moe
            result.update(bench_moe.moe_extras("reference", rank, world, steps=getattr(args, "moe_steps", 5), warmup=3))
        except Exception as e:
            result["moe_error"] = f"{type(e).__name__}: {str(e)[:200]}"
    if rank == 0:
        B.emit(result)
    dist.destroy_process_group()


def _bench_normal(deep_ep, buf, rank, world, flush, steps, warmup, B):
    sys.path.insert(0, os.path.join(REF_DIR, "ref_tests"))
    from utils import per_token_cast_to_fp8  # the reference's own helper (tests/utils.py:50-58)
    T, H, E, K = B.NORMAL_TOKENS, B.HIDDEN, B.NUM_EXPERTS, B.TOPK
    x_h, idx_h, w_h = B.make_inputs(rank + 100, T)
    x, topk_idx, topk_w = x_h.cuda(), idx_h.cuda().to(deep_ep.topk_idx_t), w_h.cuda()
    x_e4m3 = per_token_cast_to_fp8(x)
    x_e4m3 = (x_e4m3[0], x_e4m3[1].T.contiguous().T)
    deep_ep.Buffer.set_num_sms(24)
    per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(topk_idx, E)
    best = {}
    # one fresh dispatch gives the handle; the timed calls reuse it, exactly as the reference's own tuning loop does
    # (tests/test_intranode.py:200-214: tune_args = {'x': current_x, 'handle': handle, 'config': config})
    first = buf.dispatch(x_e4m3, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert,
                         topk_idx=topk_idx, topk_weights=topk_w)
    n_recv = first[0][0].size(0)
    handle_ref = first[4]
    for chunk in (8, 16, 24, 32):
        cfg = deep_ep.Config(24, chunk, 256)

        def do_dispatch():
            buf.dispatch(x_e4m3, handle=handle_ref, config=cfg)
        for _ in range(warmup):
            do_dispatch()
        ms = B.max_over_ranks(B.timed_loop(do_dispatch, steps, flush))
        gbps = n_recv * H * 2 * (1 + 4 / 128) / 2 / 1e9 / (ms / 1e3)
        if "dispatch_fp8_cached" not in best or gbps > best["dispatch_fp8_cached"]["GBps"]:
            best["dispatch_fp8_cached"] = {"ms": round(ms, 4), "GBps": round(gbps, 1), "chunk": chunk}

    def do_fresh():
        buf.dispatch(x_e4m3, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert,
                     topk_idx=topk_idx, topk_weights=topk_w, config=deep_ep.Config(24, best["dispatch_fp8_cached"]["chunk"], 256))
    for _ in range(warmup):
        do_fresh()
    ms = B.max_over_ranks(B.timed_loop(do_fresh, steps, flush))
    best["dispatch_fp8"] = {"ms": round(ms, 4), "GBps": round(n_recv * H * 2 * (1 + 4 / 128) / 2 / 1e9 / (ms / 1e3), 1)}
    y = torch.randn(n_recv, H, device="cuda").to(torch.bfloat16)
    for chunk in (2, 4, 8, 16):
        cfg = deep_ep.Config(24, chunk, 256)

        def do_combine():
            buf.combine(y, handle_ref, config=cfg)
        for _ in range(warmup):
            do_combine()
        ms = B.max_over_ranks(B.timed_loop(do_combine, steps, flush))
        gbps = n_recv * H * 2 / 1e9 / (ms / 1e3)
        if "combine_bf16" not in best or gbps > best["combine_bf16"]["GBps"]:
            best["combine_bf16"] = {"ms": round(ms, 4), "GBps": round(gbps, 1), "chunk": chunk}
    # the same two kernels at this library's default grid size (32 SMs), best chunk of the sweeps above
    try:
        deep_ep.Buffer.set_num_sms(32)
        cfg_d = deep_ep.Config(32, best["dispatch_fp8_cached"]["chunk"], 256)
        cfg_c = deep_ep.Config(32, best["combine_bf16"]["chunk"], 256)
        # a handle carries per-channel matrices, and the channel count follows the SM count: take a fresh one at 32 SMs
        handle32 = buf.dispatch(x_e4m3, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert,
                                topk_idx=topk_idx, topk_weights=topk_w, config=cfg_d)[4]
        for name, fn, nbytes in (("dispatch_fp8_cached_32sms", lambda: buf.dispatch(x_e4m3, handle=handle32, config=cfg_d), n_recv * H * 2 * (1 + 4 / 128) / 2),
                                 ("combine_bf16_32sms", lambda: buf.combine(y, handle32, config=cfg_c), n_recv * H * 2)):
            for _ in range(warmup):
                fn()
            ms = B.max_over_ranks(B.timed_loop(fn, steps, flush))
            best[name] = {"ms": round(ms, 4), "GBps": round(nbytes / 1e9 / (ms / 1e3), 1)}
    except Exception as e:
        best["equal_budget_error"] = f"{type(e).__name__}: {str(e)[:200]}"
    deep_ep.Buffer.set_num_sms(24)
    best["recv_tokens"] = int(n_recv)
    best["note"] = "24 SMs, best NVL chunk of a small sweep (the reference's own tuning protocol, tests/test_intranode.py:200-262)"
    return best
