"""Model-level benchmarks that sit on top of the communication library (bench.py holds the headline metric and calls
the functions of this file for its extra keys).

    python bench_moe.py --gpus N [--config fwd_fp8|train_bf16|decode_ll|both] [--impl ours|reference] [--steps K] [--warmup W]

* ``fwd_fp8``   DeepSeek-V3-shaped MoE layer forward: 4096 tokens/rank, hidden 7168, 256 routed experts, top-8,
                expert FFN 7168 -> 2048 -> 7168 SwiGLU, FP8 block-scaled weights ~N(0, 0.02). Our arm prints four lines:
                the fused pipeline (expert-major FP8 dispatch overlapped with an arrival-gated grouped GEMM, scatter
                epilogue, local reduce) and the unfused chain, each with fp32 block scales promoted per K block
                (``"native_scaling": false``) and with power-of-two scales applied by the tensor core (``true``).
* ``decode_ll``  the same layer for a decode step: 128 tokens/rank through low-latency dispatch -> masked grouped FP8 GEMMs
                over the landing zone -> zero-copy low-latency combine, no host synchronisation.
* ``train_bf16`` MoE training step fwd+bwd: 8192 tokens/rank, hidden 4096, 64 experts, top-6, FFN 4096 -> 1408 -> 4096
                SwiGLU in BF16, routing skewed Zipf(s=1.2) over experts; backward of dispatch is a combine and
                backward of combine is a cached-handle dispatch.

``--impl reference`` runs the same three workloads on the unmodified reference library (``baseline/_ref``): its
``Buffer.dispatch / combine`` (deep_ep/buffer.py:451-579) and ``low_latency_dispatch / low_latency_combine`` (:1816, :2460)
around a per-expert PyTorch (cuBLAS, BF16) SwiGLU loop, which is what a user of that library writes, since it ships no
expert GEMM. Its normal mode needs 2, 4 or 8 ranks.

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N bench_moe.py --gpus N``. Timing: CUDA
events around every step, max over ranks; activations (>= 58 MB per rank) plus weights exceed L2, no flush needed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from bench import init_dist, max_over_ranks, ramp_clocks  # noqa: E402

FWD = dict(T=4096, H=7168, I=2048, E=256, K=8)
DECODE = dict(T=128, H=7168, I=2048, E=256, K=8)
TRAIN = dict(T=8192, H=4096, I=1408, E=64, K=6)


def zipf_routing(tokens, num_experts, topk, s, gen):
    p = 1.0 / torch.arange(1, num_experts + 1, dtype=torch.float64) ** s
    g = -torch.log(-torch.log(torch.rand(tokens, num_experts, generator=gen, dtype=torch.float64)))
    idx = (torch.log(p / p.sum()) + g).topk(topk, dim=-1).indices.to(torch.int64)
    w = torch.softmax(torch.randn(tokens, topk, generator=gen), dim=-1).float()
    return idx, w


def uniform_inputs(rank, T, H, E, K, seed=0):
    g = torch.Generator().manual_seed(seed + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    idx = torch.rand(T, E, generator=g).topk(K, dim=-1).indices.cuda()
    w = torch.softmax(torch.randn(T, K, generator=g), dim=-1).cuda()
    return x, idx, w


def time_steps(fn, steps, warmup, per_rank=False):
    """Mean ms per step (max over ranks); with ``per_rank`` also this rank's own mean."""
    for _ in range(warmup):
        fn()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    dist.barrier()
    torch.cuda.synchronize()
    for a, b in ev:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    dist.barrier()
    mine = sum(a.elapsed_time(b) for a, b in ev) / steps
    return (max_over_ranks(mine), mine) if per_rank else max_over_ranks(mine)


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def fwd_flops(T, H, I, K):
    return 2.0 * T * K * H * (2 * I) + 2.0 * T * K * I * H  # per rank on average (uniform routing)


# ------------------------------------------------------------------------------------------------
# this library
# ------------------------------------------------------------------------------------------------
def fused_nvl_bytes(world, T, H, E, K):
    L = E // world
    rows = (world * T * min(K, L) + L * 127 + 127) // 128 * 128
    return int(rows * (H + H // 128 * 4 + 4) + T * K * H * 2) + (64 << 20)


def ours_fwd(rank, world, steps, warmup, scale_variants=(False, True), paths=("fused", "unfused"), stamps=False):
    import deepep_efa_b200 as ep
    from deepep_efa_b200.models.moe import MoEConfig, MoELayer
    T, H, I, E, K = (FWD[k] for k in "THIEK")
    peaks = load_peaks()
    rows_worst = T * world
    unfused = int(1.3 * ((rows_worst * (H + H // 128 * 4 + K * 12 + 4)) + 2 * rows_worst * H * 2)) + (64 << 20)
    nvl = (unfused if "unfused" in paths else (64 << 20)) + (2 * fused_nvl_bytes(world, T, H, E, K) if "fused" in paths else 0)
    buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=nvl, explicitly_destroy=True)
    layer = MoELayer(MoEConfig(hidden=H, intermediate=I, num_experts=E, num_topk=K, init_std=0.02), buf, seed=1)
    x, idx, w = uniform_inputs(rank, T, H, E, K)
    flops = fwd_flops(T, H, I, K)
    fp8_peak = 2.0 * peaks.get("bf16_tflops", 1657.8)  # the tensor core's FP8 rate is twice its BF16 rate
    results = []
    for native in scale_variants:
        layer.prepare_fp8(native_block_scaling=native)
        for path in paths:
            fn = (lambda: layer.forward_fused(x, idx, w)) if path == "fused" else (lambda: layer.forward_fp8(x, idx, w))
            ms = time_steps(fn, steps, max(warmup, 3))
            buf.check_status(sync=True)
            r = {"metric": "moe_layer_forward_fp8_tokens_per_s", "value": round(T * world / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world,
                 "steps": steps, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "dtype": "fp8_e4m3 (bf16 combine)",
                 "native_scaling": native, "path": path, "impl": "deepep_efa_b200",
                 "expert_gemm_tflops_per_gpu": round(flops / (ms / 1e3) / 1e12, 1),
                 "frac_of_measured_fp8_peak": round(flops / (ms / 1e3) / 1e12 / fp8_peak, 3),
                 "fp8_peak_definition": "2 x the measured cuBLAS bf16 burst rate of MEASURED_PEAKS.json",
                 "config": {"model": "DeepSeek-V3-shaped MoE layer forward", "tokens_per_rank": T, "hidden": H, "intermediate": I,
                            "num_experts": E, "topk": K, "parallelism": f"ep{world}", "l2": "working set >> L2"},
                 "data": "synthetic N(0,1) activations, uniform top-8, random-init weights N(0,0.02)"}
            if path == "fused" and stamps:
                ws = layer.fused_workspace(T)
                ws.enable_trace()
                ws.reset_trace()
                layer.forward_fused(x, idx, w)
                torch.cuda.synchronize()
                t = ws.trace.tolist()
                r["stamps_us_from_dispatch_start"] = {"dispatch_end": round((t[1] - t[0]) / 1e3, 1), "gemm1_first_tile_load": round((t[2] - t[0]) / 1e3, 1),
                                                     "gemm1_end": round((t[3] - t[0]) / 1e3, 1)}
                ws.trace = None
            results.append(r)
    del layer
    buf.destroy()
    return results


def ours_decode(rank, world, steps, warmup, scale_variants=(False, True)):
    import deepep_efa_b200 as ep
    from deepep_efa_b200.models.moe import MoEConfig, MoELayer
    T, H, I, E, K = (DECODE[k] for k in "THIEK")
    peaks = load_peaks()
    buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=2 << 20, num_rdma_bytes=ep.Buffer.get_low_latency_rdma_size_hint(T, H, world, E),
                    low_latency_mode=True, explicitly_destroy=True)
    layer = MoELayer(MoEConfig(hidden=H, intermediate=I, num_experts=E, num_topk=K, init_std=0.02), buf, seed=3)
    x, idx, w = uniform_inputs(rank, T, H, E, K, seed=200)
    L = E // world
    weight_bytes = L * (2 * I * H + H * I)  # e4m3 expert weights streamed once per step
    results = []
    for native in scale_variants:
        layer.prepare_fp8(native_block_scaling=native)
        ms = time_steps(lambda: layer.forward_low_latency(x, idx, w, num_max_tokens=T), max(steps, 20), max(warmup, 5))
        buf.check_status(sync=True)
        results.append({
            "metric": "moe_decode_layer_us", "value": round(ms * 1e3, 1), "unit": "us", "n_gpus": world, "steps": max(steps, 20),
            "ms_per_step": round(ms, 4), "higher_is_better": False, "scaling": "weak", "dtype": "fp8_e4m3 (bf16 combine)", "native_scaling": native,
            "impl": "deepep_efa_b200", "weight_stream_GBps_per_gpu": round(weight_bytes / 1e9 / (ms / 1e3), 1),
            "frac_of_measured_hbm": round(weight_bytes / 1e9 / (ms / 1e3) / peaks.get("hbm_gbs", 6551.4), 3),
            "config": {"model": "DeepSeek-V3-shaped MoE layer, decode step through the low-latency path", "tokens_per_rank": T, "hidden": H,
                       "intermediate": I, "num_experts": E, "topk": K, "parallelism": f"ep{world}",
                       "l2": "expert weights (>= 1.4 GB per rank) exceed L2"},
            "data": "synthetic N(0,1) activations, uniform top-8, random-init weights N(0,0.02)"})
    del layer
    buf.destroy()
    return results


def ours_train(rank, world, steps, warmup):
    import deepep_efa_b200 as ep
    from deepep_efa_b200.models.moe import MoEConfig, MoELayer
    T, H, I, E, K = (TRAIN[k] for k in "THIEK")
    peaks = load_peaks()
    rows_worst = T * world
    nvl = int(1.3 * 6 * rows_worst * (H * 2 + K * 12 + 4)) + (64 << 20)
    buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=nvl, explicitly_destroy=True)
    layer = MoELayer(MoEConfig(hidden=H, intermediate=I, num_experts=E, num_topk=K, init_std=0.02), buf, seed=2)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda().requires_grad_(True)
    idx, w = zipf_routing(T, E, K, 1.2, g)
    idx, w = idx.cuda(), w.cuda().requires_grad_(True)

    def step():
        layer.zero_grad(set_to_none=True)
        x.grad = None
        y = layer(x, idx, w)
        y.float().pow(2).mean().backward()

    ms, mine = time_steps(step, steps, max(warmup, 3), per_rank=True)
    buf.check_status(sync=True)
    # rows this rank's experts received (Zipf puts the hot experts on the low ranks): the step waits for the busiest rank
    recv_rows = torch.zeros(world, dtype=torch.float64, device="cuda")
    cnt = torch.bincount(idx.flatten(), minlength=E).double().view(world, E // world).sum(1)
    dist.all_reduce(cnt)
    per_rank_ms = torch.zeros(world, dtype=torch.float64, device="cuda")
    per_rank_ms[rank] = mine
    dist.all_reduce(per_rank_ms)
    flops = 3 * fwd_flops(T, H, I, K)
    busiest = float(cnt.max().item())
    busiest_flops = 3 * (2.0 * busiest * H * (2 * I) + 2.0 * busiest * I * H)
    res = {"metric": "moe_train_step_tokens_per_s", "value": round(T * world / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world,
           "steps": steps, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "impl": "deepep_efa_b200",
           "expert_gemm_tflops_per_gpu_avg": round(flops / (ms / 1e3) / 1e12, 1),
           "busiest_rank_gemm_tflops": round(busiest_flops / (ms / 1e3) / 1e12, 1),
           "busiest_rank_frac_of_measured_bf16_sustained": round(busiest_flops / (ms / 1e3) / 1e12 / peaks.get("bf16_tflops_sustained", 1408.3), 3),
           "rows_per_rank": [int(v) for v in cnt.tolist()], "ms_per_rank": [round(v, 3) for v in per_rank_ms.tolist()],
           "config": {"model": "MoE training step fwd+bwd", "tokens_per_rank": T, "hidden": H, "intermediate": I, "num_experts": E, "topk": K,
                      "routing": "Zipf(s=1.2) over experts", "parallelism": f"ep{world}"},
           "data": "synthetic N(0,1) activations, random-init weights N(0,0.02)"}
    del recv_rows
    buf.destroy()
    return [res]


# ------------------------------------------------------------------------------------------------
# reference library + per-expert PyTorch loop
# ------------------------------------------------------------------------------------------------
def _ref_weights(L, H, I, rank, seed):
    ge = torch.Generator(device="cuda").manual_seed(seed + 1 + rank)
    w13 = torch.empty(L, 2 * I, H, dtype=torch.bfloat16, device="cuda")
    w2 = torch.empty(L, H, I, dtype=torch.bfloat16, device="cuda")
    for e in range(L):
        w13[e] = (torch.randn(2 * I, H, generator=ge, device="cuda") * 0.02).to(torch.bfloat16)
        w2[e] = (torch.randn(H, I, generator=ge, device="cuda") * 0.02).to(torch.bfloat16)
    return w13, w2


def _expert_loop(recv_x, recv_idx, recv_w, w13, w2, inter):
    """What a user of the reference writes between dispatch and combine: per local expert, gather its rows, two cuBLAS
    GEMMs with SwiGLU in between, weighted accumulation back into receive order."""
    out = torch.zeros(recv_x.shape, dtype=torch.float32, device=recv_x.device)
    for e in range(w13.size(0)):
        rows, ks = (recv_idx == e).nonzero(as_tuple=True)
        if rows.numel() == 0:
            continue
        h = recv_x[rows] @ w13[e].t()
        h = torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]
        y = h @ w2[e].t()
        out.index_add_(0, rows, y.float() * recv_w[rows, ks].unsqueeze(1))
    return out.to(torch.bfloat16)


def reference_fwd(deep_ep, ref_utils, rank, world, steps, warmup):
    T, H, I, E, K = (FWD[k] for k in "THIEK")
    if world not in (2, 4, 8):
        return [{"impl": "reference", "metric": "moe_layer_forward_fp8_tokens_per_s", "unavailable": "the reference's normal mode supports 2, 4 or 8 ranks"}]
    buf = deep_ep.Buffer(dist.group.WORLD, int(2e9), 0, low_latency_mode=False, explicitly_destroy=True)
    deep_ep.Buffer.set_num_sms(24)
    L = E // world
    w13, w2 = _ref_weights(L, H, I, rank, 1)
    x, idx, w = uniform_inputs(rank, T, H, E, K)
    idx = idx.to(deep_ep.topk_idx_t)

    def step():
        xq = ref_utils.per_token_cast_to_fp8(x)  # FP8 on the wire, as in our arm (the reference's own helper, tests/utils.py:50-58)
        per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(idx, E)
        (rx, rs), ridx, rw, _, handle, _ = buf.dispatch(xq, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank,
                                                        num_tokens_per_expert=per_expert, topk_idx=idx, topk_weights=w)
        recv = ref_utils.per_token_cast_back(rx, rs)
        y = _expert_loop(recv, ridx, rw, w13, w2, I)
        out, _, _ = buf.combine(y, handle)
        return out

    ms = time_steps(step, steps, max(warmup, 3))
    res = {"metric": "moe_layer_forward_fp8_tokens_per_s", "value": round(T * world / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world,
           "steps": steps, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "impl": "reference",
           "dtype": "fp8_e4m3 dispatch, bf16 cuBLAS expert GEMMs (the reference ships no GEMM), bf16 combine",
           "expert_gemm_tflops_per_gpu": round(fwd_flops(T, H, I, K) / (ms / 1e3) / 1e12, 1),
           "config": {"model": "DeepSeek-V3-shaped MoE layer forward", "tokens_per_rank": T, "hidden": H, "intermediate": I, "num_experts": E,
                      "topk": K, "parallelism": f"ep{world}", "l2": "working set >> L2"},
           "path": "reference Buffer.dispatch/combine (24 SMs) around a per-expert PyTorch SwiGLU loop",
           "data": "synthetic N(0,1) activations, uniform top-8, random-init weights N(0,0.02)"}
    buf.destroy()
    return [res]


def reference_decode(deep_ep, ref_utils, rank, world, steps, warmup):
    T, H, I, E, K = (DECODE[k] for k in "THIEK")
    buf = deep_ep.Buffer(dist.group.WORLD, 0, 0, low_latency_mode=False, explicitly_destroy=True)
    L = E // world
    w13, w2 = _ref_weights(L, H, I, rank, 3)
    x, idx, w = uniform_inputs(rank, T, H, E, K, seed=200)
    idx = idx.to(deep_ep.topk_idx_t)

    def step():
        (px, ps), cnt, handle, _, _ = buf.low_latency_dispatch(x, idx, T, E, use_fp8=True, topk_weights=w)
        counts = cnt.tolist()
        y = torch.empty(L, px.size(1), H, dtype=torch.bfloat16, device="cuda")
        for e in range(L):
            n = counts[e]
            if n == 0:
                continue
            a = ref_utils.per_token_cast_back(px[e, :n], ps[e, :n])
            h = a @ w13[e].t()
            h = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
            y[e, :n] = h @ w2[e].t()
        out, _, _ = buf.low_latency_combine(y, idx, w, handle)
        return out

    ms = time_steps(step, max(steps, 20), max(warmup, 5))
    res = {"metric": "moe_decode_layer_us", "value": round(ms * 1e3, 1), "unit": "us", "n_gpus": world, "steps": max(steps, 20),
           "ms_per_step": round(ms, 4), "higher_is_better": False, "scaling": "weak", "impl": "reference",
           "dtype": "fp8_e4m3 dispatch, bf16 cuBLAS expert GEMMs, bf16 combine",
           "config": {"model": "DeepSeek-V3-shaped MoE layer, decode step through the low-latency path", "tokens_per_rank": T, "hidden": H,
                      "intermediate": I, "num_experts": E, "topk": K, "parallelism": f"ep{world}",
                      "l2": "expert weights (>= 1.4 GB per rank) exceed L2"},
           "path": "reference low_latency_dispatch/combine (single-node NCCL fallback) around a per-expert PyTorch SwiGLU loop",
           "data": "synthetic N(0,1) activations, uniform top-8, random-init weights N(0,0.02)"}
    buf.destroy()
    return [res]


def reference_train(deep_ep, ref_utils, rank, world, steps, warmup):
    T, H, I, E, K = (TRAIN[k] for k in "THIEK")
    if world not in (2, 4, 8):
        return [{"impl": "reference", "metric": "moe_train_step_tokens_per_s", "unavailable": "the reference's normal mode supports 2, 4 or 8 ranks"}]
    buf = deep_ep.Buffer(dist.group.WORLD, int(2e9), 0, low_latency_mode=False, explicitly_destroy=True)
    deep_ep.Buffer.set_num_sms(24)
    L = E // world
    w13, w2 = _ref_weights(L, H, I, rank, 2)
    w13.requires_grad_(True), w2.requires_grad_(True)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda().requires_grad_(True)
    idx, w = zipf_routing(T, E, K, 1.2, g)
    idx, w = idx.cuda().to(deep_ep.topk_idx_t), w.cuda().requires_grad_(True)

    # the reference documents the autograd contract (deep_ep/buffer.py:512-519): the backward of a dispatch is a combine,
    # the backward of a combine is a dispatch with the cached handle
    class Dispatch(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x_, w_):
            per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(idx, E)
            rx, ridx, rw, _, handle, _ = buf.dispatch(x_, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank,
                                                      num_tokens_per_expert=per_expert, topk_idx=idx, topk_weights=w_)
            ctx.handle = handle
            ctx.mark_non_differentiable(ridx)
            return rx, ridx, rw, _Box(handle)

        @staticmethod
        def backward(ctx, grx, _gidx, grw, _gh):
            gx, gw, _ = buf.combine(grx.contiguous(), ctx.handle, topk_weights=grw.contiguous() if grw is not None else None)
            return gx, gw

    class Combine(torch.autograd.Function):
        @staticmethod
        def forward(ctx, y, box):
            ctx.handle = box.v
            out, _, _ = buf.combine(y, box.v)
            return out

        @staticmethod
        def backward(ctx, g):
            gy, *_ = buf.dispatch(g.contiguous(), handle=ctx.handle)
            return gy, None

    def step():
        w13.grad = w2.grad = x.grad = w.grad = None
        rx, ridx, rw, box = Dispatch.apply(x, w)
        out = torch.zeros(rx.shape, dtype=torch.float32, device="cuda")
        for e in range(L):
            rows, ks = (ridx == e).nonzero(as_tuple=True)
            if rows.numel() == 0:
                continue
            h = rx[rows] @ w13[e].t()
            h = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
            yv = h @ w2[e].t()
            out = out.index_add(0, rows, yv.float() * rw[rows, ks].unsqueeze(1))
        y = Combine.apply(out.to(torch.bfloat16), box)
        y.float().pow(2).mean().backward()

    ms = time_steps(step, steps, max(warmup, 3))
    res = {"metric": "moe_train_step_tokens_per_s", "value": round(T * world / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world,
           "steps": steps, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "impl": "reference",
           "config": {"model": "MoE training step fwd+bwd", "tokens_per_rank": T, "hidden": H, "intermediate": I, "num_experts": E, "topk": K,
                      "routing": "Zipf(s=1.2) over experts", "parallelism": f"ep{world}"},
           "path": "reference Buffer.dispatch/combine (24 SMs) with autograd around a per-expert PyTorch SwiGLU loop",
           "data": "synthetic N(0,1) activations, random-init weights N(0,0.02)"}
    buf.destroy()
    return [res]


class _Box:
    """Carries a non-tensor handle through an autograd Function's outputs."""

    def __init__(self, v):
        self.v = v


def import_reference():
    """(deep_ep module, its tests/utils.py helpers) of the unmodified reference under baseline/_ref, or raises."""
    from baseline import reference_arm
    deep_ep = reference_arm._import_reference()
    sys.path.insert(0, os.path.join(reference_arm.REF_DIR, "ref_tests"))
    import utils as ref_utils
    return deep_ep, ref_utils


def moe_extras(impl, rank, world, steps=5, warmup=3, which=("fwd", "decode", "train")):
    """Compact model-level numbers for bench.py's JSON line: {"moe_fwd_ms", "decode_us", "train_step_ms", ...}; a failing
    or unavailable part becomes a string under its key instead of taking the headline down."""
    out = {}
    if impl == "reference":
        try:
            deep_ep, ref_utils = import_reference()
        except Exception as e:  # pragma: no cover
            return {"moe_error": f"reference failed to import: {type(e).__name__}: {str(e)[:200]}"}

    def run(key, fn, pick):
        try:
            out[key] = pick(fn())
        except Exception as e:
            out[key] = f"error: {type(e).__name__}: {str(e)[:200]}"
        torch.cuda.synchronize()
        torch.cuda.empty_cache()

    def first_ms(rs):
        r = rs[0]
        return r["unavailable"] if "unavailable" in r else r["ms_per_step"]

    if impl == "reference":
        if "fwd" in which:
            run("moe_fwd_ms", lambda: reference_fwd(deep_ep, ref_utils, rank, world, steps, warmup), first_ms)
        if "decode" in which:
            run("decode_us", lambda: reference_decode(deep_ep, ref_utils, rank, world, steps, warmup),
                lambda rs: round(rs[0]["ms_per_step"] * 1e3, 1))
        if "train" in which:
            run("train_step_ms", lambda: reference_train(deep_ep, ref_utils, rank, world, steps, warmup), first_ms)
        return out
    if "fwd" in which:
        # Four variants: fused / unfused pipeline, fp32 block scales (promoted on the CUDA cores) / power-of-two block scales applied
        # by the tensor core. The reported number is the fused pipeline with the tensor core's own block scaling, the form this
        # library recommends on Blackwell; all four ride along under "moe_fwd".
        run("moe_fwd", lambda: ours_fwd(rank, world, steps, warmup), lambda rs: {f"{r['path']}_{'native' if r['native_scaling'] else 'fp32scale'}": r["ms_per_step"] for r in rs})
        if isinstance(out.get("moe_fwd"), dict):
            out["moe_fwd_ms"] = out["moe_fwd"].get("fused_native")
            out["moe_fwd_variant"] = "fused pipeline, e4m3 with power-of-two 1x128 / 128x128 block scales applied by tcgen05 block-scaled MMA"
    if "decode" in which:
        run("decode", lambda: ours_decode(rank, world, steps, warmup, scale_variants=(False, True)),
            lambda rs: {("native" if r.get("native_scaling") else "fp32scale"): round(r["ms_per_step"] * 1e3, 1) for r in rs})
        if isinstance(out.get("decode"), dict):
            out["decode_us"] = min(out["decode"].values())
        else:
            out["decode_us"] = out.pop("decode")
    if "train" in which:
        run("train_step_ms", lambda: ours_train(rank, world, steps, warmup), first_ms)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="both", choices=["fwd_fp8", "train_bf16", "decode_ll", "both"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--native-scaling", action="store_true",
                    help="FP8 configs: only the variant with power-of-two scales applied by the tensor core (default: fp32 scales, then that one)")
    ap.add_argument("--stamps", action="store_true", help="fwd_fp8: add the dispatch / first-GEMM overlap stamps of one fused step")
    args = ap.parse_args()
    rank, world, local_rank = init_dist(args.gpus)
    ramp_clocks(local_rank)
    results = []
    variants = (True,) if args.native_scaling else (False, True)
    if args.impl == "reference":
        try:
            deep_ep, ref_utils = import_reference()
        except Exception as e:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}), flush=True)
            dist.destroy_process_group()
            return
        if args.config in ("fwd_fp8", "both"):
            results += reference_fwd(deep_ep, ref_utils, rank, world, args.steps, args.warmup)
        if args.config in ("train_bf16", "both"):
            results += reference_train(deep_ep, ref_utils, rank, world, args.steps, args.warmup)
        if args.config in ("decode_ll", "both"):
            results += reference_decode(deep_ep, ref_utils, rank, world, args.steps, args.warmup)
    else:
        if args.config in ("fwd_fp8", "both"):
            results += ours_fwd(rank, world, args.steps, args.warmup, variants, stamps=args.stamps)
        if args.config in ("train_bf16", "both"):
            results += ours_train(rank, world, args.steps, args.warmup)
        if args.config in ("decode_ll", "both"):
            results += ours_decode(rank, world, args.steps, args.warmup, variants)
    if rank == 0:
        for r in results:
            print(json.dumps(r), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
