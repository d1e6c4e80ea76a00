"""Model-level benchmarks that sit on top of the communication library (bench.py holds the headline metric).

    python bench_moe.py --gpus N [--config fwd_fp8|train_bf16|both] [--steps K] [--warmup W]

* ``fwd_fp8``   DeepSeek-V3-shaped MoE layer forward: 4096 tokens/rank, hidden 7168, 256 routed experts, top-8,
                expert FFN 7168 -> 2048 -> 7168 SwiGLU, FP8 block-scaled weights ~N(0, 0.02), FP8 dispatch,
                grouped tcgen05 GEMMs (SwiGLU fused), BF16 combine. Two lines: fp32 block scales promoted per K block
                (``"native_scaling": false``) and power-of-two scales applied by the tensor core (``true``).
* ``decode_ll``  the same layer for a decode step: 128 tokens/rank through low-latency dispatch -> masked grouped FP8 GEMMs
                over the landing zone -> zero-copy low-latency combine, no host synchronisation.
* ``train_bf16`` MoE training step fwd+bwd: 8192 tokens/rank, hidden 4096, 64 experts, top-6, FFN 4096 -> 1408 -> 4096
                SwiGLU in BF16, routing skewed Zipf(s=1.2) over experts; backward of dispatch is a combine and
                backward of combine is a cached-handle dispatch.

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


def zipf_routing(tokens, num_experts, topk, s, gen):
    p = 1.0 / torch.arange(1, num_experts + 1, dtype=torch.float64) ** s
    g = -torch.log(-torch.log(torch.rand(tokens, num_experts, generator=gen, dtype=torch.float64)))
    idx = (torch.log(p / p.sum()) + g).topk(topk, dim=-1).indices.to(torch.int64)
    w = torch.softmax(torch.randn(tokens, topk, generator=gen), dim=-1).float()
    return idx, w


def time_steps(fn, steps, warmup):
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
    return max_over_ranks(sum(a.elapsed_time(b) for a, b in ev) / steps)


def run(args):
    import deepep_efa_b200 as ep
    from deepep_efa_b200.models.moe import MoEConfig, MoELayer

    rank, world, local_rank = init_dist(args.gpus)
    ramp_clocks(local_rank)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    results = []
    # FP8 configs run with the DeepSeek-style fp32 scales and again with power-of-two scales applied by the tensor core
    scale_variants = [True] if args.native_scaling else [False, True]
    if args.config in ("fwd_fp8", "both"):
        T, H, I, E, K = 4096, 7168, 2048, 256, 8
        rows_worst = T * world
        nvl = int(1.3 * ((rows_worst * (H + H // 128 * 4 + K * 12 + 4)) + 2 * rows_worst * H * 2)) + (64 << 20)
        buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=nvl, explicitly_destroy=True)
        layer = MoELayer(MoEConfig(hidden=H, intermediate=I, num_experts=E, num_topk=K, init_std=0.02), buf, seed=1)
        g = torch.Generator().manual_seed(rank)
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
        idx = torch.rand(T, E, generator=g).topk(K, dim=-1).indices.cuda()
        w = torch.softmax(torch.randn(T, K, generator=g), dim=-1).cuda()
        flops = 2.0 * T * K * H * (2 * I) + 2.0 * T * K * I * H  # per rank on average (uniform routing)
        for native in scale_variants:
            layer.prepare_fp8(native_block_scaling=native)
            ms = time_steps(lambda: layer.forward_fp8(x, idx, w), args.steps, max(args.warmup, 3))
            buf.check_status(sync=True)
            results.append({
                "metric": "moe_layer_forward_fp8_tokens_per_s", "value": round(T * world / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "dtype": "fp8_e4m3 (bf16 combine)", "native_scaling": native,
                "expert_gemm_tflops_per_gpu": round(flops / (ms / 1e3) / 1e12, 1),
                "frac_of_measured_bf16_peak": round(flops / (ms / 1e3) / 1e12 / peaks.get("bf16_tflops_sustained", 1408.3), 3),
                "config": {"model": "DeepSeek-V3-shaped MoE layer forward", "tokens_per_rank": T, "hidden": H, "intermediate": I, "num_experts": E,
                           "topk": K, "parallelism": f"ep{world}", "l2": "working set >> L2"},
                "data": "synthetic N(0,1) activations, uniform top-8, random-init weights N(0,0.02)"})
        del layer
        buf.destroy()
    if args.config in ("train_bf16", "both"):
        T, H, I, E, K = 8192, 4096, 1408, 64, 6
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

        ms = time_steps(step, args.steps, max(args.warmup, 3))
        buf.check_status(sync=True)
        flops = 3 * (2.0 * T * K * H * (2 * I) + 2.0 * T * K * I * H)
        results.append({
            "metric": "moe_train_step_tokens_per_s", "value": round(T * world / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "dtype": "bf16",
            "expert_gemm_tflops_per_gpu_avg": round(flops / (ms / 1e3) / 1e12, 1),
            "config": {"model": "MoE training step fwd+bwd", "tokens_per_rank": T, "hidden": H, "intermediate": I, "num_experts": E, "topk": K,
                       "routing": "Zipf(s=1.2) over experts", "parallelism": f"ep{world}"},
            "data": "synthetic N(0,1) activations, random-init weights N(0,0.02)"})
        buf.destroy()
    if args.config in ("decode_ll", "both"):
        T, H, I, E, K = 128, 7168, 2048, 256, 8
        buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=2 << 20, num_rdma_bytes=ep.Buffer.get_low_latency_rdma_size_hint(T, H, world, E),
                        low_latency_mode=True, explicitly_destroy=True)
        layer = MoELayer(MoEConfig(hidden=H, intermediate=I, num_experts=E, num_topk=K, init_std=0.02), buf, seed=3)
        g = torch.Generator().manual_seed(200 + rank)
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
        idx = torch.rand(T, E, generator=g).topk(K, dim=-1).indices.cuda()
        w = torch.softmax(torch.randn(T, K, generator=g), dim=-1).cuda()
        L = E // world
        weight_bytes = L * (2 * I * H + H * I)  # e4m3 expert weights streamed once per step
        for native in scale_variants:
            layer.prepare_fp8(native_block_scaling=native)
            ms = time_steps(lambda: layer.forward_low_latency(x, idx, w, num_max_tokens=T), max(args.steps, 20), max(args.warmup, 5))
            buf.check_status(sync=True)
            results.append({
                "metric": "moe_decode_layer_us", "value": round(ms * 1e3, 1), "unit": "us", "n_gpus": world, "steps": max(args.steps, 20),
                "ms_per_step": round(ms, 4), "higher_is_better": False, "scaling": "weak", "dtype": "fp8_e4m3 (bf16 combine)", "native_scaling": native,
                "weight_stream_GBps_per_gpu": round(weight_bytes / 1e9 / (ms / 1e3), 1),
                "frac_of_measured_hbm": round(weight_bytes / 1e9 / (ms / 1e3) / peaks.get("hbm_gbs", 6551.4), 3),
                "config": {"model": "DeepSeek-V3-shaped MoE layer, decode step through the low-latency path", "tokens_per_rank": T, "hidden": H,
                           "intermediate": I, "num_experts": E, "topk": K, "parallelism": f"ep{world}",
                           "l2": "expert weights (>= 1.4 GB per rank) exceed L2"},
                "data": "synthetic N(0,1) activations, uniform top-8, random-init weights N(0,0.02)"})
        del layer
        buf.destroy()
    if rank == 0:
        for r in results:
            print(json.dumps(r), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="both", choices=["fwd_fp8", "train_bf16", "decode_ll", "both"])
    ap.add_argument("--native-scaling", action="store_true",
                    help="FP8 configs: only the variant with power-of-two scales applied by the tensor core (default: fp32 scales, then that one)")
    run(ap.parse_args())
