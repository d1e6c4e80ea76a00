"""Grouped expert GEMM micro-benchmark (one GPU): the tcgen05 kernel of this library against a per-expert cuBLAS loop.

    python bench_gemm.py [--experts 8] [--rows 4096] [--k 7168] [--n 4096] [--dtype bf16|fp8] [--swiglu] [--iters 20]
                         [--op fwd|dgrad|wgrad|wgrad_t]

``--op`` (bf16): ``fwd`` y = x @ w[g].T; ``dgrad`` dx = dy @ w[g] with the weight read in place (MN-major operand);
``wgrad`` dw[g] = dy.T @ x with both operands read in place; ``wgrad_t`` the same product from transposed copies (the
K-major form), the transposes not timed.

Prints one JSON line per run with achieved TFLOP/s and the fraction of the measured cuBLAS BF16 peak
(MEASURED_PEAKS.json, "of measured"). ``--rows`` is the number of rows per expert (multiple of 128). Inputs exceed L2
for the default shape (A 58 MB x experts, B 58 MB x experts), so no flush is needed; timing uses CUDA events after
a 0.7 s warm-up (idle clocks ramp slowly).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--k", type=int, default=7168)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"])
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--tile", default="auto", choices=["auto", "wide", "narrow"],
                    help="natively block-scaled fp8 only: 256- or 128-column tiles (auto: wide with --swiglu, narrow without)")
    ap.add_argument("--op", default="fwd", choices=["fwd", "dgrad", "wgrad", "wgrad_t"])
    ap.add_argument("--native-scaling", action="store_true",
                    help="fp8 only: power-of-two scales applied by the tensor core (UE8M0 block scaling) instead of per-K-block promotion")
    args = ap.parse_args()
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.ops.grouped_gemm import grouped_gemm
    C = _ext.load()
    torch.cuda.set_device(0)
    G, R, K, N = args.experts, args.rows, args.k, args.n
    M = G * R
    offs = torch.arange(0, M + 1, R, dtype=torch.int32, device="cuda")
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(G, N, K, device="cuda") * 0.02).to(torch.bfloat16)
    if args.dtype == "fp8":
        from deepep_efa_b200.ops.grouped_gemm import build_sf_atoms_a, build_sf_atoms_b
        a, a_s = C.per_token_cast_to_fp8(x, args.native_scaling, False)
        wb = w.float().view(G, N // 128, 128, K // 128, 128)
        b_s = (wb.abs().amax(dim=(2, 4)).clamp(min=1e-4) / 448.0).contiguous()
        if args.native_scaling:
            b_s = torch.exp2(torch.ceil(torch.log2(b_s))).contiguous()
        b = (wb / b_s.view(G, N // 128, 1, K // 128, 1)).view(G, N, K).to(torch.float8_e4m3fn).contiguous()
        del wb
        if args.native_scaling:
            atoms_b = build_sf_atoms_b(b_s, N, args.swiglu, None if args.tile == "auto" else args.tile == "wide")  # once per weight
            # the activation atoms are rebuilt on every call, as a layer does
            fn = lambda: grouped_gemm(a, b, offs, swiglu=args.swiglu, sfa_atoms=build_sf_atoms_a(a_s), sfb_atoms=atoms_b)
        else:
            fn = lambda: grouped_gemm(a, b, offs, swiglu=args.swiglu, a_scales=a_s, b_scales=b_s)
    elif args.op == "fwd":
        fn = lambda: grouped_gemm(x, w, offs, swiglu=args.swiglu)
    else:
        from deepep_efa_b200.ops.grouped_gemm import grouped_gemm_dgrad, grouped_gemm_wgrad, grouped_gemm_wgrad_inplace
        dy = torch.randn(M, N, device="cuda").to(torch.bfloat16)
        if args.op == "dgrad":
            fn = lambda: grouped_gemm_dgrad(dy, w, offs)
        elif args.op == "wgrad":
            fn = lambda: grouped_gemm_wgrad_inplace(dy, x, offs)
        else:
            dy_t, x_t = dy.t().contiguous(), x.t().contiguous()
            fn = lambda: grouped_gemm_wgrad(dy_t, x_t, offs)

    from bench import ClockSampler, ramp_clocks
    ramp_clocks(0)

    def timeit(f):
        import time
        t0 = time.time()
        while time.time() - t0 < 0.7:  # an idle GPU sits at 120 MHz; give the clocks time to ramp before timing
            for _ in range(5):
                f()
            torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(args.iters):
            f()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / args.iters

    sampler = ClockSampler(gpus={0})
    sampler.start()
    ms = timeit(fn)
    clocks = sampler.stop({0})
    assert C.gemm_error(0) == 0
    flops = 2.0 * M * N * K
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = peaks.get("bf16_tflops", 1590.0)
    out = {"kernel": "grouped_gemm", "op": args.op, "dtype": args.dtype, "native_scaling": bool(args.native_scaling), "swiglu": args.swiglu, "experts": G, "rows_per_expert": R, "k": K, "n": N,
           "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "frac_of_measured_bf16_cublas_peak": round(flops / ms / 1e9 / peak, 3),
           "sm_mhz_median": clocks["sm_mhz"], "throttle_reasons": clocks["reasons"],
           "ms_x_mhz": None if clocks["sm_mhz"] is None else round(ms * clocks["sm_mhz"], 1)}
    if not args.no_cublas and args.dtype == "bf16" and not args.swiglu and args.op == "fwd":
        def loop():
            for g in range(G):
                torch.matmul(x[g * R:(g + 1) * R], w[g].t())
        ms_c = timeit(loop)
        out["cublas_loop_ms"] = round(ms_c, 4)
        out["cublas_loop_tflops"] = round(flops / ms_c / 1e9, 1)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
