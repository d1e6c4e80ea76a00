"""Micro-benchmark of the memory-bound helper kernels (one GPU): layout, standalone FP8 cast, expert-major plan / gathers,
two-level bookkeeping, and the training-step elementwise kernels.

    python bench_kernels.py [--rows 32768] [--hidden 7168] [--iters 20] [--warmup 5] [--only NAME]

One JSON line per kernel: milliseconds (CUDA events, mean over --iters after --warmup launches), algorithmic bytes moved and
the fraction of the measured HBM copy bandwidth (MEASURED_PEAKS.json, "of measured"). Default inputs (470 MB of bf16 rows)
exceed L2, so no flush is needed between iterations.
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
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    from bench import ramp_clocks
    from deepep_efa_b200 import _ext
    from deepep_efa_b200.ops import hier as Hh
    from deepep_efa_b200.ops.permute import build_expert_plan
    C = _ext.load()
    torch.cuda.set_device(0)
    ramp_clocks(0)
    try:
        hbm = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("hbm_gbs", 6551.4)
    except Exception:
        hbm = 6551.4
    M, H, K, E, R = args.rows, args.hidden, 8, 256, 8
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, H, device="cuda", generator=g).to(torch.bfloat16)
    topk = torch.rand(M, E, device="cuda", generator=g).topk(K, dim=-1).indices
    local = torch.where(topk < E // R, topk, torch.full_like(topk, -1))  # local expert ids of rank 0, -1 elsewhere
    counts = [int(((local == e).sum().item() + 127) // 128 * 128) for e in range(E // R)]
    plan = build_expert_plan(local, counts)
    w = torch.rand(M, K, device="cuda", generator=g)
    y_perm = torch.randn(plan.num_rows, H, device="cuda", generator=g).to(torch.bfloat16)
    inter = 2048
    h13 = torch.randn(M, 2 * inter, device="cuda", generator=g).to(torch.bfloat16)
    dh = torch.randn(M, inter, device="cuda", generator=g).to(torch.bfloat16)
    member = torch.rand(M, 16, device="cuda", generator=g) < 0.3
    ids, cnts, prefix, pos = Hh.routing_sort(member, 8)
    S = int(prefix[-1].item())

    cases = {
        "layout_kernel": (lambda: Hh.layout_hier(topk, E, R, R), M * K * 8 + M * R),
        "fp8_cast_kernel": (lambda: C.per_token_cast_to_fp8(x, False, False), M * H * 3 + M * H // 128 * 4),
        "build_plan_kernel": (lambda: build_expert_plan(local, counts), M * K * 12 + plan.num_rows * 8),
        "gather_rows_kernel": (lambda: C.gather_rows(x, plan.src_row, None, None), 2 * plan.num_rows * H * 2),
        "gather_reduce_rows_kernel": (lambda: C.gather_reduce_rows(y_perm, plan.pos, w, None), int((plan.pos >= 0).sum()) * H * 2 + M * H * 2),
        "rowdot_kernel": (lambda: C.rowdot(y_perm, x, plan.pos), 2 * int((plan.pos >= 0).sum()) * H * 2),
        "transpose_bf16_kernel": (lambda: C.transpose_bf16(x), 2 * M * H * 2),
        "swiglu_fwd_kernel": (lambda: C.swiglu_fwd(h13), M * inter * 6),
        "swiglu_bwd_kernel": (lambda: C.swiglu_bwd(h13, dh), M * inter * 10),
        "routing_sort_kernel": (lambda: Hh.routing_sort(member, 8), M * 16 * 3 + S * 4 + M * 2 * 4),
        "topk_remap_pack_kernel": (lambda: Hh.topk_remap_pack(topk, w, ids, prefix, S, E // 2), S * K * (8 + 4 + 12)),
    }
    for name, (fn, nbytes) in cases.items():
        if args.only and args.only != name:
            continue
        for _ in range(args.warmup):
            fn()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(args.iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / args.iters
        gbs = nbytes / 1e9 / (ms / 1e3)
        print(json.dumps({"kernel": name, "ms": round(ms, 4), "algorithmic_MB": round(nbytes / 1e6, 1), "GBps": round(gbs, 1),
                          "frac_of_measured_hbm": round(gbs / hbm, 3)}), flush=True)


if __name__ == "__main__":
    main()
