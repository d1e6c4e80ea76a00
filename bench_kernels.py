"""Micro-benchmark of the memory-bound helper kernels (one GPU): layout, standalone FP8 cast (plain, masked, scale atoms),
scale-atom builders, expert-major plan / gathers, two-level bookkeeping, the training-step elementwise kernels, and the
single-rank forms of the collective kernels of the fused MoE path (count exchange, expert-major dispatch, stage reduce,
barrier).

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

    # fused-path kernels on one rank: a layer with a tiny FFN gives the workspace (rows, scales, stage) at full hidden size
    from deepep_efa_b200.models.moe import UNIT_ROWS, MoEConfig, MoELayer
    from deepep_efa_b200.ops.grouped_gemm import build_sf_atoms_a, build_sf_atoms_b
    from deepep_efa_b200.parallel.virtual import VirtualCluster
    Tf = min(M, 4096)
    rows_f = (Tf * K + E * 127 + 127) // 128 * 128
    vc = VirtualCluster(1, num_nvl_bytes=(64 << 20) + 2 * (rows_f * (H + H // 128 * 4 + 4) + Tf * K * H * 2))
    fbuf = vc.buffers[0]
    layer = MoELayer(MoEConfig(hidden=H, intermediate=128, num_experts=E, num_topk=K), fbuf)
    fw = layer.fused_workspace(Tf)
    rts = [fbuf.runtime]
    xf, idxf, wf = x[:Tf].contiguous(), topk[:Tf].contiguous(), w[:Tf].contiguous()
    notify_args = [(idxf, fw.recv_x, fw.recv_scales_raw, fw.recv_info, fw.stage, fw.my_counts, fw.sel_list, fw.send_base, fw.unit_start,
                    fw.m_offsets, fw.m_ends, fw.peer_bases)]
    disp_args = [(xf, fw.my_counts, fw.sel_list, fw.send_base, fw.unit_start, fw.peer_bases, None, None, None)]

    def em_dispatch():
        C.em_notify(rts, notify_args, E, UNIT_ROWS)
        C.em_dispatch(rts, disp_args, E, K, UNIT_ROWS, False, False, 148)

    out_f = torch.empty(Tf, H, dtype=torch.bfloat16, device="cuda")
    xs_q, xs_s = C.per_token_cast_to_fp8(x, True, False)
    b_s = torch.exp2(torch.randint(-8, 0, (E // R, 4096 // 128, H // 128), device="cuda").float())
    cnts = torch.randint(0, 129, (M // 128,), device="cuda", dtype=torch.int32)
    nrows = torch.tensor([M // 2], dtype=torch.int32, device="cuda")
    recv_prefix = torch.arange(0, M + 1, M // 8, dtype=torch.int32, device="cuda")
    in_local = torch.rand(M, 4, device="cuda", generator=g) < 0.5
    seg_n = 64
    seg = torch.tensor([[i * (M // seg_n) * H * 2, ((i * 7) % seg_n) * (M // seg_n) * H * 2, (M // seg_n) * H * 2] for i in range(seg_n)],
                       dtype=torch.int64, device="cuda")
    dst_rows = torch.empty_like(x)

    cases = {
        "em_notify_kernel": (lambda: C.em_notify(rts, notify_args, E, UNIT_ROWS), Tf * K * 8 + E * Tf * 4 // 8),
        "em_dispatch_kernel": (em_dispatch, Tf * K * (H * 2 + H + H // 128 * 4 + 4)),
        "stage_reduce_kernel": (lambda: C.stage_reduce(fw.stage, out_f, idxf, wf, E), Tf * K * H * 2 + Tf * H * 2),
        "barrier_kernel": (lambda: C.barrier(rts), 64),
        "sfa_atoms_kernel": (lambda: build_sf_atoms_a(xs_s), 2 * M * (H // 128) * 4),
        "sfb_atoms_kernel": (lambda: build_sf_atoms_b(b_s, 4096, True, True), 2 * b_s.numel() * 4),
        "fp8_cast_kernel_masked": (lambda: C.per_token_cast_to_fp8(x, False, False, cnts, 128), int(cnts.sum()) * H * 3),
        "fp8_cast_kernel_atoms_devcount": (lambda: C.per_token_cast_to_fp8(x, True, False, None, 1, None, None, nrows, True), M // 2 * H * 3),
        "recv_src_meta_kernel": (lambda: Hh.recv_src_meta(recv_prefix, in_local, M), M * 4 + M * 8),
        "segmented_copy_kernel": (lambda: Hh.segmented_copy(x, dst_rows, seg), 2 * M * H * 2),
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
