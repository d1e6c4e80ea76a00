"""Normal-mode tuning sweep: dispatch / combine bandwidth as a function of the grid size, at N ranks.

    python -m torch.distributed.run --nproc-per-node N bench_normal_sweep.py --gpus N [--sms 16,24,32,48,64]

The protocol follows the reference's tuning loop (tests/test_intranode.py:194-262): one fresh dispatch gives the handle,
every timed call reuses it, 256 MB L2 flush between calls, CUDA events, max over ranks, bytes counted as the reference
counts them (``recv_x.numel() * 2``, times (1 + 4/128)/2 for FP8, every source rank including self). The reference sweeps
its NVL chunk size at a fixed 24 SMs; this library has no chunking, so the knob is the number of CTAs. Prints one JSON
line: per grid size the GB/s of the three dispatch forms and of combine, and the best grid size of each (the values the
per-rank-count tables of ``deepep_efa_b200/config.py`` are filled from).
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
import bench as B  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--sms", default="16,24,32,48,64")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    import deepep_efa_b200 as ep
    rank, world, local_rank = B.init_dist(args.gpus)
    T, H, E, K = B.NORMAL_TOKENS, B.HIDDEN, B.NUM_EXPERTS, B.TOPK
    nvl = ep.Config(32, 6, 256, 6, 128).get_nvl_buffer_size_hint(H * 2, world, T)
    buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=nvl, explicitly_destroy=True)
    flush = torch.empty(256 << 20, dtype=torch.int8, device="cuda")
    B.ramp_clocks(local_rank)
    x_h, idx_h, w_h = B.make_inputs(rank + 100, T)
    x, topk_idx, topk_w = x_h.cuda(), idx_h.cuda(), w_h.cuda()
    per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(topk_idx, E)
    (rx, rs), _, _, _, handle, _ = buf.dispatch(x, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert,
                                                topk_idx=topk_idx, topk_weights=topk_w, quantize_fp8=True)
    n_recv = rx.size(0)
    y = buf.empty_symmetric([n_recv, H], torch.bfloat16)
    y.normal_()
    xq = B.C_ext().per_token_cast_to_fp8(x, False, False)
    fp8_bytes, bf16_bytes = n_recv * H * 2 * (1 + 4 / 128) / 2, n_recv * H * 2
    keep = {}
    table = {}
    for sms in [int(v) for v in args.sms.split(",")]:
        cfg = ep.Config(sms, 6, 256, 6, 128)
        cases = {
            "dispatch_fp8_fused_quant": (lambda: keep.__setitem__("a", buf.dispatch(x, handle=handle, quantize_fp8=True, config=cfg)), fp8_bytes),
            "dispatch_fp8_prequantized": (lambda: keep.__setitem__("b", buf.dispatch(xq, handle=handle, config=cfg)), fp8_bytes),
            "dispatch_bf16": (lambda: keep.__setitem__("c", buf.dispatch(x, handle=handle, config=cfg)), bf16_bytes),
            "combine_bf16": (lambda: keep.__setitem__("d", buf.combine(y, handle, config=cfg)), bf16_bytes),
        }
        row = {}
        for name, (fn, nbytes) in cases.items():
            for _ in range(args.warmup):
                fn()
            ms = B.max_over_ranks(B.timed_loop(fn, args.steps, flush))
            row[name] = round(nbytes / 1e9 / (ms / 1e3), 1)
        buf.check_status(sync=True)
        table[str(sms)] = row
    best = {name: max(table, key=lambda s: table[s][name]) for name in next(iter(table.values()))}
    if rank == 0:
        print(json.dumps({"metric": "normal_mode_GBps_by_num_sms", "n_gpus": world, "tokens_per_rank": T, "hidden": H, "recv_tokens": int(n_recv),
                          "GBps": table, "best_num_sms": best,
                          "bytes_definition": "recv_x.numel()*2 (x(1+4/128)/2 for FP8), all source ranks including self"}), flush=True)
    buf.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
