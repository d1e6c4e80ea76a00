"""CPU reference semantics over gloo, world_size = 2: 128 tokens/rank, hidden 7168, 64 experts, top-8 without
replacement, softmax weights, seed 0. Checks layout counts, dispatch, per-expert identity and
combine(dispatch(x)) == x * sum(w)."""
import os
import socket

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


def _worker(rank, world, port, q):
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import deepep_efa_b200 as ep
        from deepep_efa_b200.reference import oracle
        from helpers import make_routing, make_tokens
        T, H, E, K = 128, 7168, 64, 8
        L = E // world
        x = make_tokens(T, H, "cpu", seed=rank)
        topk_idx, topk_w = make_routing(T, E, K, "cpu", seed=rank)
        buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=1 << 20)
        per_rank, per_rdma, per_expert, in_rank, _ = buf.get_dispatch_layout(topk_idx, E)
        assert per_rdma is None
        for e in range(E):
            assert per_expert[e].item() == (topk_idx == e).sum().item()
        recv_x, recv_idx, recv_w, per_expert_list, handle, _ = buf.dispatch(
            x, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert,
            topk_idx=topk_idx, topk_weights=topk_w)
        # total count, local-id range, per-expert counts against an all-reduced reference
        total = per_rank.clone()
        dist.all_reduce(total)
        assert recv_x.size(0) == total[rank].item()
        assert ((recv_idx == -1) | ((recv_idx >= 0) & (recv_idx < L))).all()
        glob = per_expert.clone()
        dist.all_reduce(glob)
        assert per_expert_list == glob[rank * L:(rank + 1) * L].tolist()
        # per-expert identity: "expert" = multiply by (1 + local id), weighted by the gate
        y = torch.zeros_like(recv_x, dtype=torch.float32)
        for e in range(L):
            rows, ks = (recv_idx == e).nonzero(as_tuple=True)
            y[rows] += recv_x[rows].float() * recv_w[rows, ks].unsqueeze(1)
        combined, combined_w, _ = buf.combine(y.to(torch.bfloat16), handle, topk_weights=recv_w)
        ref = x.float() * topk_w.sum(dim=1, keepdim=True)
        assert oracle.calc_diff(ref, combined.float()) < 1e-4, oracle.calc_diff(ref, combined.float())
        assert (combined_w - topk_w).abs().max() < 1e-6
        # cached handle: only x travels
        rx2, a, b, c, d, _ = buf.dispatch(x, handle=handle)
        assert a is None and torch.equal(rx2, recv_x)
        # low latency round trip
        (px, ps), cnt, ll_handle, _, _ = buf.low_latency_dispatch(x, topk_idx, T, E, use_fp8=True)
        assert px.shape == (L, world * T, H) and cnt.shape == (L,)
        sim = oracle.per_token_cast_back(px.view(-1, H), ps.view(-1, H // 128)).view(px.shape)
        out, _, _ = buf.low_latency_combine(sim, topk_idx, topk_w, ll_handle)
        assert oracle.calc_diff(ref, out.float()) < 9e-4
        # a program written for the GPU path keeps its expert outputs in Buffer.empty_symmetric: on the CPU backend that is an
        # ordinary tensor and the call gives the same result
        sym = buf.empty_symmetric(list(sim.shape), sim.dtype)
        sym.copy_(sim)
        (_, _), _, ll_handle2, _, _ = buf.low_latency_dispatch(x, topk_idx, T, E, use_fp8=True)
        out2, _, _ = buf.low_latency_combine(sym, topk_idx, topk_w, ll_handle2)
        assert torch.equal(out2, out)
        buf.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc()))


def test_gloo_world2_reference_semantics():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, msg in res:
        assert msg == "ok", f"rank {rank}: {msg}"
