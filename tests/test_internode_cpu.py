"""Two-level path (NVLink domain x rail) on CPU: gloo world of 4 as 2 domains x 2 ranks, against the flat all-rank
oracle. The hierarchy must be invisible in the results except for the documented row order of normal dispatch."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _gather(obj, world):
    out = [None] * world
    dist.all_gather_object(out, obj)
    return out


def _worker(rank, world, port, q):
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.set_num_threads(2)
        import deepep_efa_b200 as ep
        from deepep_efa_b200.reference import oracle
        from helpers import make_routing, make_tokens
        P = 2
        nodes = world // P
        T, H, E, K = 40 + 3 * rank, 256, 16, 4
        L = E // world
        x = make_tokens(T, H, "cpu", seed=rank)
        topk_idx, topk_w = make_routing(T, E, K, "cpu", seed=rank, masked_fraction=0.15)
        topk_w = topk_w.masked_fill(topk_idx == -1, 0)
        buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=1 << 20, num_nvl_ranks=P)
        assert buf.get_num_rdma_ranks() == nodes and buf.get_rdma_rank() == rank // P
        # a gloo group serves CPU tensors as it is; only a CUDA tensor would make the transport create its NCCL twin
        from deepep_efa_b200.parallel.transport import CollectiveTransport, group_moves_cuda_tensors
        assert not group_moves_cuda_tensors(dist.group.WORLD)
        tr = CollectiveTransport(dist.group.WORLD)
        assert tr.group_for(torch.zeros(1)) is dist.group.WORLD and tr._gpu_group is None
        got = tr.all_to_all_equal(torch.full((world * 2, 3), float(rank)))
        assert torch.equal(got[:, 0], torch.arange(world, dtype=got.dtype).repeat_interleave(2))

        # ---- layout
        per_rank, per_node, per_expert, in_rank, _ = buf.get_dispatch_layout(topk_idx, E)
        o_rank, o_expert, o_in = oracle.get_dispatch_layout(topk_idx, E, world)
        assert torch.equal(per_rank, o_rank) and torch.equal(per_expert, o_expert) and torch.equal(in_rank, o_in)
        assert per_node.tolist() == [int(o_in[:, n * P:(n + 1) * P].any(1).sum()) for n in range(nodes)]

        # ---- dispatch against the flat oracle, blocks reordered to (forwarder's local index, source domain)
        recv_x, recv_idx, recv_w, per_expert_list, handle, _ = buf.dispatch(
            x, num_tokens_per_rank=per_rank, num_tokens_per_rdma_rank=per_node, is_token_in_rank=in_rank,
            num_tokens_per_expert=per_expert, topk_idx=topk_idx, topk_weights=topk_w)
        assert len(handle) == 10
        everyone = _gather((x, topk_idx, topk_w), world)
        flat = oracle.dispatch([e[0] for e in everyone], [e[1] for e in everyone], [e[2] for e in everyone], E)[rank]
        rpm = flat["rank_prefix_matrix"]
        order = [m * P + i for i in range(P) for m in range(nodes)]
        rows = torch.cat([torch.arange(int(rpm[s - 1, rank]) if s else 0, int(rpm[s, rank])) for s in order])
        assert recv_x.size(0) == rows.numel()
        assert torch.equal(recv_x, flat["recv_x"][rows])
        assert torch.equal(recv_idx, flat["recv_topk_idx"][rows])
        assert torch.equal(recv_w, flat["recv_topk_weights"][rows])
        assert per_expert_list == flat["num_recv_tokens_per_expert_list"]
        gbl = handle[6]
        assert gbl.tolist() == rpm[:, rank].tolist()

        # ---- combine: per-expert identity weighted by the gate returns x * sum(w)
        y = torch.zeros_like(recv_x, dtype=torch.float32)
        for e in range(L):
            r_, k_ = (recv_idx == e).nonzero(as_tuple=True)
            y[r_] += recv_x[r_].float() * recv_w[r_, k_].unsqueeze(1)
        bias = torch.randn(T, H).to(torch.bfloat16)
        combined, combined_w, _ = buf.combine(y.to(torch.bfloat16), handle, topk_weights=recv_w, bias=bias)
        ref = x.float() * topk_w.sum(dim=1, keepdim=True)
        assert oracle.calc_diff(ref + bias.float(), combined.float()) < 1e-4
        assert (combined_w - topk_w).abs().max() < 1e-6

        # ---- cached handle, FP8 pair
        rx2, a, b, c, d, _ = buf.dispatch(x, handle=handle)
        assert a is None and d is None and torch.equal(rx2, recv_x)
        xq, xs = oracle.per_token_cast_to_fp8(x)
        (rq, rs), _, _, _, _, _ = buf.dispatch((xq, xs), handle=handle)
        assert torch.equal(rq.view(torch.uint8), oracle.per_token_cast_to_fp8(flat["recv_x"][rows])[0].view(torch.uint8))
        assert rs.shape == (rows.numel(), H // 128)

        # ---- low latency across domains against the oracle
        M = 64
        idx_all = [e[1] for e in everyone]
        for use_fp8 in (True, False):
            want = oracle.low_latency_dispatch([e[0] for e in everyone], idx_all, M, E, use_fp8)[rank]
            res, cnt, ll_handle, _, hook = buf.low_latency_dispatch(x, topk_idx, M, E, use_fp8=use_fp8, return_recv_hook=True)
            hook()
            px, ps = res if use_fp8 else (res, None)
            assert torch.equal(cnt, want["packed_recv_count"])
            assert torch.equal(ll_handle[1], want["layout_range"])
            for le in range(L):
                n = int(cnt[le])
                assert torch.equal(ll_handle[0][le, :n], want["src_info"][le, :n])
                assert torch.equal(px[le, :n].view(torch.uint8), want["packed_recv_x"][le, :n].view(torch.uint8))
                if use_fp8:
                    assert torch.equal(ps[le, :n], want["packed_recv_x_scales"][le, :n])
            sim = oracle.per_token_cast_back(px.view(-1, H), ps.view(-1, H // 128)).view(px.shape) if use_fp8 else px
            zc = buf.get_next_low_latency_combine_buffer(ll_handle)
            zc.copy_(sim)
            out, _, _ = buf.low_latency_combine(zc, topk_idx, topk_w, ll_handle, zero_copy=True)
            assert oracle.calc_diff(ref, out.float()) < (9e-4 if use_fp8 else 1e-5)

        # ---- the MoE layer runs unchanged on top (autograd duality through both hops)
        from deepep_efa_b200.models.moe import MoEConfig, MoELayer, dense_reference
        layer = MoELayer(MoEConfig(hidden=H, intermediate=128, num_experts=E, num_topk=K, init_std=0.05), buf, seed=7)
        xg = x.clone().requires_grad_(True)
        wg = topk_w.clone().requires_grad_(True)
        yl = layer(xg, topk_idx, wg)
        (yl.float() ** 2).mean().backward()
        w13_all = torch.cat(_gather(layer.w13.detach(), world)).float().requires_grad_(True)
        w2_all = torch.cat(_gather(layer.w2.detach(), world)).float().requires_grad_(True)
        xr, wr = x.clone().requires_grad_(True), topk_w.clone().requires_grad_(True)
        dref = dense_reference(xr, topk_idx, wr, w13_all, w2_all)
        (dref ** 2).mean().backward()
        assert oracle.calc_diff(dref.detach(), yl.detach().float()) < 2e-3
        assert oracle.calc_diff(xr.grad, xg.grad.float()) < 5e-3

        mask = torch.zeros(world, dtype=torch.int32)
        buf.low_latency_update_mask_buffer(1, True)
        buf.low_latency_query_mask_buffer(mask)
        assert mask.tolist() == [0, 1, 0, 0]
        buf.low_latency_clean_mask_buffer()
        buf.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc()))


def test_two_level_path_world4_as_2x2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    world = 4
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            r, msg = q.get(timeout=240)
            results[r] = msg
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    for r in range(world):
        assert results.get(r) == "ok", f"rank {r}: {results.get(r)}"


def test_hier_ops_cpu_fallbacks():
    """routing_sort / topk_remap_pack / recv_src_meta / segmented_copy on CPU tensors (the oracle of the CUDA kernels)."""
    from deepep_efa_b200.ops import hier as H
    torch.manual_seed(0)
    T, G, P = 37, 3, 2
    member = torch.rand(T, G * P) < 0.3
    ids, counts, prefix, pos = H.routing_sort(member, P)
    grp = member.view(T, G, P).any(2)
    assert counts.tolist() == grp.sum(0).tolist() and prefix.tolist()[-1] == int(grp.sum())
    for g in range(G):
        seg = ids[prefix[g]:prefix[g + 1]].tolist()
        assert seg == grp[:, g].nonzero().flatten().tolist()
        for i, t in enumerate(seg):
            assert pos[t, g] == prefix[g] + i
    assert ((pos >= 0) == grp).all()
    K, Eg = 3, 4
    topk = torch.randint(-1, G * Eg, (T, K))
    w = torch.rand(T, K)
    S = int(prefix[-1])
    idx, ww = H.unpack_topk(H.topk_remap_pack(topk, w, ids, prefix, S, Eg), K)
    for s in range(S):
        g = int((prefix[1:] <= s).sum())
        t = int(ids[s])
        for k in range(K):
            mine = g * Eg <= topk[t, k] < (g + 1) * Eg
            assert idx[s, k] == (topk[t, k] - g * Eg if mine else -1)
            assert ww[s, k] == (w[t, k] if mine else 0)
    local = torch.rand(S, P) < 0.5
    meta = H.recv_src_meta(prefix, local, S)
    assert meta[:, 0].tolist() == [int((prefix[1:] <= s).sum()) for s in range(S)]
    assert meta[:, 1].tolist() == [int(local[s, 0]) | (int(local[s, 1]) << 1) for s in range(S)]
    src = torch.arange(100, dtype=torch.uint8)
    dst = torch.zeros(100, dtype=torch.uint8)
    H.segmented_copy(src, dst, torch.tensor([[0, 10, 5], [50, 0, 7]]))
    assert dst[10:15].tolist() == [0, 1, 2, 3, 4] and dst[:7].tolist() == list(range(50, 57))
