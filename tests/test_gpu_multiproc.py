"""Real multi-process runs: one process per GPU, CUDA IPC peer mappings, NCCL only for bootstrap.
Skipped when fewer than two GPUs are visible. Every rank checks its own outputs against the pure-PyTorch
oracle evaluated on the all-gathered inputs."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import traceback
    try:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        torch.set_num_threads(2)  # the CPU oracle runs in every rank; keep the ranks from starving each other
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import deepep_efa_b200 as ep
        from deepep_efa_b200.reference import oracle
        from helpers import make_routing, make_tokens

        def gather(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out

        def align():
            # the oracle checks between collectives take different CPU time on every rank; line the ranks up again so
            # that no rank sits in a device-side wait for seconds
            torch.cuda.synchronize()
            dist.barrier()

        T, H, E, K = 96, 2048, 8 * world, 4
        L = E // world
        buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=128 << 20,
                        num_rdma_bytes=ep.Buffer.get_low_latency_rdma_size_hint(T, H, world, E), low_latency_mode=True,
                        explicitly_destroy=True, timeout_ms=20000)
        x = make_tokens(T, H, "cuda", seed=rank)
        idx, w = make_routing(T, E, K, "cuda", seed=rank, masked_fraction=0.05)
        all_x = [t.cpu() for t in gather(x.cpu())]
        all_idx = [t.cpu() for t in gather(idx.cpu())]
        all_w = [t.cpu() for t in gather(w.cpu())]

        for it in range(3):
            # ---- normal mode, bf16 and fused fp8 ----
            per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(idx, E)
            for fused in (False, True):
                align()
                recv_x, recv_idx, recv_w, counts, handle, ev = buf.dispatch(
                    x, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert,
                    topk_idx=idx, topk_weights=w, quantize_fp8=fused, async_finish=(it == 1))
                ev.current_stream_wait()
                torch.cuda.synchronize()
                buf.check_status()
                if fused:
                    pairs = [oracle.per_token_cast_to_fp8(t) for t in all_x]
                    ref = oracle.dispatch([p[0] for p in pairs], all_idx, all_w, E, x_scales=[p[1] for p in pairs])[rank]
                    assert torch.equal(recv_x[0].cpu().view(torch.uint8), ref["recv_x"].view(torch.uint8))
                    assert torch.equal(recv_x[1].cpu(), ref["recv_x_scales"])
                    y = oracle.per_token_cast_back(recv_x[0].cpu(), recv_x[1].cpu()).cuda()
                else:
                    ref = oracle.dispatch(all_x, all_idx, all_w, E)[rank]
                    assert torch.equal(recv_x.cpu(), ref["recv_x"])
                    y = recv_x
                assert torch.equal(recv_idx.cpu(), ref["recv_topk_idx"]) and torch.equal(recv_w.cpu(), ref["recv_topk_weights"])
                assert counts == ref["num_recv_tokens_per_expert_list"]
                assert torch.equal(handle[0].cpu(), ref["rank_prefix_matrix"])
                align()
                out, out_w, _ = buf.combine(y, handle, topk_weights=recv_w)
                torch.cuda.synchronize()
                buf.check_status()
                hits = in_rank.sum(dim=1, keepdim=True).float()
                base = y.float() if False else None
                if fused:
                    want = oracle.per_token_cast_back(*oracle.per_token_cast_to_fp8(x.cpu())).float().cuda() * hits
                    assert oracle.calc_diff(want, out.float()) < 1e-4
                else:
                    assert oracle.calc_diff(x.float() * hits, out.float()) < 5e-6
                assert (out_w - w.masked_fill(idx == -1, 0)).abs().max() < 1e-6
            # cached handle
            align()
            rx2, *_ = buf.dispatch(x, handle=handle)
            assert torch.equal(rx2.cpu(), oracle.dispatch(all_x, all_idx, all_w, E)[rank]["recv_x"])

            # ---- low latency ----
            for use_fp8 in (True, False):
                stats = torch.zeros(L, dtype=torch.int32, device="cuda")
                align()
                rx, cnt, h, _, hook = buf.low_latency_dispatch(x, idx, T, E, use_fp8=use_fp8, cumulative_local_expert_recv_stats=stats,
                                                               return_recv_hook=(it == 2))
                if hook is not None:
                    hook()
                torch.cuda.synchronize()
                buf.check_status()
                ref = oracle.low_latency_dispatch(all_x, all_idx, T, E, use_fp8)[rank]
                assert torch.equal(cnt.cpu(), ref["packed_recv_count"]) and torch.equal(h[1].cpu(), ref["layout_range"])
                for le in range(L):
                    n = int(cnt[le])
                    assert torch.equal(h[0][le, :n].cpu(), ref["src_info"][le, :n])
                    if use_fp8:
                        assert torch.equal(rx[0][le, :n].cpu().view(torch.uint8), ref["packed_recv_x"][le, :n].view(torch.uint8))
                        assert torch.equal(rx[1][le, :n].cpu(), ref["packed_recv_x_scales"][le, :n])
                    else:
                        assert torch.equal(rx[le, :n].cpu(), ref["packed_recv_x"][le, :n])
                if use_fp8:
                    ysim = oracle.per_token_cast_back(rx[0].view(-1, H), rx[1].view(-1, H // 128)).view(rx[0].shape)
                else:
                    ysim = rx.clone()
                align()
                o, _, hook = buf.low_latency_combine(ysim, idx, w, h, return_recv_hook=(it == 2))
                if hook is not None:
                    hook()
                torch.cuda.synchronize()
                buf.check_status()
                want = x.float() * w.masked_fill(idx == -1, 0).sum(dim=1, keepdim=True)
                assert oracle.calc_diff(want, o.float()) < (9e-4 if use_fp8 else 1e-5)
        # ---- MoE layer forward + backward across ranks against the dense loop over all experts ----
        from deepep_efa_b200.models.moe import MoEConfig, MoELayer, dense_reference
        cfg = MoEConfig(hidden=512, intermediate=256, num_experts=E, num_topk=K, init_std=0.05)
        layer = MoELayer(cfg, buf)
        xm = make_tokens(T, 512, "cuda", seed=40 + rank).requires_grad_(True)
        mi, mw = make_routing(T, E, K, "cuda", seed=40 + rank)
        align()
        ym = layer(xm, mi, mw)
        (ym.float() ** 2).mean().backward()
        torch.cuda.synchronize()
        buf.check_status()
        w13_all = torch.cat([t.cuda() for t in gather(layer.w13.detach().cpu())]).float()
        w2_all = torch.cat([t.cuda() for t in gather(layer.w2.detach().cpu())]).float()
        xr = xm.detach().clone().requires_grad_(True)
        ref = dense_reference(xr, mi, mw, w13_all, w2_all)
        (ref ** 2).mean().backward()
        rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()
        assert rel(ym, ref) < 3e-2, rel(ym, ref)
        assert rel(xm.grad, xr.grad) < 6e-2, rel(xm.grad, xr.grad)
        align()
        layer.prepare_fp8(native_block_scaling=False)
        y8 = layer.forward_fp8(xm.detach(), mi, mw)
        torch.cuda.synchronize()
        buf.check_status()
        assert rel(y8, ref.detach()) < 8e-2, rel(y8, ref.detach())
        align()
        yl = layer.forward_low_latency(xm.detach(), mi, mw, num_max_tokens=T)
        torch.cuda.synchronize()
        buf.check_status()
        assert rel(yl, ref.detach()) < 8e-2, rel(yl, ref.detach())
        # ---- the fused pipeline with real overlap: dispatch on the communication stream, gated GEMM on this one ----
        for native in (False, True):
            layer.prepare_fp8(native_block_scaling=native)
            for rep in range(3):
                # a different input every time: a value that a kernel picks up from the step before (a scale read before its row
                # had arrived, a stage row summed before it was written) must show as an error, not repeat the right answer
                x_rep = (xm.detach() * (0.5 + rep)).contiguous()
                ref_rep = dense_reference(x_rep, mi, mw, w13_all, w2_all)
                align()
                yf = layer.forward_fused(x_rep, mi, mw)
                torch.cuda.synchronize()
                buf.check_status(sync=True)
                assert rel(yf, ref_rep) < 8e-2, (native, rep, rel(yf, ref_rep))
        # ---- a gloo group handed to the rail transport: CUDA tensors travel over a lazily created NCCL twin ----
        from deepep_efa_b200.parallel.transport import CollectiveTransport, group_moves_cuda_tensors
        gloo = dist.new_group(backend="gloo")
        dev = torch.device("cuda", rank)
        assert not group_moves_cuda_tensors(gloo) and group_moves_cuda_tensors(dist.group.WORLD)
        tr = CollectiveTransport(gloo)
        blk = torch.full((world * 3, 5), float(rank), device=dev)
        got = tr.all_to_all_equal(blk)
        assert torch.equal(got, torch.arange(world, device=dev, dtype=blk.dtype).repeat_interleave(3)[:, None].expand(-1, 5))
        assert tr.group_for(blk) is not gloo and tr.group_for(blk.cpu()) is gloo
        sp = [r + 1 for r in range(world)]
        rows = tr.all_to_all_rows(torch.full((sum(sp), 2), float(rank), device=dev), sp, [rank + 1] * world)
        assert rows.shape[0] == (rank + 1) * world and torch.equal(rows[:, 0], torch.arange(world, device=dev, dtype=rows.dtype).repeat_interleave(rank + 1))
        buf.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


def _worker_pressure(rank, world, port, q):
    """Full-size low-latency shape, 3 seeds x 20 repeats: every repeat of a seed must reproduce the first one bit for bit
    (received rows, counts, source info, combined output), in the staged and in the zero-copy (pull) form."""
    import traceback
    try:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import deepep_efa_b200 as ep
        from deepep_efa_b200.reference import oracle
        from helpers import make_routing, make_tokens
        T, H, E, K = 128, 7168, 256, 8
        L = E // world
        buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=2 << 20, num_rdma_bytes=ep.Buffer.get_low_latency_rdma_size_hint(T, H, world, E),
                        low_latency_mode=True, explicitly_destroy=True, timeout_ms=20000)
        for seed in range(3):
            x = make_tokens(T, H, "cuda", seed=100 * seed + rank)
            idx, w = make_routing(T, E, K, "cuda", seed=100 * seed + rank, masked_fraction=0.02)
            first = None
            for rep in range(20):
                (px, ps), cnt, h, _, _ = buf.low_latency_dispatch(x, idx, T, E, use_fp8=True)
                valid = torch.arange(px.size(1), device="cuda")[None, :] < cnt[:, None]
                sig = [oracle.hash_tensor(px.view(torch.uint8)[valid]), oracle.hash_tensor(ps[valid]), oracle.hash_tensor(cnt),
                       oracle.hash_tensor(h[0][valid]), oracle.hash_tensor(h[1])]
                y = oracle.per_token_cast_back(px.view(-1, H), ps.view(-1, H // 128)).view(px.shape)
                zero_copy = rep % 2 == 1
                if zero_copy:
                    buf.get_next_low_latency_combine_buffer(h).copy_(y)
                o, _, _ = buf.low_latency_combine(y, idx, w, h, zero_copy=zero_copy)
                sig.append(oracle.hash_tensor(o))
                torch.cuda.synchronize()
                buf.check_status()
                if first is None:
                    first = sig
                    want = x.float() * w.masked_fill(idx == -1, 0).sum(dim=1, keepdim=True)
                    assert oracle.calc_diff(want, o.float()) < 9e-4
                assert sig == first, f"seed {seed} repeat {rep}: results differ from the first repeat"
        # Pairs issued back to back with no host synchronisation and nothing between the two kernels: the combine then overlaps
        # the tail of its dispatch, and a fast rank can announce the next call's source before a slow rank has read this call's.
        # The zero-copy buffers of the two parities hold DIFFERENT expert outputs, so picking up the wrong announcement (or a
        # stale row number) changes the result.
        x = make_tokens(T, H, "cuda", seed=7 + rank)
        idx, w = make_routing(T, E, K, "cuda", seed=7 + rank, masked_fraction=0.02)
        want = {}
        for par in range(2):
            (px, ps), cnt, h, _, _ = buf.low_latency_dispatch(x, idx, T, E, use_fp8=True)
            y = (oracle.per_token_cast_back(px.view(-1, H), ps.view(-1, H // 128)).view(px.shape) * (1.0 + par)).to(torch.bfloat16)
            buf.get_next_low_latency_combine_buffer(h).copy_(y)
            o, _, _ = buf.low_latency_combine(y, idx, w, h, zero_copy=True)
            torch.cuda.synchronize()
            dist.barrier()
            want[par] = o.clone()
        assert not torch.equal(want[0], want[1])
        outs = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(60)]
        for it in range(60):
            if rank == world - 1 and it % 7 == 3:
                torch.cuda._sleep(300000)  # the last rank falls behind now and then
            _, _, h, _, _ = buf.low_latency_dispatch(x, idx, T, E, use_fp8=True)
            buf.low_latency_combine(y, idx, w, h, zero_copy=True, out=outs[it])
        torch.cuda.synchronize()
        buf.check_status()
        for it in range(60):
            assert torch.equal(outs[it], want[it % 2]), f"back-to-back pair {it} differs"
        buf.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


def _worker_shrink(rank, world, port, q):
    """Shrink mode with a host-made failure: rank 0 simply does not take part in one step (it sits in a host barrier, no
    kernel of this library in flight). The others' waits run out after a short limit, they mask rank 0 on the device,
    finish the step among themselves, and keep working; a collective recover() brings rank 0 back."""
    import traceback
    try:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import deepep_efa_b200 as ep
        from deepep_efa_b200.buffer import EPTimeoutError
        from deepep_efa_b200.reference import oracle
        from helpers import make_routing, make_tokens
        T, H, E, K = 32, 1024, 4 * world, 4
        L = E // world
        buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=2 << 20, num_rdma_bytes=ep.Buffer.get_low_latency_rdma_size_hint(T, H, world, E),
                        low_latency_mode=True, explicitly_destroy=True, enable_shrink=True, timeout_ms=300)
        x = make_tokens(T, H, "cuda", seed=rank)
        idx, w = make_routing(T, E, K, "cuda", seed=rank)

        def step(expect_timeout=False):
            rx, cnt, h, _, _ = buf.low_latency_dispatch(x, idx, T, E, use_fp8=False)
            o, _, _ = buf.low_latency_combine(rx.clone(), idx, w, h)
            torch.cuda.synchronize()
            if expect_timeout:
                with pytest.raises(EPTimeoutError):
                    buf.check_status()
                buf.runtime.clear_status()
            else:
                buf.check_status()
            return o

        def want(masked=()):
            keep = idx >= 0
            for m in masked:
                keep = keep & (idx // L != m)
            return x.float() * (w * keep).sum(dim=1, keepdim=True)

        torch.cuda.synchronize()
        dist.barrier()
        assert oracle.calc_diff(want(), step().float()) < 1e-5          # everybody takes part
        torch.cuda.synchronize()
        dist.barrier()
        if rank != 0:
            o = step(expect_timeout=True)                                 # rank 0 is silent: the waits run out, it gets masked
            st = torch.zeros(world, dtype=torch.int32, device="cuda")
            buf.low_latency_query_mask_buffer(st)
            assert st.tolist() == [1] + [0] * (world - 1), st.tolist()
            assert oracle.calc_diff(want(masked=(0,)), o.float()) < 1e-5
            o = step()                                                    # the survivors carry on without waiting for it
            assert oracle.calc_diff(want(masked=(0,)), o.float()) < 1e-5
        torch.cuda.synchronize()
        dist.barrier()
        buf.low_latency_clean_mask_buffer()
        buf.recover()                                                     # collective: sequence state starts over on every rank
        assert oracle.calc_diff(want(), step().float()) < 1e-5
        buf.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


def _worker_two_level(rank, world, port, q, P):
    """The group as `world / P` NVLink domains of P GPUs: rail hops over NCCL, fan-out by the NVLink kernels."""
    import traceback
    try:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        torch.set_num_threads(2)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import deepep_efa_b200 as ep
        from deepep_efa_b200.reference import oracle
        from helpers import make_routing, make_tokens

        def gather(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out

        def align():
            torch.cuda.synchronize()
            dist.barrier()

        nodes = world // P
        T, H, E, K = 200 + 8 * rank, 1024, 8 * world, 4
        L = E // world
        buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=128 << 20, explicitly_destroy=True, timeout_ms=20000, num_nvl_ranks=P)
        assert buf.get_num_rdma_ranks() == nodes
        x = make_tokens(T, H, "cuda", seed=rank)
        idx, w = make_routing(T, E, K, "cuda", seed=rank, masked_fraction=0.05)
        w = w.masked_fill(idx == -1, 0)
        all_x, all_idx, all_w = [t.cpu() for t in gather(x.cpu())], [t.cpu() for t in gather(idx.cpu())], [t.cpu() for t in gather(w.cpu())]
        flat = oracle.dispatch(all_x, all_idx, all_w, E)[rank]
        rpm = flat["rank_prefix_matrix"]
        order = [m * P + i for i in range(P) for m in range(nodes)]
        rows = torch.cat([torch.arange(int(rpm[s - 1, rank]) if s else 0, int(rpm[s, rank])) for s in order])
        ref = (x.float() * w.sum(dim=1, keepdim=True)).cpu()
        for it in range(2):
            align()
            per_rank, per_node, per_expert, in_rank, _ = buf.get_dispatch_layout(idx, E)
            o_rank, o_expert, o_in = oracle.get_dispatch_layout(all_idx[rank], E, world)
            assert torch.equal(per_rank.cpu(), o_rank) and torch.equal(per_expert.cpu(), o_expert) and torch.equal(in_rank.cpu(), o_in)
            assert per_node.tolist() == [int(o_in[:, n * P:(n + 1) * P].any(1).sum()) for n in range(nodes)]
            align()
            recv_x, recv_idx, recv_w, per_expert_list, handle, ev = buf.dispatch(
                x, num_tokens_per_rank=per_rank, num_tokens_per_rdma_rank=per_node, is_token_in_rank=in_rank,
                num_tokens_per_expert=per_expert, topk_idx=idx, topk_weights=w)
            ev.current_stream_wait()
            torch.cuda.synchronize()
            buf.check_status()
            assert torch.equal(recv_x.cpu(), flat["recv_x"][rows])
            assert torch.equal(recv_idx.cpu(), flat["recv_topk_idx"][rows])
            assert torch.equal(recv_w.cpu(), flat["recv_topk_weights"][rows])
            assert per_expert_list == flat["num_recv_tokens_per_expert_list"]
            assert handle[6].tolist() == rpm[:, rank].tolist()
            y = torch.zeros_like(recv_x, dtype=torch.float32)
            for e in range(L):
                r_, k_ = (recv_idx == e).nonzero(as_tuple=True)
                y[r_] += recv_x[r_].float() * recv_w[r_, k_].unsqueeze(1)
            align()
            combined, combined_w, _ = buf.combine(y.to(torch.bfloat16), handle, topk_weights=recv_w)
            torch.cuda.synchronize()
            buf.check_status()
            assert oracle.calc_diff(ref, combined.float().cpu()) < 1e-4
            assert (combined_w - w).abs().max() < 1e-6
            align()
            # cached handle with FP8 on both hops
            (rq, rs), a, b, c, d, _ = buf.dispatch(x, handle=handle, quantize_fp8=True)
            torch.cuda.synchronize()
            wq, ws = oracle.per_token_cast_to_fp8(flat["recv_x"][rows])
            assert a is None and torch.equal(rq.cpu().view(torch.uint8), wq.view(torch.uint8)) and torch.equal(rs.cpu(), ws)
            # low latency across domains
            align()
            M = 256
            want = oracle.low_latency_dispatch(all_x, all_idx, M, E, True)[rank]
            (px, ps), cnt, ll_handle, _, _ = buf.low_latency_dispatch(x, idx, M, E, use_fp8=True)
            torch.cuda.synchronize()
            assert torch.equal(cnt.cpu(), want["packed_recv_count"]) and torch.equal(ll_handle[1].cpu(), want["layout_range"])
            for le in range(L):
                n = int(cnt[le])
                assert torch.equal(ll_handle[0][le, :n].cpu(), want["src_info"][le, :n])
                assert torch.equal(px[le, :n].cpu().view(torch.uint8), want["packed_recv_x"][le, :n].view(torch.uint8))
                assert torch.equal(ps[le, :n].cpu(), want["packed_recv_x_scales"][le, :n])
            sim = oracle.per_token_cast_back(px.view(-1, H).cpu(), ps.view(-1, H // 128).cpu()).view(px.shape).cuda()
            align()
            out, _, _ = buf.low_latency_combine(sim, idx, w, ll_handle)
            torch.cuda.synchronize()
            assert oracle.calc_diff(ref, out.float().cpu()) < 9e-4
        buf.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


def _run_ranks(target, world, extra=()):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q) + tuple(extra)) for r in range(world)]
    for p in procs:
        p.start()
    import queue as _queue
    import time
    res, deadline = [], time.time() + 420
    while len(res) < world and time.time() < deadline:
        try:
            res.append(q.get(timeout=5))
        except _queue.Empty:
            if res and any(m != "ok" for _, m in res):
                break
    for p in procs:
        p.join(5)
        if p.is_alive():
            p.terminate()
    for rank, msg in res:
        assert msg == "ok", f"rank {rank}: {msg}"
    assert len(res) == world, f"only {len(res)} of {world} ranks reported"


@pytest.mark.parametrize("world", [2, 8])
def test_low_latency_pressure_hash_equality(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_ranks(_worker_pressure, world)


@pytest.mark.parametrize("world", [2, 4])
def test_shrink_mode_masks_a_silent_rank(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_ranks(_worker_shrink, world)


@pytest.mark.parametrize("world,P", [(2, 1), (4, 2)])
def test_two_level_path_multiprocess(world, P):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_ranks(_worker_two_level, world, (P,))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multiprocess_against_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    import queue as _queue
    import time
    res, deadline = [], time.time() + 420
    while len(res) < world and time.time() < deadline:
        try:
            res.append(q.get(timeout=5))
        except _queue.Empty:
            if res and any(m != "ok" for _, m in res):
                break  # a rank failed; the others may be stuck waiting for it
    for p in procs:
        p.join(5)
        if p.is_alive():
            p.terminate()
    for rank, msg in res:
        assert msg == "ok", f"rank {rank}: {msg}"
    assert len(res) == world, f"only {len(res)} of {world} ranks reported"

