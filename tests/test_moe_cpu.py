"""MoE layer (dispatch -> grouped GEMMs -> combine, autograd both ways) on the CPU backend: one process, and two
gloo ranks, against a dense single-process fp32 loop over all experts."""
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


def _run(rank, world, port, q):
    import traceback
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import deepep_efa_b200 as ep
        from deepep_efa_b200.models.moe import MoEConfig, MoELayer, dense_reference
        from helpers import make_routing, make_tokens
        T, H, I, E, K = 40, 64, 128, 8, 3
        buf = ep.Buffer(dist.group.WORLD, num_nvl_bytes=1 << 20)
        cfg = MoEConfig(hidden=H, intermediate=I, num_experts=E, num_topk=K, init_std=0.1)
        layer = MoELayer(cfg, buf, device=torch.device("cpu"))
        x = make_tokens(T, H, "cpu", seed=rank).requires_grad_(True)
        idx, w = make_routing(T, E, K, "cpu", seed=rank)
        w = w.requires_grad_(True)
        y = layer(x, idx, w)
        loss = (y.float() ** 2).mean()
        loss.backward()
        # dense reference with every rank's experts
        w13s, w2s = [None] * world, [None] * world
        dist.all_gather_object(w13s, layer.w13.detach())
        dist.all_gather_object(w2s, layer.w2.detach())
        w13_all = torch.cat(w13s).float().requires_grad_(True)
        w2_all = torch.cat(w2s).float().requires_grad_(True)
        xr = x.detach().clone().requires_grad_(True)
        wr = w.detach().clone().requires_grad_(True)
        ref = dense_reference(xr, idx, wr, w13_all, w2_all)
        (ref ** 2).mean().backward()
        rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()
        assert rel(y, ref) < 3e-2, rel(y, ref)
        assert rel(x.grad, xr.grad) < 6e-2, rel(x.grad, xr.grad)
        assert rel(w.grad, wr.grad) < 6e-2, rel(w.grad, wr.grad)
        # this rank's expert gradients: every rank's tokens contribute, so compare with the sum of dense grads over ranks
        L = E // world
        g13 = w13_all.grad[rank * L:(rank + 1) * L].clone()
        g2 = w2_all.grad[rank * L:(rank + 1) * L].clone()
        # dense grads above only saw this rank's tokens; add the other ranks' contributions
        parts13, parts2 = [None] * world, [None] * world
        dist.all_gather_object(parts13, w13_all.grad)
        dist.all_gather_object(parts2, w2_all.grad)
        g13 = sum(p[rank * L:(rank + 1) * L] for p in parts13)
        g2 = sum(p[rank * L:(rank + 1) * L] for p in parts2)
        assert rel(layer.w13.grad, g13) < 8e-2, rel(layer.w13.grad, g13)
        assert rel(layer.w2.grad, g2) < 8e-2, rel(layer.w2.grad, g2)
        buf.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


def _launch(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_run, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, msg in res:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_moe_layer_single_rank_cpu():
    _launch(1)


def test_moe_layer_two_gloo_ranks():
    _launch(2)
