"""Headline benchmark: low-latency dispatch + combine latency, plus normal-mode NVLink bandwidth.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Headline metric (lower is better): microseconds for one low-latency ``dispatch`` followed by one
``combine`` with 128 tokens per rank, hidden 7168, 256 experts, top-8, FP8 dispatch / BF16 combine — the
reference's tests/test_low_latency.py protocol (:245-251): inputs stay on the device, an L2 flush (256 MB
write) runs between iterations outside the timed events, every iteration is timed with CUDA events on the
launching stream, and the job-wide number is the MAX over ranks of the per-rank mean.

Also reported: the normal-mode FP8 dispatch / BF16 combine bandwidth (4096 tokens per rank, reference byte
definitions, tests/test_intranode.py:186-214) and an end-to-end number that moves each step's inputs from
pinned host memory and reads the step's result back.

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...``.
Synthetic data: N(0,1) activations, uniform top-8 without replacement, softmax weights.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

# stdout carries exactly one JSON line: whatever NCCL wants to log (its version banner, NCCL_DEBUG output) goes to stderr
os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LL_TOKENS, HIDDEN, NUM_EXPERTS, TOPK = 128, 7168, 256, 8
NORMAL_TOKENS = 4096
PUBLISHED_LL_US = 1145.0  # reference README.md:83, EP16 on 2 nodes (no single-node number is published)


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons of the given physical GPUs while a region runs; settings are only READ.

    A thread polls NVML every ``period_ms`` (the first sample is taken inside ``start``, so even a region of a few
    milliseconds has one); if NVML cannot be loaded, one ``nvidia-smi -lms`` process for all GPUs is used instead, which
    needs a second or two before its first line."""

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # NVML clocks-event-reason bits (nvml.h: nvmlClocksEventReason*)
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, period_ms: int = 20, gpus=None):
        self.period_ms = period_ms
        self.gpus = sorted(gpus) if gpus is not None else None
        self.proc, self.path = None, None
        self._nvml, self._handles, self._thread = None, [], None
        self._stop = threading.Event()
        self._sm, self._smax, self._reasons = [], [], set()

    def _sample_nvml(self):
        n = self._nvml
        for h in self._handles:
            try:
                self._sm.append(float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)))
                self._smax.append(float(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)))
                get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
                bits = int(get(h))
                for name, bit in self.REASON_BITS.items():
                    if bits & bit:
                        self._reasons.add(name)
            except Exception:
                pass

    def _loop(self):
        while not self._stop.wait(self.period_ms / 1e3):
            self._sample_nvml()

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            count = pynvml.nvmlDeviceGetCount()
            ids = self.gpus if self.gpus is not None else list(range(count))
            self._handles = [pynvml.nvmlDeviceGetHandleByIndex(i) for i in ids if i < count]
            self._nvml = pynvml
            self._sample_nvml()
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
            return
        except Exception:
            self._nvml = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms",
                                          str(max(self.period_ms, 100))], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, gpus=None):
        res = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self._nvml is not None:
            self._stop.set()
            if self._thread is not None:
                self._thread.join(timeout=2)
            self._sample_nvml()
            try:
                self._nvml.nvmlShutdown()
            except Exception:
                pass
            if self._sm:
                res.update(sm_mhz=statistics.median(self._sm), sm_max_mhz=max(self._smax), reasons=sorted(self._reasons),
                           samples=len(self._sm))
            return res
        if self.proc is None:
            return res
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, smax, reasons = [], [], set()
        try:
            for line in open(self.path):
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    if gpus is not None and int(p[1]) not in gpus:
                        continue
                    sm.append(float(p[2])), smax.append(float(p[3]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            res.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(smax), reasons=sorted(reasons), samples=len(sm))
        return res


BOUND_CPUS = None  # set by init_dist: how many GPU-local CPU cores this process was pinned to (None: not pinned)


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v for v in vis.split(",") if v != ""]
        try:
            return int(ids[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


def emit(obj) -> None:
    """Write the result line to the process's original stdout (kept on the sys module: this file can be loaded twice, as
    __main__ and as 'bench')."""
    stream = getattr(sys, "_deepep_result_stream", None) or sys.stdout
    stream.write(json.dumps(obj) + "\n")
    stream.flush()


def ramp_clocks(local_rank: int, max_seconds: float = 12.0) -> None:
    """Untimed: keep the SMs busy with a light streaming kernel until the SM clock reads (nearly) its maximum.

    An idle GPU sits at its lowest clock and some machines take several seconds to ramp up; a latency benchmark that
    starts before that measures the ramp, not the kernels. Clocks are only read (NVML), never set."""
    import time
    buf = torch.empty(64 << 20, dtype=torch.float32, device="cuda")
    handle = nvml = None
    try:
        import pynvml as nvml
        nvml.nvmlInit()
        handle = nvml.nvmlDeviceGetHandleByIndex(physical_gpu_index(local_rank))
        top = nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM)
    except Exception:
        handle = None
    t0, last = time.time(), None
    while time.time() - t0 < max_seconds:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(40):
            buf.add_(1.0)
        e.record()
        torch.cuda.synchronize()
        if handle is not None:
            try:
                if nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM) >= 0.93 * top:
                    break
                continue
            except Exception:
                handle = None
        ms = s.elapsed_time(e)  # no NVML: stop when the same work stops getting faster
        if last is not None and ms > 0.97 * last and time.time() - t0 > 1.0:
            break
        last = ms
    if nvml is not None:
        try:
            nvml.nvmlShutdown()
        except Exception:
            pass


# ------------------------------------------------------------------------------------------------
# helpers
# ------------------------------------------------------------------------------------------------
def bind_to_gpu_local_cpus(local_rank: int):
    """Pin this process to the CPU cores that NVML reports as local to its GPU (same socket / PCIe root), before any pinned
    host memory is allocated: the host-to-device and device-to-host copies of the end-to-end number then stay on one NUMA
    node. Process affinity only (nothing that outlasts the process); best effort, both arms go through it. Returns the
    number of CPUs bound to, or None when NVML or the cpuset would not allow it."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(physical_gpu_index(local_rank))
        words = pynvml.nvmlDeviceGetCpuAffinity(h, ((os.cpu_count() or 64) + 63) // 64)
        local = {i * 64 + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        cpus = local & os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return None


def init_dist(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == n_gpus, f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n_gpus}"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    global BOUND_CPUS
    BOUND_CPUS = bind_to_gpu_local_cpus(local_rank)
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
    return rank, world, local_rank


def max_over_ranks(value: float) -> float:
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed_samples(fn, steps: int, flush: torch.Tensor):
    """K iterations, each [L2 flush][event][fn][event]; returns the K per-iteration times in milliseconds."""
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    dist.barrier()
    torch.cuda.synchronize()
    for i in range(steps):
        flush.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    dist.barrier()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def timed_loop(fn, steps: int, flush: torch.Tensor):
    """Mean milliseconds per iteration of :func:`timed_samples`."""
    return sum(timed_samples(fn, steps, flush)) / steps


def spread_us(samples_ms):
    """Median and minimum (microseconds, max over ranks) next to the mean that the headline reports."""
    return {"median": round(max_over_ranks(statistics.median(samples_ms) * 1e3), 3),
            "min": round(max_over_ranks(min(samples_ms) * 1e3), 3)}


def nccl_all_to_all_floor(rank: int, world: int, topk_idx: torch.Tensor, bytes_per_selection: int, steps: int, flush: torch.Tensor,
                          per_rank_once: bool = False):
    """Time of one plain ``dist.all_to_all_single`` (NCCL over NVLink) that moves the byte volume of a dispatch or combine
    with this routing: per destination rank, ``bytes_per_selection`` for every (token, expert) selection that lives there
    (``per_rank_once``: for every token that has at least one expert there). This is the collective the reference's
    single-node low-latency path is built on (deep_ep/buffer.py:2297, 2735); no packing, casting or reduction is included."""
    L = NUM_EXPERTS // world
    dest = torch.where(topk_idx >= 0, topk_idx // L, torch.full_like(topk_idx, -1))
    if per_rank_once:
        counts = torch.stack([(dest == r).any(dim=1).sum() for r in range(world)])
    else:
        counts = torch.stack([(dest == r).sum() for r in range(world)])
    send_counts = (counts * bytes_per_selection).to(torch.int64)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts)
    send_split, recv_split = send_counts.tolist(), recv_counts.tolist()
    send = torch.empty(max(sum(send_split), 1), dtype=torch.uint8, device="cuda")
    recv = torch.empty(max(sum(recv_split), 1), dtype=torch.uint8, device="cuda")

    def fn():
        dist.all_to_all_single(recv, send, recv_split, send_split)

    for _ in range(3):
        fn()
    return max_over_ranks(timed_loop(fn, steps, flush) * 1e3)


def make_inputs(rank: int, tokens: int, masked_fraction: float = 0.0):
    g = torch.Generator(device="cpu").manual_seed(rank)
    x = torch.randn(tokens, HIDDEN, generator=g).to(torch.bfloat16)
    topk_idx = torch.rand(tokens, NUM_EXPERTS, generator=g).topk(TOPK, dim=-1).indices.to(torch.int64)
    topk_w = torch.softmax(torch.randn(tokens, TOPK, generator=g), dim=-1).float()
    if masked_fraction > 0:
        topk_idx[torch.rand(tokens, TOPK, generator=g) < masked_fraction] = -1
    return x, topk_idx, topk_w


# ------------------------------------------------------------------------------------------------
# this library
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import deepep_efa_b200 as ep
    from deepep_efa_b200.reference import oracle

    rank, world, local_rank = init_dist(args.gpus)
    group = dist.group.WORLD
    steps, warmup = args.steps, max(args.warmup, 3)
    ll_bytes = ep.Buffer.get_low_latency_rdma_size_hint(LL_TOKENS, HIDDEN, world, NUM_EXPERTS)
    nvl_bytes = ep.Config(32, 6, 256, 6, 128).get_nvl_buffer_size_hint(HIDDEN * 2, world, NORMAL_TOKENS) if not args.skip_normal else (2 << 20)
    nvl_bytes += NUM_EXPERTS * LL_TOKENS * HIDDEN * 2 + (16 << 20)  # room for the stand-in expert output [L, world*T, hidden] in symmetric memory
    buf = ep.Buffer(group, num_nvl_bytes=nvl_bytes, num_rdma_bytes=ll_bytes, low_latency_mode=True, explicitly_destroy=True)
    flush = torch.empty(256 << 20, dtype=torch.int8, device="cuda")

    # ---------------- low-latency dispatch + combine (headline) ----------------
    x_h, idx_h, w_h = make_inputs(rank, LL_TOKENS)
    x, topk_idx, topk_w = x_h.cuda(), idx_h.cuda(), w_h.cuda()
    L = NUM_EXPERTS // world
    # The stand-in for the expert GEMM's output. The headline step keeps it in symmetric memory (Buffer.empty_symmetric, where a
    # user of this library lets the last expert GEMM write): the home ranks then pull the rows they need straight from it. The same
    # values in an ordinary tensor (combine pushes them through a stage) are timed beside it as `ll_plain_tensor_us`.
    sim_gemm_plain = torch.randn(L, world * LL_TOKENS, HIDDEN, device="cuda").to(torch.bfloat16) * 0.1
    sim_gemm_out = buf.empty_symmetric([L, world * LL_TOKENS, HIDDEN], torch.bfloat16)
    sim_gemm_out.copy_(sim_gemm_plain)
    out = torch.empty(LL_TOKENS, HIDDEN, dtype=torch.bfloat16, device="cuda")

    def ll_step():
        _, _, handle, _, _ = buf.low_latency_dispatch(x, topk_idx, LL_TOKENS, NUM_EXPERTS, use_fp8=True)
        buf.low_latency_combine(sim_gemm_out, topk_idx, topk_w, handle, out=out)

    # correctness of exactly what is timed: combine(dispatch(x)) == x * sum(w) through the FP8 wire format
    (px, ps), cnt, handle, _, _ = buf.low_latency_dispatch(x, topk_idx, LL_TOKENS, NUM_EXPERTS, use_fp8=True)
    back = oracle.per_token_cast_back(px.view(-1, HIDDEN), ps.view(-1, HIDDEN // 128)).view(px.shape)
    chk, _, _ = buf.low_latency_combine(back, topk_idx, topk_w, handle)
    torch.cuda.synchronize()
    buf.check_status()
    diff = oracle.calc_diff(x.float() * topk_w.sum(1, keepdim=True), chk.float())
    assert diff < 9e-4, f"low-latency round trip is wrong: diff={diff}"

    # one sampler (rank 0) for all GPUs of the job; it runs from the warm-up through both timed regions (device-timed and
    # end-to-end), which execute the same workload back to back
    ramp_clocks(local_rank)
    sampler = ClockSampler(gpus={physical_gpu_index(r) for r in range(world)}) if rank == 0 else None
    if sampler is not None:
        sampler.start()
    for _ in range(warmup):
        ll_step()
    ll_samples = timed_samples(ll_step, steps, flush)
    buf.check_status(sync=True)
    ll_us = max_over_ranks(sum(ll_samples) / steps * 1e3)
    ll_spread = spread_us(ll_samples)

    # the same pair with the expert outputs in an ordinary device tensor: must give the same bits
    plain_us = None
    if not args.skip_breakdown:
        def ll_step_plain():
            _, _, handle, _, _ = buf.low_latency_dispatch(x, topk_idx, LL_TOKENS, NUM_EXPERTS, use_fp8=True)
            buf.low_latency_combine(sim_gemm_plain, topk_idx, topk_w, handle, out=out)

        ll_step()
        want = out.clone()
        out.zero_()
        ll_step_plain()
        torch.cuda.synchronize()
        assert torch.equal(out, want), "combine of an ordinary tensor differs from the combine of the symmetric one"
        for _ in range(warmup):
            ll_step_plain()
        plain_us = round(max_over_ranks(timed_loop(ll_step_plain, max(10, min(steps, 200)), flush) * 1e3), 3)
        buf.check_status(sync=True)

    # phase stamps of one dispatch + combine pair (first and last CTA of each kernel, %globaltimer, µs from the start of dispatch)
    stamps = None
    if args.ll_stamps:
        buf.runtime.enable_trace(True)
        for _ in range(2):
            dist.barrier()
            torch.cuda.synchronize()
            ll_step()
            torch.cuda.synchronize()
            tr = buf.runtime.read_trace()
        base = tr[(4 * 2 + 0) * 16]
        mine = {f"{name}_{'first' if slot == 0 else 'last'}_cta": [round((v - base) / 1e3, 2) if v else None for v in tr[(fam * 2 + slot) * 16:(fam * 2 + slot) * 16 + 7]]
                for fam, name in ((4, "ll_dispatch"), (5, "ll_combine")) for slot in (0, 1)}
        buf.runtime.enable_trace(False)
        allst = [None] * world
        dist.all_gather_object(allst, mine)
        stamps = {"rank0": allst[0], f"rank{world - 1}": allst[-1],
                  "legend": {"ll_dispatch_first_cta": "start, idx loaded, counts of lower ranks, rows known, rows stored, release done, exit",
                             "ll_dispatch_last_cta": "start, -, counts sent, all counts, layout out, all rows in, exit",
                             "ll_combine (pull)": "start, offset posted, -, -, peers' offsets known, rows reduced, exit"}}

    # the same pair with the expert outputs in the zero-copy combine buffer (where the decode path's last GEMM writes them):
    # pulled like the symmetric tensor, without the closing "readers done" round a caller-owned tensor needs
    zc_us = None
    if not args.skip_breakdown:
        for _ in range(2):  # both parities hold the stand-in GEMM output
            _, _, h0, _, _ = buf.low_latency_dispatch(x, topk_idx, LL_TOKENS, NUM_EXPERTS, use_fp8=True)
            buf.get_next_low_latency_combine_buffer(h0).copy_(sim_gemm_out)
            buf.low_latency_combine(sim_gemm_out, topk_idx, topk_w, h0, out=out)

        def ll_step_zero_copy():
            _, _, handle, _, _ = buf.low_latency_dispatch(x, topk_idx, LL_TOKENS, NUM_EXPERTS, use_fp8=True)
            buf.low_latency_combine(sim_gemm_out, topk_idx, topk_w, handle, zero_copy=True, out=out)

        ll_step()
        want = out.clone()
        out.zero_()
        ll_step_zero_copy()
        torch.cuda.synchronize()
        assert torch.equal(out, want), "combine from the zero-copy buffer differs from the combine of the caller's tensor"
        for _ in range(warmup):
            ll_step_zero_copy()
        zc_us = round(max_over_ranks(timed_loop(ll_step_zero_copy, max(10, min(steps, 200)), flush) * 1e3), 3)
        buf.check_status(sync=True)

    # separate dispatch / combine times (same protocol)
    state = {}

    def ll_dispatch_only():
        state["h"] = buf.low_latency_dispatch(x, topk_idx, LL_TOKENS, NUM_EXPERTS, use_fp8=True)[2]

    def ll_combine_only():
        buf.low_latency_combine(sim_gemm_out, topk_idx, topk_w, state["h"], out=out)

    sub_steps = max(10, min(steps, 200))
    disp_us = comb_us = None
    if not args.skip_breakdown:
        # dispatch and combine alternate on the wire; time each half with its own events
        d_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(sub_steps)]
        c_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(sub_steps)]
        dist.barrier()
        torch.cuda.synchronize()
        for i in range(sub_steps):
            flush.zero_()
            d_ev[i][0].record(); ll_dispatch_only(); d_ev[i][1].record()
            c_ev[i][0].record(); ll_combine_only(); c_ev[i][1].record()
        torch.cuda.synchronize()
        disp_us = max_over_ranks(sum(a.elapsed_time(b) for a, b in d_ev) / sub_steps * 1e3)
        comb_us = max_over_ranks(sum(a.elapsed_time(b) for a, b in c_ev) / sub_steps * 1e3)

    # ---------------- plain NCCL all-to-all of the same byte volumes (what a library call alone costs) ----------------
    nccl_floor = None
    if not args.skip_breakdown:
        try:
            d_us = nccl_all_to_all_floor(rank, world, topk_idx, HIDDEN + HIDDEN // 128 * 4 + 16, sub_steps, flush)
            c_us = nccl_all_to_all_floor(rank, world, topk_idx, HIDDEN * 2, sub_steps, flush)
            nccl_floor = {"ll_dispatch_bytes_us": round(d_us, 2), "ll_combine_bytes_us": round(c_us, 2), "sum_us": round(d_us + c_us, 2),
                          "what": "dist.all_to_all_single of the per-destination byte volumes only (no cast, pack, count exchange or reduce)"}
        except Exception as e:  # pragma: no cover
            nccl_floor = {"error": f"{type(e).__name__}: {str(e)[:200]}"}

    # ---------------- end to end: pinned host inputs in, result out, every step ----------------
    # The step's inputs (activations, expert ids, weights) sit packed in ONE pinned host buffer and cross PCIe as one
    # host-to-device copy; the combine kernel writes the step's result straight into pinned host memory (its stores are the
    # device-to-host transfer). Both transfers happen inside the timed region of every step.
    nx, ni, nw = x_h.numel() * 2, idx_h.numel() * 8, w_h.numel() * 4
    stage_p = torch.empty(nx + ni + nw, dtype=torch.uint8).pin_memory()
    stage_p[:nx].view(torch.bfloat16).view_as(x_h).copy_(x_h)
    stage_p[nx:nx + ni].view(torch.int64).view_as(idx_h).copy_(idx_h)
    stage_p[nx + ni:].view(torch.float32).view_as(w_h).copy_(w_h)
    stage_d = torch.empty(nx + ni + nw, dtype=torch.uint8, device="cuda")
    x_d = stage_d[:nx].view(torch.bfloat16).view_as(x)
    idx_d = stage_d[nx:nx + ni].view(torch.int64).view_as(topk_idx)
    w_d = stage_d[nx + ni:].view(torch.float32).view_as(topk_w)
    out_p = torch.empty(LL_TOKENS, HIDDEN, dtype=torch.bfloat16).pin_memory()

    x_p = stage_p[:nx].view(torch.bfloat16).view_as(x_h)     # the activations where they sit in pinned host memory
    meta_p, meta_d = stage_p[nx:], stage_d[nx:]             # (topk_idx | topk_weights), 12 KB

    def make_e2e(src, store_to_host, x_from_host=False):
        def step():
            if x_from_host:
                # ids and weights by one small copy; the dispatch kernel reads every token's row from pinned host memory
                # itself (each row exactly once), so the activations cross PCIe inside the kernel instead of in front of it
                meta_d.copy_(meta_p, non_blocking=True)
                _, _, h, _, _ = buf.low_latency_dispatch(x_p, idx_d, LL_TOKENS, NUM_EXPERTS, use_fp8=True)
            else:
                stage_d.copy_(stage_p, non_blocking=True)
                _, _, h, _, _ = buf.low_latency_dispatch(x_d, idx_d, LL_TOKENS, NUM_EXPERTS, use_fp8=True)
            if store_to_host:
                buf.low_latency_combine(src, idx_d, w_d, h, out=out_p)   # the combine kernel's stores are the device-to-host transfer
            else:
                buf.low_latency_combine(src, idx_d, w_d, h, out=out)
                out_p.copy_(out, non_blocking=True)                     # result produced on the device, copied out by the copy engine
        return step

    # the host copy of the result must equal what the device path produces
    out_p.zero_()
    make_e2e(sim_gemm_out, True)()
    ll_step()
    torch.cuda.synchronize()
    assert torch.equal(out_p, out.cpu()), "end-to-end result in pinned host memory differs from the device result"
    out_p.zero_()
    make_e2e(sim_gemm_out, True, x_from_host=True)()
    torch.cuda.synchronize()
    assert torch.equal(out_p, out.cpu()), "end-to-end result with the activations read from pinned host memory differs from the device result"
    # Which way of getting the result to the host is faster depends on the machine (where the pinned pages sit relative to the
    # GPU's PCIe root) and on where the expert outputs live; every combination is timed with the full protocol and the fastest
    # one is the reported value.
    e2e_variants = {}
    for name, fn in (("symmetric_expert_output__result_stored_to_pinned_host_by_kernel", make_e2e(sim_gemm_out, True)),
                     ("symmetric_expert_output__result_copied_out_by_copy_engine", make_e2e(sim_gemm_out, False)),
                     ("ordinary_expert_output__result_stored_to_pinned_host_by_kernel", make_e2e(sim_gemm_plain, True)),
                     ("ordinary_expert_output__result_copied_out_by_copy_engine", make_e2e(sim_gemm_plain, False)),
                     ("x_read_from_pinned_host_by_dispatch_kernel__symmetric_expert_output__result_stored_to_pinned_host_by_kernel",
                      make_e2e(sim_gemm_out, True, x_from_host=True)),
                     ("x_read_from_pinned_host_by_dispatch_kernel__symmetric_expert_output__result_copied_out_by_copy_engine",
                      make_e2e(sim_gemm_out, False, x_from_host=True))):
        for _ in range(warmup):
            fn()
        smp = timed_samples(fn, steps, flush)
        e2e_variants[name] = {"value": round(max_over_ranks(sum(smp) / steps * 1e3), 3), **spread_us(smp)}
    e2e_how = min(e2e_variants, key=lambda k: e2e_variants[k]["value"])
    e2e_us = e2e_variants[e2e_how]["value"]
    e2e_spread = {"median": e2e_variants[e2e_how]["median"], "min": e2e_variants[e2e_how]["min"]}
    h2d = stage_p.numel()
    d2h = out_p.numel() * 2
    buf.check_status(sync=True)
    clocks = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    if sampler is not None:
        clocks = sampler.stop({physical_gpu_index(r) for r in range(world)})

    # ---------------- masked-slot sweep (2 % / 5 % of the top-k slots are -1) ----------------
    masked = {}
    if not args.skip_breakdown:
        for frac in (0.02, 0.05):
            _, mi, mw = make_inputs(rank, LL_TOKENS, frac)
            mi, mw = mi.cuda(), mw.cuda()

            def masked_step():
                _, _, h, _, _ = buf.low_latency_dispatch(x, mi, LL_TOKENS, NUM_EXPERTS, use_fp8=True)
                buf.low_latency_combine(sim_gemm_out, mi, mw, h, out=out)

            for _ in range(max(warmup, 5)):
                masked_step()
            masked[f"{int(frac * 100)}pct"] = round(max_over_ranks(timed_loop(masked_step, sub_steps, flush) * 1e3), 2)

    # ---------------- normal mode: FP8 dispatch / BF16 combine bandwidth ----------------
    normal = None
    if not args.skip_normal:
        normal = bench_normal(buf, rank, world, flush, max(10, min(steps, 50)), warmup)

    buf.destroy()
    # ---------------- model-level numbers on top of the library (bench_moe.py holds the full versions) ----------------
    moe = {}
    if not args.skip_moe:
        import bench_moe
        moe = bench_moe.moe_extras("ours", rank, world, steps=args.moe_steps, warmup=3)

    result = {
        "metric": "ll_dispatch_combine_us",
        "value": round(ll_us, 3),
        "unit": "us",
        "n_gpus": world,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": round(ll_us / 1e3, 6),
        "higher_is_better": False,
        "scaling": "weak",
        "vs_baseline": round(ll_us / PUBLISHED_LL_US, 5),
        "dtype": "fp8_e4m3 dispatch / bf16 combine",
        "data": "synthetic: N(0,1) bf16 activations, uniform top-8 of 256 experts without replacement, softmax weights",
        "config": {"model": "low-latency EP dispatch+combine", "tokens_per_rank": LL_TOKENS, "global_batch": LL_TOKENS * world,
                   "seq_len": 1, "hidden": HIDDEN, "num_experts": NUM_EXPERTS, "topk": TOPK, "parallelism": f"ep{world}",
                   "l2": "256 MB flush between timed iterations", "timing": "CUDA events per iteration, max over ranks"},
        "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                   "samples": clocks["samples"]},
        "e2e": {"value": round(e2e_us, 3), "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "median": e2e_spread["median"], "min": e2e_spread["min"],
                "how": "inputs packed in one pinned buffer (x|topk_idx|topk_weights), crossing PCIe every step either by one H2D copy or "
                       "(x) by the dispatch kernel's own loads; fastest variant: " + e2e_how.replace("__", "; ").replace("_", " "),
                "process_pinned_to_gpu_local_cpus": BOUND_CPUS,
                "variants": e2e_variants},
        "value_median": ll_spread["median"],
        "value_min": ll_spread["min"],
        "ll_zero_copy_us": zc_us,
        "ll_plain_tensor_us": plain_us,
        "ll_stamps_us": stamps,
        "notes": "our arm passes out= (a preallocated result tensor) and keeps the stand-in expert output in symmetric memory "
                 "(Buffer.empty_symmetric; home ranks pull from it; ll_plain_tensor_us is the same call on an ordinary tensor); "
                 "the reference's single-node path allocates its own result and takes an ordinary tensor",
        "gpu_launches": 2 * steps,
        "ll_dispatch_us": None if disp_us is None else round(disp_us, 2),
        "ll_combine_us": None if comb_us is None else round(comb_us, 2),
        "ll_masked_us": masked,
        "nccl_all_to_all_floor": nccl_floor,
        "normal": normal,
        "impl": "deepep_efa_b200",
    }
    result.update(moe)
    if rank == 0:
        emit(result)
    dist.destroy_process_group()


def C_ext():
    from deepep_efa_b200 import _ext
    return _ext.load()


def bench_normal(buf, rank, world, flush, steps, warmup):
    """Normal-mode dispatch (BF16 in, FP8 on the wire, quantised inside the dispatch kernel) and BF16 combine."""
    import deepep_efa_b200 as ep

    x_h, idx_h, w_h = make_inputs(rank + 100, NORMAL_TOKENS)
    x, topk_idx, topk_w = x_h.cuda(), idx_h.cuda(), w_h.cuda()
    per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(topk_idx, NUM_EXPERTS)
    state = {}

    def do_dispatch():
        state["r"] = buf.dispatch(x, num_tokens_per_rank=per_rank, is_token_in_rank=in_rank, num_tokens_per_expert=per_expert,
                                  topk_idx=topk_idx, topk_weights=topk_w, quantize_fp8=True)

    do_dispatch()
    (rx, rs), _, _, _, handle, _ = state["r"]
    n_recv = rx.size(0)
    # correctness of what is timed (the reference's check, tests/test_intranode.py:80-86): a payload that is constant per
    # source rank must arrive as one constant segment per source, and combining it must give x * (ranks the token went to)
    xc = torch.full((NORMAL_TOKENS, HIDDEN), float(rank + 1), dtype=torch.bfloat16, device="cuda")
    rc, *_ = buf.dispatch(xc, handle=handle)
    rpm = handle[0].cpu()
    start = 0
    for src in range(world):
        end = int(rpm[src, rank])
        seg = rc[start:end]
        assert seg.numel() == 0 or (float(seg.float().min()) == src + 1 and float(seg.float().max()) == src + 1), f"rows of source {src} are wrong"
        start = end
    assert start == n_recv
    back, _, _ = buf.combine(rc, handle)
    hits = in_rank.sum(dim=1, keepdim=True).float()
    assert torch.equal(back.float(), xc.float() * hits), "combine(dispatch(x)) != x * hits"
    del rc, back
    y = buf.empty_symmetric([n_recv, HIDDEN], torch.bfloat16)
    y.normal_()

    def do_cached_dispatch():
        state["c"] = buf.dispatch(x, handle=handle, quantize_fp8=True)

    xq = C_ext().per_token_cast_to_fp8(x, False, False)  # pre-quantised input, the form the reference's protocol feeds

    def do_cached_dispatch_prequant():
        state["p"] = buf.dispatch(xq, handle=handle)

    def do_combine():
        state["o"] = buf.combine(y, handle)

    res = {}
    for name, fn in (("dispatch_fp8", do_dispatch), ("dispatch_fp8_cached", do_cached_dispatch),
                     ("dispatch_fp8_cached_prequantized", do_cached_dispatch_prequant), ("combine_bf16", do_combine)):
        for _ in range(warmup):
            fn()
        ms = max_over_ranks(timed_loop(fn, steps, flush))
        nbytes = n_recv * HIDDEN * 2
        if name.startswith("dispatch"):
            nbytes = nbytes * (1 + 4 / 128) / 2
        res[name] = {"ms": round(ms, 4), "GBps": round(nbytes / 1e9 / (ms / 1e3), 1)}
    # the same kernels at the reference's SM budget (24), next to the default grid above
    cfg24 = ep.Config(24, 6, 256, 6, 128)
    for name, fn in (("dispatch_fp8_cached_prequantized_24sms", lambda: state.__setitem__("p", buf.dispatch(xq, handle=handle, config=cfg24))),
                     ("combine_bf16_24sms", lambda: state.__setitem__("o", buf.combine(y, handle, config=cfg24)))):
        for _ in range(warmup):
            fn()
        ms = max_over_ranks(timed_loop(fn, steps, flush))
        nbytes = n_recv * HIDDEN * 2 * ((1 + 4 / 128) / 2 if name.startswith("dispatch") else 1)
        res[name] = {"ms": round(ms, 4), "GBps": round(nbytes / 1e9 / (ms / 1e3), 1)}
    try:
        d_us = nccl_all_to_all_floor(rank, world, topk_idx, int(HIDDEN * (1 + 4 / 128)), steps, flush, per_rank_once=True)
        c_us = nccl_all_to_all_floor(rank, world, topk_idx, HIDDEN * 2, steps, flush, per_rank_once=True)
        res["nccl_all_to_all_floor"] = {"dispatch_fp8_ms": round(d_us / 1e3, 4), "dispatch_fp8_GBps": round(n_recv * HIDDEN * 2 * (1 + 4 / 128) / 2 / 1e9 / (d_us / 1e6), 1),
                                        "combine_bf16_ms": round(c_us / 1e3, 4), "combine_bf16_GBps": round(n_recv * HIDDEN * 2 / 1e9 / (c_us / 1e6), 1),
                                        "what": "dist.all_to_all_single of the same rows, one per (token, destination rank); GB/s with the same byte definition"}
    except Exception as e:  # pragma: no cover
        res["nccl_all_to_all_floor"] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
    res["default_num_sms"] = {"dispatch": ep.Buffer.get_dispatch_config(world).num_sms, "combine": ep.Buffer.get_combine_config(world).num_sms}
    res["checked"] = "constant-per-source payload arrives as one segment per source; combine(dispatch(x)) == x * hits"
    buf.check_status(sync=True)
    res["recv_tokens"] = int(n_recv)
    res["bytes_definition"] = "recv_x.numel()*2 (x(1+4/128)/2 for FP8), all source ranks including self"
    res["note"] = ("dispatch_fp8: fresh call (count exchange + host sync + BF16->FP8 inside the kernel); *_cached reuse the handle as the "
                   "reference's tuning protocol does (tests/test_intranode.py:200-214)")
    return res


# ------------------------------------------------------------------------------------------------
# reference arm
# ------------------------------------------------------------------------------------------------
def run_reference(args):
    from baseline import reference_arm
    reference_arm.main(args)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-normal", action="store_true")
    ap.add_argument("--skip-breakdown", action="store_true")
    ap.add_argument("--skip-moe", action="store_true", help="leave out the model-level extras (fused MoE forward, decode step, training step)")
    ap.add_argument("--moe-steps", type=int, default=5)
    ap.add_argument("--ll-stamps", action="store_true", help="add the device-side phase stamps of one dispatch + combine pair")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    # Libraries (NCCL's version banner among them) write to file descriptor 1 behind Python's back; the contract is ONE
    # JSON line on stdout. Keep a private handle on the real stdout for that line and point fd 1 at stderr for everything else.
    sys._deepep_result_stream = os.fdopen(os.dup(1), "w")
    sys.stdout.flush()
    os.dup2(2, 1)
    main()
