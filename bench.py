"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Primary workload (the configuration the headline metric is quoted on): flash_attention forward +
backward, bf16, B=4, H=32, L=4096, D=128, causal, q/k/v/dO ~ N(0,1).  A step is one forward and one
backward over that batch THROUGH THE PUBLIC OPERATOR (flash_attention + torch.autograd.grad).
`value` is matmul-only TFLOP/s (the reference benchmark's convention: forward 4*B*H*M*N*D*0.5 for
causal, backward 2.5x that) with inputs resident in HBM, over exactly K steps that follow the warm-up
without a gap; `value_sustained` is the same loop run for at least a second; `e2e` is the same metric
with the inputs in pinned host memory, every step copying q, k, v, dO to the device and o, dq, dk, dv
back, next to the plain-copy ceiling of the same bytes.  The per-kernel split behind `roofline` comes
from a second pass of K steps, run back to back with the timed one, that enqueues the backward's
stages one C call at a time with CUDA events between them.

The same JSON line carries, as sub-records: "paged" (the decode workload: 64 sequences, 32/8 heads,
head 128, block 16, contexts in [1024, 32768], 512-token partitions) as HBM GB/s, "cfg3" (fp16 D=64
L=8192 non-causal with the log-normaliser), "piecewise" (B=1 H=48 L=16384 D=128, threshold 4096),
"decode", "rotary", a sequence-length "sweep" on the reference benchmark's grid, and "strong".

With N > 1 (launched by torch.distributed.run): the headline is weak scaling (every rank runs the
per-GPU workload, no data-path collective, all ranks' work over the slowest rank's device time);
"strong" splits ONE copy of the workloads over the ranks: the 128 (batch, head) pairs of the
dense configuration, and the 64 sequences of the decode configuration by longest-first assignment,
each rank holding only its sequences' KV blocks, the outputs all-gathered (NCCL) inside the timed region.

`--impl reference` times the reference's CPU implementation of the path (its PyTorch oracle, as
restated under oracle/) on the host cores, on a bounded sample of the same workload.
"""
import argparse
import ctypes
import datetime
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

_T0 = time.perf_counter()

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG1 = dict(B=2, H=4, L=256, D=64, causal=True, dtype="f32")
FLASH_CFG = dict(B=4, H=32, Hk=32, L=4096, D=128, causal=True, dtype="bf16")
CFG3 = dict(B=2, H=16, Hk=16, L=8192, D=64, causal=False, dtype="fp16")
PIECEWISE_CFG = dict(B=1, H=48, L=16384, D=128, w=4096, causal=True, dtype="bf16")
PAGED_CFG = dict(num_seqs=64, q_heads=32, kv_heads=8, head=128, block=16, ctx_lo=1024, ctx_hi=32768,
                 partition=512, num_splits=64)
SM_COUNT, EX2_PER_CLK_PER_SM = 148, 16


def flash_flops(B, H, M, N, D, causal):
    fwd = 4.0 * B * H * M * N * D * (0.5 if causal else 1.0)
    return fwd, 2.5 * fwd


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tflops_burst=p["bf16_tflops"],
                    tflops_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


def tensor_roofline(kernel, flop_per_launch, ms_per_launch, clocks=None, **extra):
    """Roofline record of a tensor-bound kernel.  The denominator follows the regime the timed loop
    actually ran in, read off the SM clocks sampled during it: the burst cuBLAS figure when the
    clock sat at its maximum with no power cap reported, the sustained figure otherwise (and when
    there is no clock record).  The fractions of both peaks ride along."""
    peaks = load_peaks()
    achieved = flop_per_launch / (ms_per_launch * 1e-3) / 1e12
    burst = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz")
                 and clocks["sm_mhz"] >= 0.97 * clocks["sm_max_mhz"]
                 and "sw_power_cap" not in clocks.get("reasons", []))
    peak = peaks["tflops_burst"] if burst else peaks["tflops_sustained"]
    out = dict(bound="tensor", kernel=kernel, achieved=round(achieved, 2), peak=peak, unit="TFLOP/s",
               frac=round(achieved / peak, 4),
               peak_source=peaks["source"] + (" (burst cuBLAS bf16: SM clock at maximum, no power cap, during the timed loop)"
                                              if burst else
                                              " (sustained cuBLAS bf16: the timed loop ran power-capped, or has no clock record)"),
               regime="burst" if burst else "sustained",
               peak_burst=peaks["tflops_burst"], frac_burst=round(achieved / peaks["tflops_burst"], 4),
               peak_sustained=peaks["tflops_sustained"],
               frac_sustained=round(achieved / peaks["tflops_sustained"], 4),
               frac_nominal_2250=round(achieved / 2250.0, 4))
    out.update(extra)
    return out


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi; `window(t0, t1)` gives the
    record of the samples taken between two time.time() stamps."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path, self.rows = index, None, None, []

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "20", "-f", self.path],
                stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        try:
            lines = [r.strip().split(", ") for r in open(self.path) if r.strip()]
            os.unlink(self.path)
        except OSError:
            lines = []
        for r in lines:
            if len(r) < 7:
                continue
            try:
                stamp = datetime.datetime.strptime(r[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                self.rows.append((stamp, float(r[1]), float(r[2]),
                                  [n for n, v in zip(self.NAMES, r[3:7]) if v.strip().lower() == "active"]))
            except ValueError:
                continue
        self.proc = None

    def window(self, t0=None, t1=None):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        rows = [r for r in self.rows if (t0 is None or r[0] >= t0) and (t1 is None or r[0] <= t1)]
        if not rows and self.rows and t0 is not None:
            # a region shorter than the sampling period: the sample nearest to its middle
            mid = 0.5 * (t0 + t1)
            rows = [min(self.rows, key=lambda r: abs(r[0] - mid))]
            out["nearest_sample_ms_away"] = round(abs(rows[0][0] - mid) * 1e3, 1)
        if rows:
            out["sm_mhz"] = statistics.median(r[1] for r in rows)
            out["sm_max_mhz"] = rows[-1][2]
            out["reasons"] = sorted({n for r in rows for n in r[3]})
            out["samples"] = len(rows)
        return out


# ------------------------------------------------------------------------------------------------
# distributed plumbing
# ------------------------------------------------------------------------------------------------
def dist_setup():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        # the communicator is built here, by a first collective, long before any timed region: a
        # barrier that builds it between a warm-up and its timed loop would leave the GPU idle for
        # seconds and hand the loop boost clocks
        t = torch.zeros(1, device=torch.device("cuda", local))
        dist.all_reduce(t)
        torch.cuda.synchronize()
        return dist, rank, world, local
    return None, 0, 1, 0


def trace(rank, what):
    """Progress marks on stderr (rank 0): if a run is cut short, the log says where it was."""
    if rank == 0:
        print("[bench %.1fs] %s" % (time.perf_counter() - _T0, what), file=sys.stderr, flush=True)


def max_over_ranks(dist, value, device):
    if dist is None:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(dist):
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()


def extra_warmup_calls(dist, device, warm, warm_seconds, spent):
    """How many more warm-up calls to make after `warm` calls took `spent` seconds, so that the
    warm-up lasts about `warm_seconds`: each rank proposes a count from its own pace and the largest
    wins, so every rank makes the same number (the timed function may hold a collective)."""
    extra = 0
    if spent < warm_seconds:
        extra = int((warm_seconds - spent) / max(spent / max(warm, 1), 1e-5)) + 1
    return int(max_over_ranks(dist, float(extra), device))


def timed(fn, steps, dist, device, warm=3, warm_seconds=0.0):
    """`warm` untimed calls (continued until `warm_seconds` of load), then, after a barrier among the
    ranks and with no idle gap on this GPU, `steps` timed calls; returns (ms per call, max over
    ranks; per-call device times of this rank)."""
    t_w = time.perf_counter()
    for _ in range(warm):
        fn()
    extra = 0
    if warm_seconds > 0.0:
        torch.cuda.synchronize()
        extra = extra_warmup_calls(dist, device, warm, warm_seconds, time.perf_counter() - t_w)
    for i in range(extra):
        fn()
        if i % 8 == 7:
            torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()       # enqueued behind the warm-up: the GPU goes straight on to the timed calls
    else:
        torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    for i in range(steps):
        fn()
        marks[i + 1].record()
    torch.cuda.synchronize()
    barrier(dist)
    ms = max_over_ranks(dist, marks[0].elapsed_time(marks[-1]), device) / steps
    return ms, [a.elapsed_time(b) for a, b in zip(marks[:-1], marks[1:])]


# ------------------------------------------------------------------------------------------------
# host memory placement for the end-to-end legs
# ------------------------------------------------------------------------------------------------
def prefer_host_memory_near_gpu(local, on=True):
    """Asks the kernel to place this thread's future page allocations on the NUMA node the GPU hangs
    off (sysfs + set_mempolicy; a no-op when the information or the permission is missing), so that
    pinned buffers allocated afterwards are local to the GPU's PCIe root.  on=False restores the
    default policy."""
    info = dict(numa_node=None, mem_policy_set=False)
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        SYS_set_mempolicy, MPOL_DEFAULT, MPOL_PREFERRED = 238, 0, 1      # x86_64
        if not on:
            libc.syscall(SYS_set_mempolicy, MPOL_DEFAULT, None, ctypes.c_ulong(0))
            return info
        props = torch.cuda.get_device_properties(local)
        bdf = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % bdf).read().strip())
        info["numa_node"] = node
        if node < 0:
            return info
        mask = ctypes.c_ulong(1 << node)
        if libc.syscall(SYS_set_mempolicy, MPOL_PREFERRED, ctypes.byref(mask), ctypes.c_ulong(64)) == 0:
            info["mem_policy_set"] = True
    except (OSError, ValueError, AttributeError):
        pass
    return info


def copy_ceiling(device, nbytes_each_way, dist, reps=4):
    """Plain pinned-memory copies of the end-to-end step's bytes, both directions at once, nothing
    else running: the ceiling of any end-to-end number on this host.  Returns GB/s per direction
    (bytes of one direction over the time both took), max time over the ranks."""
    n = nbytes_each_way // 4
    h_in = [torch.empty(n, dtype=torch.uint8).pin_memory() for _ in range(4)]
    h_out = [torch.empty(n, dtype=torch.uint8).pin_memory() for _ in range(4)]
    d_in = [torch.empty(n, dtype=torch.uint8, device=device) for _ in range(4)]
    d_out = [torch.empty(n, dtype=torch.uint8, device=device) for _ in range(4)]
    s_a, s_b = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)

    def both():
        cur = torch.cuda.current_stream(device)
        s_a.wait_stream(cur), s_b.wait_stream(cur)
        with torch.cuda.stream(s_a):
            for d, h in zip(d_in, h_in):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s_b):
            for h, d in zip(h_out, d_out):
                h.copy_(d, non_blocking=True)
        cur.wait_stream(s_a), cur.wait_stream(s_b)

    ms, _ = timed(both, reps, dist, device, warm=2)
    return nbytes_each_way / (ms * 1e-3) / 1e9, ms


def pipelined_e2e(host_in, host_out, chunks, take, compute, device, n_slots=4):
    """One end-to-end step as a three-stage pipeline over `chunks`: a copy-in stream brings chunk
    i + 1 from pinned host memory while a second stream computes chunk i and a third copies the
    results of chunk i - 1 back.  take(host_tensor, chunk) selects a chunk's slice; compute(device
    inputs) returns the device results, in the order of host_out."""
    s_in, s_cmp, s_out = (torch.cuda.Stream(device=device) for _ in range(3))
    slots = [[torch.empty(take(h, chunks[0]).shape, dtype=h.dtype, device=device) for h in host_in]
             for _ in range(n_slots)]

    def step():
        cur = torch.cuda.current_stream(device)
        for st in (s_in, s_cmp, s_out):
            st.wait_stream(cur)
        slot_free = [None] * n_slots
        for ci, ch in enumerate(chunks):
            bufs = slots[ci % n_slots]
            with torch.cuda.stream(s_in):
                if slot_free[ci % n_slots] is not None:
                    s_in.wait_event(slot_free[ci % n_slots])
                for dst, src in zip(bufs, host_in):
                    dst.copy_(take(src, ch), non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in)
                results = compute(bufs)
                ev_cmp = torch.cuda.Event()
                ev_cmp.record(s_cmp)
                slot_free[ci % n_slots] = ev_cmp
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp)
                for dst, src in zip(host_out, results):
                    src.record_stream(s_out)
                    take(dst, ch).copy_(src, non_blocking=True)
        for st in (s_in, s_cmp, s_out):
            cur.wait_stream(st)
    return step


# ------------------------------------------------------------------------------------------------
# dense workloads
# ------------------------------------------------------------------------------------------------
def staged_backward_split(fl, q, k, v, do, causal, sm_scale, steps):
    """`steps` forward + backward passes with CUDA events between the kernels of the backward (its
    stages enqueued one C call at a time); returns {stage: mean ms}."""
    names, events = [], []
    for _ in range(steps):
        e0 = torch.cuda.Event(enable_timing=True)
        e0.record()
        marks, step_names = [e0], ["fwd"]
        o, lse = fl._forward(q, k, v, causal, sm_scale)
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        marks.append(e)

        def mark(name):
            if name == "start":
                return
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append(ev)
            step_names.append(name)
        fl._backward(q, k, v, o, lse, do, causal, sm_scale, mark)
        events.append(marks)
        names = step_names
    torch.cuda.synchronize()
    per = {n: 0.0 for n in names}
    for marks in events:
        for i, n in enumerate(names):
            per[n] += marks[i].elapsed_time(marks[i + 1])
    return {n: t / steps for n, t in per.items()}


# DRAM bytes of one launch at the primary workload, from ncu captures of earlier builds of the same
# kernels (dram__bytes_read.sum + dram__bytes_write.sum); not measured by this run
NCU_TRAFFIC = {"dkdvdq": 1.304e9, "dkdv": 0.782e9, "dq": 0.662e9, "fwd": 0.522e9}


def run_flash(args, dist, rank, world, device, sampler):
    import flagattention_b200 as fa
    from flagattention_b200 import flash as fl

    c = FLASH_CFG
    B, H, L, D = c["B"], c["H"], c["L"], c["D"]
    numa = prefer_host_memory_near_gpu(device.index)
    gen = torch.Generator().manual_seed(10086 + 2 + rank)
    host = [torch.randn((B, H, L, D), generator=gen).to(torch.bfloat16).pin_memory() for _ in range(4)]
    q, k, v, do = (t.to(device, non_blocking=True) for t in host)
    torch.cuda.synchronize()
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    sm_scale = D ** -0.5
    fwd_f, bwd_f = flash_flops(B, H, L, L, D, True)

    fwd_bwd_events = []

    def step(record=False):
        if record:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
        o = fa.flash_attention(q, k, v, causal=True)
        if record:
            ev[1].record()
        torch.autograd.grad(o, (q, k, v), do)
        if record:
            ev[2].record()
            fwd_bwd_events.append(ev)

    # warm-up (W steps, continued to half a second of load), barrier among the ranks enqueued
    # behind it, then exactly K timed steps: no idle gap at any N
    t_wall0 = time.time()
    ms_step, step_ms = timed(lambda: step(True), args.steps, dist, device, warm=args.warmup, warm_seconds=0.5)
    fwd_bwd_events = fwd_bwd_events[-args.steps:]
    t_wall1 = time.time()
    # the wall-clock window of the timed steps alone: they end at t_wall1 and last steps * ms_step
    timed_window = (t_wall1 - args.steps * ms_step * 1e-3 - 0.002, t_wall1)
    # per-kernel split, back to back with the timed region
    per_kernel = staged_backward_split(fl, q.detach(), k.detach(), v.detach(), do, True, sm_scale, args.steps)
    t_staged1 = time.time()
    # the same loop for at least a second
    n_sus = max(args.steps, int(1100.0 / ms_step) + 1)
    t_sus0 = time.time()
    ms_sus, _ = timed(step, n_sus, dist, device, warm=0)
    t_sus1 = time.time()

    value = world * (fwd_f + bwd_f) / (ms_step * 1e-3) / 1e12
    ms_fwd = statistics.mean(e[0].elapsed_time(e[1]) for e in fwd_bwd_events)
    ms_bwd = statistics.mean(e[1].elapsed_time(e[2]) for e in fwd_bwd_events)

    # executed GEMMs per kernel (each 2*B*H*M*N*D*0.5 FLOP with the causal half): fwd 2; the
    # one-pass backward kernel ("dkdvdq") 5; where the backward runs as two kernels, dkdv 4, dq 3
    gemm = 2.0 * B * H * L * L * D * 0.5
    algo = dict(fwd=2 * gemm, dkdv=4 * gemm, dq=3 * gemm, dkdvdq=5 * gemm)
    algo = {n: f for n, f in algo.items() if n in per_kernel}
    dominant = max(algo, key=lambda n: per_kernel[n])
    roofline = dict(
        _kernel=dominant, _flop=algo[dominant], _ms=per_kernel[dominant],
        scope="the kernel alone (stage '%s' of the staged pass); the whole backward call of the timed "
              "region is under 'backward_call'" % dominant,
        timed_in="a second pass of K steps, back to back with the timed region, with CUDA events "
                 "between the backward's stages",
        traffic=NCU_TRAFFIC.get(dominant),
        traffic_source="ncu capture of an earlier build of this kernel at this workload, not this run",
        traffic_unit="bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum)",
        kernel_ms={n: round(t, 4) for n, t in per_kernel.items()},
        kernel_tflops={n: round(algo[n] / (per_kernel[n] * 1e-3) / 1e12, 2) for n in algo},
        forward_call=dict(ms=round(ms_fwd, 4), tflops=round(fwd_f / (ms_fwd * 1e-3) / 1e12, 2),
                          timed_in="the timed region (public operator)"),
        backward_call=dict(ms=round(ms_bwd, 4), tflops=round(bwd_f / (ms_bwd * 1e-3) / 1e12, 2),
                           timed_in="the timed region (torch.autograd.grad: delta, workspace "
                                    "preparation, the backward kernel(s), dq conversion)"))

    out = dict(value=value, ms_step=ms_step, ms_step_median=statistics.median(step_ms),
               value_sustained=world * (fwd_f + bwd_f) / (ms_sus * 1e-3) / 1e12, ms_sus=ms_sus, n_sus=n_sus,
               roofline=roofline, e2e=None, windows=dict(timed=timed_window, staged=(t_wall1, t_staged1),
                                                         sustained=(t_sus0, t_sus1), all=(t_wall0, t_sus1)),
               launches=len([n for n in per_kernel if n != "dq_zero"]) * args.steps, numa=numa)
    trace(rank, "flash: device-resident legs done")
    if args.skip_e2e:
        prefer_host_memory_near_gpu(device.index, on=False)
        return out

    # ---- end to end through the public operator, host buffers ---------------------------------
    e2e_steps = max(3, min(args.steps, 8))
    outs_host = [torch.empty((B, H, L, D), dtype=torch.bfloat16).pin_memory() for _ in range(4)]
    HG = args.e2e_heads if H % args.e2e_heads == 0 else H   # heads per pipeline chunk
    chunks = [(bi, h0) for bi in range(B) for h0 in range(0, H, HG)]

    def compute(bufs):
        qd, kd, vd = (t.detach().requires_grad_() for t in bufs[:3])
        o = fa.flash_attention(qd, kd, vd, causal=True)
        return (o.detach(), *torch.autograd.grad(o, (qd, kd, vd), bufs[3]))

    e2e_step = pipelined_e2e(host, outs_host, chunks, lambda t, ch: t[ch[0]:ch[0] + 1, ch[1]:ch[1] + HG],
                             compute, device)
    e2e_ms, e2e_step_ms = timed(e2e_step, e2e_steps, dist, device, warm=3)
    trace(rank, "flash: end-to-end leg done")
    nbytes = B * H * L * D * 2
    ceil_gbs, ceil_ms = copy_ceiling(device, 4 * nbytes, dist)
    trace(rank, "flash: copy ceiling done")
    out["e2e"] = dict(
        value=round(world * (fwd_f + bwd_f) / (e2e_ms * 1e-3) / 1e12, 2), unit="TFLOP/s",
        ms_per_step=round(e2e_ms, 3), h2d_bytes_per_step=4 * nbytes, d2h_bytes_per_step=4 * nbytes,
        steps=e2e_steps, step_ms=[round(x, 3) for x in e2e_step_ms],
        value_median_step=round(world * (fwd_f + bwd_f) / (statistics.median(e2e_step_ms) * 1e-3) / 1e12, 2),
        copy_ceiling_gbs=round(ceil_gbs, 2), copy_ceiling_ms=round(ceil_ms, 3),
        copy_ceiling_note="pinned cudaMemcpyAsync of the step's bytes (4 x 128 MiB each way), both "
                          "directions at once, nothing else running; GB/s per direction per GPU, "
                          "slowest rank",
        frac_of_copy_ceiling=round(ceil_ms / e2e_ms, 4),
        limiter=("host<->device copies: the step takes %.1f ms, the bare copies of its bytes %.1f ms, "
                 "its kernels %.1f ms" % (e2e_ms, ceil_ms, ms_step)),
        host_placement=numa)
    prefer_host_memory_near_gpu(device.index, on=False)
    return out


def run_cfg3(args, dist, rank, world, device, sampler):
    """Config 3: fp16, B=2, H=16, L=8192, D=64, non-causal, q/k/v = 0.5 N(0,1), forward returning
    the log-normaliser, then backward.  The case where the ex2 unit is as busy as the tensor pipe."""
    import flagattention_b200 as fa
    c = CFG3
    B, H, L, D = c["B"], c["H"], c["L"], c["D"]
    gen = torch.Generator(device=device).manual_seed(10086 + 3 + rank)
    mk = lambda s: (torch.randn((B, H, L, D), generator=gen, device=device) * s).to(torch.float16)
    q, k, v, do = mk(0.5), mk(0.5), mk(0.5), mk(1.0)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    ev = []

    def step():
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        o, lse, *_ = fa.flash_attention(q, k, v, causal=False, return_log_normalizer=True)
        e[1].record()
        torch.autograd.grad(o, (q, k, v), do)
        e[2].record()
        ev.append(e)

    steps = max(args.steps, 10)
    own = ClockSampler(device.index)
    own.start()
    ms, _ = timed(step, steps, dist, device, warm=3, warm_seconds=0.3)
    t1 = time.time()
    own.stop()
    ev = ev[-steps:]
    ms_f = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    ms_b = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    fwd_f, bwd_f = flash_flops(B, H, L, L, D, False)
    clocks = own.window(t1 - steps * ms * 1e-3 - 0.002, t1)
    mhz = clocks.get("sm_mhz") or 1965.0
    ex2_peak = EX2_PER_CLK_PER_SM * SM_COUNT * mhz * 1e6     # ex2 per second at the sampled clock
    scores = float(B) * H * L * L
    return dict(metric="flash_attn fwd+bwd TFLOP/s (hd64 non-causal fp16, log-normaliser returned)",
                value=round(world * (fwd_f + bwd_f) / (ms * 1e-3) / 1e12, 2), unit="TFLOP/s",
                ms_per_step=round(ms, 4), steps=steps, ms_fwd=round(ms_f, 4), ms_bwd=round(ms_b, 4),
                config=dict(workload="flash_attention fwd(+log_normalizer)+bwd fp16, device-resident", **c),
                roofline=tensor_roofline(
                    "backward call (one-pass kernel + delta + dq conversion)", bwd_f, ms_b, clocks=clocks,
                    forward=dict(tflops=round(fwd_f / (ms_f * 1e-3) / 1e12, 2),
                                 frac_sustained=round(fwd_f / (ms_f * 1e-3) / 1e12 / load_peaks()["tflops_sustained"], 4)),
                    ex2=dict(note="one ex2 per score and pass; peak = 16 / clk / SM x 148 SMs at the sampled clock",
                             sm_mhz=mhz, frac_fwd=round(scores / (ms_f * 1e-3) / ex2_peak, 4),
                             frac_bwd=round(scores / (ms_b * 1e-3) / ex2_peak, 4))),
                clocks=clocks, gpu_launches=4 * steps)


def run_piecewise(args, dist, rank, world, device, sampler):
    """piecewise_attention fwd+bwd at the Aquila-2-34B-shaped configuration: device-resident value,
    forward / backward split, and end to end from pinned host memory."""
    import flagattention_b200 as fa
    c = PIECEWISE_CFG
    B, H, L, D, w = c["B"], c["H"], c["L"], c["D"], c["w"]
    gen = torch.Generator(device=device).manual_seed(10086 + 4 + rank)
    mk = lambda: torch.randn((B, H, L, D), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    q1, k1, q2, k2, v, do = (mk() for _ in range(6))
    ins = [t.requires_grad_() for t in (q1, k1, q2, k2, v)]
    ev = []

    def step():
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        o = fa.piecewise_attention(*ins, w, causal=True)
        e[1].record()
        torch.autograd.grad(o, ins, do)
        e[2].record()
        ev.append(e)

    steps = max(3, min(args.steps, 6))
    ms, _ = timed(step, steps, dist, device, warm=3)
    ev = ev[-steps:]
    ms_f = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    ms_b = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    fwd, bwd = flash_flops(B, H, L, L, D, True)      # one score product per pair: the minimal algorithm
    ref_fwd = 1.5 * fwd                                 # the reference benchmark counts 3 forward matmuls
    ref_bwd = ref_fwd * 8.0 / 3.0
    rec = dict(metric="piecewise_attention fwd+bwd TFLOP/s", value=round(world * (fwd + bwd) / (ms * 1e-3) / 1e12, 2),
               unit="TFLOP/s", ms_per_step=round(ms, 3), steps=steps, ms_fwd=round(ms_f, 3), ms_bwd=round(ms_b, 3),
               value_reference_convention=round(world * (ref_fwd + ref_bwd) / (ms * 1e-3) / 1e12, 2),
               config=dict(workload="piecewise_attention fwd+bwd bf16, device-resident", **c,
                           flops_convention="primary: flash-equivalent (each pair needs one of the two "
                                            "score products); secondary: the reference benchmark's 3 "
                                            "forward matmuls, backward x 8/3"),
               roofline=tensor_roofline("backward call (delta + one launch of the one-pass kernel over both branches + two dq conversions)",
                                        bwd, ms_b, flops="flash-equivalent: 2.5 x forward",
                                        forward=dict(tflops=round(fwd / (ms_f * 1e-3) / 1e12, 2),
                                                     frac_sustained=round(fwd / (ms_f * 1e-3) / 1e12 / load_peaks()["tflops_sustained"], 4))),
               gpu_launches=5 * steps)   # forward, delta, the one-pass kernel, two dq conversions
    if args.skip_e2e:
        return rec
    host_in = [t.detach().cpu().pin_memory() for t in (q1, k1, q2, k2, v, do)]
    host_out = [torch.empty((B, H, L, D), dtype=torch.bfloat16).pin_memory() for _ in range(6)]
    HG = 8
    chunks = list(range(0, H, HG))

    def compute(bufs):
        xs = [t.detach().requires_grad_() for t in bufs[:5]]
        o = fa.piecewise_attention(*xs, w, causal=True)
        return (o.detach(), *torch.autograd.grad(o, xs, bufs[5]))

    e2e_step = pipelined_e2e(host_in, host_out, chunks, lambda t, h0: t[:, h0:h0 + HG], compute, device, n_slots=3)
    e2e_ms, _ = timed(e2e_step, 3, dist, device, warm=1)
    nbytes = B * H * L * D * 2
    rec["e2e"] = dict(value=round(world * (fwd + bwd) / (e2e_ms * 1e-3) / 1e12, 2), unit="TFLOP/s",
                      ms_per_step=round(e2e_ms, 3), h2d_bytes_per_step=6 * nbytes, d2h_bytes_per_step=6 * nbytes)
    return rec


def run_total(args, dist, rank, world, device):
    """total_attention (the column sums of the attention matrix, recomputed from the log-normaliser)
    at config 3's shape: one score product and one exponential per score on the tcgen05 kernel."""
    import flagattention_b200 as fa
    from flagattention_b200.total import total_attention
    c = CFG3
    B, H, L, D = c["B"], c["H"], c["L"], c["D"]
    gen = torch.Generator(device=device).manual_seed(10086 + 8 + rank)
    q, k, v = ((torch.randn((B, H, L, D), generator=gen, device=device) * 0.5).to(torch.float16) for _ in range(3))
    _, lse, *_ = fa.flash_attention(q, k, v, causal=False, return_log_normalizer=True)
    steps = max(args.steps, 10)
    own = ClockSampler(device.index)
    own.start()
    ms, _ = timed(lambda: total_attention(q, k, lse, causal=False), steps, dist, device, warm=3, warm_seconds=0.3)
    t1 = time.time()
    own.stop()
    clocks = own.window(t1 - steps * ms * 1e-3 - 0.002, t1)
    mhz = clocks.get("sm_mhz") or 1965.0
    flop = 2.0 * B * H * L * L * D
    scores = float(B) * H * L * L
    return dict(metric="total_attention TFLOP/s (one score product per pair; hd64 non-causal fp16)",
                value=round(world * flop / (ms * 1e-3) / 1e12, 2), unit="TFLOP/s", ms_per_step=round(ms, 4),
                steps=steps, config=dict(workload="total_attention fp16, device-resident", **c),
                roofline=tensor_roofline("total_attention_tc_kernel", flop, ms, clocks=clocks,
                                         ex2=dict(note="one ex2 per score; peak = 16 / clk / SM x 148 SMs at the sampled clock: "
                                                       "the unit that bounds this kernel",
                                                  sm_mhz=mhz,
                                                  frac=round(scores / (ms * 1e-3) / (EX2_PER_CLK_PER_SM * SM_COUNT * mhz * 1e6), 4))),
                clocks=clocks, gpu_launches=steps)


def run_sweep(args, dist, rank, world, device):
    """Forward and backward TFLOP/s over the sequence lengths of the reference's benchmark grid
    (benchmark/flash_benchmark.py there: batch = 32768 / L, heads = 2048 / D, causal, bf16), a few
    points; the long end of the grid is the primary workload's territory."""
    import flagattention_b200 as fa
    out = []
    for D in (64, 128):
        for L in (512, 1024, 2048, 4096):
            B, H = 32768 // L, 2048 // D
            gen = torch.Generator(device=device).manual_seed(10086 + L + D)
            q, k, v, do = (torch.randn((B, H, L, D), generator=gen, device=device).to(torch.bfloat16)
                           for _ in range(4))
            q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
            keep = []

            def fwd():
                keep[:] = [fa.flash_attention(q, k, v, causal=True)]

            def bwd():
                torch.autograd.grad(keep[0], (q, k, v), do, retain_graph=True)

            ms_f, _ = timed(fwd, 10, None, device, warm=3)
            ms_b, _ = timed(bwd, 10, None, device, warm=3)
            ff, bf = flash_flops(B, H, L, L, D, True)
            out.append(dict(D=D, L=L, B=B, H=H, fwd_tflops=round(ff / (ms_f * 1e-3) / 1e12, 1),
                            bwd_tflops=round(bf / (ms_b * 1e-3) / 1e12, 1),
                            ms_fwd=round(ms_f, 4), ms_bwd=round(ms_b, 4)))
    for r in out:
        top = next(x for x in out if x["D"] == r["D"] and x["L"] == 4096)
        r["fwd_vs_L4096"] = round(r["fwd_tflops"] / top["fwd_tflops"], 3)
        r["bwd_vs_L4096"] = round(r["bwd_tflops"] / top["bwd_tflops"], 3)
    return dict(note="device-resident, 10 calls after 3 warm-ups per point, bf16 causal, "
                     "batch = 32768 / L, heads = 2048 / D", points=out)


# ------------------------------------------------------------------------------------------------
# memory-bound workloads
# ------------------------------------------------------------------------------------------------
def paged_lens(seed):
    c = PAGED_CFG
    gen = torch.Generator().manual_seed(seed)
    lens = torch.randint(c["ctx_lo"], c["ctx_hi"] + 1, (c["num_seqs"],), generator=gen, dtype=torch.int32)
    lens[0] = c["ctx_hi"]
    return lens, gen


def make_paged_inputs(device, seed, keep=None):
    """Inputs of the decode workload; `keep` (a list of sequence indices) builds only those sequences,
    with a KV cache that holds their blocks and nothing else."""
    c = PAGED_CFG
    lens, gen = paged_lens(seed)
    q = torch.randn((c["num_seqs"], c["q_heads"], c["head"]), generator=gen).to(torch.float16)
    if keep is not None:
        idx = torch.tensor(keep, dtype=torch.long)
        lens, q = lens[idx], q[idx]
    blocks = (lens.long() + c["block"] - 1) // c["block"]
    nb = int(blocks.sum())
    perm = torch.randperm(nb, generator=gen)
    max_blocks = c["ctx_hi"] // c["block"]
    bt = torch.zeros((len(lens), max_blocks), dtype=torch.int32)
    off = 0
    for i, n in enumerate(blocks.tolist()):
        bt[i, :n] = perm[off:off + n].to(torch.int32)
        off += n
    dgen = torch.Generator(device=device).manual_seed(seed)
    kc = torch.randn((nb, c["kv_heads"], c["block"], c["head"]), generator=dgen, device=device,
                     dtype=torch.float16)
    vc = torch.randn((nb, c["kv_heads"], c["block"], c["head"]), generator=dgen, device=device,
                     dtype=torch.float16)
    return q, kc, vc, lens, bt, blocks


def paged_algo_bytes(lens, blocks, n_q_elems):
    c = PAGED_CFG
    return (int(lens.long().sum()) * c["kv_heads"] * c["head"] * 2 * 2 + int(blocks.sum()) * 4
            + 2 * n_q_elems * 2 + lens.numel() * 4)


def hbm_roofline(kernel, gbs_per_gpu):
    peaks = load_peaks()
    return dict(bound="hbm", kernel=kernel, achieved=round(gbs_per_gpu, 1), peak=peaks["hbm_gbs"], unit="GB/s",
                frac=round(gbs_per_gpu / peaks["hbm_gbs"], 4), peak_source=peaks["source"],
                frac_nominal_8000=round(gbs_per_gpu / 8000.0, 4), traffic=None)


def run_paged(args, dist, rank, world, device):
    import flagattention_b200 as fa
    c = PAGED_CFG
    q_h, kc, vc, lens_h, bt_h, blocks = make_paged_inputs(device, 10086 + 5 + rank)
    q_h, lens_h, bt_h = q_h.pin_memory(), lens_h.pin_memory(), bt_h.pin_memory()
    q, lens, bt = q_h.to(device), lens_h.to(device), bt_h.to(device)
    scale = c["head"] ** -0.5
    algo_bytes = paged_algo_bytes(lens_h, blocks, q.numel())

    def step():
        return fa.paged_attention(q, kc, vc, lens, bt, scale, c["ctx_hi"], c["num_splits"])

    steps = max(args.steps, 10)
    ms, per = timed(step, steps, dist, device, warm=max(3, args.warmup), warm_seconds=0.1)
    gbs = world * algo_bytes / (ms * 1e-3) / 1e9

    out_h = torch.empty_like(q_h).pin_memory()

    def e2e_step():
        qd, ld, bd = (t.to(device, non_blocking=True) for t in (q_h, lens_h, bt_h))
        out_h.copy_(fa.paged_attention(qd, kc, vc, ld, bd, scale, c["ctx_hi"], c["num_splits"]),
                    non_blocking=True)

    e2e_ms = float("nan")
    if not args.skip_e2e:
        e2e_ms, _ = timed(e2e_step, steps, dist, device, warm=2)
    return dict(metric="paged decode HBM GB/s", value=round(gbs, 1), unit="GB/s",
                ms_per_step=round(ms, 4), ms_per_step_median=round(statistics.median(per), 4),
                algorithmic_bytes=algo_bytes,
                config=dict(workload="paged_attention decode fp16", **c, kv_cache_bytes=2 * kc.numel() * 2,
                            l2="KV cache (4.4 GB) is larger than L2"),
                roofline=hbm_roofline("paged_decode_kernel+paged_reduce_kernel", gbs / world),
                e2e=dict(value=round(world * algo_bytes / (e2e_ms * 1e-3) / 1e9, 1), unit="GB/s",
                         h2d_bytes_per_step=q_h.numel() * 2 + lens_h.numel() * 4 + bt_h.numel() * 4,
                         d2h_bytes_per_step=q_h.numel() * 2,
                         note="KV cache stays resident in HBM, as in serving; query, context_lens and "
                              "block_tables come from pinned host memory every step"),
                gpu_launches=2 * steps)


def run_decode(args, dist, rank, world, device):
    """Single-query flash_attention over a long contiguous KV (the shape of the reference's
    benchmark/flash_decoding_benchmark.py: B=2, H=2048/D, M=1, fp16, non-causal), device-resident."""
    import flagattention_b200 as fa
    B, D, N = 2, 128, 1 << 18
    H = 2048 // D
    gen = torch.Generator(device=device).manual_seed(10086 + 6 + rank)
    q = torch.randn((B, H, 1, D), generator=gen, device=device).to(torch.float16)
    k = torch.randn((B, H, N, D), generator=gen, device=device).to(torch.float16)
    v = torch.randn((B, H, N, D), generator=gen, device=device).to(torch.float16)
    steps = max(args.steps, 10)
    ms, _ = timed(lambda: fa.flash_attention(q, k, v), steps, dist, device, warm=max(3, args.warmup))
    algo_bytes = 2 * k.numel() * 2 + 2 * q.numel() * 2
    gbs = world * algo_bytes / (ms * 1e-3) / 1e9
    return dict(metric="flash_attention single-query decode HBM GB/s", value=round(gbs, 1), unit="GB/s",
                ms_per_step=round(ms, 4), algorithmic_bytes=algo_bytes,
                config=dict(workload="flash_attention M=1 fp16 non-causal", B=B, H=H, N=N, D=D,
                            l2="K and V (4.3 GB) are larger than L2"),
                roofline=hbm_roofline("paged_decode_kernel+paged_reduce_kernel on K, V in place", gbs / world),
                gpu_launches=2 * steps)


def run_rotary(args, dist, rank, world, device):
    """rotary_pair on q and k of the piecewise workload stacked along the batch (B=2, H=48, L=16384,
    D=128, bf16): one read of x, two rotated copies written; forward and backward timed separately,
    device-resident."""
    import flagattention_b200 as fa
    B, H, L, D = 2, 48, 16384, 128
    gen = torch.Generator(device=device).manual_seed(10086 + 7 + rank)
    x = torch.randn((B, H, L, D), generator=gen, device=device).to(torch.bfloat16).requires_grad_()
    g1, g2 = torch.randn_like(x), torch.randn_like(x)
    c1, s1 = fa.rotary_tables(L, D, device=device)
    c2, s2 = fa.rotary_tables(L, D, position_scale=0.25, device=device)
    # a 384 MiB tensor read and two written per call: larger than L2 by itself
    steps = max(args.steps, 10)
    outs = []

    def fwd():
        outs[:] = [fa.rotary_pair(x, c1, s1, c2, s2)]

    def bwd():
        torch.autograd.grad(outs[0], (x,), (g1, g2), retain_graph=True)

    ms_f, _ = timed(fwd, steps, dist, device, warm=max(3, args.warmup))
    ms_b, _ = timed(bwd, steps, dist, device, warm=3)
    algo_bytes = 3 * x.numel() * 2
    gbs_f, gbs_b = algo_bytes / (ms_f * 1e-3) / 1e9, algo_bytes / (ms_b * 1e-3) / 1e9
    roof = hbm_roofline("rotary_pair_fwd_kernel", gbs_f)
    roof.update(traffic=1170e6, traffic_source="ncu capture of an earlier build at this shape, not this run",
                traffic_unit="bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum)")
    return dict(metric="rotary_pair HBM GB/s", value=round(world * gbs_f, 1), unit="GB/s",
                ms_fwd=round(ms_f, 4), ms_bwd=round(ms_b, 4), bwd_gbs=round(world * gbs_b, 1),
                algorithmic_bytes=algo_bytes,
                config=dict(workload="rotary_pair bf16, two embeddings of one tensor", B=B, H=H, L=L, D=D,
                            l2="each tensor (384 MiB) is larger than L2"),
                roofline=roof, gpu_launches=2 * steps)


# ------------------------------------------------------------------------------------------------
# strong scaling: ONE copy of the workloads, sharded over the ranks
# ------------------------------------------------------------------------------------------------
def run_strong(args, dist, rank, world, device):
    import flagattention_b200 as fa
    from flagattention_b200 import dist as fdist

    # ---- dense: the 128 (batch, head) pairs of the primary workload, contiguous runs per rank ----
    c = FLASH_CFG
    B, H, L, D = c["B"], c["H"], c["L"], c["D"]
    runs = fdist.shard_batch_heads(B, H, world, rank)
    pairs = [(b, h) for b, h0, h1 in runs for h in range(h0, h1)]
    gen = torch.Generator(device=device)

    def pair_tensor(which, b, h):
        gen.manual_seed(10086 + 2 + 1000 * which + b * H + h)      # the same pair has the same bits at any N
        return torch.randn((L, D), generator=gen, device=device).to(torch.bfloat16)

    q, k, v, do = (torch.stack([pair_tensor(w, b, h) for b, h in pairs])[None] for w in range(4))
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()

    def dense_step():
        o = fa.flash_attention(q, k, v, causal=True)
        torch.autograd.grad(o, (q, k, v), do)

    steps = args.steps
    ms, _ = timed(dense_step, steps, dist, device, warm=args.warmup, warm_seconds=0.5)
    fwd_f, bwd_f = flash_flops(B, H, L, L, D, True)
    flash_rec = dict(metric="flash_attn fwd+bwd TFLOP/s, ONE B=4 H=32 L=4096 D=128 problem over all GPUs",
                     value=round((fwd_f + bwd_f) / (ms * 1e-3) / 1e12, 2), unit="TFLOP/s",
                     ms_per_step=round(ms, 4), pairs_per_rank=len(pairs), steps=steps,
                     sharding="flagattention_b200.dist.shard_batch_heads: contiguous runs of (batch, head) "
                              "pairs; no exchange (dq, dk, dv of a pair stay with the pair)")
    del q, k, v, do
    torch.cuda.empty_cache()
    trace(rank, "strong: dense done")

    # ---- decode: the 64 sequences by longest-first assignment, outputs all-gathered ---------------
    pc = PAGED_CFG
    lens_all, _ = paged_lens(10086 + 5)
    shards = fdist.shard_sequences_lpt(lens_all.tolist(), world)
    mine = shards[rank]
    q_h, kc, vc, lens_h, bt_h, blocks = make_paged_inputs(device, 10086 + 5, keep=mine)
    q_d, lens_d, bt_d = q_h.to(device), lens_h.to(device), bt_h.to(device)
    scale = pc["head"] ** -0.5
    counts = [len(s) for s in shards]
    gathered = []

    def paged_step():
        out = fa.paged_attention(q_d, kc, vc, lens_d, bt_d, scale, pc["ctx_hi"], pc["num_splits"])
        if dist is not None:
            gathered[:] = fdist.all_gather_rows(out, counts)
        else:
            gathered[:] = [out]

    psteps = max(args.steps, 10)
    pms, _ = timed(paged_step, psteps, dist, device, warm=3, warm_seconds=0.1)
    blocks_all = (lens_all.long() + pc["block"] - 1) // pc["block"]
    total_bytes = paged_algo_bytes(lens_all, blocks_all, pc["num_seqs"] * pc["q_heads"] * pc["head"])
    loads = [int(sum(int(lens_all[i]) for i in s)) for s in shards]
    paged_rec = dict(metric="paged decode HBM GB/s, ONE 64-sequence problem over all GPUs",
                     value=round(total_bytes / (pms * 1e-3) / 1e9, 1), unit="GB/s", ms_per_step=round(pms, 4),
                     steps=psteps, seqs_per_rank=counts, tokens_per_rank=loads,
                     imbalance=round(max(loads) * world / max(1, sum(loads)), 4),
                     kv_blocks_this_rank=int(blocks.sum()),
                     sharding="flagattention_b200.dist.shard_sequences_lpt; each rank holds only its "
                              "sequences' KV blocks; all_gather_rows of out (NCCL) inside the timed region"
                              if dist is not None else "one rank: no gather")
    return dict(flash=flash_rec, paged=paged_rec)


# ------------------------------------------------------------------------------------------------
# CPU baseline / reference arm (the oracle port on the host cores)
# ------------------------------------------------------------------------------------------------
def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def cpu_cfg1(reps=25):
    """Config 1, as the baseline plan states it: the reference's PyTorch oracle, fp32, B=2, H=4,
    L=256, D=64, causal, sm_scale=1/8, both aux outputs, backward through autograd; 3 warm-ups,
    median of `reps` (>= 20) perf_counter timings, all host cores."""
    import oracle
    c = CFG1
    B, H, L, D = c["B"], c["H"], c["L"], c["D"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(10086 + 1)
    q, k, v, do = (torch.randn((B, H, L, D), generator=gen) for _ in range(4))
    times = []
    for i in range(reps + 3):
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        t0 = time.perf_counter()
        o, lse, tot = oracle.flash_attention(qq, kk, vv, True, sm_scale=0.125, return_log_normalizer=True,
                                             return_total_attention=True, upcast=True)
        torch.autograd.grad(o, (qq, kk, vv), do)
        dt = time.perf_counter() - t0
        if i >= 3:
            times.append(dt)
    sec = statistics.median(times)
    flop = 4.0 * B * H * L * L * D * 0.5 * 3.5
    return dict(median_ms=round(sec * 1e3, 3), min_ms=round(min(times) * 1e3, 3), reps=reps, warmups=3,
                gflops=round(flop / sec / 1e9, 2), counted_flop=flop, cores=cores, cpu=cpu_model(),
                kind="port", what="oracle.flash_attention (the restated flag_attn.testing.flash_attention), "
                                  "fp32, B=2 H=4 L=256 D=64 causal, log-normaliser and total attention "
                                  "returned, backward through autograd")


def cpu_flash_sample(reps, heads=4):
    """Times the reference's CPU implementation of the path (oracle port, fp32 upcast) on
    `heads` (batch, head) pairs of the primary workload; returns counted TFLOP/s."""
    import oracle
    c = FLASH_CFG
    L, D = c["L"], c["D"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(10086 + 2)
    q, k, v, do = (torch.randn((1, heads, L, D), generator=gen).to(torch.bfloat16) for _ in range(4))
    fwd_f, bwd_f = flash_flops(1, heads, L, L, D, True)
    times = []
    for i in range(reps + 1):
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        t0 = time.perf_counter()
        o = oracle.flash_attention(qq, kk, vv, True, upcast=True)
        torch.autograd.grad(o, (qq, kk, vv), do)
        dt = time.perf_counter() - t0
        if i > 0:
            times.append(dt)
    sec = statistics.median(times)
    return dict(value=round((fwd_f + bwd_f) / sec / 1e12, 5), unit="TFLOP/s", cores=cores, kind="port",
                cpu=cpu_model(),
                sample=f"oracle.flash_attention fwd+bwd (fp32 upcast, torch CPU) on {heads} of the "
                       f"{c['B'] * c['H']} (batch, head) pairs of the workload, median of {reps} runs, "
                       f"{sec:.2f} s each"), sec


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, sec = cpu_flash_sample(max(3, min(args.steps, 7)))
    base["cfg1"] = cpu_cfg1()
    c = FLASH_CFG
    line = {
        "impl": "reference", "metric": "flash_attn fwd+bwd TFLOP/s (hd128 causal bf16)",
        "value": base["value"], "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 2), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "flash_attention fwd+bwd bf16 B=4 H=32 L=4096 D=128 causal "
                               "(bounded sample: 4 (batch, head) pairs per step)", **c},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-paged", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true", help="device-resident timing only (profiling)")
    ap.add_argument("--e2e-heads", type=int, default=8, help="heads per chunk of the host-buffer pipeline")
    ap.add_argument("--skip-piecewise", action="store_true")
    ap.add_argument("--skip-extras", action="store_true", help="no cfg3 / sweep / decode / rotary / strong records")
    ap.add_argument("--backward", default="auto", choices=["auto", "one_pass", "two_kernel"],
                    help="backward kernels of the dense operators (flagattention_b200.flash.set_backward_mode)")
    ap.add_argument("--kernels", default="auto", choices=["auto", "generic", "one_cta_per_tile"],
                    help="generic: the shape-generic mma.sync kernels instead of the tcgen05 ones; "
                         "one_cta_per_tile: tcgen05, but the forward never in its persistent form (profiling)")
    ap.add_argument("--only", default=None, choices=["flash", "paged", "piecewise", "rotary", "cfg3", "sweep", "total"],
                    help="run one workload only (profiling); the JSON line is then partial")
    ap.add_argument("--paged-seqs", type=int, default=PAGED_CFG["num_seqs"],
                    help="number of sequences of the paged workload (smaller for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference(args)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    dist, rank, world, local = dist_setup()
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    sampler = ClockSampler(local)
    sampler.start()
    from flagattention_b200 import _C as fa_c
    from flagattention_b200 import flash as fa_flash
    fa_flash.set_backward_mode(args.backward)
    fa_c.load().fa_set_kernel_family({"auto": 0, "generic": 1, "one_cta_per_tile": 2}[args.kernels])

    PAGED_CFG["num_seqs"] = args.paged_seqs
    single = {"paged": lambda: run_paged(args, dist, rank, world, device),
              "rotary": lambda: run_rotary(args, dist, rank, world, device),
              "piecewise": lambda: run_piecewise(args, dist, rank, world, device, sampler),
              "cfg3": lambda: run_cfg3(args, dist, rank, world, device, sampler),
              "sweep": lambda: run_sweep(args, dist, rank, world, device),
              "total": lambda: run_total(args, dist, rank, world, device)}
    if args.only in single:
        rec = single[args.only]()
        sampler.stop()
        if rank == 0:
            print(json.dumps({"partial": True, args.only: rec}), flush=True)
        return

    trace(rank, "process group up, %d rank(s)" % world)
    fl = run_flash(args, dist, rank, world, device, sampler)
    trace(rank, "flash done")
    flash_only = args.only == "flash"
    paged = None if (args.skip_paged or flash_only) else run_paged(args, dist, rank, world, device)
    trace(rank, "paged done")
    strong = None if (args.skip_extras or flash_only) else run_strong(args, dist, rank, world, device)
    trace(rank, "strong-scaling records done")
    # the secondary records are single-GPU measurements
    extras = world == 1 and not flash_only and not args.skip_extras
    pw = run_piecewise(args, dist, rank, world, device, sampler) if (world == 1 and not flash_only and not args.skip_piecewise) else None
    cfg3 = run_cfg3(args, dist, rank, world, device, sampler) if extras else None
    sweep = run_sweep(args, dist, rank, world, device) if extras else None
    dec = run_decode(args, dist, rank, world, device) if extras and not args.skip_paged else None
    rot = run_rotary(args, dist, rank, world, device) if extras else None
    tot = run_total(args, dist, rank, world, device) if extras else None
    sampler.stop()
    cpu = None
    if rank == 0 and not args.skip_cpu and world == 1:
        cpu, _ = cpu_flash_sample(3)
        cpu["cfg1"] = cpu_cfg1()

    if rank == 0:
        c = FLASH_CFG
        w = fl["windows"]
        clk_timed, clk_sus, clk_all = (sampler.window(*w[n]) for n in ("timed", "sustained", "all"))
        mhz = clk_timed["sm_mhz"]
        rf = fl["roofline"]
        clk_staged = sampler.window(*w["staged"])
        fl["roofline"] = tensor_roofline(rf.pop("_kernel"), rf.pop("_flop"), rf.pop("_ms"), clocks=clk_staged,
                                         clocks_during=clk_staged, **rf)
        clocks = dict(clk_all)
        clocks.update(timed_region=clk_timed, sustained_loop=clk_sus,
                      note="sm_mhz / reasons: every sample from the first warm-up step to the end of the "
                           "sustained loop; timed_region: the samples inside the K timed steps")
        smhz = clk_staged["sm_mhz"]
        fl["roofline"]["ms_x_mhz"] = ({n: round(t * smhz, 1) for n, t in fl["roofline"]["kernel_ms"].items()}
                                      if smhz else None)
        line = {
            "metric": "flash_attn fwd+bwd TFLOP/s (hd128 causal bf16)",
            "value": round(fl["value"], 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(fl["ms_step"], 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "ms_per_step_median": round(fl["ms_step_median"], 4),
            "sm_mhz_median": mhz, "ms_x_mhz": round(fl["ms_step"] * mhz, 1) if mhz else None,
            "value_sustained": round(fl["value_sustained"], 2),
            "sustained": dict(steps=fl["n_sus"], ms_per_step=round(fl["ms_sus"], 4), sm_mhz_median=clk_sus["sm_mhz"],
                              ms_x_mhz=round(fl["ms_sus"] * clk_sus["sm_mhz"], 1) if clk_sus["sm_mhz"] else None),
            "config": {"workload": "flash_attention fwd+bwd bf16 B=4 H=32 L=4096 D=128 causal, per GPU, "
                                   "through flash_attention + torch.autograd.grad",
                       **c, "global_batch": c["B"] * world,
                       "parallelism": f"{world} GPU(s), one process each, every rank the per-GPU workload "
                                      "(weak); 'strong' splits one copy by (batch x head) / by sequence",
                       "flops_convention": "matmul only: fwd 4*B*H*M*N*D*0.5, bwd 2.5x",
                       "l2": "inputs (4 x 128 MiB) are larger than the 126 MB L2",
                       "timing": "warm-up (W steps, at least 0.5 s) -> rank barrier enqueued behind it -> "
                                 "K timed steps, no idle gap; CUDA events, slowest rank"},
            "roofline": fl["roofline"], "cpu_baseline": cpu, "e2e": fl["e2e"],
            "gpu_launches": fl["launches"], "clocks": clocks, "paged": paged, "strong": strong,
            "cfg3": cfg3, "piecewise": pw, "sweep": sweep, "decode": dec, "rotary": rot, "total": tot,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
