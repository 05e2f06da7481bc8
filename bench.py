"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Primary workload (the configuration the headline metric is quoted on): flash_attention forward +
backward, bf16, B=4, H=32, L=4096, D=128, causal, q/k/v/dO ~ N(0,1).  A step is one forward and one
backward over that batch.  `value` is matmul-only TFLOP/s (the reference benchmark's convention:
forward 4*B*H*M*N*D*0.5 for causal, backward 2.5x that) with inputs resident in HBM; `e2e` is the
same metric through the public operator with the inputs in pinned host memory, every step copying
q, k, v, dO to the device and o, dq, dk, dv back.  The same JSON line also carries the paged decode
workload (64 sequences, 32/8 heads, head 128, block 16, contexts in [1024, 32768], 512-token
partitions) as HBM GB/s under "paged".

With N > 1 (launched by torch.distributed.run) every rank runs the same per-GPU workload on its
own (batch x head) shard -- no data-path collective -- and the value is all ranks' work over the
slowest rank's device time (weak scaling).

`--impl reference` times the reference's CPU implementation of the path (its PyTorch oracle, as
restated under oracle/) on the host cores, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FLASH_CFG = dict(B=4, H=32, Hk=32, L=4096, D=128, causal=True, dtype="bf16")
PIECEWISE_CFG = dict(B=1, H=48, L=16384, D=128, w=4096, causal=True, dtype="bf16")
PAGED_CFG = dict(num_seqs=64, q_heads=32, kv_heads=8, head=128, block=16, ctx_lo=1024, ctx_hi=32768,
                 partition=512, num_splits=64)


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


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "50", "-f", self.path],
                stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        try:
            rows = [r.strip().split(", ") for r in open(self.path) if r.strip()]
            os.unlink(self.path)
        except OSError:
            return out
        mhz, reasons = [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in rows:
            if len(r) < 6:
                continue
            try:
                mhz.append(float(r[0]))
                out["sm_max_mhz"] = float(r[1])
            except ValueError:
                continue
            for name, val in zip(names, r[2:6]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if mhz:
            out["sm_mhz"] = statistics.median(mhz)
        out["reasons"] = sorted(reasons)
        out["samples"] = len(mhz)
        return out


# ------------------------------------------------------------------------------------------------
# distributed plumbing
# ------------------------------------------------------------------------------------------------
def dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return dist, rank, world, local
    return None, 0, 1, 0


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


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_flash(args, dist, rank, world, device):
    import flagattention_b200 as fa
    from flagattention_b200 import flash as fl

    c = FLASH_CFG
    B, H, L, D = c["B"], c["H"], c["L"], c["D"]
    gen = torch.Generator().manual_seed(10086 + 2 + rank)
    host = [torch.randn((B, H, L, D), generator=gen).to(torch.bfloat16).pin_memory() for _ in range(4)]
    q, k, v, do = (t.to(device, non_blocking=True) for t in host)
    torch.cuda.synchronize()
    sm_scale = D ** -0.5
    names = []   # kernel groups in launch order, filled by the first timed step

    def step(events=None):
        if events is not None:
            e0 = torch.cuda.Event(enable_timing=True)
            e0.record()
            marks = [e0]
        o, lse = fl._forward(q, k, v, True, sm_scale)
        if events is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            marks.append(e)

            step_names = ["fwd"]

            def mark(name):
                if name == "start":
                    return
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append(ev)
                step_names.append(name)
            fl._backward(q, k, v, o, lse, do, True, sm_scale, mark)
            events.append(marks)
            names[:] = step_names
        else:
            fl._backward(q, k, v, o, lse, do, True, sm_scale)

    # Warm-up: W steps, continued until the GPU has been under this load for half a second, with
    # the clock sampler already running, so that the clock record covers a loaded GPU even when
    # the timed region itself is shorter than nvidia-smi's sampling period.
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    t_warm = time.perf_counter()
    done = 0
    while done < args.warmup or time.perf_counter() - t_warm < 0.5:
        step()
        done += 1
        if done % 8 == 0:
            torch.cuda.synchronize()
    barrier(dist)
    events = []
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step(events)
    t1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    barrier(dist)
    ms_total = max_over_ranks(dist, t0.elapsed_time(t1), device)
    ms_step = ms_total / args.steps
    fwd_f, bwd_f = flash_flops(B, H, L, L, D, True)
    value = world * (fwd_f + bwd_f) / (ms_step * 1e-3) / 1e12

    per_kernel = {n: 0.0 for n in names}
    for marks in events:
        for i, n in enumerate(names):
            per_kernel[n] += marks[i].elapsed_time(marks[i + 1])
    per_kernel = {n: t / args.steps for n, t in per_kernel.items()}

    # executed GEMMs per kernel (each 2*B*H*M*N*D*0.5 FLOP with the causal half): fwd 2; the
    # one-pass backward kernel ("dkdvdq"; the zero-fill of its fp32 dq workspace and the dq
    # conversion are timed apart as "dq_zero" and "dq_convert") 5; where the backward runs as two
    # kernels, dkdv 4 and dq 3
    gemm = 2.0 * B * H * L * L * D * 0.5
    algo = dict(fwd=2 * gemm, dkdv=4 * gemm, dq=3 * gemm, dkdvdq=5 * gemm)
    algo = {n: f for n, f in algo.items() if n in per_kernel}
    dominant = max(algo, key=lambda n: per_kernel[n])
    peaks = load_peaks()
    achieved = algo[dominant] / (per_kernel[dominant] * 1e-3) / 1e12
    roofline = dict(bound="tensor", kernel=dominant, achieved=round(achieved, 2),
                    peak=peaks["tflops_sustained"], unit="TFLOP/s",
                    frac=round(achieved / peaks["tflops_sustained"], 4),
                    peak_source=peaks["source"] + " (sustained cuBLAS bf16)",
                    # DRAM bytes of one launch of that kernel, from the ncu captures summarised under
                    # profiles/ (not measured by this run)
                    traffic={"dkdvdq": 1.304e9, "dkdv": 0.782e9, "dq": 0.662e9, "fwd": 0.522e9}.get(dominant),
                    traffic_unit="bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum, ncu)",
                    kernel_ms={n: round(t, 4) for n, t in per_kernel.items()},
                    kernel_tflops={n: round(algo[n] / (per_kernel[n] * 1e-3) / 1e12, 2) for n in algo})

    if args.skip_e2e:
        return dict(value=value, ms_step=ms_step, roofline=roofline, e2e=None, clocks=clocks,
                    launches=4 * args.steps)

    # ---- end to end through the public operator, host buffers ---------------------------------
    e2e_steps = max(2, min(args.steps, 5))
    outs_host = [torch.empty((B, H, L, D), dtype=torch.bfloat16).pin_memory() for _ in range(4)]

    # The step is a three-stage pipeline over (batch element, group of 8 heads) chunks: one stream
    # copies chunk i+1 in while a second runs the kernels of chunk i and a third copies the
    # results of chunk i-1 out, so both PCIe directions and the SMs stay busy; the fill and drain
    # of the pipeline are one chunk (1/16 of the step) each.
    s_in, s_cmp, s_out = (torch.cuda.Stream(device=device) for _ in range(3))
    HG = args.e2e_heads if H % args.e2e_heads == 0 else H   # heads per pipeline chunk
    chunks = [(bi, h0) for bi in range(B) for h0 in range(0, H, HG)]
    NS = 4   # input slots on the device
    slots = [[torch.empty((1, HG, L, D), dtype=torch.bfloat16, device=device) for _ in range(4)]
             for _ in range(NS)]

    def e2e_step():
        cur = torch.cuda.current_stream(device)
        for st in (s_in, s_cmp, s_out):
            st.wait_stream(cur)
        slot_free = [None] * NS
        for ci, (bi, h0) in enumerate(chunks):
            bufs = slots[ci % NS]
            with torch.cuda.stream(s_in):
                if slot_free[ci % NS] is not None:
                    s_in.wait_event(slot_free[ci % NS])
                for dst, src in zip(bufs, host):
                    dst.copy_(src[bi:bi + 1, h0:h0 + HG], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in)
                qd, kd, vd = (t.detach().requires_grad_() for t in bufs[:3])
                o = fa.flash_attention(qd, kd, vd, causal=True)
                grads = torch.autograd.grad(o, (qd, kd, vd), bufs[3])
                ev_cmp = torch.cuda.Event()
                ev_cmp.record(s_cmp)
                slot_free[ci % NS] = ev_cmp
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp)
                for dst, src in zip(outs_host, (o.detach(), *grads)):
                    src.record_stream(s_out)
                    dst[bi:bi + 1, h0:h0 + HG].copy_(src, non_blocking=True)
        for st in (s_in, s_cmp, s_out):
            cur.wait_stream(st)

    for _ in range(3):   # untimed: allocator pools of the three streams settle
        e2e_step()
    barrier(dist)
    t0.record()
    marks = [t0]
    for _ in range(e2e_steps):
        e2e_step()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append(ev)
    t1.record()
    torch.cuda.synchronize()
    barrier(dist)
    e2e_ms = max_over_ranks(dist, t0.elapsed_time(t1), device) / e2e_steps
    step_ms = [round(a.elapsed_time(b), 3) for a, b in zip(marks[:-1], marks[1:])]
    nbytes = B * H * L * D * 2
    e2e = dict(value=round(world * (fwd_f + bwd_f) / (e2e_ms * 1e-3) / 1e12, 2), unit="TFLOP/s",
               ms_per_step=round(e2e_ms, 3), h2d_bytes_per_step=4 * nbytes, d2h_bytes_per_step=4 * nbytes,
               steps=e2e_steps, step_ms=step_ms)
    return dict(value=value, ms_step=ms_step, roofline=roofline, e2e=e2e, clocks=clocks,
                launches=4 * args.steps)


def run_piecewise(args, dist, rank, world, device):
    """piecewise_attention fwd+bwd at the Aquila-2-34B-shaped configuration (device-resident)."""
    import flagattention_b200 as fa
    c = PIECEWISE_CFG
    B, H, L, D, w = c["B"], c["H"], c["L"], c["D"], c["w"]
    gen = torch.Generator(device=device).manual_seed(10086 + 4 + rank)
    mk = lambda: torch.randn((B, H, L, D), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    q1, k1, q2, k2, v, do = (mk() for _ in range(6))
    ins = [t.requires_grad_() for t in (q1, k1, q2, k2, v)]

    def step():
        o = fa.piecewise_attention(*ins, w, causal=True)
        torch.autograd.grad(o, ins, do)

    for _ in range(3):
        step()
    steps = max(3, min(args.steps, 5))
    barrier(dist)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    torch.cuda.synchronize()
    barrier(dist)
    ms = max_over_ranks(dist, t0.elapsed_time(t1), device) / steps
    fwd, bwd = flash_flops(B, H, L, L, D, True)      # one score product per pair: the minimal algorithm
    ref_fwd = 1.5 * fwd                                 # the reference benchmark counts 3 forward matmuls
    ref_bwd = ref_fwd * 8.0 / 3.0
    return dict(metric="piecewise_attention fwd+bwd TFLOP/s", value=round(world * (fwd + bwd) / (ms * 1e-3) / 1e12, 2),
                unit="TFLOP/s", ms_per_step=round(ms, 3), steps=steps,
                value_reference_convention=round(world * (ref_fwd + ref_bwd) / (ms * 1e-3) / 1e12, 2),
                config=dict(workload="piecewise_attention fwd+bwd bf16, device-resident", **c,
                            flops_convention="primary: flash-equivalent (each pair needs one of the two "
                                             "score products); secondary: the reference benchmark's 3 "
                                             "forward matmuls, backward x 8/3"))


def make_paged_inputs(device, seed):
    c = PAGED_CFG
    gen = torch.Generator().manual_seed(seed)
    lens = torch.randint(c["ctx_lo"], c["ctx_hi"] + 1, (c["num_seqs"],), generator=gen, dtype=torch.int32)
    lens[0] = c["ctx_hi"]
    blocks = (lens.long() + c["block"] - 1) // c["block"]
    nb = int(blocks.sum())
    perm = torch.randperm(nb, generator=gen)
    max_blocks = c["ctx_hi"] // c["block"]
    bt = torch.zeros((c["num_seqs"], max_blocks), dtype=torch.int32)
    off = 0
    for i, n in enumerate(blocks.tolist()):
        bt[i, :n] = perm[off:off + n].to(torch.int32)
        off += n
    dgen = torch.Generator(device=device).manual_seed(seed)
    kc = torch.randn((nb, c["kv_heads"], c["block"], c["head"]), generator=dgen, device=device,
                     dtype=torch.float16)
    vc = torch.randn((nb, c["kv_heads"], c["block"], c["head"]), generator=dgen, device=device,
                     dtype=torch.float16)
    q = torch.randn((c["num_seqs"], c["q_heads"], c["head"]), generator=gen).to(torch.float16)
    return q, kc, vc, lens, bt, blocks


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
    for _ in range(max(3, args.warmup)):
        fa.flash_attention(q, k, v)
    steps = max(args.steps, 10)
    barrier(dist)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        fa.flash_attention(q, k, v)
    t1.record()
    torch.cuda.synchronize()
    barrier(dist)
    ms = max_over_ranks(dist, t0.elapsed_time(t1), device) / steps
    algo_bytes = 2 * k.numel() * 2 + 2 * q.numel() * 2
    gbs = world * algo_bytes / (ms * 1e-3) / 1e9
    peaks = load_peaks()
    return dict(metric="flash_attention single-query decode HBM GB/s", value=round(gbs, 1), unit="GB/s",
                ms_per_step=round(ms, 4), algorithmic_bytes=algo_bytes,
                config=dict(workload="flash_attention M=1 fp16 non-causal", B=B, H=H, N=N, D=D,
                            l2="K and V (4.3 GB) are larger than L2"),
                roofline=dict(bound="hbm", kernel="paged_decode_kernel+paged_reduce_kernel on K, V in place",
                              achieved=round(gbs / world, 1), peak=peaks["hbm_gbs"], unit="GB/s",
                              frac=round(gbs / world / peaks["hbm_gbs"], 4), peak_source=peaks["source"],
                              traffic=None),
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
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]

    def run(n, timed):
        if timed:
            ev[0].record()
        outs = None
        for _ in range(n):
            outs = fa.rotary_pair(x, c1, s1, c2, s2)
        if timed:
            ev[1].record()
        for _ in range(n):
            torch.autograd.grad(outs, (x,), (g1, g2), retain_graph=True)
        if timed:
            ev[2].record()

    run(max(3, args.warmup), False)
    barrier(dist)
    run(steps, True)
    torch.cuda.synchronize()
    barrier(dist)
    ms_f = max_over_ranks(dist, ev[0].elapsed_time(ev[1]), device) / steps
    ms_b = max_over_ranks(dist, ev[1].elapsed_time(ev[2]), device) / steps
    algo_bytes = 3 * x.numel() * 2
    peaks = load_peaks()
    gbs_f, gbs_b = algo_bytes / (ms_f * 1e-3) / 1e9, algo_bytes / (ms_b * 1e-3) / 1e9
    return dict(metric="rotary_pair HBM GB/s", value=round(world * gbs_f, 1), unit="GB/s",
                ms_fwd=round(ms_f, 4), ms_bwd=round(ms_b, 4), bwd_gbs=round(world * gbs_b, 1),
                algorithmic_bytes=algo_bytes,
                config=dict(workload="rotary_pair bf16, two embeddings of one tensor", B=B, H=H, L=L, D=D,
                            l2="each tensor (384 MiB) is larger than L2"),
                roofline=dict(bound="hbm", kernel="rotary_pair_fwd_kernel", achieved=round(gbs_f, 1),
                              peak=peaks["hbm_gbs"], unit="GB/s", frac=round(gbs_f / peaks["hbm_gbs"], 4),
                              peak_source=peaks["source"],
                              traffic=1170e6 * B / 2,   # ncu capture of this shape at B=2 (profiles/)
                              traffic_unit="bytes per launch (dram__bytes.sum, ncu)"),
                gpu_launches=2 * steps)


def run_paged(args, dist, rank, world, device):
    import flagattention_b200 as fa
    c = PAGED_CFG
    q_h, kc, vc, lens_h, bt_h, blocks = make_paged_inputs(device, 10086 + 5 + rank)
    q_h, lens_h, bt_h = q_h.pin_memory(), lens_h.pin_memory(), bt_h.pin_memory()
    q, lens, bt = q_h.to(device), lens_h.to(device), bt_h.to(device)
    scale = c["head"] ** -0.5
    algo_bytes = (int(lens_h.long().sum()) * c["kv_heads"] * c["head"] * 2 * 2 + int(blocks.sum()) * 4
                  + 2 * q.numel() * 2 + lens.numel() * 4)

    def step():
        return fa.paged_attention(q, kc, vc, lens, bt, scale, c["ctx_hi"], c["num_splits"])

    for _ in range(max(3, args.warmup)):
        step()
    steps = max(args.steps, 10)
    barrier(dist)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    torch.cuda.synchronize()
    barrier(dist)
    ms = max_over_ranks(dist, t0.elapsed_time(t1), device) / steps
    gbs = world * algo_bytes / (ms * 1e-3) / 1e9

    out_h = torch.empty_like(q_h).pin_memory()

    def e2e_step():
        qd, ld, bd = (t.to(device, non_blocking=True) for t in (q_h, lens_h, bt_h))
        out_h.copy_(fa.paged_attention(qd, kc, vc, ld, bd, scale, c["ctx_hi"], c["num_splits"]),
                    non_blocking=True)

    e2e_ms = float("nan")
    if not args.skip_e2e:
        e2e_step()
        barrier(dist)
        t0.record()
        for _ in range(steps):
            e2e_step()
        t1.record()
        torch.cuda.synchronize()
        barrier(dist)
        e2e_ms = max_over_ranks(dist, t0.elapsed_time(t1), device) / steps
    peaks = load_peaks()
    return dict(metric="paged decode HBM GB/s", value=round(gbs, 1), unit="GB/s",
                ms_per_step=round(ms, 4), algorithmic_bytes=algo_bytes,
                config=dict(workload="paged_attention decode fp16", **c, kv_cache_bytes=2 * kc.numel() * 2,
                            l2="KV cache (4.4 GB) is larger than L2"),
                roofline=dict(bound="hbm", kernel="paged_decode_kernel+paged_reduce_kernel",
                              achieved=round(gbs / world, 1), peak=peaks["hbm_gbs"], unit="GB/s",
                              frac=round(gbs / world / peaks["hbm_gbs"], 4),
                              peak_source=peaks["source"], traffic=None),
                e2e=dict(value=round(world * algo_bytes / (e2e_ms * 1e-3) / 1e9, 1), unit="GB/s",
                         h2d_bytes_per_step=q_h.numel() * 2 + lens_h.numel() * 4 + bt_h.numel() * 4,
                         d2h_bytes_per_step=q_h.numel() * 2,
                         note="KV cache stays resident in HBM, as in serving; query, context_lens and "
                              "block_tables come from pinned host memory every step"),
                gpu_launches=2 * steps)


# ------------------------------------------------------------------------------------------------
# CPU baseline / reference arm (the oracle port on the host cores)
# ------------------------------------------------------------------------------------------------
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
                sample=f"oracle.flash_attention fwd+bwd (fp32 upcast, torch CPU) on {heads} of the "
                       f"{c['B'] * c['H']} (batch, head) pairs of the workload, median of {reps} runs, "
                       f"{sec:.2f} s each"), sec


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, sec = cpu_flash_sample(max(1, min(args.steps, 3)))
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
    ap.add_argument("--only", default=None, choices=["flash", "paged", "piecewise", "rotary"],
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
    dist, rank, world, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)

    PAGED_CFG["num_seqs"] = args.paged_seqs
    if args.only == "paged":
        paged = run_paged(args, dist, rank, world, device)
        if rank == 0:
            print(json.dumps({"partial": True, "paged": paged}), flush=True)
        return
    if args.only == "rotary":
        rot = run_rotary(args, dist, rank, world, device)
        if rank == 0:
            print(json.dumps({"partial": True, "rotary": rot}), flush=True)
        return
    if args.only == "piecewise":
        pw = run_piecewise(args, dist, rank, world, device)
        if rank == 0:
            print(json.dumps({"partial": True, "piecewise": pw}), flush=True)
        return
    fl = run_flash(args, dist, rank, world, device)
    paged = None if (args.skip_paged or args.only == "flash") else run_paged(args, dist, rank, world, device)
    pw = None if (args.skip_piecewise or args.only == "flash") else run_piecewise(args, dist, rank, world, device)
    dec = None if (args.skip_paged or args.only == "flash") else run_decode(args, dist, rank, world, device)
    rot = None if (args.skip_piecewise or args.only == "flash") else run_rotary(args, dist, rank, world, device)
    cpu = None
    if rank == 0 and not args.skip_cpu and world == 1:
        cpu, _ = cpu_flash_sample(2)

    if rank == 0:
        c = FLASH_CFG
        line = {
            "metric": "flash_attn fwd+bwd TFLOP/s (hd128 causal bf16)",
            "value": round(fl["value"], 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(fl["ms_step"], 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "flash_attention fwd+bwd bf16 B=4 H=32 L=4096 D=128 causal, per GPU",
                       **c, "global_batch": c["B"] * world, "parallelism": f"batch x head shards over {world} GPU(s), no collective",
                       "flops_convention": "matmul only: fwd 4*B*H*M*N*D*0.5, bwd 2.5x",
                       "l2": "inputs (4 x 128 MiB) are larger than the 126 MB L2"},
            "roofline": fl["roofline"], "cpu_baseline": cpu, "e2e": fl["e2e"],
            "gpu_launches": fl["launches"], "clocks": fl["clocks"], "paged": paged,
            "piecewise": pw, "decode": dec, "rotary": rot,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
