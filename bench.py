#!/usr/bin/env python
"""Benchmark of the block-FP8 hot path (activation quantiser -> W8A8 block-FP8 GEMM
[-> bf16 exchange when N is sharded]) on synthetic data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (all GPU counts): the tensor-parallel MLP GEMM of the benchmark
configurations, M = 8192 tokens, K = 7168, N = 18432, bf16 activations ~N(0,1)
quantised per 1x128 group, weights ~N(0,0.02) quantised per 128x128 block, bf16 output;
N is sharded column-parallel over the GPUs and every GPU ends up with the whole [M, N]
result (strong scaling: total work is fixed).  One step = quantise A, multiply, exchange.
Inputs are drawn on the CPU from seed 0 (activations first, then the weight), so that the
CPU checker sees the same bits: after the timed regions a sample of rows of the LAST timed
step's result - all N columns, i.e. every rank's slice - is compared with the checker.
Prints ONE JSON line on rank 0.  For N > 1 launch with torchrun, one rank per GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, K, N = 8192, 7168, 18432
WORKLOAD = "tensor-parallel block-FP8 MLP GEMM M=8192 K=7168 N=18432 (bf16 act quantised 1x128, e4m3 weight 128x128 scales, bf16 out)"
METRIC = "block-FP8 GEMM TFLOPS"
FLOPS = 2.0 * M * N * K
PARITY_ROWS = 32


def load_peaks():
    """Measured roofline denominators of this GPU pool; fallback = an earlier measurement."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def make_inputs_cpu():
    """Seed 0 on the CPU: activations, then the weight, then a second activation set that only
    serves to rotate the per-step input (every rank draws the same tensors)."""
    g = torch.Generator().manual_seed(0)
    a0 = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    a1 = torch.randn(M, K, generator=g).to(torch.bfloat16)
    return [a0, a1], w


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU while a region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "10"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def window(self, t0: float, t1: float):
        """Summary of the samples taken between two wall-clock times (None if there are none)."""
        inside = [r for (t, r) in list(self.rows) if t0 <= t <= t1 and len(r) >= 9]
        if not inside:
            return None
        sm = [float(r[1]) for r in inside]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[5 + i].lower().startswith("active") for r in inside)]
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(inside[0][2]), "samples": len(inside),
                "power_w_max": max(float(r[3]) for r in inside), "reasons": reasons}

    def stop(self):
        if self.proc is None:
            return
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()


# --------------------------------------------------------------------------- CPU arm (reference's own CPU path)

def cpu_threads() -> int:
    """Use every host core: under torchrun the launcher exports OMP_NUM_THREADS=1, which would make
    the CPU arm at N > 1 a different baseline from the one at N = 1."""
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_step(a, B, Bs):
    """One CPU step: quantise the activations, then the reference's CPU formulation
    (dequantise, fp32 matmul, cast) - finegrained-fp8-helion/bench.py:11-14."""
    from oracle import fp8_oracle as oracle

    A, As = oracle.quant_act(a)
    return oracle.gemm_dequant(A, B, As, Bs).to(torch.bfloat16)


def run_cpu_baseline(steps: int, warmup: int, rows: int = M):
    from oracle import fp8_oracle as oracle

    threads = cpu_threads()
    a_sets, w = make_inputs_cpu()
    a = a_sets[0][:rows]
    B, Bs = oracle.quant_weight(w)
    del w
    for _ in range(warmup):
        cpu_step(a, B, Bs)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(a, B, Bs)
    dt = (time.perf_counter() - t0) / steps
    tflops = 2.0 * rows * N * K / dt / 1e12
    what = "the whole workload" if rows == M else f"first {rows} of {M} token rows against the full {N}x{K} weight"
    return {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{what} ({2.0 * rows * N * K / 1e9:.1f} GFLOP per step, {dt:.2f} s per step, {steps} step(s), "
                      f"torch threads set to the host's {os.cpu_count()} logical CPUs)"}, dt


def main_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # the whole workload per step (about 1.5-2 s on 16 cores); bounded number of steps
    steps, warmup = max(1, min(args.steps, 20)), max(1, min(args.warmup, 2))
    base, dt = run_cpu_baseline(steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp32 (dequantised e4m3)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "reference's CPU formulation (torch dequantise-then-matmul) on all host cores, "
                                                 "every step the whole M x N x K problem"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm

def graph_ms(fn, iters: int, reps: int = 3) -> float:
    """Average device time of one fn() call: `iters` calls captured in a CUDA graph and
    replayed (no host launch overhead between them), CUDA events on the replay stream."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / iters)
    return best


def eager_ms(fn, iters: int = 50) -> float:
    """Average time of one eager fn() call, host launch cost included: `iters` calls back to back
    from Python between two CUDA events (how the reference times its op: scripts/rebench_llm.py:47-54)."""
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def measured_fp8_peak(dev):
    """Yardstick only, never on the product path: the vendor library's dense e4m3 x e4m3 GEMM
    (per-tensor scales, bf16 out) at 8192^3 on this GPU, best of 10 launches."""
    try:
        n = 8192
        a = (torch.randn(n, n, device=dev) * 0.3).to(torch.float8_e4m3fn)
        b = (torch.randn(n, n, device=dev) * 0.3).to(torch.float8_e4m3fn)
        one = torch.ones((), device=dev)
        fn = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / best / 1e9
    except Exception:  # noqa: BLE001 - a yardstick: its absence must not fail the bench
        return None


def extra_shapes(dev, peaks):
    """Other benchmark configurations, device-timed (CUDA-graph replay), rank 0 at N=1 only. Every
    shape whose operands fit the 126 MB L2 rotates over enough distinct operand sets to exceed it."""
    import hf_kernels_helion_b200 as pkg
    from hf_kernels_helion_b200 import runtime

    fp8_peak = 2.0 * peaks["bf16_tflops"]
    out = {}

    def mk(m, n, k):
        a = (torch.randn(m, k, device=dev) * 0.3).to(torch.float8_e4m3fn)
        b = (torch.randn(n, k, device=dev) * 0.3).to(torch.float8_e4m3fn)
        sa = torch.rand(m, k // 128, device=dev) * 0.5 + 0.5
        sb = torch.rand(n // 128, k // 128, device=dev) * 0.5 + 0.5
        return a, b, sa, sb

    for name, (m, n, k, nsets) in {"gemm_2048x2048x4096": (2048, 2048, 4096, 6), "gemm_4096x4096x8192": (4096, 4096, 8192, 3)}.items():
        sets = [mk(m, n, k) + (torch.empty(m, n, dtype=torch.bfloat16, device=dev),) for _ in range(nsets)]
        i = [0]

        def run():
            a, b, sa, sb, c = sets[i[0] % nsets]
            i[0] += 1
            runtime.gemm(a, b, sa, sb, 128, 128, torch.bfloat16, out=c)

        ms = graph_ms(run, 4 * nsets if nsets == 6 else 18)
        tf = 2.0 * m * n * k / ms / 1e9
        out[name] = {"ms": round(ms, 5), "tflops": round(tf, 1), "frac_of_fp8_peak": round(tf / fp8_peak, 3),
                     "operand_sets_rotated": nsets}
        del sets
    for m in (1, 16, 64, 256):
        n, k = 28672, 8192
        a, b, sa, sb = mk(m, n, k)
        c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        ms = graph_ms(lambda: runtime.gemm(a, b, sa, sb, 128, 128, torch.bfloat16, out=c), 20)
        # the drop-in call as a user makes it (allocates its result; host launch cost included)
        op_ms = eager_ms(lambda: pkg.w8a8_block_fp8_matmul(a, b, sa, sb, [128, 128], torch.bfloat16))
        byts = m * k + n * k + 4 * m * (k // 128) + 4 * (n // 128) * (k // 128) + 2 * m * n
        gbs = byts / ms / 1e6
        # bf16 activations in, one library call: the quantiser is the GEMM's own prep launch
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        lin_ms = graph_ms(lambda: runtime.linear(x, b, sb, torch.bfloat16, out=c), 20)
        out[f"decode_M{m}_N28672_K8192"] = {"ms": round(ms, 5), "gbs": round(gbs, 1),
                                            "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 3),
                                            "op_level_eager_ms": round(op_ms, 5),
                                            "fp8_linear_bf16_in_ms": round(lin_ms, 5)}
        if m == 256:   # near the ridge: the tensor-side fraction beside the bandwidth-side one
            tf = 2.0 * m * n * k / ms / 1e9
            out[f"decode_M{m}_N28672_K8192"].update({"tflops": round(tf, 1), "frac_of_fp8_peak": round(tf / fp8_peak, 3)})
        del a, b, sa, sb, c
    # the same GEMM with one B scale per ROW of B (deep-gemm-helion's operand layout)
    m, n, k = 4096, 4096, 8192
    a, b, sa, _ = mk(m, n, k)
    sb_row = torch.rand(n, k // 128, device=dev) * 0.5 + 0.5
    ms = graph_ms(lambda: runtime.gemm_rowscale(a, b, sa, sb_row, 128, torch.bfloat16), 10)
    tf = 2.0 * m * n * k / ms / 1e9
    out["gemm_rowscale_4096x4096x8192"] = {"ms": round(ms, 5), "tflops": round(tf, 1), "frac_of_fp8_peak": round(tf / fp8_peak, 3)}
    del a, b, sa, sb_row
    xs = [torch.randn(4096, 8192, device=dev).to(torch.bfloat16) for _ in range(3)]   # 3 x 64 MiB > L2
    i = [0]

    def q():
        pkg.fp8_act_quant(xs[i[0] % 3])
        i[0] += 1

    ms = graph_ms(q, 18)
    gbs = (4096 * 8192 * 3 + 4096 * 64 * 4) / ms / 1e6
    out["quant_act_4096x8192"] = {"ms": round(ms, 5), "gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 3)}
    out["published_reference_ms_4096x4096x8192"] = {"helion_pretuned": 1.4669, "helion_autotuned": 1.2803, "upstream_triton": 0.9582}
    return out


def parity_sample(out_dev: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    return out_dev[rows.to(out_dev.device)].clone()


def main_ours(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the package has no CPU implementation)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))   # host-side checker work, shared by the ranks

    import hf_kernels_helion_b200 as pkg
    from hf_kernels_helion_b200 import _lib, runtime, tp

    peaks = load_peaks()
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    # ---- synthetic inputs from the CPU generator (seed 0); every rank keeps its slice of the weight
    a_cpu, w_cpu = make_inputs_cpu()
    a_sets = [a.to(dev) for a in a_cpu]          # rotate: the per-step input never sits in L2
    n0, n1 = tp.shard_bounds(N, world, rank)
    B, Bs = pkg.fp8_weight_quant(w_cpu[n0:n1].to(dev))
    n_local = n1 - n0
    parity_rows = torch.randperm(M, generator=torch.Generator().manual_seed(1234))[:PARITY_ROWS].sort().values
    slots = torch.empty((world, M, n_local), dtype=torch.bfloat16, device=dev)      # gather buffer, slot r = rank r's columns
    fulls = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]   # results alternate between two buffers
    turn = [0]

    lin = tp.ShardedFp8Linear(B, Bs) if world > 1 else None
    if world > 1 and args.exchange == "auto":
        # measured on 2, 4 and 8 GPUs: the per-GPU NVLink ingress bounds both fused forms, and the
        # multicast form also receives its own slice back through the switch, so peer stores win
        args.exchange = "fused"
    elif world > 1 and args.exchange == "multimem":
        # every rank must take the same path: agree on multicast support through an all-reduce
        ok = torch.tensor([1.0 if tp.multicast_supported(dev) else 0.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) <= 0:
            raise SystemExit("--exchange multimem: this box reports no NVLink multicast support")
    elif world == 1:
        args.exchange = "none"

    def step(a_bf16, reader_done=None):
        """One pass of the hot path on this rank; returns the contiguous [M, N] bf16 result."""
        q, s = pkg.fp8_act_quant(a_bf16)
        if world == 1:
            out = fulls[turn[0]]
            turn[0] ^= 1
            runtime.gemm(q, B, s, Bs, 128, 128, torch.bfloat16, out=out)
            return out
        if args.exchange == "multimem":
            return lin.forward_multimem(q, s, torch.bfloat16)
        if args.exchange == "fused":
            return lin.forward_fused(q, s, torch.bfloat16, reader_done=reader_done)
        mine = slots[rank]
        runtime.gemm(q, B, s, Bs, 128, 128, torch.bfloat16, out=mine)
        dist.all_gather_into_tensor(slots.view(-1), mine.view(-1))
        out = fulls[turn[0]]
        turn[0] ^= 1
        out.view(M, world, n_local).copy_(slots.permute(1, 0, 2))
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed region: exactly `steps` steps between barrier + synchronize
    for i in range(warmup):
        step(a_sets[i % 2])
    runtime.check_device_status()
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    last_out, last_set = None, 0
    for i in range(steps):
        last_out, last_set = step(a_sets[i % 2]), i % 2
    e1.record()
    barrier()
    t1 = time.time()
    ms_total = e0.elapsed_time(e1)
    runtime.check_device_status()
    samples = {"timed": parity_sample(last_out, parity_rows)}   # every rank checks its own assembled [M, N]
    timed_set = last_set

    # ---- the same steps for at least two seconds, device-timed: the rate the part sustains under its
    #      power limit, with the clocks sampled over exactly this region
    sus_iters = max(10, int(2200.0 / max(ms_total / steps, 1e-3)) + 1)
    if world > 1:
        # every rank must run the same number of steps (they meet in a barrier every step)
        n_it = torch.tensor([sus_iters], dtype=torch.int64, device=dev)
        dist.broadcast(n_it, src=0)
        sus_iters = int(n_it.item())
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ts0 = time.time()
    s0.record()
    for i in range(sus_iters):
        step(a_sets[i % 2])
    s1.record()
    barrier()
    ts1 = time.time()
    sus_ms_total = s0.elapsed_time(s1)
    sampler.stop()
    clocks = sampler.window(t0, t1)
    clocks_sus = sampler.window(ts0 + 0.2, ts1)
    if clocks is None or clocks["samples"] < 2:
        # the K-step region is shorter than two sampling periods of nvidia-smi: report the samples of
        # the first 0.3 s of the sustained region that follows it directly (same steps, same load)
        clocks = sampler.window(ts0, ts0 + 0.3) or clocks_sus or {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        clocks["sampled_over"] = "first 0.3 s of the sustained region that directly follows the timed region"
    else:
        clocks["sampled_over"] = "timed region"
    runtime.check_device_status()

    # ---- end-to-end through the public API with HOST buffers (pinned): H2D of the activations,
    #      quantise + GEMM (+ exchange), D2H of the result, every step.
    #      The result read-back of step i runs on a second stream and overlaps the upload and
    #      the math of step i + 1 (PCIe is full duplex); buffers alternate and are guarded by events.
    # N > 1: the host holds the activations once; rank r uploads rows [r M / world, (r + 1) M / world)
    # and the ranks all-gather them over NVLink (the N-sharded layout needs all of A on every GPU);
    # every rank holds the whole [M, N] result and the host needs it once, so rank r reads back the
    # row block [r M / world, (r + 1) M / world) and the ranks' host buffers together hold C
    r0, r1 = rank * M // world, (rank + 1) * M // world
    host_a = [a[r0:r1].contiguous().pin_memory() for a in a_cpu]
    dev_rows = [torch.empty((r1 - r0, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    host_c = [torch.empty((r1 - r0, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    dev_a = [torch.empty((M, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    d2h_stream = torch.cuda.Stream()
    d2h_done = [None, None]
    phase_ev = {}

    def e2e_step(i, record_phases=False):
        b = i % 2
        comp = torch.cuda.current_stream()

        def mark(name):
            if record_phases:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(comp)
                phase_ev[name] = ev

        if d2h_done[b] is not None:
            comp.wait_event(d2h_done[b])       # host_c[b] and the result buffer about to be rewritten have been read back
        mark("start")
        if world == 1:
            dev_a[b].copy_(host_a[b], non_blocking=True)
            mark("h2d")
        else:
            dev_rows[b].copy_(host_a[b], non_blocking=True)
            mark("h2d")
            dist.all_gather_into_tensor(dev_a[b].view(-1), dev_rows[b].view(-1))
        mark("a_allgather")
        # the read-back of the previous step's result (other buffer set) must be over before peers may
        # overwrite that buffer: the fused exchange waits for it ahead of its barrier
        out = step(dev_a[b], reader_done=d2h_done[b ^ 1])
        mark("step")
        ready = torch.cuda.Event()
        ready.record(comp)
        d2h_stream.wait_event(ready)
        with torch.cuda.stream(d2h_stream):
            host_c[b].copy_(out[r0:r1], non_blocking=True)
            done = torch.cuda.Event(enable_timing=record_phases)
            done.record(d2h_stream)
        d2h_done[b] = done
        return out

    e2e_steps = max(2, min(steps, 10))
    for i in range(2):
        e2e_step(i)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.current_stream().wait_stream(d2h_stream)   # the last read-backs are inside the timed region
    f1.record()
    barrier()
    e2e_ms_total = f0.elapsed_time(f1)
    # what the host received in the last end-to-end step: this rank's row block of C
    last_b = (e2e_steps - 1) % 2
    mine = (parity_rows >= r0) & (parity_rows < r1)
    if bool(mine.any()):
        samples["e2e_host"] = host_c[last_b][parity_rows[mine] - r0].clone()
    e2e_host_set = last_b

    # ---- one end-to-end step taken apart (events between its phases, nothing overlapping it), and the
    #      host link alone: every rank moving its row blocks at the same time, no compute
    barrier()
    e2e_step(e2e_steps, record_phases=True)
    torch.cuda.current_stream().wait_stream(d2h_stream)
    barrier()
    pe = phase_ev
    e2e_phases = {"h2d_ms": pe["start"].elapsed_time(pe["h2d"]), "a_allgather_ms": pe["h2d"].elapsed_time(pe["a_allgather"]),
                  "step_ms": pe["a_allgather"].elapsed_time(pe["step"]), "d2h_ms": pe["step"].elapsed_time(d2h_done[e2e_steps % 2])}
    c0, c1, c2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    barrier()
    c0.record()
    for _ in range(3):
        dev_rows[0].copy_(host_a[0], non_blocking=True)
    c1.record()
    src = fulls[0][r0:r1] if world == 1 else last_out[r0:r1]
    for _ in range(3):
        host_c[0].copy_(src, non_blocking=True)
    c2.record()
    barrier()
    e2e_phases["pinned_copy_only_h2d_ms"] = c0.elapsed_time(c1) / 3
    e2e_phases["pinned_copy_only_d2h_ms"] = c1.elapsed_time(c2) / 3

    # ---- dominant kernel alone (the GEMM launch of one step), CUDA events on its stream
    q, s = pkg.fp8_act_quant(a_sets[0])
    gemm_out = fulls[0] if world == 1 else slots[rank]
    for _ in range(3):
        runtime.gemm(q, B, s, Bs, 128, 128, torch.bfloat16, out=gemm_out)
    torch.cuda.synchronize()
    k_iters = 10
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(k_iters):
        runtime.gemm(q, B, s, Bs, 128, 128, torch.bfloat16, out=gemm_out)
    g1.record()
    torch.cuda.synchronize()
    gemm_ms = g0.elapsed_time(g1) / k_iters
    quant_ms = graph_ms(lambda: pkg.fp8_act_quant(a_sets[0]), 10)

    # ---- N > 1: the exchange by itself against the library collective on the same bytes
    exchange = None
    if world > 1:
        fused_ms = nccl_ms = None
        if args.exchange == "fused":
            for _ in range(3):
                lin.forward_fused(q, s, torch.bfloat16)
            barrier()
            x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            x0.record()
            for _ in range(k_iters):
                lin.forward_fused(q, s, torch.bfloat16)
            x1.record()
            barrier()
            fused_ms = x0.elapsed_time(x1) / k_iters
        mine_slot = slots[rank]
        for _ in range(3):
            dist.all_gather_into_tensor(slots.view(-1), mine_slot.view(-1))
        barrier()
        y0, y1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        y0.record()
        for _ in range(k_iters):
            dist.all_gather_into_tensor(slots.view(-1), mine_slot.view(-1))
        y1.record()
        barrier()
        nccl_ms = y0.elapsed_time(y1) / k_iters
        exchange = {"fused_ms": fused_ms, "nccl_allgather_ms": nccl_ms}

    # ---- checker (host, outside every timed region): sampled rows, all N columns, of the last timed
    #      step's result on THIS rank, and of what the host received in the last end-to-end step
    # (the slice identity C[:, n0:n1] = A . B[n0:n1]^T rests on torch-ext/finegrained_fp8_helion/fp8.py:30-36)
    worst = {}
    from oracle import fp8_oracle as oracle
    Bq_cpu, Bs_cpu = oracle.quant_weight(w_cpu)
    refs = {}
    for set_idx in {timed_set, e2e_host_set}:
        Aq_cpu, As_cpu = oracle.quant_act(a_cpu[set_idx][parity_rows])
        refs[set_idx] = oracle.gemm_dequant(Aq_cpu, Bq_cpu, As_cpu, Bs_cpu)
    worst["timed"] = float(oracle.bf16_ulp_error(samples["timed"].cpu(), refs[timed_set]))
    if "e2e_host" in samples:
        worst["e2e_host"] = float(oracle.bf16_ulp_error(samples["e2e_host"], refs[e2e_host_set][mine]))
    max_ulp = max(worst.values())
    ok_local = 1.0 if max_ulp <= 1.0 else 0.0

    # ---- max over ranks
    vals = torch.tensor([ms_total, e2e_ms_total, gemm_ms, quant_ms, sus_ms_total, max_ulp,
                         exchange["fused_ms"] or 0.0 if exchange else 0.0, exchange["nccl_allgather_ms"] if exchange else 0.0]
                        + [e2e_phases[k] for k in sorted(e2e_phases)], dtype=torch.float64, device=dev)
    oks = torch.tensor([ok_local], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(oks, op=dist.ReduceOp.SUM)
    v = [float(x) for x in vals.tolist()]
    ms_total, e2e_ms_total, gemm_ms, quant_ms, sus_ms_total, max_ulp, fused_ms, nccl_ms = v[:8]
    e2e_phases = {k: round(x, 4) for k, x in zip(sorted(e2e_phases), v[8:])}
    ranks_ok = int(round(float(oks.item())))

    if rank == 0:
        ms_per_step = ms_total / steps
        value = FLOPS / (ms_per_step * 1e-3) / 1e12
        sus_ms = sus_ms_total / sus_iters
        e2e_value = FLOPS / (e2e_ms_total / e2e_steps * 1e-3) / 1e12
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        gemm_flops = 2.0 * M * n_local * K
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
        variant = _lib.load().b200fp8_gemm_pick_variant(M, n_local, K)
        # (the 256-wide forms stage their output and store it by TMA: the *_multi_kernel instantiations, one destination at N = 1)
        kernel = {1: "gemm_tile_kernel<128>", 2: "gemm_tile_multi_kernel<256>", 3: "gemm_streamk_kernel",
                  4: "gemm_tile_kernel<256> with tail split-K", 5: "gemm_pair_multi_kernel<false>",
                  6: "gemm_pair_multi_kernel<true>", 7: "gemm_pair_multi_sk_kernel"}[variant]
        if world > 1 and args.exchange == "fused" and variant == 2 and M > 128:
            kernel = "gemm_pair_multi_kernel<true>"   # several destinations: AUTO takes the pair form whenever M > 128
        # DRAM bytes of one GEMM launch at 1 GPU, from one profiler capture of this kernel on this shape
        # (dram__bytes_read.sum / dram__bytes_write.sum); at N > 1 scaled by the share of the weight and of
        # the output a rank touches (A is read whole by every rank). Not re-measured by this run.
        traffic_1gpu = {"read": 482.3e6, "write": 295.5e6}
        traffic = (M * K + (traffic_1gpu["read"] - M * K) / world) + traffic_1gpu["write"] / world
        if world == 1:
            step_desc = "fp8_act_quant(A bf16) + w8a8_block_fp8_matmul"
        elif args.exchange == "fused":
            step_desc = ("fp8_act_quant(A bf16) + w8a8_block_fp8_matmul whose epilogue stores the slice into every GPU's [M,N] "
                         "buffer over NVLink + " + ("flag-exchange barrier kernel (b200fp8_peer_barrier)" if lin.device_barrier
                                                    else "1-element all_reduce as barrier"))
        elif args.exchange == "multimem":
            step_desc = ("fp8_act_quant(A bf16) + w8a8_block_fp8_matmul whose epilogue writes the slice once to the NVLink "
                         "multicast view of every GPU's [M,N] buffer (multimem.st) + 1-element all_reduce as barrier")
        else:
            step_desc = "fp8_act_quant(A bf16) + w8a8_block_fp8_matmul + all_gather + slot->[M,N] copy"
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8_e4m3 x fp8_e4m3 -> fp32 accumulate -> bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "parallelism": f"N sharded over {world} GPU(s), exchange={args.exchange}" if world > 1 else "single GPU",
                       "step": step_desc,
                       "barrier": None if world == 1 else ("peer_flags" if args.exchange == "fused" and lin.device_barrier else "all_reduce" if args.exchange != "nccl" else "nccl"),
                       "inputs": "torch CPU generator, seed 0: activations, then weight (a second activation set rotates the per-step input)",
                       "l2": "per-step traffic (A bf16 117 MB rotating over 2 buffers, C bf16 302 MB) exceeds the 126 MB L2; no flush"},
            "clocks": clocks,
            "value_sustained": {"value": FLOPS / (sus_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": sus_iters, "ms_per_step": sus_ms,
                                "seconds": sus_ms_total / 1e3, "clocks": clocks_sus,
                                "ms_x_median_sm_mhz": (sus_ms * clocks_sus["sm_mhz"]) if clocks_sus and clocks_sus.get("sm_mhz") else None,
                                "note": "the same steps back to back for >= 2 s, CUDA events, max over ranks; clocks sampled over this region (first 0.2 s left out)"},
            "parity": {"rows": PARITY_ROWS, "columns": N, "max_ulp": max_ulp, "ok": ranks_ok == world, "ranks_ok": ranks_ok,
                       "checked": "sampled rows x all N columns of the last timed step's [M,N] on every rank, and of the row block the host "
                                  "received in the last end-to-end step, against the CPU checker (quantise + dequantise-then-matmul); bound 1 bf16 ulp"},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                    "steps": e2e_steps, "ms_per_step": e2e_ms_total / e2e_steps, "phases_one_step_serial": e2e_phases,
                    "note": "bytes are job totals: the pinned bf16 activations go up once per step (each rank uploads its M/n_gpus row block and the ranks all-gather the rows over NVLink, "
                            "since the N-sharded layout needs all of A on every GPU), the [M,N] bf16 result comes back to pinned host memory once per step "
                            "(each rank reads back its M/n_gpus row block of the assembled result); "
                            "read-back of step i overlaps upload + math of step i+1 (second stream); the quantised weight is a resident parameter; "
                            "phases_one_step_serial: one extra step with events between its phases and nothing overlapping, max over ranks, plus the pinned copies alone"},
            # per step: quant_act_contig_kernel, tile_prep_kernel, the GEMM kernel; N > 1 adds the exchange's
            # barrier kernel (fused) or NCCL's all-gather plus the slot -> [M,N] copy (not counted: not ours)
            # per step: quantiser, scale re-layout, GEMM; + the split-K fix-up pass where AUTO takes such a form;
            # + the barrier kernel of the fused exchange
            "gpu_launches": steps * (3 + (1 if variant in (4, 7) and world == 1 else 0)
                                     + (1 if world > 1 and args.exchange == "fused" else 0)),
            "roofline": {"bound": "tensor", "kernel": kernel, "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s",
                         "frac": achieved / fp8_peak, "traffic": traffic,
                         "peak_source": f"2 x bf16_tflops ({peaks['bf16_tflops']}) of MEASURED_PEAKS.json ({peaks['source']}): "
                                        "dense e4m3 runs at twice the dense bf16 rate; the file holds no fp8 figure",
                         "frac_of_nominal_4500": achieved / 4500.0, "launch_ms": gemm_ms,
                         "algorithmic_flops_per_launch": gemm_flops},
            "phases_ms": {"quant_act": quant_ms, "gemm": gemm_ms, "step": ms_per_step},
        }
        if exchange is not None:
            bytes_in = (world - 1) * M * n_local * 2
            line["exchange"] = {"fused_ms": fused_ms or None, "nccl_allgather_ms": nccl_ms, "bytes_in_per_gpu": bytes_in,
                                "gbs_fused": (bytes_in / fused_ms / 1e6) if fused_ms else None, "gbs_nccl": bytes_in / nccl_ms / 1e6,
                                "nvlink_ceiling_ms_at_900_gbs": bytes_in / 900e9 * 1e3,
                                "note": "fused_ms = GEMM with peer stores + barrier (device time, max over ranks); nccl_allgather_ms = one in-place "
                                        "all_gather_into_tensor of the same slices, no GEMM; both outside the timed step"}
        if world == 1:
            pk = measured_fp8_peak(dev)
            if pk is not None:
                line["roofline"]["peak_fp8_measured"] = pk
                line["roofline"]["frac_of_measured_fp8"] = achieved / pk
                line["roofline"]["peak_fp8_measured_how"] = "torch._scaled_mm e4m3 x e4m3 8192^3, per-tensor scales, bf16 out, best of 10 (yardstick, not on the product path)"
            line["extra_shapes"] = extra_shapes(dev, peaks)
            base, _ = run_cpu_baseline(2, 1)
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
        if ranks_ok != world:
            print(f"PARITY FAILED: {world - ranks_ok} rank(s) beyond 1 bf16 ulp (max {max_ulp})", file=sys.stderr, flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if ranks_ok != world:
        sys.exit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--exchange", choices=["auto", "multimem", "fused", "nccl"], default="auto",
                    help="N > 1: how the column slices reach every GPU: GEMM epilogue multicast stores through the "
                         "NVSwitch, GEMM epilogue peer stores, or NCCL all-gather; auto = fused (fastest measured)")
    args = ap.parse_args()
    if args.impl == "reference":
        main_reference(args)
    else:
        main_ours(args)


if __name__ == "__main__":
    main()
