#!/usr/bin/env python
"""Benchmark of the Stream-K GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--sweep FILE]

Headline workload (every N): configuration 5, the large fp16 NT GEMM
M=8192 N=28672 K=8192 (A ~ N(0,1), B ~ N(0,0.02), seeded, synthetic).  With N GPUs the
weight rows (output columns) are sharded N-ways, each GPU runs its own Stream-K launch on
its slab and no collective is on the data path (strong scaling: the total work is fixed).
A step is one GEMM over the whole problem.  Rank 0 prints ONE JSON line.

--sweep FILE additionally times configurations 2, 3 and 4 (24 fp16 shapes x schedules, 9
W4A16 shapes) L2-cold on one GPU and writes the table to FILE as JSON.

--impl reference times the reference's CPU expression for the path
(`torch.matmul(A.float(), B.float().T)` on the host cores) on a bounded row slice.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M5, N5, K5 = 8192, 28672, 8192
BASE_SLAB = N5 // 8            # B is generated in eight 3584-row slabs, whatever N is
CPU_SAMPLE_ROWS = 256
NOMINAL_TFLOPS = 2250.0
NOMINAL_HBM_GBS = 8000.0


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons; stop(t0, t1) keeps the samples whose
    timestamp falls inside the timed region [t0, t1] (wall clock, seconds)."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu), "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
        except OSError:
            self.proc = None

    def stop(self, t0: float, t1: float) -> dict:
        import datetime
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        rows = []
        for line in out.strip().split("\n"):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[1]), float(f[2]), float(f[3]), f[5:9]))
            except ValueError:
                continue
        inside = [r for r in rows if t0 <= r[0] <= t1]
        note = "samples inside the timed region"
        if not inside:                       # region shorter than the sampling period
            inside = [r for r in rows if t0 - 0.05 <= r[0] <= t1 + 0.05] or rows
            note = "no sample fell inside the timed region; nearest samples used"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        reasons = set()
        for r in inside:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), r[4]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": max(r[2] for r in inside),
                "samples": len(inside), "power_w_max": max(r[3] for r in inside),
                "reasons": sorted(reasons), "note": note}


def cpu_gemm_sample(A_rows, B, reps: int) -> tuple[float, int]:
    """Seconds per `torch.matmul(A.float(), B.float().T)` on the host, threads used."""
    import torch
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    Af, Bf = A_rows.float(), B.float()
    torch.matmul(Af, Bf.t())  # warm the thread pool
    t0 = time.perf_counter()
    torch.matmul(Af, Bf.t())
    one = time.perf_counter() - t0
    reps = max(reps, min(200, int(10.0 / max(one, 1e-3))))   # about 10 s of CPU work
    t0 = time.perf_counter()
    for _ in range(reps):
        torch.matmul(Af, Bf.t())
    return (time.perf_counter() - t0) / reps, torch.get_num_threads()


def make_operands(rank: int, world: int, device):
    """A (full) and this rank's slab of B, identical global values for every world size."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(5000)
    A = torch.randn(M5, K5, generator=g, device=device, dtype=torch.float32).half()
    per = 8 // world
    slabs = []
    for s in range(rank * per, (rank + 1) * per):
        g.manual_seed(5001 + s)
        slabs.append((0.02 * torch.randn(BASE_SLAB, K5, generator=g, device=device,
                                         dtype=torch.float32)).half())
    return A, torch.cat(slabs, 0)


def reference_arm(args, rank: int) -> None:
    if rank != 0:
        return
    import torch
    g = torch.Generator().manual_seed(5000)
    A = torch.randn(CPU_SAMPLE_ROWS, K5, generator=g).half()
    B = (0.02 * torch.randn(N5, K5, generator=g)).half()
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    Af, Bf = A.float(), B.float()
    for _ in range(max(args.warmup, 1)):
        torch.matmul(Af, Bf.t())
    t0 = time.perf_counter()
    for _ in range(args.steps):
        torch.matmul(Af, Bf.t())
    dt = (time.perf_counter() - t0) / args.steps
    tflops = 2.0 * CPU_SAMPLE_ROWS * N5 * K5 / dt / 1e12
    sample = (f"{CPU_SAMPLE_ROWS}-row slice of A (1/{M5 // CPU_SAMPLE_ROWS} of the problem) against the "
              f"full B; torch.matmul(A.float(), B.float().T) on host cores")
    print(json.dumps({
        "impl": "reference", "metric": "Stream-K fp16 GEMM TFLOP/s", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": f"cfg5 fp16 NT GEMM M={M5} N={N5} K={K5}", "sampled": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------- sweep
def time_rotating(launch, n_copies: int, est_us: float, batches: int = 25):
    """p50/p10/p90 per-launch microseconds; launch(i) uses operand copy i (L2-cold rotation).

    A batch of launches is captured once into a CUDA graph and replayed, so the figure is
    device time per kernel, not the host's launch rate."""
    import torch
    n = max(n_copies, int(math.ceil(1000.0 / max(est_us, 1.0))))
    n = min(n, 512)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(max(3, min(n_copies, 8))):
            launch(i % n_copies)        # also creates this stream's workspace before capture
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(n):
            launch(i % n_copies)
    times = []
    with torch.cuda.stream(side):
        for _ in range(3):
            graph.replay()
        side.synchronize()
        for _ in range(batches):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            graph.replay()
            e1.record(side)
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / n)
    torch.cuda.current_stream().wait_stream(side)
    times.sort()
    return times[len(times) // 2], times[len(times) // 10], times[(len(times) * 9) // 10]


def run_sweep(path: str, peaks: dict) -> None:
    import torch
    import oracle
    import streamk_b200 as sk
    dev = torch.device("cuda", torch.cuda.current_device())
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    rows = []

    def roof(flops, nbytes):
        t_nom = max(flops / (NOMINAL_TFLOPS * 1e12), nbytes / (NOMINAL_HBM_GBS * 1e9))
        t_meas = max(flops / (peaks["bf16_tflops"] * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9))
        bound = "tensor" if flops / (peaks["bf16_tflops"] * 1e12) > nbytes / (peaks["hbm_gbs"] * 1e9) else "hbm"
        return t_nom * 1e6, t_meas * 1e6, bound

    def record(cfg, name, M, N, K, variant, us, flops, nbytes, extra=None):
        t_nom, t_meas, bound = roof(flops, nbytes)
        r = {"cfg": cfg, "entry": name, "M": M, "N": N, "K": K, "variant": variant,
             "p50_us": round(us[0], 3), "p10_us": round(us[1], 3), "p90_us": round(us[2], 3),
             "tflops": round(flops / us[0] / 1e6, 2), "gbs": round(nbytes / us[0] / 1e3, 1),
             "bound": bound, "frac_of_nominal_roof": round(t_nom / us[0], 4),
             "frac_of_measured_roof": round(t_meas / us[0], 4)}
        if extra:
            r.update(extra)
        rows.append(r)
        print(json.dumps(r), file=sys.stderr, flush=True)

    def fp16_case(cfg, case):
        c = oracle.make_case(cfg, case)
        M, N, K = c["M"], c["N"], c["K"]
        A = c["A"].to(dev)
        wbytes = 2 * N * K
        copies = min(int(math.ceil(2 * l2 / wbytes)) + 1, 40)
        Bs = [c["B"].to(dev).clone() for _ in range(copies)]
        out = torch.empty(M, N, dtype=torch.float16, device=dev)
        flops, nbytes = 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
        est = max(nbytes / 6.5e3, flops / 1.5e9) / 1e3 + 3
        ref = oracle.gemm_ref(c["A"], c["B"], "nt")
        # tile None = the library's own choice (operands swapped for M <= 64, CTA pairs for
        # large problems); explicit 128 x 256 tiles are timed as well where they make sense
        variants = [("auto", "block_reduce", None), ("streamk", "atomic", None),
                    ("streamk", "block_reduce", None), ("hybrid", "block_reduce", None),
                    ("dp", "atomic", None)]
        if M > 64 and N * M >= 256 * 4096:
            variants += [("streamk", "block_reduce", 256), ("dp", "atomic", 256)]
        # split-K inside clusters, where there are few enough tiles for it
        try:
            if sk.schedule_info(M, N, K, schedule="cluster")["cluster"] > 0:
                variants.append(("cluster", "block_reduce", None))
        except sk.StreamKError:
            pass
        # the library's choice once more, launched with SK_FLAG_PDL: in a chain of launches the
        # start-up of one overlaps the tail of the one before (what the graph replay times)
        variants.append(("auto+pdl", "block_reduce", None))
        for schedule, fixup, tile_n in variants:
            pdl = schedule.endswith("+pdl")
            schedule = schedule.split("+")[0]
            fn = lambda i: sk.streamk_fp16_nt(A, Bs[i], schedule=schedule, fixup=fixup, out=out, tile_n=tile_n,
                                              pdl=pdl)
            fn(0)
            sk.check_status()
            err = oracle.rel_err(out, ref)
            us = time_rotating(fn, copies, est)
            info = sk.schedule_info(M, N, K, schedule=schedule, tile_n=tile_n)
            names = {v: k for k, v in sk.SCHEDULES.items()}
            how = f"cluster of {info['cluster']}" if info["cluster"] else fixup
            label = schedule if schedule != "auto" else f"auto={names[info['schedule']]}"
            if pdl:
                label = "pdl " + label
            record(cfg, "streamk_fp16_nt", M, N, K,
                   f"{label}/{how}/tile{info['tile_m']}x{info['tile_n']}", us, flops, nbytes,
                   {"rel_err": float(f"{err:.3e}")})
        fn = lambda i: torch.matmul(A, Bs[i].t(), out=out)
        us = time_rotating(fn, copies, est)
        record(cfg, "cublas torch.matmul", M, N, K, "data-parallel library GEMM", us, flops, nbytes)

    def q4_case(case):
        c = oracle.make_case(4, case)
        M, N, K = c["M"], c["N"], c["K"]
        A = c["A"].to(dev)
        wbytes = N * K // 2
        copies = min(int(math.ceil(2 * l2 / wbytes)) + 1, 64)
        P0 = sk.q4_prepack(c["qweight"].to(dev), c["scales"].to(dev), c["zeros"].to(dev))
        Ps = [P0] + [sk.PackedQ4(P0.data.clone(), N, K) for _ in range(copies - 1)]
        out = torch.empty(M, N, dtype=torch.float16, device=dev)
        flops = 2.0 * M * N * K
        nbytes = 2.0 * M * K + N * K / 2 + 3.0 * N * K / 128 + 2.0 * M * N
        est = max(nbytes / 6.5e3, flops / 1.5e9) / 1e3 + 3
        ref = oracle.w4a16_ref(c["A"], c["q"], c["scales"], c["zeros"])
        for schedule, fixup in (("auto", "block_reduce"), ("streamk", "block_reduce"),
                                ("hybrid", "block_reduce"), ("streamk", "atomic"), ("auto+pdl", "block_reduce")):
            pdl = schedule.endswith("+pdl")
            schedule = schedule.split("+")[0]
            fn = lambda i: sk.streamk_fp16_ladder_block_reduce_q4(A, Ps[i], schedule=schedule, fixup=fixup, out=out,
                                                                  pdl=pdl)
            fn(0)
            sk.check_status()
            err = oracle.rel_err(out, ref)
            us = time_rotating(fn, copies, est)
            record(4, "streamk_fp16_ladder_block_reduce_q4", M, N, K, f"{'pdl ' if pdl else ''}{schedule}/{fixup}", us, flops, nbytes,
                   {"rel_err": float(f"{err:.3e}")})
        W = sk.dequant_w4(P0)
        Ws = [W.clone() for _ in range(min(copies, int(math.ceil(2 * l2 / (2 * N * K))) + 1))]
        fn = lambda i: torch.matmul(A, Ws[i % len(Ws)].t(), out=out)
        us = time_rotating(fn, len(Ws), est)
        record(4, "cublas on dequantised fp16 W", M, N, K, "library GEMM, 4x the weight bytes", us, flops, nbytes)

    fp16_case(2, 0)
    for case in range(len(oracle.CONFIGS[3]["shapes"])):
        fp16_case(3, case)
    for case in range(len(oracle.CONFIGS[4]["shapes"])):
        q4_case(case)
    json.dump({"peaks": peaks, "protocol": "L2-cold: weights rotate through ceil(2*L2/bytes)+1 copies; "
               "CUDA events around CUDA-graph replays of >= 1 ms batches; p50 over 25 replays", "rows": rows},
              open(path, "w"), indent=1)


# ------------------------------------------------------------------------- main arm
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sweep", default=None, help="also time configs 2-4 and write the table here")
    ap.add_argument("--schedule", default=os.environ.get("SK_BENCH_SCHEDULE", "auto"))
    ap.add_argument("--fixup", default=os.environ.get("SK_BENCH_FIXUP", "block_reduce"))
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist
    import streamk_b200 as sk

    if world not in (1, 2, 4, 8):
        raise SystemExit("the column sharding of configuration 5 supports 1, 2, 4 or 8 GPUs")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL writes a version banner to standard output when its first communicator comes up;
        # standard output is for the one JSON line, so the banner goes to standard error.
        sys.stdout.flush()
        keep = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=dev)
        t = torch.zeros(1, device=dev)
        dist.all_reduce(t)
        torch.cuda.synchronize()
        sys.stdout.flush()
        os.dup2(keep, 1)
        os.close(keep)
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    n_slab = N5 // world
    A, B = make_operands(rank, world, dev)
    C = torch.empty(M5, n_slab, dtype=torch.float16, device=dev)
    step = lambda: sk.streamk_fp16_nt(A, B, out=C, schedule=args.schedule, fixup=args.fixup)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    info = sk.schedule_info(M5, n_slab, K5, kind="f16_pairs", schedule=args.schedule, num_sms=sms // 2)

    # ---- device-resident timing -------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    sk.check_status()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    t_wall1 = time.time()
    my_ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    total_ms = max_over_ranks(my_ms)
    sk.check_status()
    flops_total = 2.0 * M5 * N5 * K5
    value = flops_total * args.steps / (total_ms * 1e-3) / 1e12

    # spot check of the timed output against an fp32 product of the same operands
    rows = torch.arange(0, M5, M5 // 16, device=dev)[:16]
    ref = A[rows].float() @ B.float().t()
    check = float((C[rows].float() - ref).abs().max() / ref.abs().max())

    # cuBLAS fp16 on the same operands, for context (library data-parallel GEMM)
    for _ in range(3):
        torch.matmul(A, B.t(), out=C)
    barrier()
    e0.record()
    for _ in range(args.steps):
        torch.matmul(A, B.t(), out=C)
    e1.record()
    barrier()
    cublas_ms = max_over_ranks(e0.elapsed_time(e1))
    cublas_tflops = flops_total * args.steps / (cublas_ms * 1e-3) / 1e12
    step()

    # ---- end to end: host buffers in, host result out ---------------------------
    e2e_steps = max(1, min(args.steps, 5))
    A_h = torch.empty(A.shape, dtype=A.dtype).pin_memory(); A_h.copy_(A)
    B_h = torch.empty(B.shape, dtype=B.dtype).pin_memory(); B_h.copy_(B)
    C_h = torch.empty(C.shape, dtype=C.dtype).pin_memory()

    # the library's host-buffer entry point: B and C move in column slabs, copies in, GEMMs and
    # copies out overlapping on three streams (every byte still crosses PCIe inside the timed region)
    e2e_slabs = max(2, 8 // world)

    def e2e_step():
        sk.streamk_fp16_nt_host(A_h, B_h, C_h, slabs=e2e_slabs, schedule=args.schedule, fixup=args.fixup)

    e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    e2e_value = flops_total * e2e_steps / (e2e_ms * 1e-3) / 1e12
    torch.cuda.synchronize()
    e2e_check = float((C_h[rows.cpu()].float().to(dev) - ref).abs().max() / ref.abs().max())
    h2d = (A_h.numel() + B_h.numel()) * 2 * world
    d2h = C_h.numel() * 2 * world

    # ---- optional collective, timed on its own (not part of `value`) -------------
    gather_ms = None
    if world > 1:
        parts = torch.empty(world, M5, n_slab, dtype=torch.float16, device=dev)
        for _ in range(2):
            dist.all_gather_into_tensor(parts, C)
        barrier()
        e0.record()
        for _ in range(5):
            step()
            dist.all_gather_into_tensor(parts, C)
        e1.record()
        barrier()
        gather_ms = max_over_ranks(e0.elapsed_time(e1)) / 5

    # ---- the same product with the all-gather fused into the epilogue (peer stores) ----
    fused = None
    if world > 1:
        res, err = None, ""
        try:
            res = sk.GatheredResult(M5, N5)   # (raises on every rank or on none)
        except Exception as e:
            err = f"{type(e).__name__}: {e}"
        if res is not None:
            for _ in range(2):
                sk.streamk_fp16_nt_gather(A, B, res, schedule=args.schedule, fixup=args.fixup)
            barrier()
            e0.record()
            for _ in range(5):
                sk.streamk_fp16_nt_gather(A, B, res, schedule=args.schedule, fixup=args.fixup)
            e1.record()
            barrier()
            fused_ms = max_over_ranks(e0.elapsed_time(e1)) / 5
            sk.check_status()
            # every block of the gathered matrix against what NCCL delivered (same kernels, same bits
            # with the block-reduce fixup; the atomic fixup's summation order is free)
            same = all(torch.equal(res.full[:, r * n_slab:(r + 1) * n_slab], parts[r]) for r in range(world))
            worst = max(float((res.full[:, r * n_slab:(r + 1) * n_slab].float() - parts[r].float()).abs().max())
                        for r in range(world))
            agree = torch.tensor([1.0 if same else 0.0, -worst], device=dev)
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            scale = torch.tensor([float(parts.float().abs().max())], device=dev)
            dist.all_reduce(scale, op=dist.ReduceOp.MAX)
            # (bitwise equality needs the same tiling in both runs; a link-bound gather drops the
            # 256 x 512 units, which moves the split tiles and with them the summation order)
            fused = {"gemm_fused_allgather_ms": fused_ms, "bitwise_equal_to_nccl_gather": bool(agree[0].item() == 1.0),
                     "max_rel_diff_to_nccl_gather": float(-agree[1].item()) / float(scale.item()),
                     "bytes_pushed_per_gpu": M5 * n_slab * 2 * (world - 1)}
            res.close()
        else:
            fused = {"error": err}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant (only) kernel ---------------------------------
    launch_ms = my_ms / args.steps
    achieved = 2.0 * M5 * n_slab * K5 / (launch_ms * 1e-3) / 1e12
    timed_s = total_ms * 1e-3
    # The kernel is timed back to back: once that lasts long enough for the power cap to set
    # the clock (sw_power_cap seen, or a quarter second of sustained work) the sustained
    # cuBLAS figure is the like-for-like peak; a short burst is compared with the burst one.
    capped = bool(clocks and "sw_power_cap" in (clocks.get("reasons") or []))
    peak_key = "bf16_tflops_sustained" if (capped or timed_s >= 0.25) else "bf16_tflops"
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    if os.path.exists(tpath):
        t = json.load(open(tpath)).get("sk_gemm_f16_kernel_cfg5")
        if t:
            traffic = t["dram_bytes_per_launch_full_problem"] / world
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks[peak_key], "unit": "TFLOP/s",
                "frac": achieved / peaks[peak_key], "traffic": traffic,
                "peak_source": f"{peaks['source']} {peak_key}",
                "frac_of_burst_peak": achieved / peaks["bf16_tflops"],
                "frac_of_nominal_2250": achieved / NOMINAL_TFLOPS,
                "kernel": "sk_gemm_f16_2cta_kernel (CTA pairs; 256x256x64 tiles, data-parallel part in 256x512 units)"}

    cpu_baseline = None
    if world == 1:
        rows_s = A[:CPU_SAMPLE_ROWS].cpu()
        sec, threads = cpu_gemm_sample(rows_s, B.cpu(), reps=3)
        cpu_baseline = {"value": 2.0 * CPU_SAMPLE_ROWS * N5 * K5 / sec / 1e12, "unit": "TFLOP/s",
                        "cores": threads, "kind": "port",
                        "sample": f"{CPU_SAMPLE_ROWS}-row slice of A against the full B, "
                                  f"torch.matmul(A.float(), B.float().T), {sec:.3f} s per product, "
                                  f"repeated for about 10 s"}

    out = {
        "metric": "Stream-K fp16 GEMM TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": f"cfg5 fp16 NT GEMM M={M5} N={N5} K={K5}, N sharded {world}-way",
                   "schedule": {v: k for k, v in __import__("streamk_b200")._lib.SCHEDULES.items()}[info["schedule"]]
                   + (" (auto)" if args.schedule == "auto" else ""),
                   "fixup": args.fixup, "tile": [info["tile_m"], info["tile_n"], 64],
                   "sk_tiles": info["sk_tiles"], "dp_tiles": info["dp_tiles"],
                   "dp_units_256x512": info["wide_units"],
                   "l2": "operands (>= 0.25 GB per GPU) exceed the 126 MB L2; no flush needed"},
        "per_gpu_tflops": value / world,
        "roofline": roofline, "cpu_baseline": cpu_baseline,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "call": f"streamk_fp16_nt_host, {e2e_slabs} column slabs per GPU", "check_rel_err": e2e_check},
        "gpu_launches": args.steps, "clocks": clocks, "check_rel_err": check,
        "cublas_fp16_tflops_same_operands": cublas_tflops,
    }
    if gather_ms is not None:
        out["gemm_plus_allgather_ms"] = gather_ms
    if fused is not None:
        out["fused_allgather"] = fused
    if args.sweep and world == 1:
        run_sweep(args.sweep, peaks)
        out["sweep_file"] = args.sweep
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
