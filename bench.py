#!/usr/bin/env python
"""Benchmark of the Stream-K GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--no-summary] [--sweep FILE] [--tune FILE]
    python bench.py --case KIND M N K [--schedule S] [--fixup F] [--tile-m T] [--tile-n T]
                    [--iters I] [--cublas] [--peers P]

Headline workload (every N): configuration 5, the large fp16 NT GEMM
M=8192 N=28672 K=8192 (A ~ N(0,1), B ~ N(0,0.02), seeded, synthetic).  With N GPUs the
weight rows (output columns) are sharded N-ways, each GPU runs its own Stream-K launch on
its slab and no collective is on the data path (strong scaling: the total work is fixed).
A step is one GEMM over the whole problem.  Rank 0 prints ONE JSON line; besides the
contract's keys it carries

  p50_us            median device time of one launch (per-launch CUDA events)
  sustained         the same kernel in a >= 2 s loop after a pre-heat: the power-capped regime
  sweep_summary     (N = 1) a fixed subset of configurations 1-4, L2-cold p50 per launch beside
                    cuBLAS, the reference's own Triton kernel where available, the measured roof
                    and the CPU baseline of each shape; every result is checked against the oracle
                    and the run FAILS if one is out of tolerance
  with_gather       (N > 1) the product including the all-gather of C: NCCL after the GEMM, and
                    fused into the epilogue, with the efficiency against one GPU of the same box

--sweep FILE times every shape of configurations 2-4 with every schedule and writes FILE.
--tune FILE   times the tile / schedule candidates of every shape of configurations 2-4,
              rejects any whose result is out of tolerance, and writes the table the
              library's SK_SCHED_AUTO consults (csrc/sk_tuned_table.inc format) to FILE.
--case        runs one entry point on one shape a few times and exits: the command line the
              ncu captures under profiles/ are taken from.
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
TOL16, TOL32 = 1e-2, 1e-4
PREHEAT = 10                   # untimed launches ahead of the warm-up steps (clock ramp of an idle GPU)
METRIC = "Stream-K fp16 GEMM TFLOP/s"


def headline_config(world: int) -> dict:
    """The `config` object, identical in both arms."""
    return {"workload": f"cfg5 fp16 NT GEMM M={M5} N={N5} K={K5}, N sharded {world}-way",
            "l2": "operands (>= 0.25 GB per GPU) exceed the 126 MB L2; no flush needed",
            "preheat": f"{PREHEAT} untimed launches ahead of the warm-up steps of every timed kernel"}


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


def cpu_time(fn, budget_s: float = 1.0, min_reps: int = 2) -> tuple[float, int]:
    """Seconds per call of a CPU function: one warm call, then repeats for about budget_s."""
    fn()
    t0 = time.perf_counter()
    fn()
    one = time.perf_counter() - t0
    reps = max(min_reps, min(200, int(budget_s / max(one, 1e-4))))
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    return (time.perf_counter() - t0) / reps, reps


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
    sample = (f"each step: a {CPU_SAMPLE_ROWS}-row slice of A (1/{M5 // CPU_SAMPLE_ROWS} of the problem) against "
              f"the full B; torch.matmul(A.float(), B.float().T) on host cores; the rate is reported")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": headline_config(max(args.gpus, 1)),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------- timing helpers
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


def time_rotating_eager(launch, n_copies: int, est_us: float, batches: int = 9):
    """The same figure for a callable that cannot be captured into a CUDA graph (a Triton kernel
    that allocates its result): plain launches, back to back, >= 1 ms per batch."""
    import torch
    n = min(max(n_copies, int(math.ceil(1000.0 / max(est_us, 1.0)))), 256)
    for i in range(3):
        launch(i % n_copies)
    torch.cuda.synchronize()
    times = []
    for _ in range(batches):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            launch(i % n_copies)
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / n)
    times.sort()
    return times[len(times) // 2], times[len(times) // 10], times[(len(times) * 9) // 10]


def roof_us(flops: float, nbytes: float, peaks: dict):
    t_nom = max(flops / (NOMINAL_TFLOPS * 1e12), nbytes / (NOMINAL_HBM_GBS * 1e9))
    tc, tm = flops / (peaks["bf16_tflops"] * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)
    return t_nom * 1e6, max(tc, tm) * 1e6, "tensor" if tc > tm else "hbm"


class ParityError(SystemExit):
    pass


def require(err: float, tol: float, what: str) -> float:
    if not (err <= tol):
        raise ParityError(f"bench.py: {what}: rel_err {err:.3e} exceeds {tol:g}; no number is reported for a wrong result")
    return err


# ------------------------------------------------------------------------- per-shape cases
class Fp16Case:
    """One fp16 NT shape: operands on the device (weights in L2-cold rotation), oracle result."""

    def __init__(self, cfg, case, dev, l2, shape=None):
        import torch
        import oracle
        self.c = c = oracle.make_case(cfg, case, shape=shape)
        self.cfg, self.M, self.N, self.K = cfg, c["M"], c["N"], c["K"]
        self.A = c["A"].to(dev)
        wbytes = 2 * self.N * self.K
        self.copies = min(int(math.ceil(2 * l2 / wbytes)) + 1, 40)
        self.Bs = [c["B"].to(dev).clone() for _ in range(self.copies)]
        self.out = torch.empty(self.M, self.N, dtype=torch.float16, device=dev)
        self.flops = 2.0 * self.M * self.N * self.K
        self.nbytes = 2.0 * (self.M * self.K + self.N * self.K + self.M * self.N)
        self.est = max(self.nbytes / 6.5e3, self.flops / 1.5e9) / 1e3 + 3
        self.ref = oracle.gemm_ref(c["A"], c["B"], "nt")

    def run(self, sk, **kw):
        return lambda i: sk.streamk_fp16_nt(self.A, self.Bs[i], out=self.out, **kw)

    def check(self, sk, fn, what):
        import oracle
        fn(0)
        sk.check_status()
        return require(oracle.rel_err(self.out, self.ref), TOL16, f"{what} {self.M}x{self.N}x{self.K}")

    def cublas(self):
        import torch
        return lambda i: torch.matmul(self.A, self.Bs[i].t(), out=self.out)

    def cpu_baseline(self):
        import torch
        Af, Bf = self.c["A"].float(), self.c["B"].float()
        sec, reps = cpu_time(lambda: torch.matmul(Af, Bf.t()))
        return {"us": sec * 1e6, "cores": torch.get_num_threads(), "reps": reps,
                "what": "torch.matmul(A.float(), B.float().T) on host cores"}


class Q4Case:
    """One W4A16 shape."""

    def __init__(self, case, dev, l2, shape=None):
        import torch
        import oracle
        import streamk_b200 as sk
        self.c = c = oracle.make_case(4, case, shape=shape)
        self.cfg, self.M, self.N, self.K = 4, c["M"], c["N"], c["K"]
        self.A = c["A"].to(dev)
        wbytes = self.N * self.K // 2
        self.copies = min(int(math.ceil(2 * l2 / wbytes)) + 1, 64)
        P0 = sk.q4_prepack(c["qweight"].to(dev), c["scales"].to(dev), c["zeros"].to(dev))
        self.Ps = [P0] + [sk.PackedQ4(P0.data.clone(), self.N, self.K) for _ in range(self.copies - 1)]
        self.out = torch.empty(self.M, self.N, dtype=torch.float16, device=dev)
        self.flops = 2.0 * self.M * self.N * self.K
        self.nbytes = 2.0 * self.M * self.K + self.N * self.K / 2 + 3.0 * self.N * self.K / 128 + 2.0 * self.M * self.N
        self.est = max(self.nbytes / 6.5e3, self.flops / 1.5e9) / 1e3 + 3
        self.ref = oracle.w4a16_ref(c["A"], c["q"], c["scales"], c["zeros"])
        W = sk.dequant_w4(P0)
        require(0.0 if torch.equal(W.cpu().view(torch.int16),
                                   oracle.dequant_ref(c["q"], c["scales"], c["zeros"]).view(torch.int16)) else 1.0,
                0.0, f"dequantisation (bitwise) {self.N}x{self.K}")
        self.Ws = [W.clone() for _ in range(min(self.copies, int(math.ceil(2 * l2 / (2 * self.N * self.K))) + 1))]

    def run(self, sk, **kw):
        return lambda i: sk.streamk_fp16_ladder_block_reduce_q4(self.A, self.Ps[i], out=self.out, **kw)

    def check(self, sk, fn, what):
        import oracle
        fn(0)
        sk.check_status()
        return require(oracle.rel_err(self.out, self.ref), TOL16, f"{what} {self.M}x{self.N}x{self.K}")

    def cublas(self):
        import torch
        return lambda i: torch.matmul(self.A, self.Ws[i % len(self.Ws)].t(), out=self.out)

    def cpu_baseline(self):
        """The reference's CPU path for q4: dequantise, then matmul (both timed, separately)."""
        import torch
        import oracle
        c = self.c
        dq, _ = cpu_time(lambda: oracle.dequant_ref(c["q"], c["scales"], c["zeros"]), budget_s=0.5, min_reps=1)
        Wf, Af = oracle.dequant_ref(c["q"], c["scales"], c["zeros"]).float(), c["A"].float()
        mm, reps = cpu_time(lambda: torch.matmul(Af, Wf.t()))
        return {"us": (dq + mm) * 1e6, "dequant_us": dq * 1e6, "matmul_us": mm * 1e6,
                "cores": torch.get_num_threads(), "reps": reps,
                "what": "(q.half() - z.half()) * s, then torch.matmul(A.float(), W.float().T), on host cores"}


def triton_column(case, ref_mod):
    """p50 microseconds of the reference's own Triton Stream-K kernel on the same operands
    (its `matmul(a, b)` takes B as [K, N] and returns a fresh fp32 C), checked against the oracle."""
    import torch
    Bnn = [b.t().contiguous() for b in case.Bs[:min(case.copies, 8)]]
    c = ref_mod.matmul(case.A, Bnn[0])
    torch.cuda.synchronize()
    err = float((c.cpu() - case.ref).abs().max() / case.ref.abs().max())
    require(err, TOL16, f"reference Triton kernel {case.M}x{case.N}x{case.K}")
    us = time_rotating_eager(lambda i: ref_mod.matmul(case.A, Bnn[i % len(Bnn)]), len(Bnn), case.est * 4)
    return us[0]


# ------------------------------------------------------------------------- sweeps
SUMMARY_FP16 = [(2, 0)] + [(3, i) for i in (0, 1, 4, 5, 16, 17, 20, 21)]     # cfg2; M in {1,16,128,256} x two (N,K)
SUMMARY_Q4 = [0, 5, 7]                                                        # 1x4096x4096, 16x4096x11008, 128x11008x4096
SUMMARY_TRITON = {(2, 0), (3, 20)}                                            # (a recompilation per shape: two shapes)


def sweep_summary(peaks: dict) -> dict:
    """A fixed subset of configurations 1-4 for the default run (about a minute)."""
    import torch
    import oracle
    import streamk_b200 as sk
    dev = torch.device("cuda", torch.cuda.current_device())
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    torch.set_num_threads(os.cpu_count() or 1)
    ref_mod = oracle.load_triton_ref()
    names = {v: k for k, v in sk.SCHEDULES.items()}
    rows = []

    # configuration 1: fp32 NN 256 x 256 x 1024 (FFMA kernel; CPU torch.matmul is oracle and baseline)
    c = oracle.make_case(1)
    A, B = c["A"].to(dev), c["B"].to(dev)
    out = torch.empty(256, 256, device=dev)
    fn = lambda i: sk.streamk_fp32(A, B, out=out)
    fn(0)
    sk.check_status()
    err = require(oracle.rel_err(out, oracle.gemm_ref(c["A"], c["B"], "nn")), TOL32, "cfg1 fp32")
    us = time_rotating(fn, 1, 10.0)
    cub = time_rotating(lambda i: torch.matmul(A, B, out=out), 1, 10.0)
    sec, reps = cpu_time(lambda: torch.matmul(c["A"], c["B"]), budget_s=0.5)
    flops, nbytes = 2.0 * 256 * 256 * 1024, 4.0 * (256 * 1024 * 2 + 256 * 256)
    rows.append({"cfg": 1, "entry": "streamk_fp32", "M": 256, "N": 256, "K": 1024, "p50_us": round(us[0], 2),
                 "cublas_us": round(cub[0], 2), "rel_err": float(f"{err:.2e}"),
                 "cpu_us": round(sec * 1e6, 1), "cpu_cores": torch.get_num_threads(),
                 "note": "L2-resident (1.3 MB); fp32 FFMA kernel, cuBLAS column is torch.matmul fp32 (no TF32)"})

    def one(case, entry, triton):
        fn = case.run(sk)
        err = case.check(sk, fn, entry)
        us = time_rotating(fn, case.copies, case.est)
        pdl = time_rotating(case.run(sk, pdl=True), case.copies, case.est)
        cub = time_rotating(case.cublas(), case.copies, case.est)
        _, t_meas, bound = roof_us(case.flops, case.nbytes, peaks)
        kind = "w4a16" if case.cfg == 4 else "f16"
        info = sk.schedule_info(case.M, case.N, case.K, kind=kind)
        cpu = case.cpu_baseline()
        r = {"cfg": case.cfg, "entry": entry, "M": case.M, "N": case.N, "K": case.K,
             "auto": f"{names[info['schedule']]}" + (f"/cluster{info['cluster']}" if info["cluster"] else "")
                     + f"/tile{info['tile_m']}x{info['tile_n']}",
             "p50_us": round(us[0], 2), "p50_us_pdl": round(pdl[0], 2), "cublas_us": round(cub[0], 2),
             "vs_cublas": round(cub[0] / us[0], 3), "bound": bound,
             "frac_of_measured_roof": round(t_meas / us[0], 3),
             "gbs": round(case.nbytes / us[0] / 1e3, 1), "tflops": round(case.flops / us[0] / 1e6, 2),
             "rel_err": float(f"{err:.2e}"), "cpu_us": round(cpu["us"], 1), "cpu_cores": cpu["cores"]}
        if "dequant_us" in cpu:
            r["cpu_dequant_us"] = round(cpu["dequant_us"], 1)
            r["cpu_matmul_us"] = round(cpu["matmul_us"], 1)
        if triton and ref_mod is not None:
            try:
                r["ref_triton_us"] = round(triton_column(case, ref_mod), 2)
            except ParityError:
                raise
            except Exception as e:      # the comparator is not the product: note and go on
                r["ref_triton_error"] = f"{type(e).__name__}: {e}"[:160]
        rows.append(r)

    for cfg, i in SUMMARY_FP16:
        one(Fp16Case(cfg, i, dev, l2), "streamk_fp16_nt", (cfg, i) in SUMMARY_TRITON)
    for i in SUMMARY_Q4:
        one(Q4Case(i, dev, l2), "streamk_fp16_ladder_block_reduce_q4", False)
    geo = [r["vs_cublas"] for r in rows if "vs_cublas" in r]
    return {"protocol": "L2-cold: weights rotate through ceil(2*L2/bytes)+1 copies; CUDA-graph replays of >= 1 ms "
                        "batches, p50 of 25; cuBLAS = torch.matmul on the same operands (cfg 4: on the dequantised "
                        "fp16 weights, 4x the bytes); cpu_us = the reference's CPU expression on this host",
            "reference_triton_kernel": "available" if ref_mod is not None else "oracle/_ref/triton_streamk.py absent",
            "geomean_vs_cublas": round(math.exp(sum(math.log(x) for x in geo) / len(geo)), 3),
            "rows": rows}


def run_sweep(path: str, peaks: dict) -> None:
    """Every shape of configurations 2-4, every schedule, beside cuBLAS (and, for M in {16, 256}
    and configuration 2, the reference's Triton kernel).  Results are checked, not just recorded."""
    import torch
    import oracle
    import streamk_b200 as sk
    dev = torch.device("cuda", torch.cuda.current_device())
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    ref_mod = oracle.load_triton_ref()
    names = {v: k for k, v in sk.SCHEDULES.items()}
    rows = []

    def record(cfg, name, M, N, K, variant, us, flops, nbytes, extra=None):
        t_nom, t_meas, bound = roof_us(flops, nbytes, peaks)
        r = {"cfg": cfg, "entry": name, "M": M, "N": N, "K": K, "variant": variant,
             "p50_us": round(us[0], 3), "p10_us": round(us[1], 3), "p90_us": round(us[2], 3),
             "tflops": round(flops / us[0] / 1e6, 2), "gbs": round(nbytes / us[0] / 1e3, 1),
             "bound": bound, "frac_of_nominal_roof": round(t_nom / us[0], 4),
             "frac_of_measured_roof": round(t_meas / us[0], 4)}
        if extra:
            r.update(extra)
        rows.append(r)
        print(json.dumps(r), file=sys.stderr, flush=True)

    def fp16_case(cfg, i):
        case = Fp16Case(cfg, i, dev, l2)
        M, N, K = case.M, case.N, case.K
        # tile None = the library's own choice (operands swapped for M <= 64, CTA pairs for
        # large problems); explicit 128 x 256 tiles are timed as well where they make sense
        variants = [("auto", "block_reduce", None), ("streamk", "atomic", None),
                    ("streamk", "block_reduce", None), ("hybrid", "block_reduce", None),
                    ("dp", "atomic", None)]
        if M > 64 and N * M >= 256 * 4096:
            variants += [("streamk", "block_reduce", 256), ("dp", "atomic", 256)]
        try:   # split-K inside clusters, where there are few enough tiles for it
            if sk.schedule_info(M, N, K, schedule="cluster")["cluster"] > 0:
                variants.append(("cluster", "block_reduce", None))
        except sk.StreamKError:
            pass
        variants.append(("auto+pdl", "block_reduce", None))
        for schedule, fixup, tile_n in variants:
            pdl = schedule.endswith("+pdl")
            schedule = schedule.split("+")[0]
            fn = case.run(sk, schedule=schedule, fixup=fixup, tile_n=tile_n, pdl=pdl)
            err = case.check(sk, fn, f"{schedule}/{fixup}")
            us = time_rotating(fn, case.copies, case.est)
            info = sk.schedule_info(M, N, K, schedule=schedule, tile_n=tile_n)
            how = f"cluster of {info['cluster']}" if info["cluster"] else fixup
            label = schedule if schedule != "auto" else f"auto={names[info['schedule']]}"
            if pdl:
                label = "pdl " + label
            record(cfg, "streamk_fp16_nt", M, N, K, f"{label}/{how}/tile{info['tile_m']}x{info['tile_n']}", us,
                   case.flops, case.nbytes, {"rel_err": float(f"{err:.3e}")})
        record(cfg, "cublas torch.matmul", M, N, K, "data-parallel library GEMM",
               time_rotating(case.cublas(), case.copies, case.est), case.flops, case.nbytes)
        if ref_mod is not None and (cfg == 2 or M in (16, 256)):
            try:
                t = triton_column(case, ref_mod)
                record(cfg, "reference triton_impl.matmul", M, N, K, "the reference's own Triton Stream-K kernel "
                       "(256x256x32 tiles, fp32 result, zero-filled C included)", (t, t, t), case.flops, case.nbytes)
            except ParityError:
                raise
            except Exception as e:
                print(f"reference Triton kernel failed on {M}x{N}x{K}: {e}", file=sys.stderr)

    def q4_case(i):
        case = Q4Case(i, dev, l2)
        for schedule, fixup in (("auto", "block_reduce"), ("streamk", "block_reduce"),
                                ("hybrid", "block_reduce"), ("streamk", "atomic"), ("dp", "block_reduce"),
                                ("auto+pdl", "block_reduce")):
            pdl = schedule.endswith("+pdl")
            schedule = schedule.split("+")[0]
            fn = case.run(sk, schedule=schedule, fixup=fixup, pdl=pdl)
            err = case.check(sk, fn, f"w4a16 {schedule}/{fixup}")
            us = time_rotating(fn, case.copies, case.est)
            info = sk.schedule_info(case.M, case.N, case.K, kind="w4a16", schedule=schedule)
            how = f"cluster of {info['cluster']}" if info["cluster"] else fixup
            label = schedule if schedule != "auto" else f"auto={names[info['schedule']]}"
            record(4, "streamk_fp16_ladder_block_reduce_q4", case.M, case.N, case.K,
                   f"{'pdl ' if pdl else ''}{label}/{how}/tile{info['tile_m']}x{info['tile_n']}", us,
                   case.flops, case.nbytes, {"rel_err": float(f"{err:.3e}")})
        record(4, "cublas on dequantised fp16 W", case.M, case.N, case.K, "library GEMM, 4x the weight bytes",
               time_rotating(case.cublas(), len(case.Ws), case.est), case.flops, case.nbytes)

    fp16_case(2, 0)
    for i in range(len(oracle.CONFIGS[3]["shapes"])):
        fp16_case(3, i)
    for i in range(len(oracle.CONFIGS[4]["shapes"])):
        q4_case(i)
    json.dump({"peaks": peaks, "protocol": "L2-cold: weights rotate through ceil(2*L2/bytes)+1 copies; "
               "CUDA events around CUDA-graph replays of >= 1 ms batches; p50 over 25 replays; every timed "
               "variant's result checked against the CPU oracle (rel_err <= 1e-2) before it is timed", "rows": rows},
              open(path, "w"), indent=1)


def run_tune(path: str, peaks: dict) -> None:
    """Offline tuner (the counterpart of the reference's autotune/streamk_fp16_autotune.py:36-94,
    which sweeps tile / stage configurations per shape but skips the result check, :93-94).
    For every shape of configurations 2-4: time the library's candidates, drop any whose result
    is out of tolerance, and emit one table row where a candidate beats the built-in rules by
    more than 3 %.  The output is the body of csrc/sk_tuned_table.inc."""
    import torch
    import oracle
    import streamk_b200 as sk
    dev = torch.device("cuda", torch.cuda.current_device())
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    entries, report = [], []

    def candidates_f16(M, N, K):
        c = [dict(schedule="streamk"), dict(schedule="hybrid"), dict(schedule="dp")]
        if M <= 4:
            c.append(dict(schedule="gemv"))
        if M <= 64:
            tm = (M + 15) // 16 * 16
            for tn in (64, 80, 96, 112, 128):
                c.append(dict(schedule="dp", tile_m=tm, tile_n=tn))
            c.append(dict(schedule="streamk", tile_m=tm, tile_n=128))
        else:
            for tn in (64, 96, 128, 160, 192, 256):
                c.append(dict(schedule="dp", tile_m=128, tile_n=tn))
                c.append(dict(schedule="streamk", tile_m=128, tile_n=tn))
            if M > 128:
                for tn in (96, 128, 160, 192, 256):
                    c.append(dict(schedule="dp", tile_m=256, tile_n=tn))
                    c.append(dict(schedule="streamk", tile_m=256, tile_n=tn))
        try:
            if sk.schedule_info(M, N, K, schedule="cluster", no_table=True)["cluster"] > 0:
                c.append(dict(schedule="cluster"))
                if M > 64:
                    for tn in (64, 96, 128, 192):
                        c.append(dict(schedule="cluster", tile_m=128, tile_n=tn))
        except sk.StreamKError:
            pass
        return c

    def candidates_q4(M, N, K):
        c = [dict(schedule="streamk"), dict(schedule="hybrid"), dict(schedule="dp"),
             dict(schedule="streamk", fixup="atomic")]
        if M <= 16:
            c.append(dict(schedule="gemv"))
        # narrower tiles along M: more tiles (more CTAs streaming, cluster split-K within reach) for
        # the price of dequantising every weight once per tile column
        widths = sorted({w for w in (16, 32, 48, 64, 96, 112) if w < ((M + 15) // 16 * 16) and M > 16})
        for tm in [None] + widths:
            for sched in ("streamk", "dp", "cluster"):
                kw = dict(schedule=sched) if tm is None else dict(schedule=sched, tile_m=tm)
                if kw in c:
                    continue
                try:
                    info = sk.schedule_info(M, N, K, kind="w4a16", no_table=True, **kw)
                except sk.StreamKError:
                    continue
                if sched == "cluster" and info["cluster"] == 0:
                    continue
                if sched == "dp" and info["total_tiles"] > 2 * sms:
                    continue
                c.append(kw)
        return c

    def tune(case, kind, cands):
        base_fn = case.run(sk, no_table=True)
        case.check(sk, base_fn, "rules")
        base = time_rotating(base_fn, case.copies, case.est, batches=15)[0]
        best, best_us, rejected = None, base, 0
        for kw in cands:
            try:
                fn = case.run(sk, no_table=True, **kw)
                fn(0)
                sk.check_status()
            except sk.StreamKError:
                try:
                    sk.reset_workspace()
                except sk.StreamKError:
                    pass
                continue
            if oracle.rel_err(case.out, case.ref) > TOL16:      # the check the reference's tuner skips
                rejected += 1
                continue
            us = time_rotating(fn, case.copies, case.est, batches=15)[0]
            if us < best_us:
                best, best_us = kw, us
        row = {"kind": kind, "M": case.M, "N": case.N, "K": case.K, "rules_us": round(base, 2),
               "best_us": round(best_us, 2), "best": best, "rejected": rejected}
        report.append(row)
        print(json.dumps(row), file=sys.stderr, flush=True)
        if best is not None and best_us < 0.97 * base and best.get("fixup") is None:
            entries.append((1 if kind == "f16" else 2, case.M, case.N, case.K, sms, sk.SCHEDULES[best["schedule"]],
                            int(best.get("tile_m") or 0), int(best.get("tile_n") or 0)))

    tune(Fp16Case(2, 0, dev, l2), "f16", candidates_f16(384, 384, 8192))
    for i, (M, N, K) in enumerate(oracle.CONFIGS[3]["shapes"]):
        tune(Fp16Case(3, i, dev, l2), "f16", candidates_f16(M, N, K))
    for i, (M, N, K) in enumerate(oracle.CONFIGS[4]["shapes"]):
        tune(Q4Case(i, dev, l2), "w4a16", candidates_q4(M, N, K))
    with open(path, "w") as f:
        f.write("// Written by `python bench.py --tune FILE` on a %d-SM device: shapes where a timed,\n"
                "// result-checked candidate beat the built-in rules of sk_resolve_auto by more than 3 %%.\n"
                "// {kernel kind, M, N, K, SMs, schedule, tile_m, tile_n}\n" % sms)
        for e in entries:
            f.write("{%d, %d, %d, %d, %d, %d, %d, %d},\n" % e)
    json.dump(report, open(path + ".json", "w"), indent=1)


# ------------------------------------------------------------------------- one case (profiling driver)
def run_case(a) -> None:
    import ctypes as C
    import torch
    import streamk_b200 as sk
    kind = a.case[0]
    M, N, K = (int(x) for x in a.case[1:4])
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    kw = dict(schedule=a.schedule, fixup=a.fixup, tile_m=a.tile_m, tile_n=a.tile_n, group_m=a.group_m)
    if kind == "f32":
        A = torch.rand(M, K, generator=g, device=dev) * 2 - 1
        B = torch.rand(K, N, generator=g, device=dev) * 2 - 1
        for k in ("tile_m", "tile_n", "group_m"):
            kw.pop(k)
        fn = lambda: sk.streamk_fp32(A, B, **kw)
        ref = lambda: torch.matmul(A, B)
    elif kind in ("f16", "w4a16"):
        A = torch.randn(M, K, generator=g, device=dev).half()
        W = (0.02 * torch.randn(N, K, generator=g, device=dev)).half()
        out = torch.empty(M, N, dtype=torch.float16, device=dev)
        ref = lambda: torch.matmul(A, W.t(), out=out)
        if kind == "f16" and a.peers > 0:
            # the fused all-gather kernel with P further matrices of the same GPU standing in for
            # the peer GPUs' (what a one-GPU capture can show: the kernel's own cost of issuing P
            # extra copies of every store); plain C-ABI calls with a workspace of its own
            from streamk_b200 import _lib as L
            lib = L.load()
            mats = [torch.empty(M, N, dtype=torch.float16, device=dev) for _ in range(a.peers)]
            ptrs = (C.c_void_p * a.peers)(*[m.data_ptr() for m in mats])
            prob = L.SkProblem(M=M, N=N, K=K, lda=K, ldb=K, ldc=N, layout=L.LAYOUTS["nt"],
                               schedule=L.SCHEDULES[a.schedule], fixup=L.FIXUPS[a.fixup],
                               tile_m=a.tile_m or 0, tile_n=a.tile_n or 0, group_m=a.group_m or 0)
            nbytes = int(lib.sk_workspace_bytes(torch.cuda.get_device_properties(0).multi_processor_count))
            ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            stream = torch.cuda.current_stream().cuda_stream
            L.check(lib.sk_workspace_init(ws.data_ptr(), nbytes, stream), "sk_workspace_init")

            def fn():
                L.check(lib.sk_gemm_f16_gather(C.byref(prob), A.data_ptr(), W.data_ptr(), out.data_ptr(), ptrs,
                                               a.peers, ws.data_ptr(), nbytes, stream), "sk_gemm_f16_gather")
        elif kind == "f16":
            fn = lambda: sk.streamk_fp16_nt(A, W, out=out, **kw)
        else:
            q = torch.randint(0, 16, (N, K // 8, 8), generator=g, device=dev, dtype=torch.int64)
            word = sum(q[:, :, j] << (4 * j) for j in range(8))
            word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
            z = torch.randint(0, 16, (N, K // 128), generator=g, device=dev, dtype=torch.uint8)
            s = (0.002 + 0.018 * torch.rand(N, K // 128, generator=g, device=dev)).half()
            P = sk.q4_prepack(word, s, z)
            kw.pop("group_m")
            fn = lambda: sk.streamk_fp16_ladder_block_reduce_q4(A, P, out=out, **kw)
    else:
        raise SystemExit("--case KIND must be f16, w4a16 or f32")
    for _ in range(a.iters):
        fn()
    torch.cuda.synchronize()
    if a.timeline:
        case_timeline(a, kind, M, N, K, kw, dev)
    if a.time:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        e1.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / a.iters
        print(json.dumps({"case": a.case, "schedule": a.schedule, "tile_m": a.tile_m, "tile_n": a.tile_n,
                          "group_m": a.group_m, "us_per_launch": round(us, 2),
                          "tflops": round(2.0 * M * N * K / us / 1e6, 1)}))
    if a.cublas:
        for _ in range(a.iters):
            ref()
    torch.cuda.synchronize()
    sk.check_status()
    print("done")


def case_timeline(a, kind, M, N, K, kw, dev) -> None:
    """--case ... --timeline: per-CTA %globaltimer stamps of ONE launch in the middle of a
    back-to-back sequence on rotating weight copies (the state the timed runs see; no cache flush:
    a memset before the launch leaves the L2 full of dirty lines whose write-back slows the
    kernel under test).  Needs the trace build of the library: run with STREAMK_B200_TRACE=1
    (`STREAMK_B200_TRACE=1 python stream-k.tvm_b200/build.py` builds it)."""
    import torch
    import streamk_b200 as sk
    from streamk_b200 import _lib as L
    if os.environ.get("STREAMK_B200_TRACE") != "1":
        raise SystemExit("--timeline needs STREAMK_B200_TRACE=1 (the trace build of the library)")
    if kind not in ("f16", "w4a16"):
        raise SystemExit("--timeline: KIND f16 or w4a16")
    lib = L.load()
    l2 = torch.cuda.get_device_properties(0).L2_cache_size
    g = torch.Generator(device=dev).manual_seed(1)
    A = torch.randn(M, K, generator=g, device=dev).half()
    out = torch.empty(M, N, dtype=torch.float16, device=dev)
    wbytes = 2 * N * K if kind == "f16" else N * K // 2
    copies = min(max(3, 2 * l2 // wbytes + 2), 40)
    if kind == "f16":
        Ws = [(0.02 * torch.randn(N, K, generator=g, device=dev)).half() for _ in range(copies)]
        fn = lambda i: sk.streamk_fp16_nt(A, Ws[i % copies], out=out, **kw)
    else:
        def packed():
            q = torch.randint(0, 16, (N, K // 8, 8), generator=g, device=dev, dtype=torch.int64)
            word = sum(q[:, :, j] << (4 * j) for j in range(8))
            word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
            z = torch.randint(0, 16, (N, K // 128), generator=g, device=dev, dtype=torch.uint8)
            s = (0.002 + 0.018 * torch.rand(N, K // 128, generator=g, device=dev)).half()
            return sk.q4_prepack(word, s, z)
        Ps = [packed() for _ in range(copies)]
        kw = {k: v for k, v in kw.items() if k != "group_m"}
        fn = lambda i: sk.streamk_fp16_ladder_block_reduce_q4(A, Ps[i % copies], out=out, **kw)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    buf = torch.zeros(2 * sms * 16, dtype=torch.int64, device=dev)
    names = {0: "entry", 1: "barriers up", 2: "first load issued", 3: "first MMA", 4: "last MMA",
             6: "epilogue done", 7: "exit"}
    for rep in range(3):
        for i in range(2 * copies):
            fn(i)
        buf.zero_()
        for i in range(copies):
            fn(i)
        L.check(lib.sk_debug_set_trace(buf.data_ptr()), "sk_debug_set_trace")
        fn(0)
        lib.sk_debug_set_trace(None)
        fn(1)
        torch.cuda.synchronize()
        t = buf.view(-1, 16).cpu().double()
        t = t[t[:, 0] > 0]
        if len(t) == 0:
            raise SystemExit("no stamps: is this the trace build?")
        t0 = float(t[:, 0].min())
        row = {"ctas": int(len(t))}
        for slot, name in names.items():
            x = t[:, slot]
            x = x[x > 1e15]            # (globaltimer values; other slots may hold cycle counts)
            if len(x):
                row[name] = [round((float(x.median()) - t0) / 1e3, 2), round((float(x.max()) - t0) / 1e3, 2)]
        print(json.dumps({"case": a.case, "schedule": a.schedule, "timeline_us_median_max": row}))


# ------------------------------------------------------------------------- main arm
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sweep", default=None, help="also time every shape of configs 2-4 and write the table here")
    ap.add_argument("--tune", default=None, help="time the tile/schedule candidates of configs 2-4, write the table here")
    ap.add_argument("--no-summary", action="store_true", help="skip sustained loop and sweep summary")
    ap.add_argument("--schedule", default=os.environ.get("SK_BENCH_SCHEDULE", "auto"))
    ap.add_argument("--fixup", default=os.environ.get("SK_BENCH_FIXUP", "block_reduce"))
    ap.add_argument("--case", nargs=4, default=None, metavar=("KIND", "M", "N", "K"))
    ap.add_argument("--tile-m", type=int, default=None)
    ap.add_argument("--tile-n", type=int, default=None)
    ap.add_argument("--group-m", type=int, default=None)
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--cublas", action="store_true", help="--case: also run torch.matmul on the same operands")
    ap.add_argument("--time", action="store_true", help="--case: print the time per launch of a second batch")
    ap.add_argument("--peers", type=int, default=0)
    ap.add_argument("--timeline", action="store_true",
                    help="--case: per-CTA timestamps of one launch in a replayed sequence (trace build)")
    args = ap.parse_args()
    if args.case:
        run_case(args)
        return
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

    def timed(fn, n):
        """ms for n back-to-back calls, max over ranks, bracketed by barrier + synchronize."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)), e0.elapsed_time(e1)

    n_slab = N5 // world
    A, B = make_operands(rank, world, dev)
    C = torch.empty(M5, n_slab, dtype=torch.float16, device=dev)
    step = lambda: sk.streamk_fp16_nt(A, B, out=C, schedule=args.schedule, fixup=args.fixup)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    info = sk.schedule_info(M5, n_slab, K5, kind="f16", schedule=args.schedule, num_sms=sms)
    flops_total = 2.0 * M5 * N5 * K5

    # ---- device-resident timing (the headline) ----------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # An idle GPU takes tens of milliseconds of load to reach its working clocks; whichever kernel
    # is timed first on a fresh box would otherwise pay for the ramp (the first launches of a
    # 20-step region ran 5 % slower than its median).  PREHEAT untimed launches come before the W
    # warm-up steps of each timed kernel, ours and cuBLAS alike.
    for _ in range(PREHEAT):
        step()
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
    value = flops_total * args.steps / (total_ms * 1e-3) / 1e12

    # spot check of the timed output against an fp32 product of the same operands
    rows = torch.arange(0, M5, M5 // 16, device=dev)[:16]
    ref = A[rows].float() @ B.float().t()
    check = float((C[rows].float() - ref).abs().max() / ref.abs().max())
    require(check, TOL16, "configuration 5, timed output")

    # per-launch latency: one event pair per launch
    lat = []
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(min(max(args.steps, 10), 50))]
    barrier()
    for a, b in evs:
        a.record(); step(); b.record()
    torch.cuda.synchronize()
    lat = sorted(a.elapsed_time(b) * 1e3 for a, b in evs)
    p50_us = max_over_ranks(lat[len(lat) // 2])

    # cuBLAS fp16 on the same operands, for context (library data-parallel GEMM)
    cub = lambda: torch.matmul(A, B.t(), out=C)
    for _ in range(PREHEAT + args.warmup):
        cub()
    cublas_ms, _ = timed(cub, args.steps)
    cublas_tflops = flops_total * args.steps / (cublas_ms * 1e-3) / 1e12
    step()

    # ---- the same kernel in the sustained (power-capped) regime -------------------
    sustained = None
    if not args.no_summary:
        def loop(fn, seconds):
            n, t0 = 0, time.time()
            while time.time() - t0 < seconds:
                for _ in range(10):
                    fn()
                torch.cuda.synchronize()
                n += 10
            return n
        sustained = {}
        for name, fn in (("ours", step), ("cublas", cub)):
            loop(fn, 1.0)                                   # pre-heat
            smp = ClockSampler(local_rank)
            if rank == 0:
                smp.start()
            barrier()
            w0 = time.time()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            n = loop(fn, 2.0)
            s1.record()
            torch.cuda.synchronize()
            w1 = time.time()
            ms = max_over_ranks(s0.elapsed_time(s1) / n) * n
            ck = smp.stop(w0, w1) if rank == 0 else None
            tf = flops_total * n / (ms * 1e-3) / 1e12
            sustained[name] = {"tflops": tf, "launches": n, "seconds": ms * 1e-3}
            if ck and ck.get("sm_mhz"):
                sustained[name].update({"sm_mhz": ck["sm_mhz"], "reasons": ck["reasons"], "power_w_max": ck.get("power_w_max"),
                                        "tflops_at_max_clock": tf * ck["sm_max_mhz"] / ck["sm_mhz"]})
        sustained["frac_of_measured_sustained_peak"] = sustained["ours"]["tflops"] / world / peaks["bf16_tflops_sustained"]
        sustained["vs_cublas"] = sustained["ours"]["tflops"] / sustained["cublas"]["tflops"]

    # ---- end to end: host buffers in, host result out ---------------------------
    # Every rank holds its column block of B and C in pinned host memory and 1/N of A's rows;
    # the library copies its part of A in and all-gathers the parts over NVLink (NCCL), so A
    # crosses PCIe once for the whole job whatever N is.
    e2e_steps = max(1, min(args.steps, 5))
    rows_part = M5 // world
    A_h = torch.empty(rows_part, K5, dtype=A.dtype).pin_memory(); A_h.copy_(A[rank * rows_part:(rank + 1) * rows_part])
    B_h = torch.empty(B.shape, dtype=B.dtype).pin_memory(); B_h.copy_(B)
    C_h = torch.empty(C.shape, dtype=C.dtype).pin_memory()
    e2e_slabs = max(2, 8 // world)
    group = dist.group.WORLD if world > 1 else None

    def e2e_step():
        sk.streamk_fp16_nt_host(A_h, B_h, C_h, slabs=e2e_slabs, schedule=args.schedule, fixup=args.fixup,
                                group=group)

    e2e_step()
    e2e_ms, _ = timed(e2e_step, e2e_steps)
    e2e_value = flops_total * e2e_steps / (e2e_ms * 1e-3) / 1e12
    torch.cuda.synchronize()
    e2e_check = float((C_h[rows.cpu()].float().to(dev) - ref).abs().max() / ref.abs().max())
    require(e2e_check, TOL16, "configuration 5, end-to-end output")
    h2d = (A_h.numel() + B_h.numel()) * 2 * world
    d2h = C_h.numel() * 2 * world
    del A_h, B_h, C_h
    sk.release_cached_memory()

    # ---- the product INCLUDING the all-gather of C, both ways (N > 1) --------------
    with_gather = None
    if world > 1:
        with_gather = {}
        parts = torch.empty(world, M5, n_slab, dtype=torch.float16, device=dev)

        def nccl_step():
            step()
            dist.all_gather_into_tensor(parts, C)
        for _ in range(2):
            nccl_step()
        nccl_ms = timed(nccl_step, 5)[0] / 5
        with_gather["gemm_ms"] = total_ms / args.steps
        with_gather["nccl_ms"] = nccl_ms
        res, err = None, ""
        try:
            res = sk.GatheredResult(M5, N5)   # (raises on every rank or on none)
        except Exception as e:
            err = f"{type(e).__name__}: {e}"
        if res is not None:
            failure = ""
            try:
                fused_step = lambda: sk.streamk_fp16_nt_gather(A, B, res, schedule=args.schedule, fixup=args.fixup)
                for _ in range(2):
                    fused_step()
                fused_ms = timed(fused_step, 5)[0] / 5
                sk.check_status()
                # Like for like: the fused call may tile differently from the plain one (a link-bound
                # gather runs data-parallel 256 x 256 tiles); the NCCL-gathered comparison product is
                # computed with the tiling the fused call used, so that "bitwise equal" says
                # something about the push path itself.
                fi = sk.schedule_info(M5, n_slab, K5, kind="f16", schedule=args.schedule, num_sms=sms,
                                      gather_peers=world - 1)
                like = sk.streamk_fp16_nt(A, B, schedule=sk.SCHEDULE_NAMES[fi["schedule"]], fixup=args.fixup,
                                          tile_m=256 if fi["tile_m"] == 256 and fi["wide_units"] == 0 else None)
                parts_like = torch.empty_like(parts)
                dist.all_gather_into_tensor(parts_like, like)
                same = all(torch.equal(res.full[:, r * n_slab:(r + 1) * n_slab], parts_like[r]) for r in range(world))
                worst = max(float((res.full[:, r * n_slab:(r + 1) * n_slab].float() - parts[r].float()).abs().max())
                            for r in range(world))
                scale_l = float(parts.float().abs().max())
            except Exception as e:       # agreed below: nobody is left alone in a collective
                failure = f"{type(e).__name__}: {e}"
                same, worst, scale_l, fused_ms = False, float("inf"), 1.0, float("nan")
            ok_all = res.all_agree(not failure)
            agree = torch.tensor([1.0 if same else 0.0, -worst], device=dev)
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            scale = torch.tensor([scale_l], device=dev)
            dist.all_reduce(scale, op=dist.ReduceOp.MAX)
            res.close()
            if ok_all:
                with_gather.update({"fused_ms": fused_ms,
                                    "fused_bitwise_equal_to_nccl_gather_of_like_tiled_product": bool(agree[0].item() == 1.0),
                                    "fused_max_rel_diff_to_nccl_gather_of_default_product": float(-agree[1].item()) / float(scale.item()),
                                    "fused_tiling": f"{sk.SCHEDULE_NAMES[fi['schedule']]}, tile {fi['tile_m']}x{fi['tile_n']}, "
                                                    f"256x512 units: {fi['wide_units']}",
                                    "bytes_pushed_per_gpu": M5 * n_slab * 2 * (world - 1)})
            else:
                with_gather["fused_error"] = failure or "another rank failed"
        else:
            with_gather["fused_error"] = err
        # one GPU of this box on the whole problem, for the collective-inclusive efficiency
        Bfull = torch.cat([make_operands(r, world, dev)[1] for r in range(world)], 0) if rank == 0 else None
        single_ms = None
        if rank == 0:
            Cfull = torch.empty(M5, N5, dtype=torch.float16, device=dev)
            one = lambda: sk.streamk_fp16_nt(A, Bfull, out=Cfull, schedule=args.schedule, fixup=args.fixup)
            for _ in range(3):
                one()
            torch.cuda.synchronize()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(5):
                one()
            s1.record()
            s1.synchronize()
            single_ms = s0.elapsed_time(s1) / 5
            del Bfull, Cfull
        barrier()
        if rank == 0:
            with_gather["one_gpu_whole_problem_ms"] = single_ms
            with_gather["efficiency_gemm_only"] = single_ms / (world * with_gather["gemm_ms"])
            with_gather["efficiency_nccl"] = single_ms / (world * nccl_ms)
            if "fused_ms" in with_gather:
                with_gather["efficiency_fused"] = single_ms / (world * with_gather["fused_ms"])
                with_gather["tflops_fused"] = flops_total / (with_gather["fused_ms"] * 1e-3) / 1e12
            with_gather["tflops_nccl"] = flops_total / (nccl_ms * 1e-3) / 1e12

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
    alg_bytes = 2.0 * (M5 * K5 + n_slab * K5 + M5 * n_slab)
    traffic, traffic_note = None, None
    tpath = os.path.join(ROOT, "profiles", "sk_gemm_f16_2cta_kernel_dram_traffic.json")
    if os.path.exists(tpath):
        t = json.load(open(tpath))
        traffic = t["dram_bytes_over_algorithmic_bytes"] * alg_bytes
        traffic_note = t["note"]
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks[peak_key], "unit": "TFLOP/s",
                "frac": achieved / peaks[peak_key], "traffic": traffic, "traffic_note": traffic_note,
                "algorithmic_bytes": alg_bytes,
                "peak_source": f"{peaks['source']} {peak_key}",
                "frac_of_burst_peak": achieved / peaks["bf16_tflops"],
                "frac_of_nominal_2250": achieved / NOMINAL_TFLOPS,
                "kernel": "sk_gemm_f16_2cta_kernel (CTA pairs; 256x256x64 tiles, data-parallel part in 256x512 units)"}

    cpu_baseline = None
    if world == 1:
        torch.set_num_threads(os.cpu_count() or 1)
        Af, Bf = A[:CPU_SAMPLE_ROWS].cpu().float(), B.cpu().float()
        sec, reps = cpu_time(lambda: torch.matmul(Af, Bf.t()), budget_s=10.0, min_reps=3)
        cpu_baseline = {"value": 2.0 * CPU_SAMPLE_ROWS * N5 * K5 / sec / 1e12, "unit": "TFLOP/s",
                        "cores": torch.get_num_threads(), "kind": "port",
                        "sample": f"{CPU_SAMPLE_ROWS}-row slice of A against the full B, "
                                  f"torch.matmul(A.float(), B.float().T), {sec:.3f} s per product, "
                                  f"{reps} repeats (about 10 s)"}
        del Af, Bf

    out = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": headline_config(world),
        "plan": {"schedule": sk.SCHEDULE_NAMES[info["schedule"]] + (" (auto)" if args.schedule == "auto" else ""),
                 "fixup": args.fixup, "tile": [info["tile_m"], info["tile_n"], 64], "grid": info["grid"],
                 "sk_tiles": info["sk_tiles"], "dp_tiles": info["dp_tiles"], "dp_units_256x512": info["wide_units"],
                 "group_m": info["group_m"]},
        "per_gpu_tflops": value / world, "p50_us": p50_us,
        "roofline": roofline, "cpu_baseline": cpu_baseline,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "call": f"streamk_fp16_nt_host, {e2e_slabs} column slabs per GPU"
                        + (f", A copied in {world} row parts and all-gathered over NVLink" if world > 1 else ""),
                "check_rel_err": e2e_check},
        "gpu_launches": args.steps, "clocks": clocks, "check_rel_err": check,
        "cublas_fp16_tflops_same_operands": cublas_tflops,
    }
    if sustained is not None:
        out["sustained"] = sustained
    if with_gather is not None:
        out["with_gather"] = with_gather
    if world == 1 and not args.no_summary:
        out["sweep_summary"] = sweep_summary(peaks)
    if args.sweep and world == 1:
        run_sweep(args.sweep, peaks)
        out["sweep_file"] = args.sweep
    if args.tune and world == 1:
        run_tune(args.tune, peaks)
        out["tune_file"] = args.tune
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
