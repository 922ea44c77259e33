"""The library's host scheduler (C, sk_schedule) against the CPU oracle."""
import ctypes as C
import random

import pytest

import oracle


def _sched(lib, M, N, K, kind, schedule, P, tile_n=0, group_m=0):
    from streamk_b200 import _lib as L
    prob = L.SkProblem(M=M, N=N, K=K, lda=K, ldb=K, ldc=N, layout=1, schedule=L.SCHEDULES[schedule],
                       fixup=0, tile_n=tile_n, num_sms=0, group_m=group_m, fixup_timeout_us=0)
    info = L.SkScheduleInfo()
    st = lib.sk_schedule(C.byref(prob), kind, P, C.byref(info))
    assert st == 0, st
    return info.as_dict(), info


def test_hybrid_equals_reference_formula(lib):
    rnd = random.Random(0)
    for _ in range(300):
        M, N, K = rnd.randint(1, 9000), rnd.randint(1, 30000), rnd.randint(1, 12000)
        P = rnd.choice([1, 2, 3, 5, 108, 132, 148])
        tn = rnd.choice([128, 256])
        d, _ = _sched(lib, M, N, K, 1, "hybrid", P, tile_n=tn)
        r = oracle.reference_schedule(M, N, K, 128, tn, 64, P)
        assert d["total_tiles"] == r["total_tiles"]
        assert d["iters_per_tile"] == r["iters_per_tile"]
        assert d["sk_tiles"] == r["streamk_tiles"]
        assert d["dp_tiles"] == r["blocking_tiles"]
        if d["grid"] == P:   # the library shrinks the grid when there is less work than CTAs
            assert d["sk_iters_per_cta"] == r["streamk_full_tiles"]
            assert d["sk_iters_rem"] == r["streamk_partial_tiles"]
        else:
            assert r["streamk_iters"] < P and d["grid"] == max(r["streamk_iters"], 1)


def test_worked_values_for_148_sms(lib):
    # shape -> (tiles, iters/tile, SK tiles, DP tiles, f, r) for 128x128x64 tiles on 148 SMs
    table = {
        (384, 384, 8192, 128): (9, 128, 9, 0, 7, 116),
        (128, 4096, 4096, 128): (32, 64, 32, 0, 13, 124),
        (128, 11008, 4096, 128): (86, 64, 86, 0, 37, 28),
        (128, 4096, 11008, 128): (32, 172, 32, 0, 37, 28),
        (128, 12288, 4096, 128): (96, 64, 96, 0, 41, 76),
        (256, 11008, 4096, 128): (172, 64, 24, 148, 10, 56),
        (256, 12288, 4096, 128): (192, 64, 44, 148, 19, 4),
        (8192, 28672, 8192, 256): (7168, 128, 212, 6956, 183, 52),
        (8192, 3584, 8192, 256): (896, 128, 156, 740, 134, 136),
    }
    for (M, N, K, tn), want in table.items():
        d, _ = _sched(lib, M, N, K, 1, "hybrid", 148, tile_n=tn)
        got = (d["total_tiles"], d["iters_per_tile"], d["sk_tiles"], d["dp_tiles"],
               d["sk_iters_per_cta"], d["sk_iters_rem"])
        assert got == want, (M, N, K, got, want)


@pytest.mark.parametrize("schedule", ["streamk", "hybrid", "hybrid_dp_first", "dp"])
def test_every_iteration_covered_exactly_once(lib, schedule):
    rnd = random.Random(hash(schedule) & 0xFFFF)
    for _ in range(60):
        kind = rnd.choice([0, 1])
        M, N, K = rnd.randint(1, 900), rnd.randint(1, 2500), rnd.randint(1, 1500)
        P = rnd.choice([1, 2, 3, 5, 7, 108, 132, 148])
        d, info = _sched(lib, M, N, K, kind, schedule, P, tile_n=rnd.choice([0, 128, 256]) if kind else 0)
        assert 1 <= d["grid"] <= P
        cov = oracle.coverage(d)
        assert len(cov) == d["total_tiles"] * d["iters_per_tile"], (M, N, K, P, d)
        assert set(cov.values()) == {1}
        # interval endpoints agree with the reference formula p*f + min(p, r)
        b, e = C.c_int64(), C.c_int64()
        for p in (0, d["grid"] // 2, d["grid"] - 1):
            assert lib.sk_cta_interval(C.byref(info), p, C.byref(b), C.byref(e)) == 0
            f, r = d["sk_iters_per_cta"], d["sk_iters_rem"]
            assert b.value == p * f + min(p, r) and e.value == (p + 1) * f + min(p + 1, r)


def test_tile_rasterisation_is_a_bijection(lib):
    rnd = random.Random(7)
    for _ in range(40):
        M, N = rnd.randint(1, 3000), rnd.randint(1, 3000)
        gm = rnd.choice([0, 1, 2, 3, 8, 16])
        d, info = _sched(lib, M, N, 512, 1, "hybrid", 148, tile_n=128, group_m=gm)
        seen = set()
        tm, tn = C.c_int(), C.c_int()
        for t in range(d["total_tiles"]):
            assert lib.sk_tile_coords(C.byref(info), t, C.byref(tm), C.byref(tn)) == 0
            assert (tm.value, tn.value) == oracle.tile_coords(t, d["tiles_m"], d["tiles_n"], d["group_m"])
            assert 0 <= tm.value < d["tiles_m"] and 0 <= tn.value < d["tiles_n"]
            seen.add((tm.value, tn.value))
        assert len(seen) == d["total_tiles"]


def test_bad_arguments(lib):
    from streamk_b200 import _lib as L
    info = L.SkScheduleInfo()
    prob = L.SkProblem(M=0, N=4, K=4, schedule=1)
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == L.SK_ERR_SHAPE
    prob = L.SkProblem(M=4, N=4, K=4, schedule=9)
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == L.SK_ERR_ARG
    prob = L.SkProblem(M=4, N=4, K=4, schedule=1, tile_n=72)
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == L.SK_ERR_ARG


def test_short_m_swaps_operands(lib):
    from streamk_b200 import _lib as L
    for M, want_tm in ((1, 16), (16, 16), (17, 32), (33, 48), (64, 64)):
        prob = L.SkProblem(M=M, N=4096, K=4096, schedule=1)
        info = L.SkScheduleInfo()
        assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == 0
        d = info.as_dict()
        assert (d["swap_ab"], d["tile_m"], d["tile_n"]) == (1, want_tm, 128)
        assert (d["tiles_m"], d["tiles_n"], d["total_tiles"]) == (1, 32, 32)
        assert lib.sk_schedule(C.byref(prob), 2, 148, C.byref(info)) == 0      # W4A16 too
        assert info.swap_ab == 1
    prob = L.SkProblem(M=65, N=4096, K=4096, schedule=1)
    info = L.SkScheduleInfo()
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == 0
    assert (info.swap_ab, info.tile_m, info.tile_n) == (0, 128, 128)
    # explicit forms
    prob = L.SkProblem(M=200, N=4096, K=4096, schedule=1, tile_m=208)
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == 0
    assert (info.swap_ab, info.tile_m, info.tiles_m, info.tiles_n) == (1, 208, 1, 32)
    prob = L.SkProblem(M=16, N=4096, K=4096, schedule=1, tile_m=128)
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == 0
    assert info.swap_ab == 0
    prob = L.SkProblem(M=16, N=4096, K=4096, schedule=1, tile_m=24)      # not a multiple of 16
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == L.SK_ERR_ARG
    # tile coordinates are reported in logical (M, N) order either way
    prob = L.SkProblem(M=100, N=1000, K=512, schedule=1, tile_m=64)
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == 0
    seen = set()
    tm, tn = C.c_int(), C.c_int()
    for t in range(info.total_tiles):
        assert lib.sk_tile_coords(C.byref(info), t, C.byref(tm), C.byref(tn)) == 0
        assert 0 <= tm.value < info.tiles_m == 2 and 0 <= tn.value < info.tiles_n == 8
        seen.add((tm.value, tn.value))
    assert len(seen) == 16


def test_auto_schedule_resolution(lib):
    from streamk_b200 import _lib as L
    AUTO = L.SCHEDULES["auto"]
    def plan(M, N, K, kind=1):
        prob = L.SkProblem(M=M, N=N, K=K, schedule=AUTO, layout=1)
        info = L.SkScheduleInfo()
        assert lib.sk_schedule(C.byref(prob), kind, 148, C.byref(info)) == 0
        return info.as_dict()
    names = {v: k for k, v in L.SCHEDULES.items()}
    d = plan(16, 4096, 4096)          # 32 swapped tiles: every SM has to stream; clusters of 4
    assert (names[d["schedule"]], d["swap_ab"], d["cluster"], d["grid"]) == ("cluster", 1, 4, 128)
    d = plan(24, 4096, 4096, kind=2)  # the W4A16 kernel alike (beyond the small-M path's 16 rows)
    assert (names[d["schedule"]], d["swap_ab"], d["cluster"]) == ("cluster", 1, 4)
    d = plan(16, 4096, 256)           # shallow K: nothing to split
    assert names[d["schedule"]] == "streamk"
    d = plan(16, 12288, 4096)         # whole swapped tiles, 88 weight rows each: 140 of 148 SMs busy
    assert (names[d["schedule"]], d["swap_ab"], d["tile_n"], d["total_tiles"]) == ("dp", 1, 88, 140)
    d = plan(16, 11008, 4096)
    assert (names[d["schedule"]], d["tile_m"], d["tile_n"], d["total_tiles"]) == ("dp", 16, 80, 138)
    d = plan(16, 12288, 4096, kind=2)  # (W4A16 weights come in blocks of 128 rows)
    assert (d["swap_ab"], d["tile_n"], d["total_tiles"]) == (1, 128, 96)
    d = plan(256, 12288, 4096)        # CTA pairs, 256-row tiles, width fitted to the 74 pairs
    assert (names[d["schedule"]], d["tile_m"], d["tile_n"], d["total_tiles"], d["grid"]) == ("dp", 256, 192, 64, 64)
    d = plan(512, 4096, 4096)         # two tile rows of 256: 37 pairs per row
    assert (names[d["schedule"]], d["tile_m"], d["tile_n"], d["total_tiles"]) == ("dp", 256, 128, 64)
    d = plan(100, 12288, 4096)        # one 128-row tile row: single CTAs, 128-wide tiles kept
    assert (names[d["schedule"]], d["tile_m"], d["tile_n"], d["total_tiles"]) == ("dp", 128, 128, 96)
    d = plan(128, 4096, 4096)         # 32 tiles: clusters of 4 on 128 x 128 tiles
    assert (names[d["schedule"]], d["tile_m"], d["tile_n"], d["cluster"]) == ("cluster", 128, 128, 4)
    d = plan(128, 9000, 4096)         # 71 tiles: clusters of 2
    assert (names[d["schedule"]], d["cluster"], d["grid"]) == ("cluster", 2, 142)
    d = plan(128, 4096, 256)          # shallow K and too narrow to fit whole tiles: Stream-K
    assert (names[d["schedule"]], d["tile_m"], d["tile_n"]) == ("streamk", 128, 128)
    d = plan(8192, 28672, 8192, kind=3)
    assert names[d["schedule"]] == "hybrid" and d["tile_m"] == 256
    # a single row of activations: the small-M path; fp16: row groups of 128 x a split of K
    d = plan(1, 4096, 4096)
    assert (names[d["schedule"]], d["tile_m"], d["tile_n"], d["tiles_n"], d["iters_per_tile"], d["tile_k"],
            d["grid"]) == ("gemv", 1, 128, 32, 16, 256, 512)
    d = plan(2, 4096, 4096)                  # from M = 2 the tensor cores are ahead
    assert names[d["schedule"]] == "cluster"
    d = plan(1, 148 * 4 * 128 + 1, 4096)     # more row groups than the workspace has counters: tensor cores
    assert names[d["schedule"]] != "gemv"
    # W4A16 (scale groups of 128): 32 rows per CTA over all of K, up to eight rows of activations
    for M in (1, 8):
        d = plan(M, 11008, 4096, kind=2)
        assert (names[d["schedule"]], d["tile_m"], d["tile_n"], d["tiles_n"], d["iters_per_tile"], d["tile_k"],
                d["grid"]) == ("gemv", M, 32, 344, 1, 4096, 344)
    d = plan(9, 11008, 4096, kind=2)          # 9 to 16 rows: only up to one CTA per SM
    assert names[d["schedule"]] != "gemv"
    d = plan(16, 4096, 4096, kind=2)
    assert (names[d["schedule"]], d["tile_m"], d["grid"]) == ("gemv", 16, 128)
    d = plan(17, 4096, 4096, kind=2)
    assert names[d["schedule"]] == "cluster"
    d = plan(4, 1024, 8192, kind=2)          # too few rows for half of the SMs: K split over 4 CTAs as well
    assert (names[d["schedule"]], d["tiles_n"], d["iters_per_tile"], d["tile_k"], d["grid"]) == ("gemv", 32, 4, 2048, 128)
    # scale groups of 32 or 64: the CUDA-core kernel, chosen at M = 1 and taken up to M = 4
    g64 = 0x200
    prob = L.SkProblem(M=1, N=11008, K=4096, schedule=L.SCHEDULES["auto"], layout=1, flags=g64)
    info = L.SkScheduleInfo()
    assert lib.sk_schedule(C.byref(prob), 2, 148, C.byref(info)) == 0 and names[info.schedule] == "gemv"
    prob = L.SkProblem(M=2, N=11008, K=4096, schedule=L.SCHEDULES["auto"], layout=1, flags=g64)
    assert lib.sk_schedule(C.byref(prob), 2, 148, C.byref(info)) == 0 and names[info.schedule] != "gemv"
    prob = L.SkProblem(M=4, N=11008, K=4096, schedule=L.SCHEDULES["gemv"], layout=1, flags=g64)
    assert lib.sk_schedule(C.byref(prob), 2, 148, C.byref(info)) == 0 and info.grid == 344
    prob = L.SkProblem(M=5, N=11008, K=4096, schedule=L.SCHEDULES["gemv"], layout=1, flags=g64)
    assert lib.sk_schedule(C.byref(prob), 2, 148, C.byref(info)) == L.SK_ERR_SHAPE
    # ... which an explicit request may still take up to M = 4 (fp16) or 16 (W4A16, groups of 128)
    prob = L.SkProblem(M=4, N=11008, K=4096, schedule=L.SCHEDULES["gemv"], layout=1)
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == 0 and info.grid == 516
    prob = L.SkProblem(M=5, N=11008, K=4096, schedule=L.SCHEDULES["gemv"], layout=1)
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == L.SK_ERR_SHAPE
    prob = L.SkProblem(M=16, N=11008, K=4096, schedule=L.SCHEDULES["gemv"], layout=1)
    assert lib.sk_schedule(C.byref(prob), 2, 148, C.byref(info)) == 0
    prob = L.SkProblem(M=17, N=11008, K=4096, schedule=L.SCHEDULES["gemv"], layout=1)
    assert lib.sk_schedule(C.byref(prob), 2, 148, C.byref(info)) == L.SK_ERR_SHAPE
    cov = oracle.coverage(plan(300, 5000, 1000))
    assert set(cov.values()) == {1}


def test_cluster_split(lib):
    """SK_SCHED_CLUSTER: cluster size from the SM budget, K ranges per rank, coverage."""
    from streamk_b200 import _lib as L
    d, info = _sched(lib, 384, 384, 8192, 1, "cluster", 148)
    assert (d["total_tiles"], d["cluster"], d["grid"]) == (9, 8, 72)
    d, info = _sched(lib, 128, 4096, 4096, 1, "cluster", 148)
    assert (d["total_tiles"], d["cluster"], d["grid"], d["sk_iters_per_cta"]) == (32, 4, 128, 16)
    d, info = _sched(lib, 256, 4096, 4096, 1, "cluster", 148)
    assert (d["total_tiles"], d["cluster"], d["grid"]) == (64, 2, 128)
    d, info = _sched(lib, 16, 4096, 4096, 1, "cluster", 64)       # the SM budget caps the size
    assert (d["swap_ab"], d["cluster"], d["grid"]) == (1, 2, 64)
    rnd = random.Random(11)
    for _ in range(40):
        M, N, K = rnd.randint(1, 600), rnd.randint(1, 1200), rnd.randint(1, 3000)
        prob = L.SkProblem(M=M, N=N, K=K, lda=K, ldb=K, ldc=N, layout=1, schedule=L.SCHEDULES["cluster"])
        info = L.SkScheduleInfo()
        st = lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info))
        d = info.as_dict()
        if st != 0:   # more tiles than half the SMs: no cluster fits
            tiles = -(-M // 128) * -(-N // 128) if M > 64 else -(-N // 128)
            assert st == L.SK_ERR_SHAPE and 2 * tiles > 148
            continue
        assert d["cluster"] in (2, 4, 8) and d["grid"] == d["total_tiles"] * d["cluster"] <= 148
        assert d["cluster"] == 8 or 2 * d["cluster"] * d["total_tiles"] > 148
        cov = oracle.coverage(d)
        assert len(cov) == d["total_tiles"] * d["iters_per_tile"] and set(cov.values()) == {1}
        b, e = C.c_int64(), C.c_int64()
        for p in range(d["grid"]):
            assert lib.sk_cta_interval(C.byref(info), p, C.byref(b), C.byref(e)) == 0
            segs = oracle.cluster_segments(p, iters_per_tile=d["iters_per_tile"], cluster=d["cluster"])
            I = d["iters_per_tile"]
            if segs:
                t, k0, k1 = segs[0]
                assert (b.value, e.value) == (t * I + k0, t * I + k1)
            else:
                assert b.value == e.value
    # other kernels do not take it
    prob = L.SkProblem(M=128, N=512, K=512, schedule=L.SCHEDULES["cluster"])
    assert lib.sk_schedule(C.byref(prob), 0, 148, C.byref(info)) == L.SK_ERR_ARG
    assert lib.sk_schedule(C.byref(prob), 3, 74, C.byref(info)) == L.SK_ERR_ARG
    assert lib.sk_schedule(C.byref(prob), 2, 148, C.byref(info)) == 0 and info.cluster == 8


def test_pair_kernel_wide_units(lib):
    """CTA-pair kernel, hybrid schedule: full waves of 256 x 512 units + Stream-K over the halves
    of the remaining units; every 256 x 256 tile is covered exactly once."""
    from streamk_b200 import _lib as L
    def plan(M, N, K, pairs=74, **kw):
        prob = L.SkProblem(M=M, N=N, K=K, lda=K, ldb=K, ldc=N, layout=1, schedule=L.SCHEDULES["hybrid"], **kw)
        info = L.SkScheduleInfo()
        assert lib.sk_schedule(C.byref(prob), 3, pairs, C.byref(info)) == 0
        return info.as_dict(), info
    d, info = plan(8192, 28672, 8192)      # configuration 5: 32 x 112 tiles = 32 x 56 units
    assert (d["total_tiles"], d["wide_units"], d["dp_tiles"], d["sk_tiles"], d["dp_waves"]) == (3584, 1776, 3552, 32, 24)
    assert (d["grid"], d["sk_iters_per_cta"], d["sk_iters_rem"]) == (74, 32 * 128 // 74, 32 * 128 % 74)
    d, _ = plan(8192, 28672, 8192, tile_m=256)     # asked for by the caller: plain 256 x 256 tiles
    assert (d["wide_units"], d["sk_tiles"]) == (0, 3584 % 74 + 74)
    d, _ = plan(8192, 28416, 8192)                 # 111 tile columns: odd, no pairing
    assert d["wide_units"] == 0
    rnd = random.Random(5)
    for _ in range(25):
        M, N, K = rnd.randint(200, 3000), rnd.randint(2000, 12000), rnd.randint(64, 2048)
        pairs = rnd.choice([3, 10, 74])
        d, info = plan(M, N, K, pairs=pairs)
        tiles_m, tiles_n = d["tiles_m"], d["tiles_n"]
        assert d["total_tiles"] == tiles_m * tiles_n == d["sk_tiles"] + d["dp_tiles"]
        seen = {}
        U = d["wide_units"]
        if U:
            assert tiles_n % 2 == 0 and U % d["grid"] == 0 and d["dp_tiles"] == 2 * U
            for u in range(U):      # the first U units of the rasterised tiles_m x tiles_n/2 grid
                tm, tnw = oracle.tile_coords(u, tiles_m, tiles_n // 2, d["group_m"])
                for h in (0, 1):
                    seen[(tm, 2 * tnw + h)] = seen.get((tm, 2 * tnw + h), 0) + 1
            tm, tn = C.c_int(), C.c_int()
            for t in range(d["sk_tiles"]):
                assert lib.sk_tile_coords(C.byref(info), t, C.byref(tm), C.byref(tn)) == 0
                seen[(tm.value, tn.value)] = seen.get((tm.value, tn.value), 0) + 1
            assert len(seen) == tiles_m * tiles_n and set(seen.values()) == {1}
            # the Stream-K part splits its iterations evenly over the pairs
            tot = d["sk_tiles"] * d["iters_per_tile"]
            assert d["sk_iters_per_cta"] * d["grid"] + d["sk_iters_rem"] == tot


def test_inspection_call_reports_what_the_fp16_entry_point_runs(lib):
    """sk_schedule(kind 1, auto) and sk_gemm_f16 share one decision (sk_f16_dispatch): for a
    large NT problem the entry point runs the CTA-pair kernel (256 x 256 tiles, 74 pairs,
    256 x 512 units), and the inspection call must say so, not describe 128-row tiles."""
    from streamk_b200 import _lib as L
    info = L.SkScheduleInfo()
    prob = L.SkProblem(M=8192, N=3584, K=8192, lda=8192, ldb=8192, ldc=3584, layout=1,
                       schedule=L.SCHEDULES["auto"])
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == 0
    d = info.as_dict()
    assert (d["tile_m"], d["tile_n"], d["grid"]) == (256, 256, 74)
    assert d["wide_units"] == 222 and d["sk_tiles"] == 4 and d["schedule"] == L.SCHEDULES["hybrid"]
    # the same problem in the NN layout has no pair kernel: single-CTA tiles on every SM
    prob.layout = 0
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == 0
    assert (info.tile_m, info.grid, info.wide_units) == (128, 148, 0)
    # an odd SM count cannot pair up either
    prob.layout = 1
    assert lib.sk_schedule(C.byref(prob), 1, 147, C.byref(info)) == 0
    assert (info.tile_m, info.grid) == (128, 147)
    # a zero-initialised problem with only the shape filled in is a valid question
    z = L.SkProblem()
    z.M, z.N, z.K = 384, 384, 8192
    assert lib.sk_schedule(C.byref(z), 1, 148, C.byref(info)) == 0 and info.total_tiles > 0


def test_tuned_table_is_consulted_first(lib):
    """SK_SCHED_AUTO looks a shape up in the table the offline tuner wrote (csrc/sk_tuned_table.inc)
    before applying its rules; SK_FLAG_NO_TABLE gives the rules alone.  Rows are read from the
    file, so the test follows whatever the last tuner run installed."""
    import os
    import re
    from streamk_b200 import _lib as L
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "stream-k.tvm_b200",
                        "csrc", "sk_tuned_table.inc")
    rows = [tuple(int(x) for x in m.groups()) for m in
            re.finditer(r"^\{(\d+), (\d+), (\d+), (\d+), (\d+), (\d+), (\d+), (\d+)\},", open(path).read(), re.M)]
    info = L.SkScheduleInfo()
    for kind, M, N, K, sms, schedule, tile_m, tile_n in rows:
        prob = L.SkProblem(M=M, N=N, K=K, lda=K, ldb=K, ldc=N, layout=1, schedule=L.SCHEDULES["auto"])
        assert lib.sk_schedule(C.byref(prob), kind, sms, C.byref(info)) == 0
        assert info.schedule == schedule
        if tile_m:
            assert info.tile_m == tile_m
        if tile_n:
            assert info.tile_n == tile_n
        # another SM count, or the flag: the rules answer (they may agree, but must not fail)
        prob.flags = L.SK_FLAG_NO_TABLE
        assert lib.sk_schedule(C.byref(prob), kind, sms, C.byref(info)) == 0
    # a shape that is not in the table is untouched by it
    prob = L.SkProblem(M=123, N=4567, K=896, lda=896, ldb=896, ldc=4567, layout=1, schedule=L.SCHEDULES["auto"])
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == 0
    a = info.as_dict()
    prob.flags = L.SK_FLAG_NO_TABLE
    assert lib.sk_schedule(C.byref(prob), 1, 148, C.byref(info)) == 0
    assert info.as_dict() == a


def test_small_m_plans_cover_the_matrix(lib):
    """SK_SCHED_GEMV: whatever the shape, the grid covers every weight row and all of K exactly once."""
    from streamk_b200 import _lib as L
    rnd = random.Random(23)
    for _ in range(300):
        kind = rnd.choice([1, 2])
        flags = rnd.choice([0, 0, 0x100, 0x200, 0x300]) if kind == 2 else 0
        small_groups = flags in (0x100, 0x200)
        M = rnd.randint(1, 4 if (kind == 1 or small_groups) else 16)
        N = rnd.choice([1, 31, 32, 33, 127, 128, 129, rnd.randint(1, 40000)])
        K = 128 * rnd.randint(1, 200) if kind == 2 else 8 * rnd.randint(1, 4000)
        prob = L.SkProblem(M=M, N=N, K=K, lda=K, ldb=K, ldc=N, layout=1, schedule=L.SCHEDULES["gemv"], flags=flags)
        info = L.SkScheduleInfo()
        st = lib.sk_schedule(C.byref(prob), kind, 148, C.byref(info))
        d = info.as_dict()
        assert st == 0, (kind, M, N, K, flags, st)
        rows = 128 if kind == 1 else 32
        assert d["tile_m"] == M and d["tile_n"] == rows
        assert d["tiles_n"] == (N + rows - 1) // rows                    # row groups
        assert d["grid"] == d["tiles_n"] * d["iters_per_tile"]           # x splits of K
        assert d["tile_k"] * d["iters_per_tile"] >= K                    # the splits reach the end of K ...
        assert d["tile_k"] * (d["iters_per_tile"] - 1) < K               # ... and none is empty
        if kind == 2:
            assert d["tile_k"] % 128 == 0                                # whole steps of the kernels
    # beyond the kernels' rows of activations: refused, nothing planned
    for kind, M, flags in ((1, 5, 0), (2, 17, 0), (2, 5, 0x100)):
        prob = L.SkProblem(M=M, N=4096, K=4096, lda=4096, ldb=4096, ldc=4096, layout=1, schedule=L.SCHEDULES["gemv"], flags=flags)
        assert lib.sk_schedule(C.byref(prob), kind, 148, C.byref(L.SkScheduleInfo())) == L.SK_ERR_SHAPE
