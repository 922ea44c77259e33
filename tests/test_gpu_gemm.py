"""GPU parity: every entry point, through the C ABI, against the CPU oracle.

Tolerances: fp16 / W4A16  max|C - C_ref| <= 1e-2 * max|C_ref|  (the benchmark's bar; the
reference itself uses rtol = atol = 1e-2, streamk_fp16.py:399); fp32  1e-4 relative.
"""
import os

import numpy as np
import pytest
import torch

import oracle
import streamk_b200 as sk

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL16 = 1e-2
TOL32 = 1e-4
GOLD = os.path.join(os.path.dirname(__file__), "golden")
SCHEDULES = ("streamk", "hybrid", "hybrid_dp_first", "dp", "auto")
FIXUPS = ("atomic", "block_reduce")


def _rand16(M, N, K, seed, layout="nt"):
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(M, K, generator=g).half()
    B = (torch.randn((N, K) if layout == "nt" else (K, N), generator=g) / K ** 0.5).half()
    return A, B


def _check(C, ref, tol):
    sk.check_status()
    err = oracle.rel_err(C, ref)
    assert err <= tol, err


# ----------------------------------------------------------------------------- golden
def test_golden_vectors():
    z = np.load(os.path.join(GOLD, "gemm_golden.npz"))
    A, B = torch.from_numpy(z["nt_A"]), torch.from_numpy(z["nt_B"])
    for fixup in FIXUPS:
        _check(sk.streamk_fp16_nt(A.to(DEV), B.to(DEV), fixup=fixup, schedule="streamk"),
               torch.from_numpy(z["nt_C"]), TOL16)
    A, B = torch.from_numpy(z["nn_A"]), torch.from_numpy(z["nn_B"])
    _check(sk.streamk_fp16_nn(A.to(DEV), B.to(DEV)), torch.from_numpy(z["nn_C"]), TOL16)
    A, B = torch.from_numpy(z["nn32_A"]), torch.from_numpy(z["nn32_B"])
    for fixup in FIXUPS:
        _check(sk.streamk_fp32(A.to(DEV), B.to(DEV), fixup=fixup, schedule="streamk"),
               torch.from_numpy(z["nn32_C"]), TOL32)


# ----------------------------------------------------------------------------- fp32
@pytest.mark.parametrize("fixup", FIXUPS)
def test_fp32_config1(fixup):
    c = oracle.make_case(1)
    ref = oracle.gemm_ref(c["A"], c["B"], "nn")
    for schedule in SCHEDULES:
        _check(sk.streamk_fp32(c["A"].to(DEV), c["B"].to(DEV), fixup=fixup, schedule=schedule),
               ref, TOL32)


@pytest.mark.parametrize("shape", [(32, 64, 32), (64, 64, 64), (1, 1, 1), (100, 90, 70), (257, 130, 513)])
def test_fp32_shapes_and_grids(shape):
    M, N, K = shape
    g = torch.Generator().manual_seed(M * 7 + N)
    A = torch.rand(M, K, generator=g) * 2 - 1
    B = torch.rand(K, N, generator=g) * 2 - 1
    ref = oracle.gemm_ref(A, B, "nn")
    for fixup in FIXUPS:
        for sms in (None, 1, 2, 3, 5):
            _check(sk.streamk_fp32(A.to(DEV), B.to(DEV), fixup=fixup, schedule="streamk", num_sms=sms),
                   ref, TOL32)
    # NT form of the same product
    _check(sk.streamk_fp32(A.to(DEV), B.t().contiguous().to(DEV), trans_b=True), ref, TOL32)


# ----------------------------------------------------------------------------- fp16
@pytest.mark.parametrize("fixup", FIXUPS)
def test_fp16_config2_deep_k_nine_tiles(fixup):
    c = oracle.make_case(2)
    ref = oracle.gemm_ref(c["A"], c["B"], "nt")
    A, B = c["A"].to(DEV), c["B"].to(DEV)
    for schedule in SCHEDULES:
        _check(sk.streamk_fp16_nt(A, B, fixup=fixup, schedule=schedule, tile_n=128), ref, TOL16)
    info = sk.schedule_info(384, 384, 8192, tile_n=128)
    assert info["total_tiles"] == 9 and info["sk_tiles"] == 9


@pytest.mark.parametrize("shape", [
    (128, 128, 64), (128, 128, 1024), (256, 1024, 512), (512, 512, 512),   # reference smoke shapes
    (1, 128, 128), (7, 200, 136), (33, 520, 1000), (255, 300, 72), (300, 520, 1032)])
def test_fp16_nt_ragged_shapes_schedules_fixups(shape):
    M, N, K = shape
    A, B = _rand16(M, N, K, seed=M + N + K)
    ref = oracle.gemm_ref(A, B, "nt")
    A, B = A.to(DEV), B.to(DEV)
    for fixup in FIXUPS:
        for schedule in SCHEDULES:
            for tile_n in (128, 256):
                _check(sk.streamk_fp16_nt(A, B, fixup=fixup, schedule=schedule, tile_n=tile_n), ref, TOL16)


@pytest.mark.parametrize("sms", [1, 2, 3, 5, 37, 148])
def test_fp16_grid_sizes(sms):
    A, B = _rand16(300, 700, 1032, seed=sms)
    ref = oracle.gemm_ref(A, B, "nt")
    for fixup in FIXUPS:
        _check(sk.streamk_fp16_nt(A.to(DEV), B.to(DEV), fixup=fixup, schedule="streamk", num_sms=sms),
               ref, TOL16)


@pytest.mark.parametrize("M", [1, 8, 16, 17, 33, 64])
def test_fp16_short_m_swapped_operands(M):
    """Short M: the weights feed the UMMA M dimension and C is stored transposed."""
    N, K = 1000, 1032
    A, B = _rand16(M, N, K, seed=M)
    ref = oracle.gemm_ref(A, B, "nt")
    assert sk.schedule_info(M, N, K)["swap_ab"] == 1
    for fixup in FIXUPS:
        for schedule in SCHEDULES:
            _check(sk.streamk_fp16_nt(A.to(DEV), B.to(DEV), fixup=fixup, schedule=schedule), ref, TOL16)
    # the same problem with the operands in the ordinary order, and swapped with several row tiles
    _check(sk.streamk_fp16_nt(A.to(DEV), B.to(DEV), tile_m=128, schedule="streamk"), ref, TOL16)
    LB = sk.ladder_prepack(B.to(DEV))
    _check(sk.streamk_fp16_ladder(A.to(DEV), LB, schedule="streamk", fixup="block_reduce"), ref, TOL16)
    Bn = B.t().contiguous()
    _check(sk.streamk_fp16_nn(A.to(DEV), Bn.to(DEV), schedule="streamk"), ref, TOL16)


@pytest.mark.parametrize("M", [1, 16, 40, 64])
def test_fp16_swapped_with_fitted_weight_tiles(M):
    """Swapped operands with fewer than 128 weight rows per tile (tile_n < 128): the UMMA
    still spans 128 rows, whose tail holds stale data that must never reach C."""
    N, K = 1000, 1032
    A, B = _rand16(M, N, K, seed=100 + M)
    ref = oracle.gemm_ref(A, B, "nt")
    Ad, Bd = A.to(DEV), B.to(DEV)
    tm = (M + 15) // 16 * 16
    for tile_n in (24, 80, 104, 120):
        info = sk.schedule_info(M, N, K, schedule="streamk", tile_m=tm, tile_n=tile_n)
        assert (info["swap_ab"], info["tile_n"], info["tiles_n"]) == (1, tile_n, -(-N // tile_n))
        for schedule in SCHEDULES:
            for fixup in FIXUPS:
                _check(sk.streamk_fp16_nt(Ad, Bd, tile_m=tm, tile_n=tile_n, schedule=schedule, fixup=fixup), ref, TOL16)
        if info["total_tiles"] * 2 <= 148:
            _check(sk.streamk_fp16_nt(Ad, Bd, tile_m=tm, tile_n=tile_n, schedule="cluster"), ref, TOL16)
    # the library's own choice for many weight rows: data-parallel tiles of fitted height
    A2, B2 = _rand16(M, 11008, 512, seed=7)
    info = sk.schedule_info(M, 11008, 512)
    if M == 1:      # (a single row goes to the CUDA-core path)
        assert sk.SCHEDULE_NAMES[info["schedule"]] == "gemv"
        info = sk.schedule_info(M, 11008, 512, no_table=True, schedule="dp", tile_m=16, tile_n=80)
    assert (info["swap_ab"], info["tile_n"], info["total_tiles"]) == (1, 80, 138)
    _check(sk.streamk_fp16_nt(A2.to(DEV), B2.to(DEV)), oracle.gemm_ref(A2, B2, "nt"), TOL16)
    with pytest.raises(Exception):     # other layouts come in 128-row units
        sk.streamk_fp16_nn(Ad, B.t().contiguous().to(DEV), tile_m=tm, tile_n=80)


def test_fp16_explicit_swap_with_several_m_tiles():
    A, B = _rand16(200, 520, 1000, seed=77)
    ref = oracle.gemm_ref(A, B, "nt")
    for tile_m in (16, 64, 112, 208, 256):
        for fixup in FIXUPS:
            _check(sk.streamk_fp16_nt(A.to(DEV), B.to(DEV), tile_m=tile_m, fixup=fixup, schedule="streamk"),
                   ref, TOL16)


def test_fp16_odd_k_is_padded():
    A, B = _rand16(20, 40, 77, seed=3)
    _check(sk.streamk_fp16_nt(A.to(DEV), B.to(DEV)), oracle.gemm_ref(A, B, "nt"), TOL16)
    A, B = _rand16(20, 44, 77, seed=4, layout="nn")
    _check(sk.streamk_fp16_nn(A.to(DEV), B.to(DEV)), oracle.gemm_ref(A, B, "nn"), TOL16)


@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 384, 512), (100, 200, 136), (16, 1024, 1024)])
def test_fp16_nn(shape):
    M, N, K = shape
    A, B = _rand16(M, N, K, seed=11, layout="nn")
    ref = oracle.gemm_ref(A, B, "nn")
    for tile_n in (128, 256):
        for fixup in FIXUPS:
            _check(sk.streamk_fp16_nn(A.to(DEV), B.to(DEV), fixup=fixup, schedule="streamk", tile_n=tile_n),
                   ref, TOL16)


@pytest.mark.parametrize("shape", [(128, 128, 64), (128, 256, 512), (100, 200, 136), (16, 4096, 4096)])
def test_fp16_ladder(shape):
    M, N, K = shape
    A, B = _rand16(M, N, K, seed=12)
    ref = oracle.gemm_ref(A, B, "nt")
    LB = sk.ladder_prepack(B.to(DEV))
    for tile_n in (128, 256):
        _check(sk.streamk_fp16_ladder(A.to(DEV), LB, schedule="streamk", tile_n=tile_n), ref, TOL16)
        _check(sk.streamk_fp16_ladder_block_reduce(A.to(DEV), LB, tile_n=tile_n), ref, TOL16)


@pytest.mark.parametrize("shape", [
    (384, 384, 8192),                    # configuration 2: 9 tiles, clusters of 8
    (16, 4096, 4096), (128, 4096, 4096), (256, 4096, 4096), (1, 4096, 11008),   # 4, 4, 2, 4 CTAs per tile
    (7, 300, 64), (33, 129, 200), (100, 1000, 520), (300, 260, 1000), (128, 512, 128)])
def test_fp16_cluster_split_k(shape):
    """SK_SCHED_CLUSTER: the partial tiles of a cluster meet in distributed shared memory.
    Ragged shapes, fewer K iterations than CTAs (empty ranks), every layout; bitwise reproducible."""
    M, N, K = shape
    A, B = _rand16(M, N, K, seed=M + 3 * N + K)
    ref = oracle.gemm_ref(A, B, "nt")
    Ad, Bd = A.to(DEV), B.to(DEV)
    first = sk.streamk_fp16_nt(Ad, Bd, schedule="cluster")
    _check(first, ref, TOL16)
    info = sk.schedule_info(M, N, K, schedule="cluster")
    assert info["cluster"] in (2, 4, 8) and info["grid"] == info["total_tiles"] * info["cluster"]
    for _ in range(3):
        assert torch.equal(sk.streamk_fp16_nt(Ad, Bd, schedule="cluster"), first)
    if N * K <= 1 << 20:
        for sms in (2 * info["total_tiles"], 4 * info["total_tiles"]):     # smaller clusters
            _check(sk.streamk_fp16_nt(Ad, Bd, schedule="cluster", num_sms=sms), ref, TOL16)
        _check(sk.streamk_fp16_nn(Ad, B.t().contiguous().to(DEV), schedule="cluster"), ref, TOL16)
        _check(sk.streamk_fp16_ladder(Ad, sk.ladder_prepack(Bd), schedule="cluster"), ref, TOL16)
        if M > 64:
            for tile_n in (48, 96, 192):     # (wider tiles leave no room for the exchange buffers)
                _check(sk.streamk_fp16_nt(Ad, Bd, schedule="cluster", tile_m=128, tile_n=tile_n), ref, TOL16)


def test_fp16_cluster_needs_room_for_two_ctas_per_tile():
    A, B = _rand16(256, 8192, 256, seed=1)     # 128 tiles: no cluster of 2 per tile fits 148 SMs
    with pytest.raises(Exception):
        sk.streamk_fp16_nt(A.to(DEV), B.to(DEV), schedule="cluster")


@pytest.mark.parametrize("shape", [(256, 1024, 512), (300, 520, 1000), (512, 768, 1032), (200, 2000, 264)])
def test_fp16_cta_pairs_with_narrow_tiles(shape):
    """The CTA-pair kernel (tile_m = 256) with tile widths other than 256: every schedule and
    fixup, ragged edges, small grids."""
    M, N, K = shape
    A, B = _rand16(M, N, K, seed=M + N)
    ref = oracle.gemm_ref(A, B, "nt")
    Ad, Bd = A.to(DEV), B.to(DEV)
    for tile_n in (32, 64, 96, 160, 192, 256):
        for schedule in ("dp", "streamk", "hybrid"):
            for fixup in FIXUPS:
                _check(sk.streamk_fp16_nt(Ad, Bd, tile_m=256, tile_n=tile_n, schedule=schedule, fixup=fixup), ref, TOL16)
        _check(sk.streamk_fp16_nt(Ad, Bd, tile_m=256, tile_n=tile_n, schedule="streamk", num_sms=6), ref, TOL16)
    with pytest.raises(Exception):
        sk.streamk_fp16_nt(Ad, Bd, tile_m=256, tile_n=72)
    # what auto makes of more than one 128-row tile row with many columns: pairs, fitted width
    A2, B2 = _rand16(256, 11008, 256, seed=9)
    info = sk.schedule_info(256, 11008, 256)
    assert (info["tile_m"], info["tile_n"], info["total_tiles"]) == (256, 160, 69)
    _check(sk.streamk_fp16_nt(A2.to(DEV), B2.to(DEV)), oracle.gemm_ref(A2, B2, "nt"), TOL16)


def test_fp16_config3_sample_of_the_sweep():
    # the full 24-shape sweep is the benchmark's job; parity on its extremes here
    for case in (0, 7, 22):
        c = oracle.make_case(3, case)
        ref = oracle.gemm_ref(c["A"], c["B"], "nt")
        A, B = c["A"].to(DEV), c["B"].to(DEV)
        for schedule in ("streamk", "hybrid", "dp"):
            _check(sk.streamk_fp16_nt(A, B, schedule=schedule, fixup="block_reduce"), ref, TOL16)


def test_programmatic_dependent_launch_changes_nothing_but_timing():
    """SK_FLAG_PDL: same bits as a plain launch, whatever runs before it in the stream (a torch
    kernel that knows nothing of it, another launch of this library, a copy)."""
    A, B = _rand16(48, 1000, 2056, seed=31)
    Ad, Bd = A.to(DEV), B.to(DEV)
    A2, B2 = _rand16(300, 520, 1032, seed=32)
    A2d, B2d = A2.to(DEV), B2.to(DEV)
    c = oracle.make_case(4, shape=(16, 512, 512))
    P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
    Aq = c["A"].to(DEV)
    for schedule in ("auto", "streamk", "hybrid", "dp", "cluster"):
        plain = sk.streamk_fp16_nt(Ad, Bd, schedule=schedule, fixup="block_reduce")
        scratch = torch.zeros(1 << 20, device=DEV)
        scratch.add_(1.0)                                   # a foreign kernel right before
        a = sk.streamk_fp16_nt(Ad, Bd, schedule=schedule, fixup="block_reduce", pdl=True)
        b = sk.streamk_fp16_nt(Ad, Bd, schedule=schedule, fixup="block_reduce", pdl=True)   # after one of ours
        Ad2 = Ad.clone()                                    # a copy right before
        d = sk.streamk_fp16_nt(Ad2, Bd, schedule=schedule, fixup="block_reduce", pdl=True)
        assert torch.equal(a, plain) and torch.equal(b, plain) and torch.equal(d, plain)
    if True:
        plain = sk.streamk_fp16_nt(A2d, B2d, schedule="hybrid", fixup="block_reduce", tile_n=128)
        outs = [sk.streamk_fp16_nt(A2d, B2d, schedule="hybrid", fixup="block_reduce", tile_n=128, pdl=True)
                for _ in range(5)]
        assert all(torch.equal(o, plain) for o in outs)
        plain = sk.streamk_fp16_ladder_block_reduce_q4(Aq, P)
        outs = [sk.streamk_fp16_ladder_block_reduce_q4(Aq, P, pdl=True) for _ in range(5)]
        assert all(torch.equal(o, plain) for o in outs)
    _check(a, oracle.gemm_ref(A, B, "nt"), TOL16)


def test_out_argument_and_views():
    A, B = _rand16(64, 256, 256, seed=5)
    big = torch.zeros(64, 512, dtype=torch.float16, device=DEV)
    out = big[:, :256]
    r = sk.streamk_fp16_nt(A.to(DEV), B.to(DEV), out=out)
    assert r.data_ptr() == out.data_ptr()
    _check(out, oracle.gemm_ref(A, B, "nt"), TOL16)
    assert float(big[:, 256:].abs().max()) == 0.0


# ----------------------------------------------------------------------------- W4A16
@pytest.mark.parametrize("shape", [(1, 128, 128), (4, 300, 256), (16, 4096, 4096)])
def test_dequant_is_bit_exact(shape):
    c = oracle.make_case(4, shape=shape)
    P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
    W = sk.dequant_w4(P).cpu()
    Wref = oracle.dequant_ref(c["q"], c["scales"], c["zeros"])
    assert torch.equal(W.view(torch.int16), Wref.view(torch.int16))
    # reference semantics: no scale, no zero-point; int8 low-nibble-first storage accepted
    q8 = c["qweight"].view(torch.int8).reshape(c["N"], c["K"] // 2)
    assert torch.equal(sk.dequant_w4(sk.q4_prepack(q8.to(DEV))).cpu(), c["q"].half())


@pytest.mark.parametrize("shape", [(128, 128, 128), (16, 512, 512), (33, 300, 256), (1, 4096, 4096),
                                   (128, 4096, 4096)])
def test_w4a16_gemm(shape):
    c = oracle.make_case(4, shape=shape)
    ref = oracle.w4a16_ref(c["A"], c["q"], c["scales"], c["zeros"])
    P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
    A = c["A"].to(DEV)
    for schedule, fixup in (("dp", "atomic"), ("streamk", "block_reduce"), ("hybrid", "atomic"),
                            ("hybrid_dp_first", "block_reduce")):
        _check(sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule=schedule, fixup=fixup), ref, TOL16)


@pytest.mark.parametrize("shape", [(16, 512, 512), (33, 300, 256), (1, 4096, 4096), (128, 4096, 4096),
                                   (16, 4096, 11008), (128, 128, 128), (200, 700, 1280)])
def test_w4a16_cluster_split_k(shape):
    """SK_SCHED_CLUSTER on the W4A16 kernel: K ranges that start inside a scale group, empty
    ranks, both operand orders; bitwise reproducible."""
    M, N, K = shape
    c = oracle.make_case(4, shape=shape)
    ref = oracle.w4a16_ref(c["A"], c["q"], c["scales"], c["zeros"])
    P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
    A = c["A"].to(DEV)
    first = sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="cluster")
    _check(first, ref, TOL16)
    info = sk.schedule_info(M, N, K, kind="w4a16", schedule="cluster")
    assert info["cluster"] in (2, 4, 8) and info["grid"] == info["total_tiles"] * info["cluster"]
    for _ in range(2):
        assert torch.equal(sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="cluster"), first)
    if N * K <= 1 << 20:
        for sms in (2 * info["total_tiles"], 4 * info["total_tiles"]):
            _check(sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="cluster", num_sms=sms), ref, TOL16)


def test_w4a16_both_operand_orders():
    c = oracle.make_case(4, shape=(48, 640, 1024))
    ref = oracle.w4a16_ref(c["A"], c["q"], c["scales"], c["zeros"])
    P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
    A = c["A"].to(DEV)
    assert sk.schedule_info(48, 640, 1024, kind="w4a16")["swap_ab"] == 1
    for tile_m in (None, 128, 16, 64):
        for fixup in FIXUPS:
            _check(sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="streamk", fixup=fixup, tile_m=tile_m),
                   ref, TOL16)


def test_w4a16_reference_semantics_no_scale_no_zero():
    c = oracle.make_case(4, shape=(32, 1024, 1024))         # the reference's q4 check shape
    ref = oracle.w4a16_ref(c["A"], c["q"])                   # A @ unpack(qB).T
    P = sk.q4_prepack(c["qweight"].to(DEV))
    _check(sk.streamk_fp16_ladder_block_reduce_q4(c["A"].to(DEV), P), ref, TOL16)


def test_w4a16_config4_extremes():
    for case in (0, 8):
        c = oracle.make_case(4, case)
        ref = oracle.w4a16_ref(c["A"], c["q"], c["scales"], c["zeros"])
        P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
        _check(sk.streamk_fp16_ladder_block_reduce_q4(c["A"].to(DEV), P), ref, TOL16)


@pytest.mark.parametrize("shape,slabs", [((300, 1000, 520), 3), ((64, 4096, 256), 8), ((256, 777, 128), 5), ((16, 100, 64), 1)])
def test_fp16_nt_host_pipeline(shape, slabs):
    """Host operands in, host result out, B and C moving in column slabs over three streams."""
    M, N, K = shape
    A, B = _rand16(M, N, K, seed=N)
    ref = oracle.gemm_ref(A, B, "nt")
    A_h, B_h = A.pin_memory(), B.pin_memory()
    out = sk.streamk_fp16_nt_host(A_h, B_h, slabs=slabs)
    torch.cuda.synchronize()
    _check(out, ref, TOL16)
    out2 = torch.empty(M, N, dtype=torch.float16).pin_memory()
    for _ in range(3):                                    # staging buffers are reused across calls
        assert sk.streamk_fp16_nt_host(A_h, B_h, out2, slabs=slabs) is out2
    torch.cuda.synchronize()
    assert torch.equal(out2, out)
    with pytest.raises(TypeError):
        sk.streamk_fp16_nt_host(A.to(DEV), B_h)
