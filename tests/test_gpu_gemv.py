"""The small-M path (schedule `gemv`): kernels that stream the weights once, with partial sums added in a
fixed order.  fp16 / bf16 NT and W4A16 with scale groups of 32 or 64 on the CUDA cores (M <= 4; what `auto`
runs at M = 1), W4A16 with groups of 128 and more through register-level tensor-core instructions (M <= 16;
what `auto` runs up to M = 8, and up to 16 on matrices of at most 32 rows per SM).

The reference has no such path (its kernels are tensor-core tiled at every M,
streamk_fp16.py:143-371, ..._q4.py:143-522); the oracle is the same CPU product as for every
other schedule, the tolerance the configurations' 1e-2 * max|C_ref| (streamk_fp16.py:389-399),
and the result must be the same bits on every launch.
"""
import pytest
import torch

import oracle
import streamk_b200 as sk

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL16 = 1e-2

SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (1000, 520), (130, 64), (1, 8), (129, 2056)]


@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("NK", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_fp16_small_m(M, NK):
    N, K = NK
    c = oracle.make_case(3, shape=(M, N, K))
    ref = oracle.gemm_ref(c["A"], c["B"], "nt")
    A, B = c["A"].to(DEV), c["B"].to(DEV)
    info = sk.schedule_info(M, N, K)
    assert (sk.SCHEDULE_NAMES[info["schedule"]] == "gemv") == (M == 1)   # what the default call runs
    first = sk.streamk_fp16_nt(A, B, schedule="gemv")
    sk.check_status()
    assert oracle.rel_err(first, ref) <= TOL16, info
    assert torch.equal(sk.streamk_fp16_nt(A, B, schedule="gemv"), first)   # split order is fixed: same bits
    if M == 1:
        assert torch.equal(sk.streamk_fp16_nt(A, B), first)
    assert torch.equal(sk.streamk_fp16_nt(A, B, schedule="gemv", fixup="atomic", pdl=True), first)
    if N >= 64 and K >= 64:   # and the tensor-core kernels on the same operands agree within the tolerance
        other = sk.streamk_fp16_nt(A, B, schedule="streamk")
        sk.check_status()
        assert oracle.rel_err(other, ref) <= TOL16
        assert oracle.rel_err(first, other.cpu()) <= TOL16


def test_bf16_small_m():
    g = torch.Generator().manual_seed(5)
    for M, N, K in ((1, 4096, 4096), (3, 777, 1032)):
        A = torch.randn(M, K, generator=g).bfloat16()
        B = (0.02 * torch.randn(N, K, generator=g)).bfloat16()
        ref = A.float() @ B.float().t()
        C = sk.streamk_fp16_nt(A.to(DEV), B.to(DEV), schedule="gemv")
        sk.check_status()
        assert C.dtype == torch.bfloat16
        assert oracle.rel_err(C.float(), ref) <= TOL16
        assert torch.equal(sk.streamk_fp16_nt(A.to(DEV), B.to(DEV), schedule="gemv"), C)


def test_strided_operands_and_output():
    """Leading dimensions larger than the extents (a view into wider matrices)."""
    g = torch.Generator().manual_seed(6)
    M, N, K = 2, 300, 1024
    Aw = torch.randn(M, K + 64, generator=g).half().to(DEV)
    Bw = (0.02 * torch.randn(N, K + 128, generator=g)).half().to(DEV)
    out = torch.full((M, N + 8), 7.0, dtype=torch.float16, device=DEV)
    A, B = Aw[:, :K], Bw[:, :K]
    sk.streamk_fp16_nt(A, B, out=out[:, :N], schedule="gemv")
    sk.check_status()
    ref = A.float().cpu() @ B.float().cpu().t()
    assert oracle.rel_err(out[:, :N], ref) <= TOL16
    assert bool((out[:, N:] == 7.0).all())                           # nothing written past N


def test_limits_and_other_layouts():
    c = oracle.make_case(3, shape=(5, 512, 512))
    A, B = c["A"].to(DEV), c["B"].to(DEV)
    with pytest.raises(sk.StreamKError):
        sk.streamk_fp16_nt(A, B, schedule="gemv")                     # M > 4
    c = oracle.make_case(3, shape=(1, 512, 512))
    A, B = c["A"].to(DEV), c["B"].to(DEV)
    ref = oracle.gemm_ref(c["A"], c["B"], "nt")
    with pytest.raises(sk.StreamKError):
        sk.streamk_fp16_nn(A, B.t().contiguous(), schedule="gemv")    # row-major [N, K] weights only
    C = sk.streamk_fp16_nn(A, B.t().contiguous())                    # auto: the tensor-core kernel
    sk.check_status()
    assert oracle.rel_err(C, ref) <= TOL16
    C = sk.streamk_fp16_nt(A, B, tile_m=16)                          # a tile size given: tensor cores too
    sk.check_status()
    assert oracle.rel_err(C, ref) <= TOL16


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 7, 8, 9, 13, 16])
@pytest.mark.parametrize("NK", [(4096, 4096), (11008, 4096), (4096, 11008), (200, 256), (129, 1152), (1024, 8192),
                                (31, 128)], ids=lambda s: "x".join(map(str, s)))
def test_w4a16_small_m(M, NK):
    N, K = NK
    c = oracle.make_case(4, shape=(M, N, K))
    ref = oracle.w4a16_ref(c["A"], c["q"], c["scales"], c["zeros"])
    P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
    A = c["A"].to(DEV)
    auto = sk.SCHEDULE_NAMES[sk.schedule_info(M, N, K, kind="w4a16")["schedule"]]     # what the default call runs
    assert (auto == "gemv") == (M <= 8 or N <= 32 * 148)
    first = sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="gemv")
    sk.check_status()
    assert oracle.rel_err(first, ref) <= TOL16
    assert torch.equal(sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="gemv"), first)
    if auto == "gemv":
        assert torch.equal(sk.streamk_fp16_ladder_block_reduce_q4(A, P), first)
    assert torch.equal(sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="gemv", pdl=True), first)
    other = sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="streamk")
    sk.check_status()
    assert oracle.rel_err(other, ref) <= TOL16


def test_w4a16_limits_and_activation_ranges():
    c = oracle.make_case(4, shape=(17, 512, 512))
    P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
    assert sk.SCHEDULE_NAMES[sk.schedule_info(17, 512, 512, kind="w4a16")["schedule"]] != "gemv"
    with pytest.raises(sk.StreamKError):
        sk.streamk_fp16_ladder_block_reduce_q4(c["A"].to(DEV), P, schedule="gemv")      # M > 16
    # activations far from 1 (the kernel multiplies them as they are, against nibbles read as
    # fp16 subnormals: neither end of the fp16 range may cost accuracy), zeros, and one outlier
    c = oracle.make_case(4, shape=(3, 640, 1024))
    P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
    for factor in (1.0, 2000.0, 1e-4, 0.0):
        A = (c["A"].float() * factor).half()
        if factor == 1.0:
            A[1, 77] = 30000.0
        ref = oracle.w4a16_ref(A, c["q"], c["scales"], c["zeros"])
        C = sk.streamk_fp16_ladder_block_reduce_q4(A.to(DEV), P, schedule="gemv")
        sk.check_status()
        assert bool(torch.isfinite(C).all())
        assert oracle.rel_err(C, ref) <= (TOL16 if factor else 0.0), factor


@pytest.mark.parametrize("group", [32, 64, 0])
def test_w4a16_small_m_formats(group):
    M, N, K = 3, 640, 1280
    g = torch.Generator().manual_seed(group + 11)
    A = torch.randn(M, K, generator=g).half()
    G = K // group if group else 1
    q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
    z = torch.randint(0, 16, (N, G), generator=g, dtype=torch.uint8)
    s = (0.002 + 0.018 * torch.rand(N, G, generator=g)).half()
    Wref = oracle.dequant_ref(q, s, z, group=group if group else K)
    P = sk.q4_prepack(oracle.pack_u4_int32(q).to(DEV), s.to(DEV), z.to(DEV), group_size=group)
    C = sk.streamk_fp16_ladder_block_reduce_q4(A.to(DEV), P, schedule="gemv")
    sk.check_status()
    assert oracle.rel_err(C, oracle.gemm_ref(A, Wref, "nt")) <= TOL16
    # signed int4 (stored as q ^ 8 with zero-point 8)
    qs = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int8)
    nib = (qs.to(torch.int16) & 0xF).to(torch.uint8)
    P = sk.q4_prepack(oracle.pack_u4_int32(nib).to(DEV), s.to(DEV), None, group_size=group, signed=True)
    Wref = qs.half() * s.repeat_interleave(group if group else K, dim=1)
    C = sk.streamk_fp16_ladder_block_reduce_q4(A.to(DEV), P, schedule="gemv")
    sk.check_status()
    assert oracle.rel_err(C, oracle.gemm_ref(A, Wref, "nt")) <= TOL16


def test_workspace_is_left_clean_for_the_other_fixups():
    """The small-M path counts arrivals in the workspace words the block-reduce fixup uses as
    flags; it must leave them zero."""
    c1 = oracle.make_case(3, shape=(1, 11008, 4096))
    c2 = oracle.make_case(3, shape=(128, 1024, 4096))
    A1, B1 = c1["A"].to(DEV), c1["B"].to(DEV)
    A2, B2 = c2["A"].to(DEV), c2["B"].to(DEV)
    ref2 = oracle.gemm_ref(c2["A"], c2["B"], "nt")
    for fixup in ("block_reduce", "atomic"):
        for _ in range(3):
            sk.streamk_fp16_nt(A1, B1)
            C = sk.streamk_fp16_nt(A2, B2, schedule="streamk", fixup=fixup, tile_n=128)
            sk.check_status()
            assert oracle.rel_err(C, ref2) <= TOL16


def test_w4a16_small_m_random_shapes():
    """Random M, N, K, group size, now and then strided activations and PDL: within tolerance of the oracle,
    finite, and the same bits on a second launch."""
    import random
    rnd = random.Random(7)
    for it in range(24):
        group = rnd.choice([128, 128, 128, 0, 32, 64])
        M = rnd.randint(1, 16 if group in (128, 0) else 4)
        K = 128 * rnd.randint(1, 40)
        if group == 0 and K == 128:
            K = 256
        N = rnd.choice([rnd.randint(1, 300), rnd.randint(300, 6000), rnd.randint(4000, 9000)])
        while N * K > 6_000_000:
            N //= 2
        g = torch.Generator().manual_seed(it)
        A = torch.randn(M, K, generator=g).half()
        G = K // group if group else 1
        q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
        z = torch.randint(0, 16, (N, G), generator=g, dtype=torch.uint8)
        s = (0.002 + 0.018 * torch.rand(N, G, generator=g)).half()
        ref = oracle.gemm_ref(A, oracle.dequant_ref(q, s, z, group=group if group else K), "nt")
        P = sk.q4_prepack(oracle.pack_u4_int32(q).to(DEV), s.to(DEV), z.to(DEV), group_size=group)
        Ad = A.to(DEV)
        if it % 5 == 0:                                            # a view into a wider matrix
            wide = torch.zeros(M, K + 64, dtype=torch.float16, device=DEV)
            wide[:, :K] = Ad
            Ad = wide[:, :K]
        C = sk.streamk_fp16_ladder_block_reduce_q4(Ad, P, schedule="gemv", pdl=(it % 3 == 0))
        sk.check_status()
        assert bool(torch.isfinite(C).all()), (M, N, K, group)
        assert oracle.rel_err(C, ref) <= TOL16, (M, N, K, group)
        assert torch.equal(sk.streamk_fp16_ladder_block_reduce_q4(Ad, P, schedule="gemv"), C), (M, N, K, group)
