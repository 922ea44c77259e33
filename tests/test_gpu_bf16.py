"""bfloat16 through the fp16 entry points (SK_FLAG_BF16): same kernels, bf16 operands, fp32
accumulation in TMEM, bf16 result.  The reference is fp16 only (its README lists further
dtypes as open work, README.md:20-21); the oracle is the same fp32 product of the operands'
own values, the bar the same max|C - C_ref| <= 1e-2 * max|C_ref|.
"""
import pytest
import torch

import oracle
import streamk_b200 as sk

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-2


def _rand(M, N, K, seed, layout="nt"):
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(M, K, generator=g).bfloat16()
    B = (torch.randn((N, K) if layout == "nt" else (K, N), generator=g) / K ** 0.5).bfloat16()
    return A, B


def _check(C, ref):
    sk.check_status()
    assert C.dtype == torch.bfloat16
    err = oracle.rel_err(C, ref)
    assert err <= TOL, err


@pytest.mark.parametrize("shape", [(128, 128, 64), (300, 520, 1032), (7, 200, 136), (33, 1000, 2056), (512, 768, 1024)])
def test_bf16_nt_every_schedule_and_fixup(shape):
    M, N, K = shape
    A, B = _rand(M, N, K, seed=M + N)
    ref = oracle.gemm_ref(A, B, "nt")
    Ad, Bd = A.to(DEV), B.to(DEV)
    for fixup in ("atomic", "block_reduce"):
        for schedule in ("auto", "streamk", "hybrid", "dp"):
            _check(sk.streamk_fp16_nt(Ad, Bd, schedule=schedule, fixup=fixup), ref)
    info = sk.schedule_info(M, N, K, schedule="cluster")
    if info["cluster"]:
        first = sk.streamk_fp16_nt(Ad, Bd, schedule="cluster")
        _check(first, ref)
        assert torch.equal(sk.streamk_fp16_nt(Ad, Bd, schedule="cluster"), first)
    if M > 128:
        for tile_n in (96, 256):        # the CTA-pair kernel
            _check(sk.streamk_fp16_nt(Ad, Bd, tile_m=256, tile_n=tile_n, schedule="hybrid"), ref)


def test_bf16_nn_ladder_and_mixed_types():
    A, B = _rand(100, 384, 520, seed=5, layout="nn")
    ref = oracle.gemm_ref(A, B, "nn")
    _check(sk.streamk_fp16_nn(A.to(DEV), B.to(DEV), schedule="streamk"), ref)
    Bt = B.t().contiguous().to(DEV)
    LB = sk.ladder_prepack(Bt)
    assert LB.dtype == torch.bfloat16
    _check(sk.streamk_fp16_ladder(A.to(DEV), LB), ref)
    with pytest.raises(TypeError):       # operands must agree
        sk.streamk_fp16_nt(A.to(DEV), Bt.half())
    with pytest.raises(TypeError):
        sk.streamk_fp16_ladder(A.to(DEV).half(), LB)


@pytest.mark.parametrize("case", [4, 13, 20, 23])      # 16x4096x4096, 64x11008x4096, 256x4096x4096, 256x12288x4096
def test_bf16_on_sweep_shapes(case):
    c = oracle.make_case(3, case)
    A, B = c["A"].bfloat16(), c["B"].bfloat16()
    ref = oracle.gemm_ref(A, B, "nt")
    Ad, Bd = A.to(DEV), B.to(DEV)
    first = sk.streamk_fp16_nt(Ad, Bd)
    _check(first, ref)
    assert torch.equal(sk.streamk_fp16_nt(Ad, Bd), first)        # deterministic fixup: same bits
    # against the fp16 run of the same (bf16-representable) values: only the output rounding differs
    C16 = sk.streamk_fp16_nt(Ad.half(), Bd.half())
    sk.check_status()
    scale = float(ref.abs().max())
    assert float((first.float() - C16.float()).abs().max()) <= 6e-3 * scale
