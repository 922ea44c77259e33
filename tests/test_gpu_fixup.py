"""Fixup properties on the GPU: bitwise reproducibility, self-cleaning workspace,
bounded waits that report instead of hanging."""
import pytest
import torch

import oracle
import streamk_b200 as sk

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_block_reduce_is_bitwise_reproducible():
    c = oracle.make_case(2)
    A, B = c["A"].to(DEV), c["B"].to(DEV)
    first = sk.streamk_fp16_block_reduce(A, B, schedule="streamk", tile_n=128).clone()
    for _ in range(20):
        assert torch.equal(first, sk.streamk_fp16_block_reduce(A, B, schedule="streamk", tile_n=128))
    sk.check_status()
    c1 = oracle.make_case(1)
    A32, B32 = c1["A"].to(DEV), c1["B"].to(DEV)
    f32 = sk.streamk_fp32(A32, B32, fixup="block_reduce", schedule="streamk").clone()
    for _ in range(20):
        assert torch.equal(f32, sk.streamk_fp32(A32, B32, fixup="block_reduce", schedule="streamk"))
    sk.check_status()


def test_w4a16_block_reduce_is_bitwise_reproducible():
    c = oracle.make_case(4, shape=(16, 1024, 4096))
    P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
    A = c["A"].to(DEV)
    first = sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="streamk").clone()
    for _ in range(10):
        assert torch.equal(first, sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="streamk"))
    sk.check_status()


def test_atomic_fixup_within_tolerance_and_workspace_stays_clean():
    """The atomic workspace must return to all-zero after every call: alternating shapes
    and tile sizes on the same workspace would otherwise see each other's leftovers."""
    g = torch.Generator().manual_seed(9)
    cases = []
    for (M, N, K, tn) in [(300, 520, 1032, 128), (384, 384, 8192, 128), (260, 1000, 520, 256), (16, 4096, 1024, 128)]:
        A = torch.randn(M, K, generator=g).half()
        B = (torch.randn(N, K, generator=g) / K ** 0.5).half()
        cases.append((A.to(DEV), B.to(DEV), oracle.gemm_ref(A, B, "nt"), tn))
    for _ in range(3):
        for A, B, ref, tn in cases:
            C = sk.streamk_fp16_atomic(A, B, schedule="streamk", tile_n=tn)
            assert oracle.rel_err(C, ref) <= 1e-2
    sk.check_status()


def test_linearity_at_full_config_sizes():
    """Size-independent property at a full-size sweep shape: C(A1 + A2) = C(A1) + C(A2)
    up to fp16 rounding of the outputs."""
    c = oracle.make_case(3, 23)   # M=256, N=12288, K=4096
    A1, B = c["A"].to(DEV), c["B"].to(DEV)
    A2 = torch.roll(A1, 1, 0)
    C1 = sk.streamk_fp16_nt(A1, B).float()
    C2 = sk.streamk_fp16_nt(A2, B).float()
    C12 = sk.streamk_fp16_nt((A1.float() + A2.float()).half(), B).float()
    sk.check_status()
    scale = float(C12.abs().max())
    assert float((C12 - (C1 + C2)).abs().max()) <= 1e-2 * scale
    # a row permutation of A permutes the rows of C (split points differ per tile, so
    # compare within the output rounding, not bitwise)
    assert float((C2 - torch.roll(C1, 1, 0)).abs().max()) <= 2e-3 * scale


@pytest.mark.parametrize("kind", ["f16", "f32", "w4a16"])
def test_lost_flag_times_out_and_reports(kind):
    """Two CTAs share one tile; the peer is told not to publish its flag.  The owner's
    wait is bounded: it gives up, the kernel returns, the status word says which tile and
    which CTA, and the next ordinary launch works."""
    if kind == "f16":
        A = torch.randn(128, 1024).half().to(DEV)
        B = (torch.randn(128, 1024) / 32).half().to(DEV)
        run = lambda **kw: sk.streamk_fp16_block_reduce(A, B, schedule="streamk", num_sms=2, **kw)
        ref = oracle.gemm_ref(A, B, "nt")
    elif kind == "f32":
        A = torch.randn(64, 256).to(DEV)
        B = torch.randn(256, 64).to(DEV)
        run = lambda **kw: sk.streamk_fp32(A, B, fixup="block_reduce", schedule="streamk", num_sms=2, **kw)
        ref = oracle.gemm_ref(A, B, "nn")
    else:
        c = oracle.make_case(4, shape=(16, 128, 1024))
        P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
        A = c["A"].to(DEV)
        run = lambda **kw: sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="streamk", num_sms=2, **kw)
        ref = oracle.w4a16_ref(c["A"], c["q"], c["scales"], c["zeros"])
    run(timeout_us=2000, _drop_flag_cta=1)
    with pytest.raises(sk.StreamKError) as ei:
        sk.check_status()
    assert ei.value.status == 6          # SK_ERR_FIXUP_TIMEOUT
    assert "detail 0, 1" in str(ei.value)  # tile 0, awaited CTA 1
    C = run()
    sk.check_status()
    assert oracle.rel_err(C, ref) <= 1e-2
