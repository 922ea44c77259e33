"""Full-size configuration 5 on one GPU: checked on every element against the reference's
own oracle expression evaluated on the GPU (`torch.matmul(A, B.T)`, streamk_fp16.py:389)
and on a 64-row sample against the CPU oracle."""
import pytest
import torch

import oracle
import streamk_b200 as sk

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_config5_full_size_single_gpu():
    M, N, K = 8192, 28672, 8192
    g = torch.Generator(device=DEV).manual_seed(5000)
    A = torch.randn(M, K, generator=g, device=DEV, dtype=torch.float32).half()
    B = (0.02 * torch.randn(N, K, generator=g, device=DEV, dtype=torch.float32)).half()
    C = sk.streamk_fp16_nt(A, B, schedule="hybrid", fixup="block_reduce")
    sk.check_status()
    ref_gpu = torch.matmul(A, B.t())
    scale = float(ref_gpu.float().abs().max())
    worst = 0.0
    for r0 in range(0, M, 1024):
        d = (C[r0:r0 + 1024].float() - ref_gpu[r0:r0 + 1024].float()).abs().max()
        worst = max(worst, float(d))
    assert worst <= 1e-2 * scale
    rows = torch.arange(0, M, M // 64)[:64]
    ref_cpu = oracle.gemm_ref(A[rows.to(DEV)].cpu(), B.cpu(), "nt")
    assert oracle.rel_err(C[rows.to(DEV)], ref_cpu) <= 1e-2
    # the three schedules agree bitwise on whole (unsplit) tiles and within tolerance overall
    C_dp = sk.streamk_fp16_nt(A, B, schedule="dp")
    sk.check_status()
    assert float((C_dp.float() - C.float()).abs().max()) <= 1e-2 * scale


@pytest.mark.parametrize("case", [
    ("f16", (16, 4096, 4096), "auto"), ("f16", (16, 11008, 4096), "auto"), ("f16", (256, 4096, 4096), "auto"),
    ("f16", (128, 4096, 4096), "streamk"), ("w4a16", (16, 4096, 11008), "auto"), ("w4a16", (16, 11008, 4096), "dp")])
@pytest.mark.parametrize("pdl", [False, True])
def test_back_to_back_launches_on_cold_weights(case, pdl):
    """Hundreds of launches without a host synchronisation in between, the weights rotating
    through more copies than the L2 holds (so loads land late and out of order, as in the
    benchmark's graph replays and unlike the small parity cases): every launch of a deterministic
    schedule must give the bits of the first, and no device wait may run out.  Guards the
    pipeline's mbarrier phase tracking (two issuing threads, grouped dequantisation) and, with
    pdl, the overlap of a launch's start-up with the tail of the launch before it."""
    kind, (M, N, K), schedule = case
    g = torch.Generator(device=DEV).manual_seed(M + N)
    A = torch.randn(M, K, generator=g, device=DEV).half()
    copies = 7 if kind == "f16" else 16
    if kind == "f16":
        W0 = (0.02 * torch.randn(N, K, generator=g, device=DEV)).half()
        Ws = [W0.clone() for _ in range(copies)]
        run = lambda i, out: sk.streamk_fp16_nt(A, Ws[i % copies], out=out, schedule=schedule, fixup="block_reduce",
                                                pdl=pdl)
    else:
        c = oracle.make_case(4, shape=(M, N, K))
        A = c["A"].to(DEV)
        P0 = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
        Ws = [P0] + [sk.PackedQ4(P0.data.clone(), N, K) for _ in range(copies - 1)]
        run = lambda i, out: sk.streamk_fp16_ladder_block_reduce_q4(A, Ws[i % copies], out=out, schedule=schedule,
                                                                    fixup="block_reduce", pdl=pdl)
    first = torch.empty(M, N, dtype=torch.float16, device=DEV)
    run(0, first)
    outs = [torch.empty_like(first) for _ in range(4)]
    for i in range(300):
        run(i, outs[i % 4])
    torch.cuda.synchronize()
    sk.check_status()
    for o in outs:
        assert torch.equal(o, first)


@pytest.mark.parametrize("shape", [(1024, 10240, 512), (1100, 10000, 520), (2048, 9728, 320), (512, 37888, 128)])
def test_pair_kernel_wide_units(shape):
    """The CTA-pair kernel's 256 x 512 units (hybrid schedule, the library's own tile choice):
    against the fp32 product on every element, both fixups, bitwise reproducible with block
    reduce, and level with the plain 256 x 256 path."""
    M, N, K = shape
    g = torch.Generator(device=DEV).manual_seed(M + N)
    A = torch.randn(M, K, generator=g, device=DEV).half()
    B = (torch.randn(N, K, generator=g, device=DEV) / K ** 0.5).half()
    info = sk.schedule_info(M, N, K, kind="f16_pairs", schedule="hybrid", num_sms=74)
    assert info["wide_units"] > 0 and info["wide_units"] % 74 == 0
    ref = torch.matmul(A.float(), B.float().t())
    scale = float(ref.abs().max())
    first = sk.streamk_fp16_nt(A, B, fixup="block_reduce")
    sk.check_status()
    assert float((first.float() - ref).abs().max()) <= 1e-2 * scale
    assert torch.equal(sk.streamk_fp16_nt(A, B, fixup="block_reduce"), first)
    other = sk.streamk_fp16_nt(A, B, fixup="atomic")
    sk.check_status()
    assert float((other.float() - ref).abs().max()) <= 1e-2 * scale
    plain = sk.streamk_fp16_nt(A, B, tile_m=256, schedule="hybrid", fixup="block_reduce")
    assert float((plain.float() - first.float()).abs().max()) <= 1e-2 * scale
    rows = torch.arange(0, M, max(M // 16, 1))[:16].to(DEV)
    assert oracle.rel_err(first[rows], oracle.gemm_ref(A[rows].cpu(), B.cpu(), "nt")) <= 1e-2
