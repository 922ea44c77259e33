"""GPU parity against the reference's OWN GPU implementation: the Triton Stream-K kernel of
streamk.fp32.breakdown/triton_impl.py:14-238 (`first_wave` + `full_tiles` + `mac_loop`, host
`matmul`), run unmodified except for the three host-side repairs oracle/make_triton_ref.py
documents.  `matmul(a, b)` takes fp16 A [M,K] and B [K,N] and returns fp32 C, so the library's
NN entry point is the like-for-like call; its fp16 result must agree with the reference kernel's
within the configurations' bar, and both with the CPU oracle.

Skipped when oracle/_ref/triton_streamk.py has not been generated (it is made from a reference
checkout and never committed) or triton is missing.
"""
import pytest
import torch

import oracle
import streamk_b200 as sk

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL16 = 1e-2

ref_mod = oracle.load_triton_ref()
needs_ref = pytest.mark.skipif(ref_mod is None, reason="oracle/_ref/triton_streamk.py or triton not available")


@needs_ref
@pytest.mark.parametrize("shape", [(512, 512, 512),        # the reference's own check (triton_impl.py:247-264)
                                   (256, 4096, 4096),      # configuration 3, largest M
                                   (16, 11008, 4096)])     # configuration 3, short M, ragged tile count
def test_library_matches_the_reference_triton_kernel(shape):
    M, N, K = shape
    g = torch.Generator().manual_seed(0)
    if shape == (512, 512, 512):
        A = torch.randn(M, K, generator=g).half()
        Bnn = torch.randn(K, N, generator=g).half()
    else:
        A = torch.randn(M, K, generator=g).half()
        Bnn = (0.02 * torch.randn(K, N, generator=g)).half()
    Ad, Bd = A.to(DEV), Bnn.to(DEV)
    theirs = ref_mod.matmul(Ad, Bd)                       # fp32 [M, N]
    torch.cuda.synchronize()
    ours = sk.streamk_fp16_nn(Ad, Bd)
    sk.check_status()
    want = oracle.gemm_ref(A, Bnn, "nn")
    scale = float(want.abs().max())
    assert float((theirs.cpu() - want).abs().max()) <= TOL16 * scale          # the comparator itself is sound
    assert float((ours.float().cpu() - theirs.cpu()).abs().max()) <= TOL16 * scale
    assert oracle.rel_err(ours, want) <= TOL16
    # the NT entry point on the transposed weight gives the same product
    ours_nt = sk.streamk_fp16_nt(Ad, Bd.t().contiguous())
    sk.check_status()
    assert float((ours_nt.float().cpu() - theirs.cpu()).abs().max()) <= TOL16 * scale


@needs_ref
def test_reference_kernel_as_written_is_still_correct():
    """With the host's tile extents left as the reference wrote them (32 x 64 against kernels
    compiled for 256 x 256) out-of-range tiles are masked: same result, different split."""
    g = torch.Generator().manual_seed(0)
    A = torch.randn(512, 512, generator=g).half().to(DEV)
    B = torch.randn(512, 512, generator=g).half().to(DEV)
    c1 = ref_mod.matmul(A, B, as_written=True)
    torch.cuda.synchronize()
    want = oracle.gemm_ref(A.cpu(), B.cpu(), "nn")
    assert float((c1.cpu() - want).abs().max()) <= TOL16 * float(want.abs().max())
