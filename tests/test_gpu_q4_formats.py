"""W4A16 quantisation formats beyond the benchmark's (uint4, group 128): group sizes 32 and 64,
per-channel scales, signed int4.  The reference has none of them (its q4 kernels apply no scale
at all, ..._q4.py:544-557, and list the rest as open work, README.md:20-21); the oracle is the
same fp16 expression W = (q - z) * s evaluated on the CPU with the matching group size:
dequantisation bit-exact, GEMM within 1e-2 * max|C_ref|.
"""
import pytest
import torch

import oracle
import streamk_b200 as sk

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(M, N, K, group, seed, signed=False):
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(M, K, generator=g).half()
    G = K // group if group else 1
    q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
    z = torch.randint(0, 16, (N, G), generator=g, dtype=torch.uint8)
    s = (0.002 + 0.018 * torch.rand(N, G, generator=g)).half()
    return A, q, z, s


@pytest.mark.parametrize("group", [32, 64, 128, 0])
@pytest.mark.parametrize("shape", [(16, 384, 512), (1, 1024, 2048), (100, 300, 1280), (128, 1024, 1024)])
def test_group_sizes(shape, group):
    M, N, K = shape
    A, q, z, s = _case(M, N, K, group, seed=M + N + group)
    gsz = group if group else K
    Wref = oracle.dequant_ref(q, s, z, group=gsz)
    P = sk.q4_prepack(oracle.pack_u4_int32(q).to(DEV), s.to(DEV), z.to(DEV), group_size=group)
    assert torch.equal(sk.dequant_w4(P).cpu().view(torch.int16), Wref.view(torch.int16))
    ref = oracle.gemm_ref(A, Wref, "nt")
    Ad = A.to(DEV)
    for schedule in ("auto", "streamk", "dp"):
        C = sk.streamk_fp16_ladder_block_reduce_q4(Ad, P, schedule=schedule)
        sk.check_status()
        assert oracle.rel_err(C, ref) <= 1e-2, (schedule, group)
    if sk.schedule_info(M, N, K, kind="w4a16", schedule="cluster")["cluster"]:
        C = sk.streamk_fp16_ladder_block_reduce_q4(Ad, P, schedule="cluster")
        sk.check_status()
        assert oracle.rel_err(C, ref) <= 1e-2


@pytest.mark.parametrize("group", [64, 128, 0])
def test_signed_int4(group):
    M, N, K = 16, 512, 1024
    g = torch.Generator().manual_seed(group + 7)
    A = torch.randn(M, K, generator=g).half()
    qs = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int8)          # the signed values
    G = K // group if group else 1
    s = (0.002 + 0.018 * torch.rand(N, G, generator=g)).half()
    nib = (qs.to(torch.int16) & 0xF).to(torch.uint8)                           # two's-complement nibbles
    P = sk.q4_prepack(oracle.pack_u4_int32(nib).to(DEV), s.to(DEV), None, group_size=group, signed=True)
    Wref = qs.half() * s.repeat_interleave(group if group else K, dim=1)       # W = q * s, one rounding
    assert torch.equal(sk.dequant_w4(P).cpu().view(torch.int16), Wref.view(torch.int16))
    C = sk.streamk_fp16_ladder_block_reduce_q4(A.to(DEV), P)
    sk.check_status()
    assert oracle.rel_err(C, oracle.gemm_ref(A, Wref, "nt")) <= 1e-2
    with pytest.raises(ValueError):
        sk.q4_prepack(oracle.pack_u4_int32(nib).to(DEV), s.to(DEV), torch.zeros(N, G, dtype=torch.uint8, device=DEV),
                      group_size=group, signed=True)
