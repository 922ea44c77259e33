"""Seeded synthetic inputs for the benchmark configurations.  Test infrastructure.

No dataset is involved: the configurations are GEMM shapes with stated value
distributions.  Tensors are drawn from a CPU torch.Generator so the values do not
depend on the machine, in the fixed order A, B (or q), zeros, scales.
Seeds: 0 for configurations 1 and 2 (the reference seeds with
`torch.manual_seed(0)`, streamk_fp16.py:19); 1000 * cfg + case index for the sweeps.
"""
from __future__ import annotations

import math

import torch

from .gemm_ref import pack_u4_int32

CONFIGS = {
    1: dict(kind="f32", layout="nn", shapes=[(256, 256, 1024)]),
    2: dict(kind="f16", layout="nt", shapes=[(384, 384, 8192)]),
    3: dict(kind="f16", layout="nt",
            shapes=[(m, n, k) for m in (1, 16, 32, 64, 128, 256)
                    for (n, k) in ((4096, 4096), (11008, 4096), (4096, 11008), (12288, 4096))]),
    4: dict(kind="w4a16", layout="nt",
            shapes=[(m, n, k) for m in (1, 16, 128)
                    for (n, k) in ((4096, 4096), (11008, 4096), (4096, 11008))]),
    5: dict(kind="f16", layout="nt", shapes=[(8192, 28672, 8192)]),
}


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def make_case(cfg: int, case: int = 0, shape: tuple | None = None) -> dict:
    """Inputs of configuration `cfg`, case index `case` (or an explicit smaller `shape`
    with the same distributions).  Returns CPU tensors."""
    M, N, K = shape if shape is not None else CONFIGS[cfg]["shapes"][case]
    if cfg == 1:
        g = _gen(0)
        A = torch.rand(M, K, generator=g) * 2 - 1          # streamk_fp32.py:19-22
        B = torch.rand(K, N, generator=g) * 2 - 1
        return dict(A=A, B=B, layout="nn", M=M, N=N, K=K)
    if cfg == 2:
        g = _gen(0)
        A = torch.randn(M, K, generator=g).half()
        B = (torch.randn(N, K, generator=g) / math.sqrt(K)).half()
        return dict(A=A, B=B, layout="nt", M=M, N=N, K=K)
    if cfg in (3, 5):
        g = _gen(1000 * cfg + case)
        A = torch.randn(M, K, generator=g).half()
        B = (0.02 * torch.randn(N, K, generator=g)).half()
        return dict(A=A, B=B, layout="nt", M=M, N=N, K=K)
    if cfg == 4:
        g = _gen(1000 * cfg + case)
        A = torch.randn(M, K, generator=g).half()
        q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
        z = torch.randint(0, 16, (N, K // 128), generator=g, dtype=torch.uint8)
        s = (0.002 + 0.018 * torch.rand(N, K // 128, generator=g)).half()
        return dict(A=A, q=q, qweight=pack_u4_int32(q), zeros=z, scales=s, layout="nt",
                    M=M, N=N, K=K)
    raise ValueError(f"unknown configuration {cfg}")


def slab_case(slab: int, n_slab: int, K: int, seed_base: int = 5000) -> torch.Tensor:
    """Rows [slab*n_slab, (slab+1)*n_slab) of configuration 5's weight B: generated per
    slab of 3584 rows from a seed derived from the slab index, so that 1/2/4/8-GPU runs
    see the same global B."""
    g = _gen(seed_base + 1 + slab)
    return (0.02 * torch.randn(n_slab, K, generator=g)).half()
