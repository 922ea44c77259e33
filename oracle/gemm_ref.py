"""CPU restatement of the reference's result expressions.  Test infrastructure."""
from __future__ import annotations

import torch


def gemm_ref(A: torch.Tensor, B: torch.Tensor, layout: str = "nt") -> torch.Tensor:
    """fp32 C = A @ B (nn) or A @ B.T (nt) on the CPU, from the operands' own values.

    The reference compares every kernel with `torch.matmul(A, B)` (streamk_fp32.py:204)
    or `torch.matmul(A, B.T)` (streamk_fp16.py:389).  Evaluated in fp32 so that the
    oracle itself adds no fp16 rounding."""
    A = A.detach().to("cpu", torch.float32)
    B = B.detach().to("cpu", torch.float32)
    return A @ (B.t() if layout == "nt" else B)


def unpack_u4(qB: torch.Tensor) -> torch.Tensor:
    """int8/uint8 [N, K/2] -> uint8 [N, K], low nibble = even k.

    `((qB.unsqueeze(-1) >> (4 * arange(2))) & 0xF)` viewed as [N, K]
    (streamk_fp16_ladder_block_reduce_q4.py:552-554)."""
    q = qB.detach().to("cpu").to(torch.uint8)
    shifts = torch.tensor([0, 4], dtype=torch.uint8)
    out = (q.unsqueeze(-1) >> shifts) & 0xF
    return out.reshape(q.shape[0], q.shape[1] * 2)


def pack_u4_int32(q: torch.Tensor) -> torch.Tensor:
    """uint8 [N, K] values 0..15 -> int32 [N, K/8]; nibble j of word w = element 8w + j.
    Byte-identical to the reference's int8 [N, K/2] low-nibble-first storage."""
    q = q.detach().to("cpu").to(torch.int64)
    N, K = q.shape
    q = q.reshape(N, K // 8, 8)
    word = torch.zeros((N, K // 8), dtype=torch.int64)
    for j in range(8):
        word |= q[:, :, j] << (4 * j)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32)


def dequant_ref(q: torch.Tensor, scales: torch.Tensor | None, zeros: torch.Tensor | None,
                group: int = 128) -> torch.Tensor:
    """fp16 W[N,K] = (q.half() - z.half()) * s, every operation rounded to fp16
    (the subtraction is exact).  scales None = 1, zeros None = 0: then W = q.half(),
    the reference's `qB_expanded...to(torch.half)` (…q4.py:552)."""
    q = q.detach().to("cpu")
    N, K = q.shape
    W = q.to(torch.float16)
    if zeros is not None:
        z = zeros.detach().to("cpu").to(torch.float16).repeat_interleave(group, dim=1)
        W = W - z
    if scales is not None:
        s = scales.detach().to("cpu").to(torch.float16).repeat_interleave(group, dim=1)
        W = W * s
    return W


def w4a16_ref(A: torch.Tensor, q: torch.Tensor, scales=None, zeros=None, group: int = 128):
    """fp32 C = A @ dequant(q).T  (`torch.matmul(A, B.T)`, …q4.py:556-557,601)."""
    return gemm_ref(A, dequant_ref(q, scales, zeros, group), "nt")


def rel_err(C: torch.Tensor, C_ref: torch.Tensor) -> float:
    """max|C - C_ref| / max|C_ref|: the acceptance measure (bar 1e-2; 1e-4 for fp32)."""
    C = C.detach().to("cpu", torch.float32)
    C_ref = C_ref.detach().to("cpu", torch.float32)
    denom = float(C_ref.abs().max())
    return float((C - C_ref).abs().max()) / (denom if denom > 0 else 1.0)
