"""Generates the golden fixtures in this directory from the reference's own source.

Run once where a checkout of the reference project (LeiWang1999/Stream-k.tvm) is at hand:

    python tests/golden/make_golden.py /path/to/reference

It executes, verbatim and on the CPU, the few self-contained host lines of the
reference that pin behaviour on the hot path:

* sched_golden.json   - the host scheduler block of streamk_fp16.py (from
                        `streamk_programs = total_sm` to `sm_patition_factor = ...`)
                        run for a list of shapes, tile sizes and SM counts;
* q4_unpack_golden.json - the uint4 unpack expression of
                        streamk_fp16_ladder_block_reduce_q4.py (the line that builds
                        `qB_expanded`) on a seeded int8 tensor;
* gemm_golden.npz     - small seeded operands with `torch.matmul(A, B.T)` /
                        `torch.matmul(A, B)` evaluated in fp32 on the CPU, the
                        expression every reference script checks against.

The fixtures travel with the repository; the reference checkout does not.
"""
from __future__ import annotations

import json
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
REF = sys.argv[1]


def _slice(path: str, first_marker: str, last_marker: str) -> str:
    lines = open(path).read().split("\n")
    i0 = next(i for i, l in enumerate(lines) if l.startswith(first_marker))
    i1 = next(i for i, l in enumerate(lines) if l.startswith(last_marker) and i >= i0)
    return "\n".join(lines[i0:i1 + 1])


def sched_golden() -> None:
    src = _slice(os.path.join(REF, "streamk_fp16.py"), "streamk_programs = total_sm",
                 "sm_patition_factor")
    cases = []
    shapes = [
        (16, 16384, 8192, 16, 128, 32, 108),      # the script's own problem
        (384, 384, 8192, 128, 128, 64, 148),
        (256, 256, 1024, 64, 64, 16, 148),
        (8192, 28672, 8192, 128, 256, 64, 148),
        (8192, 3584, 8192, 128, 256, 64, 148),
        (256, 1024, 512, 16, 16, 32, 108),        # the scripts' verification shape
        (512, 512, 512, 32, 64, 32, 108),
    ]
    for m in (1, 16, 32, 64, 128, 256):
        for (n, k) in ((4096, 4096), (11008, 4096), (4096, 11008), (12288, 4096)):
            shapes.append((m, n, k, 128, 128, 64, 148))
            shapes.append((m, n, k, 128, 256, 64, 132))
    for (M, N, K, BM, BN, BK, P) in shapes:
        ns = dict(total_sm=P, block_row_warps=1, warp_row_tiles=BM, block_col_warps=1,
                  warp_col_tiles=BN, chunk=BK, A=types.SimpleNamespace(shape=(M, K)),
                  B=types.SimpleNamespace(shape=(N, K)), cdiv=lambda a, b: math.ceil(a / b),
                  print=lambda *a, **k: None, math=math, max=max)
        exec(src, ns)
        cases.append(dict(M=M, N=N, K=K, BM=BM, BN=BN, BK=BK, P=P,
                          total_tiles=ns["total_tiles"], iters_per_tile=ns["iters_per_tile"],
                          streamk_tiles=ns["streamk_tiles"], blocking_tiles=ns["blocking_tiles"],
                          streamk_full_tiles=ns["streamk_full_tiles"],
                          streamk_partial_tiles=ns["streamk_partial_tiles"]))
    json.dump(dict(source="streamk_fp16.py host scheduler block, executed verbatim", cases=cases),
              open(os.path.join(HERE, "sched_golden.json"), "w"), indent=1)


def q4_golden() -> None:
    path = os.path.join(REF, "streamk.fp16.breakdown", "streamk_fp16_ladder_block_reduce_q4.py")
    line = next(l for l in open(path).read().split("\n") if l.startswith("qB_expanded ="))
    g = torch.Generator().manual_seed(0)
    qB = torch.randint(0, 127, (8, 16), generator=g, dtype=torch.int8)   # same range as the script
    ns = dict(torch=torch, qB=qB)
    exec(line, ns)
    exp = ns["qB_expanded"].view(8, 32)
    json.dump(dict(source=line.strip(), qB=qB.tolist(), expanded=exp.to(torch.int32).tolist()),
              open(os.path.join(HERE, "q4_unpack_golden.json"), "w"))


def gemm_golden() -> None:
    torch.manual_seed(0)
    out = {}
    # fp16 NT, ragged in every dimension
    A = (torch.rand(45, 136) * 2 - 1).half()
    B = (torch.rand(70, 136) * 2 - 1).half()
    out["nt_A"], out["nt_B"] = A.numpy(), B.numpy()
    out["nt_C"] = torch.matmul(A.float(), B.float().T).numpy()
    # fp32 NN
    A = torch.rand(33, 50) * 2 - 1
    B = torch.rand(50, 41) * 2 - 1
    out["nn32_A"], out["nn32_B"] = A.numpy(), B.numpy()
    out["nn32_C"] = torch.matmul(A, B).numpy()
    # fp16 NN
    A = (torch.rand(20, 72) * 2 - 1).half()
    B = (torch.rand(72, 24) * 2 - 1).half()
    out["nn_A"], out["nn_B"] = A.numpy(), B.numpy()
    out["nn_C"] = torch.matmul(A.float(), B.float()).numpy()
    np.savez_compressed(os.path.join(HERE, "gemm_golden.npz"), **out)


if __name__ == "__main__":
    sched_golden()
    q4_golden()
    gemm_golden()
    print("wrote fixtures to", HERE)
