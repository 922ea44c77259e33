"""Runs one entry point on one shape a few times: the command line that ncu captures
are taken from (see profiles/).

    python stream-k.tvm_b200/profile_case.py --kind f16 --shape 8192 3584 8192 \
        [--schedule hybrid] [--fixup block_reduce] [--tile-m N] [--tile-n N] [--iters 4] [--cublas]
        [--peers P]     # f16: the fused all-gather kernel, with P further matrices of the same
                        # GPU standing in for the peer GPUs' (what a one-GPU capture can show:
                        # the kernel's own cost of issuing P extra copies of every store)
"""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", default="f16", choices=["f16", "w4a16", "f32"])
    ap.add_argument("--shape", type=int, nargs=3, required=True, metavar=("M", "N", "K"))
    ap.add_argument("--schedule", default="hybrid")
    ap.add_argument("--fixup", default="block_reduce")
    ap.add_argument("--tile-m", type=int, default=None)
    ap.add_argument("--tile-n", type=int, default=None)
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--cublas", action="store_true", help="also run torch.matmul on the same operands")
    ap.add_argument("--peers", type=int, default=0)
    a = ap.parse_args()
    import torch
    import streamk_b200 as sk
    M, N, K = a.shape
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    kw = dict(schedule=a.schedule, fixup=a.fixup, tile_m=a.tile_m, tile_n=a.tile_n)
    if a.kind == "f32":
        A = torch.rand(M, K, generator=g, device=dev) * 2 - 1
        B = torch.rand(K, N, generator=g, device=dev) * 2 - 1
        kw.pop("tile_m"); kw.pop("tile_n")
        fn = lambda: sk.streamk_fp32(A, B, **kw)
        ref = lambda: torch.matmul(A, B)
    else:
        A = torch.randn(M, K, generator=g, device=dev).half()
        W = (0.02 * torch.randn(N, K, generator=g, device=dev)).half()
        out = torch.empty(M, N, dtype=torch.float16, device=dev)
        ref = lambda: torch.matmul(A, W.t(), out=out)
        if a.kind == "f16" and a.peers > 0:
            import ctypes as C
            from streamk_b200 import _lib as L
            from streamk_b200 import ops as _ops
            lib = L.load()
            mats = [torch.empty(M, N, dtype=torch.float16, device=dev) for _ in range(a.peers)]
            ptrs = (C.c_void_p * a.peers)(*[m.data_ptr() for m in mats])
            prob = L.SkProblem(M=M, N=N, K=K, lda=K, ldb=K, ldc=N, layout=L.LAYOUTS["nt"],
                               schedule=L.SCHEDULES[a.schedule], fixup=L.FIXUPS[a.fixup],
                               tile_m=a.tile_m or 0, tile_n=a.tile_n or 0, test_drop_flag_cta=-1)
            ws = _ops._workspace(torch.device(dev, torch.cuda.current_device()))

            def fn():
                L.check(lib.sk_gemm_f16_gather(C.byref(prob), A.data_ptr(), W.data_ptr(), out.data_ptr(), ptrs,
                                               a.peers, ws.buf.data_ptr(), ws.nbytes,
                                               torch.cuda.current_stream().cuda_stream), "sk_gemm_f16_gather")
        elif a.kind == "f16":
            fn = lambda: sk.streamk_fp16_nt(A, W, out=out, **kw)
        else:
            q = torch.randint(0, 16, (N, K // 8, 8), generator=g, device=dev, dtype=torch.int64)
            word = sum(q[:, :, j] << (4 * j) for j in range(8))
            word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
            z = torch.randint(0, 16, (N, K // 128), generator=g, device=dev, dtype=torch.uint8)
            s = (0.002 + 0.018 * torch.rand(N, K // 128, generator=g, device=dev)).half()
            P = sk.q4_prepack(word, s, z)
            fn = lambda: sk.streamk_fp16_ladder_block_reduce_q4(A, P, out=out, **kw)
    for _ in range(a.iters):
        fn()
    if a.cublas:
        for _ in range(a.iters):
            ref()
    torch.cuda.synchronize()
    sk.check_status()
    print("done")


if __name__ == "__main__":
    main()
