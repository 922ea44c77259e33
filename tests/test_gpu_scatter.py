"""sk_gemm_f16_scatter + sk_reduce_partials: the K-sharded product whose epilogue writes every fp32
partial tile into the receive slot of the GPU that owns its column block (fused reduce-scatter).

On one GPU the ranks are played one after the other through the C ABI, with every receive slot
a buffer of the same GPU: that exercises the kernel's store path (tile -> column block -> slot),
ragged edges and the fixed-order reduction.  With two or more GPUs the real thing runs as one
process per GPU over CUDA IPC mapped slots and is checked against the CPU oracle.
"""
import ctypes as C
import os
import socket
import sys

import pytest
import torch

import oracle
import streamk_b200 as sk
from streamk_b200 import _lib as L
from streamk_b200 import ops as _ops

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _scatter_on_one_gpu(A, B, G, tile_n, dtype=torch.float16, num_sms=0):
    """A [M, K], B [N, K] on the device; returns the [M, N] result assembled from the G blocks."""
    lib = L.load()
    M, K = A.shape
    N = B.shape[0]
    Nb, Kg = N // G, K // G
    recv = torch.full((G, G, M, Nb), float("nan"), dtype=torch.float32, device=DEV)   # [owner][sender]
    ws = _ops._workspace(DEV)
    for g in range(G):
        Ag = A[:, g * Kg:(g + 1) * Kg].contiguous()
        Bg = B[:, g * Kg:(g + 1) * Kg].contiguous()
        prob = L.SkProblem(M=M, N=N, K=Kg, lda=Kg, ldb=Kg, ldc=N, layout=L.LAYOUTS["nt"], tile_n=tile_n,
                           num_sms=num_sms, flags=L.SK_FLAG_BF16 if dtype == torch.bfloat16 else 0)
        dst = (C.c_void_p * G)(*[recv[j, g].data_ptr() for j in range(G)])
        st = lib.sk_gemm_f16_scatter(C.byref(prob), Ag.data_ptr(), Bg.data_ptr(), dst, G, ws.buf.data_ptr(),
                                     ws.nbytes, _ops._stream_ptr(DEV))
        assert st == 0, lib.sk_status_string(st)
    sk.check_status()
    assert not bool(torch.isnan(recv).any())          # every element of every slot was written
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    for j in range(G):
        blk = torch.empty(M, Nb, dtype=dtype, device=DEV)
        st = lib.sk_reduce_partials(recv[j].data_ptr(), G, M, Nb, blk.data_ptr(), Nb,
                                    L.SK_FLAG_BF16 if dtype == torch.bfloat16 else 0, _ops._stream_ptr(DEV))
        assert st == 0
        out[:, j * Nb:(j + 1) * Nb] = blk
    torch.cuda.synchronize()
    return out, recv


@pytest.mark.parametrize("shape,G,tile_n", [((256, 512, 512), 2, 256), ((300, 512, 1056), 4, 128),
                                            ((520, 768, 776), 2, 96), ((1000, 2048, 2048), 8, 256),
                                            ((64, 256, 264), 8, 32)])
def test_scatter_matches_the_full_product(shape, G, tile_n):
    M, N, K = shape
    K = K // (8 * G) * (8 * G)                   # K shards of a multiple of 8
    g = torch.Generator().manual_seed(M + N)
    A = torch.randn(M, K, generator=g).half()
    B = (torch.randn(N, K, generator=g) / K ** 0.5).half()
    ref = oracle.gemm_ref(A, B, "nt")
    out, recv = _scatter_on_one_gpu(A.to(DEV), B.to(DEV), G, tile_n)
    assert oracle.rel_err(out, ref) <= 1e-2
    # the slots hold the exact fp32 partial sums: their total is within fp32 rounding of the oracle
    total = recv.sum(dim=1).permute(1, 0, 2).reshape(M, N).cpu()
    assert float((total - ref).abs().max()) <= 2e-3 * float(ref.abs().max())
    out2, _ = _scatter_on_one_gpu(A.to(DEV), B.to(DEV), G, tile_n, num_sms=6)
    assert torch.equal(out, out2)                 # fixed-order reduction: same bits, whatever the grid


def test_scatter_bf16_and_argument_checks():
    g = torch.Generator().manual_seed(3)
    A = torch.randn(256, 512, generator=g).bfloat16()
    B = (torch.randn(512, 512, generator=g) / 22).bfloat16()
    out, _ = _scatter_on_one_gpu(A.to(DEV), B.to(DEV), 2, 256, dtype=torch.bfloat16)
    assert oracle.rel_err(out, oracle.gemm_ref(A, B, "nt")) <= 1e-2
    lib = L.load()
    ws = _ops._workspace(DEV)
    Ad, Bd = A.to(DEV), B.to(DEV)
    slot = torch.zeros(2, 256, 256, dtype=torch.float32, device=DEV)
    dst = (C.c_void_p * 2)(slot[0].data_ptr(), slot[1].data_ptr())
    call = lambda **kw: lib.sk_gemm_f16_scatter(
        C.byref(L.SkProblem(**dict(dict(M=256, N=512, K=512, lda=512, ldb=512, ldc=512, layout=1), **kw))),
        Ad.data_ptr(), Bd.data_ptr(), dst, 2, ws.buf.data_ptr(), ws.nbytes, _ops._stream_ptr(DEV))
    assert call(tile_n=192) == L.SK_ERR_SHAPE        # 256-column blocks are not whole 192-wide tiles
    assert call(layout=0) == L.SK_ERR_SHAPE          # NN has no CTA-pair kernel
    assert call(tile_m=128) == L.SK_ERR_ARG
    assert lib.sk_gemm_f16_scatter(C.byref(L.SkProblem(M=256, N=512, K=512, lda=512, ldb=512, layout=1)),
                                   Ad.data_ptr(), Bd.data_ptr(), dst, 9, ws.buf.data_ptr(), ws.nbytes,
                                   _ops._stream_ptr(DEV)) == L.SK_ERR_ARG
    torch.cuda.synchronize()


# ----------------------------------------------------------------------------- two or more GPUs
def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str):
    import datetime
    import traceback
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        M, N, K = 768, 512 * world, 512 * world
        g = torch.Generator().manual_seed(99)
        A = torch.randn(M, K, generator=g).half()
        B = (torch.randn(N, K, generator=g) / K ** 0.5).half()
        ref = oracle.gemm_ref(A, B, "nt")
        Kg, Nb = K // world, N // world
        Ad = A[:, rank * Kg:(rank + 1) * Kg].contiguous().to(dev)
        Bd = B[:, rank * Kg:(rank + 1) * Kg].contiguous().to(dev)
        failure = ""
        with sk.ScatteredResult(M, N) as res:
            first = None
            for it in range(3):
                try:
                    blk = sk.streamk_fp16_nt_reduce_scatter(Ad, Bd, res)
                    torch.cuda.synchronize(dev)
                    sk.check_status(dev)
                    want = ref[:, rank * Nb:(rank + 1) * Nb]
                    err = float((blk.float().cpu() - want).abs().max()) / float(ref.abs().max())
                    assert err <= 1e-2, (rank, it, err)
                    if first is None:
                        first = blk.clone()
                    assert torch.equal(blk, first)          # bitwise reproducible
                except Exception:
                    failure = traceback.format_exc()
                if not res.all_agree(not failure):
                    break
        open(os.path.join(out_dir, ("fail" if failure else "ok") + str(rank)), "w").write(failure or "ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_reduce_scatter_across_gpus(tmp_path):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 8)
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    fails = [open(tmp_path / f"fail{r}").read() for r in range(world) if os.path.exists(tmp_path / f"fail{r}")]
    assert not fails, "\n".join(fails)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))
