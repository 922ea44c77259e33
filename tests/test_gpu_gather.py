"""sk_gemm_f16_gather: the GEMM whose epilogue also writes every tile into peer matrices.

On one GPU the "peers" are further matrices of the same GPU, handed to the C ABI as plain
pointers: that exercises every store path of the kernel (TMA stores of whole tiles, the
register path of ragged tiles, both fixups' final writers, the 256 x 512 units).  With two or
more GPUs the real thing runs as one process per GPU: CUDA IPC mapped matrices, peer stores
over NVLink, checked against the CPU oracle and against the unfused product.
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


def _call_gather(A, B, full, peers_full, col0, schedule, fixup, tile_m=256, tile_n=0, num_sms=0):
    """C ABI call: this GPU's block goes to columns col0.. of `full` and of every matrix in
    peers_full (all [M, n_total], same pitch)."""
    lib = L.load()
    M, K = A.shape
    N = B.shape[0]
    prob = L.SkProblem(M=M, N=N, K=K, lda=A.stride(0), ldb=B.stride(0), ldc=full.stride(0),
                       layout=L.LAYOUTS["nt"], schedule=L.SCHEDULES[schedule], fixup=L.FIXUPS[fixup],
                       tile_m=tile_m, tile_n=tile_n, num_sms=num_sms)
    ptrs = (C.c_void_p * max(1, len(peers_full)))(*[p[:, col0:].data_ptr() for p in peers_full])
    ws = _ops._workspace(DEV)
    st = lib.sk_gemm_f16_gather(C.byref(prob), A.data_ptr(), B.data_ptr(), full[:, col0:].data_ptr(), ptrs,
                                len(peers_full), ws.buf.data_ptr(), ws.nbytes, _ops._stream_ptr(DEV))
    return st


@pytest.mark.parametrize("shape", [(256, 512, 256), (300, 520, 1000), (512, 776, 328), (200, 2000, 264)])
def test_gather_writes_every_peer_like_the_plain_product(shape):
    M, N, K = shape
    g = torch.Generator().manual_seed(M * 7 + N)
    A = torch.randn(M, K, generator=g).half().to(DEV)
    B = (torch.randn(N, K, generator=g) / K ** 0.5).half().to(DEV)
    ref = oracle.gemm_ref(A.cpu(), B.cpu(), "nt")
    n_total, col0 = 2 * N + 64, N + 32          # the block sits in the middle of wider matrices
    for schedule in ("dp", "streamk", "hybrid"):
        for fixup in ("atomic", "block_reduce"):
            for tile_n in (0, 96):
                plain = sk.streamk_fp16_nt(A, B, tile_m=256, tile_n=tile_n or None, schedule=schedule,
                                           fixup=fixup)
                sk.check_status()
                assert oracle.rel_err(plain, ref) <= 1e-2
                mats = [torch.full((M, n_total), 7.0, dtype=torch.float16, device=DEV) for _ in range(4)]
                st = _call_gather(A, B, mats[0], mats[1:], col0, schedule, fixup, tile_n=tile_n)
                assert st == 0, L.load().sk_status_string(st)
                sk.check_status()
                for m in mats:
                    got = m[:, col0:col0 + N]
                    if fixup == "block_reduce":
                        assert torch.equal(got, plain)          # same summation order: same bits
                    else:
                        assert oracle.rel_err(got, ref) <= 1e-2
                    assert torch.equal(got, mats[0][:, col0:col0 + N])   # all copies identical
                    # nothing outside the block was touched
                    assert bool((m[:, :col0] == 7.0).all()) and bool((m[:, col0 + N:] == 7.0).all())


def test_gather_with_wide_units_and_seven_peers():
    """The library's own tiling of a large block.  Few peers and a deep K: the 256 x 512 units
    stay (the transfer hides under the mainloop).  Bytes to push worth 60 % of the mainloop or
    more: plain 256 x 256 tiles, so that the transfer starts earlier.  More than the whole
    mainloop: those tiles data-parallel, so that nothing is left for the end.  Either way every
    copy carries the bits of the unfused product with the same tiling."""
    g = torch.Generator(device=DEV).manual_seed(11)
    for K, n_peers, how in ((4096, 1, "units"), (2304, 1, "tiles"), (256, 7, "tiles_dp")):
        M, N = 1024, 10240
        A = torch.randn(M, K, generator=g, device=DEV).half()
        B = (torch.randn(N, K, generator=g, device=DEV) / K ** 0.5).half()
        info = sk.schedule_info(M, N, K, kind="f16_pairs", schedule="hybrid", num_sms=74)
        assert info["wide_units"] > 0
        info = sk.schedule_info(M, N, K, gather_peers=n_peers)
        assert (info["wide_units"] > 0) == (how == "units")
        assert sk.SCHEDULE_NAMES[info["schedule"]] == ("dp" if how == "tiles_dp" else "hybrid")
        if how == "units":
            plain = sk.streamk_fp16_nt(A, B, fixup="block_reduce")
        elif how == "tiles":
            plain = sk.streamk_fp16_nt(A, B, tile_m=256, schedule="hybrid", fixup="block_reduce")
        else:
            plain = sk.streamk_fp16_nt(A, B, tile_m=256, schedule="dp", fixup="block_reduce")
        ref = torch.matmul(A.float(), B.float().t())
        assert float((plain.float() - ref).abs().max()) <= 1e-2 * float(ref.abs().max())
        mats = [torch.zeros(M, N, dtype=torch.float16, device=DEV) for _ in range(n_peers + 1)]
        st = _call_gather(A, B, mats[0], mats[1:], 0, "auto", "block_reduce", tile_m=0)
        assert st == 0, L.load().sk_status_string(st)
        sk.check_status()
        for m in mats:
            assert torch.equal(m, plain)


def test_gather_argument_checks():
    A = torch.zeros(256, 256, dtype=torch.float16, device=DEV)
    B = torch.zeros(512, 256, dtype=torch.float16, device=DEV)
    full = torch.zeros(256, 1024, dtype=torch.float16, device=DEV)
    peer = torch.zeros(256, 1024, dtype=torch.float16, device=DEV)
    # a kernel other than the CTA-pair one cannot gather
    assert _call_gather(A, B, full, [peer], 0, "streamk", "atomic", tile_m=128, tile_n=128) == L.SK_ERR_SHAPE
    # peer blocks must take 16-byte stores
    assert _call_gather(A, B, full, [peer], 4, "dp", "atomic") == L.SK_ERR_ALIGN
    # more peers than the parameter block holds
    assert _call_gather(A, B, full, [peer] * 8, 0, "dp", "atomic") == L.SK_ERR_ARG
    # no peers: the plain product
    assert _call_gather(A, B, full, [], 0, "dp", "atomic") == 0
    torch.cuda.synchronize()


# ----------------------------------------------------------------------------- two or more GPUs
def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str):
    """One rank of the multi-GPU test.  A failed check on one rank must not strand the others
    in a collective: every iteration ends with an agreed verdict (all_agree), all ranks leave
    the loop together, and the process group has a short timeout as a last resort."""
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
        M, K, n_total = 512, 384, 1024 * world
        g = torch.Generator().manual_seed(77)
        A = torch.randn(M, K, generator=g).half()
        Bfull = (torch.randn(n_total, K, generator=g) / K ** 0.5).half()
        ref = oracle.gemm_ref(A, Bfull, "nt")
        col0, width = sk.column_block(rank, world, n_total)
        Ad, Bd = A.to(dev), Bfull[col0:col0 + width].to(dev)
        failure = ""
        with sk.GatheredResult(M, n_total) as res:
            for it, (schedule, fixup) in enumerate((("hybrid", "block_reduce"), ("streamk", "atomic"),
                                                    ("dp", "block_reduce"))):
                try:
                    res.full.fill_(float(it))          # stale contents the call must replace everywhere
                    out = sk.streamk_fp16_nt_gather(Ad, Bd, res, schedule=schedule, fixup=fixup)
                    torch.cuda.synchronize(dev)
                    mine = out.contiguous()
                except Exception:
                    failure = traceback.format_exc()
                    mine = torch.zeros(M, n_total, dtype=torch.float16, device=dev)
                # (the collectives below are reached by every rank whatever happened above)
                parts = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(parts, mine)
                if not failure:
                    try:
                        sk.check_status(dev)
                        assert oracle.rel_err(out.cpu(), ref) <= 1e-2, (rank, schedule, fixup)
                        own = sk.streamk_fp16_nt(Ad, Bd, tile_m=256, schedule=schedule, fixup=fixup)
                        if fixup == "block_reduce":
                            assert torch.equal(out[:, col0:col0 + width], own)
                        # every rank ends up with the same bits
                        assert all(torch.equal(p, mine) for p in parts)
                    except Exception:
                        failure = traceback.format_exc()
                if not res.all_agree(not failure):
                    break
        if failure:
            open(os.path.join(out_dir, f"fail{rank}"), "w").write(failure)
        else:
            open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_gather_across_gpus(tmp_path):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 8)
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    fails = [open(tmp_path / f"fail{r}").read() for r in range(world) if os.path.exists(tmp_path / f"fail{r}")]
    assert not fails, "\n".join(fails)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))
