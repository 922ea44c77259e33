"""Python operator surface: the reference's entry points, backed by the C ABI.

The reference (LeiWang1999/Stream-k.tvm) has no importable API; each script
builds `tl_matmul_streamk(...)` and calls `tl_mod(A, B, C)` on CUDA tensors
(streamk_fp32.py:57-202, streamk_fp16.py:116-387, streamk_fp16_ladder.py,
streamk_fp16_ladder_block_reduce_q4.py).  The functions here keep those names
and argument meanings (A [M,K]; B [K,N] for NN, [N,K] for NT; C [M,N]) but
return a fresh C instead of accumulating into a pre-zeroed one.

Everything runs on the GPU through libstreamk_b200.so; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib as L

__all__ = [
    "streamk_fp32", "streamk_fp16_nn", "streamk_fp16_nt", "streamk_fp16_nt_host", "streamk_fp16_atomic",
    "streamk_fp16_block_reduce", "ladder_prepack", "streamk_fp16_ladder",
    "streamk_fp16_ladder_block_reduce", "q4_prepack", "dequant_w4",
    "streamk_fp16_ladder_block_reduce_q4", "schedule_info", "check_status",
    "SCHEDULE_NAMES", "reset_workspace", "release_cached_memory", "cached_memory_bytes", "device_info", "LadderWeight", "PackedQ4", "StreamKError", "SCHEDULES", "FIXUPS",
]

StreamKError = L.StreamKError
SCHEDULES = L.SCHEDULES   # name -> SK_SCHED_* value
FIXUPS = L.FIXUPS
SCHEDULE_NAMES = {v: k for k, v in L.SCHEDULES.items()}   # SK_SCHED_* value -> name
GROUP_SIZE = 128


# --------------------------------------------------------------------------- state
class _Workspace:
    __slots__ = ("buf", "nbytes", "status_host")

    def __init__(self, device: torch.device, stream_ptr: int):
        lib = L.load()
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.nbytes = int(lib.sk_workspace_bytes(sms))
        self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        L.check(lib.sk_workspace_init(self.buf.data_ptr(), self.nbytes, stream_ptr),
                "sk_workspace_init")


# Device memory this module keeps between calls: one workspace (sk_workspace_bytes, about
# 57 MB on 148 SMs) per (device, stream) that ever launched a GEMM, and the staging buffers of
# streamk_fp16_nt_host per (device, shape, slab).  cached_memory_bytes() reports them,
# release_cached_memory() drops them.
_workspaces: dict[tuple[int, int], _Workspace] = {}


def _stream_ptr(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def _workspace(device: torch.device) -> _Workspace:
    """One workspace per (device, stream): launches that may overlap never share one."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           _stream_ptr(device))
    ws = _workspaces.get(key)
    if ws is None:
        with torch.cuda.device(device):
            ws = _Workspace(device, key[1])
        _workspaces[key] = ws
    return ws


def reset_workspace(device=None) -> None:
    """Re-zero the workspace of the current stream (needed after a device-reported error)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ws = _workspace(device)
    with torch.cuda.device(device):
        L.check(L.load().sk_workspace_init(ws.buf.data_ptr(), ws.nbytes, _stream_ptr(device)),
                "sk_workspace_init")


def cached_memory_bytes() -> int:
    """Device bytes held by the cached workspaces and host-pipeline staging buffers."""
    n = sum(ws.nbytes for ws in _workspaces.values())
    for pipe in _host_pipes.values():
        n += pipe.nbytes
    return n


def release_cached_memory() -> None:
    """Drop every cached workspace and staging buffer (all devices).  Synchronises the devices
    first, so nothing in flight still uses them; the next call allocates afresh."""
    for dev in {k[0] for k in _workspaces} | {k[0] for k in _host_pipes}:
        torch.cuda.synchronize(dev)
    _workspaces.clear()
    _host_pipes.clear()


def check_status(device=None) -> None:
    """Synchronise the current stream and raise if a kernel reported a timeout."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ws = _workspace(device)
    lib = L.load()
    with torch.cuda.device(device):
        st = C.cast(ws.status_host.data_ptr(), C.POINTER(L.SkStatus))
        L.check(lib.sk_poll_status(ws.buf.data_ptr(), st, _stream_ptr(device)), "sk_poll_status")
        torch.cuda.current_stream(device).synchronize()
    code, cta, d0, d1 = (int(x) & 0xFFFFFFFF for x in ws.status_host.tolist())
    if code != L.SK_OK:
        reset_workspace(device)
        raise StreamKError(code, "device status", f"[cta {cta}, detail {d0}, {d1}]")


def device_info(device: int = 0) -> dict:
    info = L.SkDeviceInfo()
    st = L.load().sk_query(device, C.byref(info))
    d = {n: getattr(info, n) for n, _ in info._fields_}
    d["status"] = st
    return d


# --------------------------------------------------------------------------- helpers
_OPTION_KEYS = ("tile_m", "tile_n", "num_sms", "group_m", "out", "timeout_us", "pdl", "no_table",
                "_drop_flag_cta", "_bf16")


def _options(kw: dict) -> dict:
    """Common keyword arguments of every GEMM entry point:
    tile_m / tile_n  tile extents (None = choose; tile_m < 128 puts the weights on the UMMA
                     M dimension, the short-M form), num_sms (grid bound), group_m (tile
                     rasterisation), out (result buffer), timeout_us (bound of every device
                     wait), pdl (True: programmatic dependent launch, the kernel's start-up may
                     overlap the tail of the previous kernel of the stream; fp16 / W4A16),
                     no_table (True: schedule "auto" by the built-in rules only, ignoring the table
                     of tuned shapes),
                     _drop_flag_cta (test hook: index of a CTA that withholds its flag)."""
    unknown = set(kw) - set(_OPTION_KEYS)
    if unknown:
        raise TypeError(f"unexpected keyword argument(s): {sorted(unknown)}")
    return {k: kw.get(k) for k in _OPTION_KEYS}


def _problem(M, N, K, lda, ldb, ldc, layout, schedule, fixup, o: dict) -> L.SkProblem:
    if schedule not in L.SCHEDULES:
        raise ValueError(f"schedule must be one of {sorted(L.SCHEDULES)}, got {schedule!r}")
    if fixup not in L.FIXUPS:
        raise ValueError(f"fixup must be one of {sorted(L.FIXUPS)}, got {fixup!r}")
    return L.SkProblem(M=M, N=N, K=K, lda=lda, ldb=ldb, ldc=ldc, layout=L.LAYOUTS[layout],
                       schedule=L.SCHEDULES[schedule], fixup=L.FIXUPS[fixup],
                       tile_m=int(o["tile_m"] or 0), tile_n=int(o["tile_n"] or 0),
                       num_sms=int(o["num_sms"] or 0), group_m=int(o["group_m"] or 0),
                       fixup_timeout_us=int(o["timeout_us"] or 0),
                       # (the C field is 0 = off, n = CTA n - 1)
                       test_drop_flag_cta=0 if o["_drop_flag_cta"] is None else int(o["_drop_flag_cta"]) + 1,
                       flags=(L.SK_FLAG_PDL if o["pdl"] else 0) | (L.SK_FLAG_NO_TABLE if o["no_table"] else 0)
                             | (L.SK_FLAG_BF16 if o["_bf16"] else 0))


def schedule_info(M: int, N: int, K: int, *, kind: str = "f16", schedule: str = "auto",
                  num_sms: int = 148, gather_peers: int = 0, **kw) -> dict:
    """Host scheduler integers (streamk_fp16.py:83-113) and the tile plan for a problem;
    needs no GPU.  kind: "f32", "f16" (what the fp16 NT entry point runs: single-CTA tiles, or
    for large problems the CTA-pair kernel, described over num_sms / 2 pairs), "w4a16", or
    "f16_pairs" (the CTA-pair kernel with num_sms pairs).  gather_peers > 0: the plan of the
    fused all-gather call with that many peers."""
    o = _options(kw)
    prob = _problem(M, N, K, K, K, N, "nt", schedule, "atomic", o)
    info = L.SkScheduleInfo()
    kinds = {"f32": 0, "f16": 1, "w4a16": 2, "f16_pairs": 3}
    if gather_peers:
        L.check(L.load().sk_schedule_gather(C.byref(prob), gather_peers, num_sms, C.byref(info)),
                "sk_schedule_gather")
    else:
        L.check(L.load().sk_schedule(C.byref(prob), kinds[kind], num_sms, C.byref(info)), "sk_schedule")
    return info.as_dict()


HALF_TYPES = (torch.float16, torch.bfloat16)


def _check_matrix(name: str, t: torch.Tensor, dtype) -> None:
    """dtype: one torch dtype, or a tuple of acceptable ones."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    ok = t.dtype in dtype if isinstance(dtype, tuple) else t.dtype == dtype
    if not ok:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if t.dim() != 2:
        raise ValueError(f"{name} must be 2-D, got shape {tuple(t.shape)}")


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    # The reference asserts contiguity (triton_impl.py:199-201); row-major views
    # with a padded leading dimension are accepted here as well.
    if t.stride(1) == 1 and t.stride(0) >= t.shape[1]:
        return t
    return t.contiguous()


def _out(out, M, N, dtype, device):
    if out is None:
        return torch.empty((M, N), dtype=dtype, device=device)
    if out.shape != (M, N) or out.dtype != dtype or out.device != device or out.stride(1) != 1:
        raise ValueError("out must be a row-major [M,N] tensor of the result dtype on A's device")
    return out


def _pad_k8(t: torch.Tensor, k_dim: int) -> torch.Tensor:
    """TMA needs 16-byte row pitches: pad the K extent of an fp16 operand to a multiple of 8."""
    k = t.shape[k_dim]
    pad = (-k) % 8
    if pad == 0:
        return t
    spec = (0, pad) if k_dim == 1 else (0, 0, 0, pad)
    return torch.nn.functional.pad(t, spec)


def _aligned16(t: torch.Tensor) -> torch.Tensor:
    if t.data_ptr() % 16 == 0 and t.stride(0) % 8 == 0:
        return t
    n = torch.empty((t.shape[0], (t.shape[1] + 7) // 8 * 8), dtype=t.dtype, device=t.device)
    n[:, : t.shape[1]].copy_(t)
    return n[:, : t.shape[1]]


# --------------------------------------------------------------------------- fp32
def streamk_fp32(A: torch.Tensor, B: torch.Tensor, *, fixup: str = "atomic",
                 schedule: str = "auto", trans_b: bool = False, **kw) -> torch.Tensor:
    """C = A @ B in fp32 (FFMA, no TF32).  A [M,K]; B [K,N] (or [N,K] with trans_b).

    Mirrors `tl_matmul_streamk(..., "float32", "float32", "float32", ...)` of
    streamk_fp32.py:57-202.  `schedule="hybrid"` is the reference's split.
    """
    o = _options(kw)
    _check_matrix("A", A, torch.float32)
    _check_matrix("B", B, torch.float32)
    A = _rowmajor(A)
    B = _rowmajor(B)
    M, K = A.shape
    if trans_b:
        N, Kb = B.shape
    else:
        Kb, N = B.shape
    if K != Kb:
        raise ValueError(f"Incompatible dimensions: A {tuple(A.shape)} B {tuple(B.shape)}")
    Cout = _out(o["out"], M, N, torch.float32, A.device)
    prob = _problem(M, N, K, A.stride(0), B.stride(0), Cout.stride(0), "nt" if trans_b else "nn",
                    schedule, fixup, o)
    with torch.cuda.device(A.device):
        ws = _workspace(A.device)
        L.check(L.load().sk_gemm_f32(C.byref(prob), A.data_ptr(), B.data_ptr(), Cout.data_ptr(),
                                     ws.buf.data_ptr(), ws.nbytes, _stream_ptr(A.device)),
                "sk_gemm_f32")
    return Cout


# --------------------------------------------------------------------------- fp16
def _gemm_f16(A, B, layout, fixup, schedule, kw):
    """fp16 operands, or bfloat16 ones (both operands alike; the result has their type)."""
    o = _options(kw)
    _check_matrix("A", A, HALF_TYPES)
    dtype = A.dtype
    o["_bf16"] = dtype == torch.bfloat16
    M, K = A.shape
    if layout == "ladder":
        if not isinstance(B, LadderWeight):
            raise TypeError("B must come from ladder_prepack()")
        if B.K != K:
            raise ValueError(f"Incompatible dimensions: A {tuple(A.shape)} weight K={B.K}")
        if B.dtype != dtype:
            raise TypeError(f"A is {dtype} but the weight image was packed from {B.dtype}")
        N = B.N
        Bt, ldb = B.data, 0
        A = _aligned16(_rowmajor(_pad_k8(A, 1)))
    else:
        _check_matrix("B", B, dtype)
        if layout == "nt":
            N, Kb = B.shape
        else:
            Kb, N = B.shape
        if K != Kb:
            raise ValueError(f"Incompatible dimensions: A {tuple(A.shape)} B {tuple(B.shape)}")
        A = _aligned16(_rowmajor(_pad_k8(A, 1)))
        if layout == "nt":
            Bt = _aligned16(_rowmajor(_pad_k8(B, 1)))
        else:
            # NN: rows of B are K; the N pitch must be a multiple of 8 halves
            Bt = _aligned16(_rowmajor(_pad_k8(B, 0)))
        ldb = Bt.stride(0)
    Cout = _out(o["out"], M, N, dtype, A.device)
    prob = _problem(M, N, A.shape[1], A.stride(0), ldb, Cout.stride(0), layout, schedule, fixup, o)
    with torch.cuda.device(A.device):
        ws = _workspace(A.device)
        L.check(L.load().sk_gemm_f16(C.byref(prob), A.data_ptr(), Bt.data_ptr(), Cout.data_ptr(),
                                     ws.buf.data_ptr(), ws.nbytes, _stream_ptr(A.device)),
                "sk_gemm_f16")
    return Cout


def streamk_fp16_nt(A, B, *, fixup="block_reduce", schedule="auto", **kw):
    """C = A @ B.T, fp16 in, fp32 accumulate, fp16 out.  A [M,K], B [N,K].
    (bfloat16 tensors are accepted as well, here and in the NN and ladder forms: same kernels,
    bf16 operands, fp32 accumulation, bf16 result; the reference is fp16 only.)

    Mirrors `tl_matmul_streamk(M, N, K, streamk_tiles, "float16", "float16", ...)` +
    `tl_mod(A, B, C)` of streamk_fp16.py:116-387 and streamk_fp16_nt.py:57-192.
    schedule: "auto" (the library picks by shape), "hybrid" (the reference's split),
    "hybrid_dp_first", "streamk", "dp".  fixup: "block_reduce" (deterministic) or "atomic".
    Keyword options: see _options().
    """
    return _gemm_f16(A, B, "nt", fixup, schedule, kw)


class _HostPipe:
    """Device staging buffers, streams and events of streamk_fp16_nt_host for one shape."""

    def __init__(self, M, N, K, slab, device):
        self.key = (M, N, K, slab)
        self.A = torch.empty(M, K, dtype=torch.float16, device=device)
        self.B = [torch.empty(slab, K, dtype=torch.float16, device=device) for _ in range(2)]
        self.C = [torch.empty(M, slab, dtype=torch.float16, device=device) for _ in range(2)]
        self.s_in, self.s_mm, self.s_out = (torch.cuda.Stream(device) for _ in range(3))
        self.nbytes = 2 * (M * K + 2 * slab * K + 2 * M * slab)
        self.busy = None     # event recorded at the end of the last call that used these buffers


_host_pipes: dict[tuple, _HostPipe] = {}
_HOST_PIPES_MAX = 4     # staging sets kept; the least recently used one is dropped beyond that


def streamk_fp16_nt_host(A_host, B_host, out_host=None, *, slabs: int = 8, device=None,
                         fixup="block_reduce", schedule="auto", group=None, **kw):
    """C = A @ B.T for operands and result in (pinned) HOST memory: A [M,K], B [N,K] fp16 CPU
    tensors, result [M,N] fp16 CPU tensor (out_host, or a new pinned tensor).

    Column-sharded use (one process per GPU, `group` = a torch.distributed NCCL group of G
    ranks, B_host / out_host = this rank's column block): A_host is then only this rank's
    1/G of A's rows, [M/G, K]; every rank copies its part from the host and the parts are
    all-gathered into each GPU's memory over NVLink (NCCL, ahead of the first slab's GEMM), so
    that A crosses PCIe once for the whole group instead of once per GPU.

    B and C move in `slabs` column slabs through double-buffered device staging: the
    host-to-device copy of slab i+1, the GEMM of slab i and the device-to-host copy of slab i-1
    run on three streams at once, so a step costs about the larger of the two PCIe directions
    instead of their sum plus the GEMM.  The calling stream waits for the result; the host has
    to synchronise that stream (or the device) before reading out_host.  Each slab is one call of
    streamk_fp16_nt (same keyword options)."""
    for name, t in (("A_host", A_host), ("B_host", B_host)):
        if not isinstance(t, torch.Tensor) or t.is_cuda or t.dtype != torch.float16 or t.dim() != 2:
            raise TypeError(f"{name} must be a 2-D fp16 CPU tensor")
    Mpart, K = A_host.shape
    world = 1
    if group is not None:
        import torch.distributed as dist
        world = dist.get_world_size(group)
    M = Mpart * world
    N = B_host.shape[0]
    if B_host.shape[1] != K:
        raise ValueError("A_host [M,K] and B_host [N,K] disagree on K")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    slabs = max(1, min(int(slabs), N))
    slab = -(-N // slabs)
    slab = (slab + 15) // 16 * 16          # whole 16-column groups: aligned rows in the staging tiles
    slabs = -(-N // slab)
    if out_host is None:
        out_host = torch.empty(M, N, dtype=torch.float16).pin_memory()
    if out_host.shape != (M, N) or out_host.dtype != torch.float16 or out_host.is_cuda or out_host.stride(1) != 1:
        raise ValueError("out_host must be a row-major fp16 CPU tensor of shape [M, N]")
    if not (A_host.is_contiguous() and B_host.is_contiguous()):
        raise ValueError("A_host and B_host must be contiguous")
    key = (device.index, M, N, K, slab)
    pipe = _host_pipes.pop(key, None)
    if pipe is None:
        while len(_host_pipes) >= _HOST_PIPES_MAX:
            old = _host_pipes.pop(next(iter(_host_pipes)))
            if old.busy is not None:
                old.busy.synchronize()      # its last call may still be running
        pipe = _HostPipe(M, N, K, slab, device)
    _host_pipes[key] = pipe                 # (most recently used last)
    cur = torch.cuda.current_stream(device)
    for st in (pipe.s_in, pipe.s_mm, pipe.s_out):
        st.wait_stream(cur)
        # The staging buffers are free again only when the previous call that used them has
        # finished, whichever stream that call was made from.
        if pipe.busy is not None:
            st.wait_event(pipe.busy)
    with torch.cuda.stream(pipe.s_in):
        if world == 1:
            pipe.A.copy_(A_host, non_blocking=True)
        else:
            rank = dist.get_rank(group)
            pipe.A[rank * Mpart:(rank + 1) * Mpart].copy_(A_host, non_blocking=True)
            # row blocks are contiguous: the gather lands in place (NCCL kernel on the copy-in
            # stream; no peer pointer is handed to a GEMM kernel as an operand)
            dist.all_gather_into_tensor(pipe.A, pipe.A[rank * Mpart:(rank + 1) * Mpart], group=group)
    mm_done = [None, None]                  # per staging buffer: GEMM that last read B / wrote C
    out_done = [None, None]                 # per staging buffer: copy-out that last read C
    for i in range(slabs):
        b = i & 1
        n0, n1 = i * slab, min(N, (i + 1) * slab)
        w = n1 - n0
        with torch.cuda.stream(pipe.s_in):
            if mm_done[b] is not None:
                pipe.s_in.wait_event(mm_done[b])
            pipe.B[b][:w].copy_(B_host[n0:n1], non_blocking=True)
            loaded = torch.cuda.Event()
            loaded.record(pipe.s_in)
        with torch.cuda.stream(pipe.s_mm):
            pipe.s_mm.wait_event(loaded)
            if out_done[b] is not None:
                pipe.s_mm.wait_event(out_done[b])
            Cb = pipe.C[b] if w == slab else pipe.C[b][:, :w]
            _gemm_f16(pipe.A, pipe.B[b][:w], "nt", fixup, schedule, dict(kw, out=Cb))
            mm_done[b] = torch.cuda.Event()
            mm_done[b].record(pipe.s_mm)
        with torch.cuda.stream(pipe.s_out):
            pipe.s_out.wait_event(mm_done[b])
            # a pitched DMA straight into the column slab of the row-major host matrix (a strided
            # Tensor.copy_ would go through a staging buffer and a CPU-side scatter)
            L.check(L.load().sk_memcpy2d_async(
                out_host.data_ptr() + n0 * 2, out_host.stride(0) * 2, Cb.data_ptr(), Cb.stride(0) * 2,
                w * 2, M, int(pipe.s_out.cuda_stream)), "sk_memcpy2d_async")
            out_done[b] = torch.cuda.Event()
            out_done[b].record(pipe.s_out)
    cur.wait_stream(pipe.s_out)
    cur.wait_stream(pipe.s_mm)
    cur.wait_stream(pipe.s_in)
    pipe.busy = torch.cuda.Event()
    pipe.busy.record(cur)
    return out_host


def streamk_fp16_nn(A, B, *, fixup="block_reduce", schedule="auto", **kw):
    """C = A @ B, fp16.  A [M,K], B [K,N]  (streamk_fp16_nn.py:57-177)."""
    return _gemm_f16(A, B, "nn", fixup, schedule, kw)


def streamk_fp16_atomic(A, B, **kw):
    """NT GEMM with the order-nondeterministic fp32 red.global.add fixup
    (the role of T.atomic_addx2 in streamk_fp16.py:248-255)."""
    return streamk_fp16_nt(A, B, fixup="atomic", **kw)


def streamk_fp16_block_reduce(A, B, **kw):
    """NT GEMM with the deterministic flag-synchronised fixup.  Keeps the entry name of
    streamk_fp16_block_reduce.py; the intra-CTA split-K it performs there is subsumed by
    TMEM accumulation, the name now denotes the bitwise-reproducible cross-CTA reduction."""
    return streamk_fp16_nt(A, B, fixup="block_reduce", **kw)


@dataclass
class LadderWeight:
    """Weight pre-laid-out by ladder_prepack (opaque image + logical shape)."""
    data: torch.Tensor
    N: int
    K: int
    dtype: torch.dtype = torch.float16


def ladder_prepack(B: torch.Tensor) -> LadderWeight:
    """Re-lay B [N,K] fp16 into the streaming image of the ladder mainloop.

    Replaces `bitblas.ops.LadderPermutate(...)(B.cpu())` (streamk_fp16_ladder.py:468-477);
    runs on the GPU."""
    _check_matrix("B", B, HALF_TYPES)
    B = _rowmajor(B)
    N, K = B.shape
    lib = L.load()
    nbytes = int(lib.sk_ladder_bytes(N, K))
    out = torch.empty(nbytes, dtype=torch.uint8, device=B.device)
    with torch.cuda.device(B.device):
        L.check(lib.sk_prepack_ladder(B.data_ptr(), N, K, B.stride(0), out.data_ptr(), nbytes,
                                      _stream_ptr(B.device)), "sk_prepack_ladder")
    return LadderWeight(out, N, K, B.dtype)


def streamk_fp16_ladder(A, LB: LadderWeight, *, fixup="block_reduce", schedule="auto", **kw):
    """C = A @ W.T with W pre-laid-out (streamk_fp16_ladder.py:137-486)."""
    return _gemm_f16(A, LB, "ladder", fixup, schedule, kw)


def streamk_fp16_ladder_block_reduce(A, LB: LadderWeight, **kw):
    """Ladder path with the deterministic fixup (streamk_fp16_ladder_block_reduce.py)."""
    return streamk_fp16_ladder(A, LB, fixup="block_reduce", **kw)


# --------------------------------------------------------------------------- W4A16
@dataclass
class PackedQ4:
    """uint4 weight + group scales/zeros packed by q4_prepack (opaque image + shape)."""
    data: torch.Tensor
    N: int
    K: int
    group_size: int = GROUP_SIZE     # 32, 64, 128, or 0 = one group per weight row (per-channel)
    signed: bool = False


def q4_prepack(qweight: torch.Tensor, scales: torch.Tensor | None = None,
               zeros: torch.Tensor | None = None, group_size: int = GROUP_SIZE,
               signed: bool = False) -> PackedQ4:
    """Pack 4-bit weights for the W4A16 mainloop.

    qweight: int32 [N, K/8] (nibble j of word w = element 8w+j) or int8/uint8 [N, K/2]
    (low nibble = even k, the reference's storage, …_q4.py:28-30,545-554).
    scales: fp16 [N, K/group_size] or None (=1).  zeros: uint8 [N, K/group_size] in 0..15 or None
    (=0).  With scales=None, zeros=None the GEMM reproduces the reference's `A @ unpack(qB).T`.
    group_size: 128 (the benchmark's), 64, 32, or 0 / K for per-channel scales ([N, 1]).
    signed: the nibbles are two's-complement int4 (-8..7), W = q * s (no zero-points).
    Replaces LadderPermutate + LOP3Permutate on the CPU (…_q4.py:568-595); formats beyond plain
    uint4 have no counterpart in the reference.
    """
    if not qweight.is_cuda:
        raise ValueError("qweight must be a CUDA tensor (this library has no CPU path)")
    if qweight.dtype in (torch.int8, torch.uint8):
        N, Kh = qweight.shape
        K = Kh * 2
    elif qweight.dtype == torch.int32:
        N, Kw = qweight.shape
        K = Kw * 8
    else:
        raise TypeError("qweight must be int32 [N,K/8] or int8/uint8 [N,K/2]")
    if K % GROUP_SIZE:
        raise ValueError("K must be a multiple of 128")
    if group_size == K and K > 128:
        group_size = 0
    if group_size not in (0, 32, 64, 128):
        raise ValueError("group_size must be 32, 64, 128, or 0 / K (per-channel)")
    if signed and zeros is not None:
        raise ValueError("signed int4 is symmetric (W = q * s): zeros must be None")
    qweight = qweight.contiguous()
    G = K // group_size if group_size else 1
    sp = zp = None
    if scales is not None:
        if scales.shape != (N, G) or scales.dtype != torch.float16:
            raise ValueError(f"scales must be fp16 [{N},{G}]")
        scales = scales.contiguous(); sp = scales.data_ptr()
    if zeros is not None:
        if zeros.shape != (N, G) or zeros.dtype != torch.uint8:
            raise ValueError(f"zeros must be uint8 [{N},{G}]")
        zeros = zeros.contiguous(); zp = zeros.data_ptr()
    lib = L.load()
    nbytes = int(lib.sk_q4_bytes_ex(N, K, group_size))
    out = torch.empty(nbytes, dtype=torch.uint8, device=qweight.device)
    with torch.cuda.device(qweight.device):
        L.check(lib.sk_prepack_q4_ex(qweight.data_ptr(), sp, zp, N, K, group_size, 1 if signed else 0,
                                     out.data_ptr(), nbytes, _stream_ptr(qweight.device)), "sk_prepack_q4_ex")
    return PackedQ4(out, N, K, group_size, bool(signed))


def dequant_w4(QLB: PackedQ4) -> torch.Tensor:
    """W [N,K] fp16 = (q - z) * s, bit-exact with the fp16 expression evaluated on the CPU."""
    W = torch.empty((QLB.N, QLB.K), dtype=torch.float16, device=QLB.data.device)
    with torch.cuda.device(W.device):
        L.check(L.load().sk_dequant_q4_ex(QLB.data.data_ptr(), QLB.N, QLB.K, QLB.group_size, W.data_ptr(),
                                          W.stride(0), _stream_ptr(W.device)), "sk_dequant_q4_ex")
    return W


def streamk_fp16_ladder_block_reduce_q4(A, QLB: PackedQ4, *, fixup="block_reduce",
                                        schedule="auto", **kw):
    """W4A16: C = A @ ((q - z) * s).T, fp16 activations, uint4 weights.

    Mirrors `tl_mod(A, QLB, C)` of streamk_fp16_ladder_block_reduce_q4.py:143-599."""
    o = _options(kw)
    _check_matrix("A", A, torch.float16)
    if not isinstance(QLB, PackedQ4):
        raise TypeError("QLB must come from q4_prepack()")
    M, K = A.shape
    if K != QLB.K:
        raise ValueError(f"Incompatible dimensions: A {tuple(A.shape)} weight K={QLB.K}")
    A = _aligned16(_rowmajor(A))
    Cout = _out(o["out"], M, QLB.N, torch.float16, A.device)
    prob = _problem(M, QLB.N, K, A.stride(0), 0, Cout.stride(0), "nt", schedule, fixup, o)
    prob.flags |= L.SK_FLAG_Q4_GROUP[QLB.group_size]
    with torch.cuda.device(A.device):
        ws = _workspace(A.device)
        L.check(L.load().sk_gemm_w4a16(C.byref(prob), A.data_ptr(), QLB.data.data_ptr(),
                                       Cout.data_ptr(), ws.buf.data_ptr(), ws.nbytes,
                                       _stream_ptr(A.device)), "sk_gemm_w4a16")
    return Cout
