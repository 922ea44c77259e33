"""Column-sharded product with the all-gather fused into the GEMM's epilogue.

The sharded configuration splits B[N, K] by rows over the GPUs of a process group (one
process per GPU); GPU g computes the column block C[:, g*N/G : (g+1)*N/G].  The plain way
to give every GPU the whole C is an NCCL all-gather after the GEMM.  Here every GPU holds
the full matrix in memory that its peers have mapped (CUDA IPC, `sk_peer_*` of the C ABI),
and the kernel's epilogue writes each finished tile into the local matrix and into every
peer's (`sk_gemm_f16_gather`), so the transfer runs under the mainloop, tile by tile.  No
kernel waits on another GPU; the ranks meet in two stream-ordered NCCL all-reduces of one
element, one before the kernel (nobody still reads the matrix that is about to be
overwritten) and one after it (every rank's stores have landed).

The reference is a single-GPU study and has no counterpart of this file.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib as L
from . import ops as _ops

__all__ = ["column_block", "peer_order", "GatheredResult", "streamk_fp16_nt_gather", "ScatteredResult",
           "streamk_fp16_nt_reduce_scatter"]

MAX_PEERS = 7   # SK_MAX_PEERS


def column_block(rank: int, world: int, n_total: int) -> tuple[int, int]:
    """(first column, width) of rank's block; blocks are equal and 16-byte aligned."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    if n_total % world != 0 or (n_total // world) % 8 != 0:
        raise ValueError(f"N = {n_total} does not split into {world} column blocks of a multiple of 8")
    w = n_total // world
    return rank * w, w


def peer_order(rank: int, world: int) -> list[int]:
    """The order in which a rank writes to its peers: rank+1, rank+2, ... (mod world), so that
    at any moment the ranks address different destinations."""
    return [(rank + i) % world for i in range(1, world)]


class _DeviceBytes:
    """A raw device allocation as something torch.as_tensor understands."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class _SharedAllocation:
    """One device allocation per rank, mapped into every process of `group` (CUDA IPC through
    the C ABI's sk_peer_*).  Collective: every rank constructs and closes it at the same point of
    the program; a failure on one rank raises on all of them."""

    def __init__(self, nbytes: int, what: str, group=None, device=None):
        if not dist.is_initialized():
            raise RuntimeError(f"{what} needs an initialised torch.distributed process group")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = (torch.device("cuda", torch.cuda.current_device()) if device is None
                       else torch.device(device))
        self.nbytes = int(nbytes)
        lib = L.load()
        self._own = C.c_void_p()
        self._peer_base = {}
        handle = C.create_string_buffer(64)
        with torch.cuda.device(self.device):
            # Every rank takes part in both exchanges whatever happened to it before, so that a
            # failure on one rank (no memory, no peer access) raises on all of them instead of
            # leaving the others waiting in a collective call.
            err = ""
            try:
                L.check(lib.sk_peer_alloc(self.nbytes, C.byref(self._own), handle), "sk_peer_alloc")
            except Exception as e:
                err = f"rank {self.rank}: {e}"
            said = [None] * self.world
            dist.all_gather_object(said, (err, handle.raw), group=group)
            if not any(e for e, _ in said):
                try:
                    for r in peer_order(self.rank, self.world):
                        p = C.c_void_p()
                        L.check(lib.sk_peer_open(said[r][1], C.byref(p)), "sk_peer_open")
                        self._peer_base[r] = p.value
                except Exception as e:
                    err = f"rank {self.rank}: {e}"
            errs = [None] * self.world
            dist.all_gather_object(errs, err or next((e for e, _ in said if e), ""), group=group)
            if any(errs):
                for p in self._peer_base.values():
                    lib.sk_peer_close(p)
                dist.barrier(group=group)      # mappings first, then the memory they map
                if self._own.value:
                    lib.sk_peer_free(self._own)
                raise RuntimeError(f"{what}: " + "; ".join(sorted({e for e in errs if e})))
            self.bytes = torch.as_tensor(_DeviceBytes(self._own.value, self.nbytes), device=self.device)
            if self.bytes.data_ptr() != self._own.value:
                raise RuntimeError("the tensor over the shared allocation is a copy, not a view")
            self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._open = True

    def base_of(self, r: int) -> int:
        """Address, in this process, of rank r's allocation."""
        return self._own.value if r == self.rank else self._peer_base[r]

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self.close()
        return False

    def all_agree(self, ok: bool) -> bool:
        """Collective AND of a per-rank flag (an all-reduce MIN, synchronising): ranks use it at
        fixed points to decide together whether to go on, so that a failure on one rank never
        leaves the others inside a collective that will not be matched."""
        t = torch.tensor([1.0 if ok else 0.0], device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return bool(t.item() == 1.0)

    def meet(self) -> None:
        """Stream-ordered rendezvous of the group (an all-reduce of one element)."""
        dist.all_reduce(self._token, group=self.group)

    def _drop_views(self) -> None:
        self.bytes = None

    def close(self) -> None:
        if not self._open:
            return
        self._open = False
        lib = L.load()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)          # nobody still writes into a peer
            for p in self._peer_base.values():
                lib.sk_peer_close(p)
            self._drop_views()
            dist.barrier(group=self.group)          # every mapping is gone before the memory is
            lib.sk_peer_free(self._own)


class GatheredResult(_SharedAllocation):
    """The full fp16 result [M, N_total] on this GPU, mapped into every process of `group`.

    `full` is the local matrix (a torch tensor over the library's allocation), `block` the
    view of this rank's own columns.  Collective: every rank of the group constructs it (and
    closes it) at the same point of the program.  Usable as a context manager; leaving the
    block closes it, also on an exception -- but close() is itself collective, so ranks that
    may fail independently must first agree on the outcome (all_agree) and leave together.
    """

    def __init__(self, M: int, n_total: int, group=None, device=None):
        if dist.is_initialized() and dist.get_world_size(group) - 1 > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS + 1} ranks")
        self.M, self.n_total = int(M), int(n_total)
        if dist.is_initialized():
            self.col0, self.width = column_block(dist.get_rank(group), dist.get_world_size(group), self.n_total)
        super().__init__(self.M * self.n_total * 2, "GatheredResult", group, device)
        self.full = self.bytes.view(torch.float16).view(self.M, self.n_total)
        self.block = self.full[:, self.col0:self.col0 + self.width]
        off = self.col0 * 2
        self._peer_ptrs = (C.c_void_p * max(1, self.world - 1))(
            *[self._peer_base[r] + off for r in peer_order(self.rank, self.world)])

    def _drop_views(self) -> None:
        self.full = self.block = self.bytes = None


class ScatteredResult(_SharedAllocation):
    """Receive side of the fused reduce-scatter: this rank's fp32 slots [world, M, N_total / world]
    (slot g = the partial sum sender g computed for this rank's column block), mapped into every
    process of `group`, and the 16-bit result block [M, N_total / world] the slots are reduced
    into.  Collective like GatheredResult."""

    def __init__(self, M: int, n_total: int, group=None, device=None, dtype=torch.float16):
        if dtype not in (torch.float16, torch.bfloat16):
            raise TypeError("dtype must be float16 or bfloat16")
        self.M, self.n_total, self.dtype = int(M), int(n_total), dtype
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if world > 8:
            raise ValueError("at most 8 ranks")
        if self.n_total % world or (self.n_total // world) % 32:
            raise ValueError(f"N = {n_total} does not split into {world} column blocks of a multiple of 32")
        self.width = self.n_total // world
        super().__init__(world * self.M * self.width * 4, "ScatteredResult", group, device)
        self.parts = self.bytes.view(torch.float32).view(self.world, self.M, self.width)
        self.block = torch.empty(self.M, self.width, dtype=dtype, device=self.device)
        slot = self.M * self.width * 4
        # where THIS rank's partial of column block j goes: slot `rank` of rank j's buffer
        self._dst = (C.c_void_p * self.world)(*[self.base_of(j) + self.rank * slot for j in range(self.world)])

    def _drop_views(self) -> None:
        self.parts = self.bytes = None


def streamk_fp16_nt_gather(A: torch.Tensor, B_block: torch.Tensor, result: GatheredResult, *,
                           fixup: str = "block_reduce", schedule: str = "auto", **kw) -> torch.Tensor:
    """result.full = A @ B.T for B = the ranks' B_block stacked by rows: each rank computes its
    column block with the CTA-pair Stream-K kernel, whose epilogue writes every tile into all
    ranks' matrices.  A [M, K] fp16 (the same on every rank), B_block [N_total / world, K] fp16.
    Returns result.full, complete on every rank once the stream reaches the point after this
    call.  Options as for streamk_fp16_nt (tile_m: None or 256, the CTA-pair kernel).
    """
    o = _ops._options(kw)
    _ops._check_matrix("A", A, torch.float16)
    _ops._check_matrix("B_block", B_block, torch.float16)
    M, K = A.shape
    if (M, B_block.shape[0]) != (result.M, result.width) or B_block.shape[1] != K:
        raise ValueError(f"Incompatible dimensions: A {tuple(A.shape)} B_block {tuple(B_block.shape)} "
                         f"result {result.M} x {result.width} of {result.n_total}")
    if o["out"] is not None:
        raise TypeError("the result lives in `result`; `out` is not accepted")
    if o["tile_m"] not in (None, 256):
        raise ValueError("the fused gather runs on the CTA-pair kernel: tile_m must be 256")
    if o["tile_m"] is None:
        # Large blocks: the library's own choice is the CTA-pair kernel (with its 256 x 512
        # units); smaller ones are steered to it.
        sms = int(o["num_sms"] or torch.cuda.get_device_properties(A.device).multi_processor_count)
        tiles = ((M + 255) // 256) * ((result.width + 255) // 256)
        if tiles < 2 * (sms // 2):
            o["tile_m"] = 256
    if o["tile_m"] == 256 and schedule == "auto":
        schedule = "hybrid"   # (the automatic choice would weigh kernels that cannot gather)
    A = _ops._aligned16(_ops._rowmajor(_ops._pad_k8(A, 1)))
    Bt = _ops._aligned16(_ops._rowmajor(_ops._pad_k8(B_block, 1)))
    prob = _ops._problem(M, result.width, A.shape[1], A.stride(0), Bt.stride(0), result.n_total, "nt",
                         schedule, fixup, o)
    with torch.cuda.device(A.device):
        ws = _ops._workspace(A.device)
        result.meet()   # the peers are done with the previous contents
        L.check(L.load().sk_gemm_f16_gather(C.byref(prob), A.data_ptr(), Bt.data_ptr(),
                                            result.block.data_ptr(), result._peer_ptrs, result.world - 1,
                                            ws.buf.data_ptr(), ws.nbytes, _ops._stream_ptr(A.device)),
                "sk_gemm_f16_gather")
        result.meet()   # every rank's kernel, hence every store into this GPU, has finished
    return result.full


def streamk_fp16_nt_reduce_scatter(A_shard: torch.Tensor, B_shard: torch.Tensor, result: ScatteredResult, *,
                                   tile_n: int | None = None, **kw) -> torch.Tensor:
    """result.block = columns [rank N/G, (rank+1) N/G) of A @ B.T for A = the ranks' A_shard side by
    side along K and B likewise: A_shard [M, K/G], B_shard [N, K/G] (fp16, or bf16 to match
    `result`).  Each rank multiplies its K shard over the full [M, N] with the CTA-pair kernel,
    whose epilogue writes every fp32 partial tile straight into the owning rank's receive slot
    (peer stores under the mainloop); after a stream-ordered rendezvous each rank adds its slots in
    rank order (bitwise reproducible) and rounds once.  Returns result.block, valid once the
    stream reaches the point after this call.  tile_n: tile width (a divisor of N/G, multiple of
    32; default 256, narrower for small blocks)."""
    o = _ops._options(kw)
    _ops._check_matrix("A_shard", A_shard, result.dtype)
    _ops._check_matrix("B_shard", B_shard, result.dtype)
    M, K = A_shard.shape
    if (M, B_shard.shape[0]) != (result.M, result.n_total) or B_shard.shape[1] != K:
        raise ValueError(f"Incompatible dimensions: A_shard {tuple(A_shard.shape)} B_shard {tuple(B_shard.shape)} "
                         f"result {result.M} x {result.n_total}")
    if o["out"] is not None:
        raise TypeError("the result lives in `result`; `out` is not accepted")
    if tile_n is None:
        tile_n = next(t for t in (256, 128, 64, 32) if result.width % t == 0)
    o["tile_n"] = tile_n
    o["_bf16"] = result.dtype == torch.bfloat16
    A = _ops._aligned16(_ops._rowmajor(_ops._pad_k8(A_shard, 1)))
    Bt = _ops._aligned16(_ops._rowmajor(_ops._pad_k8(B_shard, 1)))
    prob = _ops._problem(M, result.n_total, A.shape[1], A.stride(0), Bt.stride(0), result.n_total, "nt", "dp",
                         "block_reduce", o)
    lib = L.load()
    with torch.cuda.device(A.device):
        ws = _ops._workspace(A.device)
        stream = _ops._stream_ptr(A.device)
        result.meet()   # every rank has reduced (read) the previous contents of its slots
        L.check(lib.sk_gemm_f16_scatter(C.byref(prob), A.data_ptr(), Bt.data_ptr(), result._dst, result.world,
                                        ws.buf.data_ptr(), ws.nbytes, stream), "sk_gemm_f16_scatter")
        result.meet()   # every rank's kernel, hence every store into this GPU's slots, has finished
        L.check(lib.sk_reduce_partials(result.parts.data_ptr(), result.world, M, result.width,
                                       result.block.data_ptr(), result.block.stride(0),
                                       L.SK_FLAG_BF16 if o["_bf16"] else 0, stream), "sk_reduce_partials")
    return result.block
