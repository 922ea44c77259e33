"""ctypes binding of the C ABI declared in include/streamk_b200.h.

There is no fallback: if the shared library is missing or a symbol cannot be
resolved, importing or calling raises.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

# ---- enums (mirror include/streamk_b200.h) --------------------------------
SK_OK = 0
SK_ERR_ARCH, SK_ERR_ALIGN, SK_ERR_SHAPE, SK_ERR_WORKSPACE, SK_ERR_LAUNCH = 1, 2, 3, 4, 5
SK_ERR_FIXUP_TIMEOUT, SK_ERR_PIPE_TIMEOUT, SK_ERR_ARG, SK_ERR_LIMIT = 6, 7, 8, 9

LAYOUTS = {"nn": 0, "nt": 1, "ladder": 2}
SCHEDULES = {"streamk": 0, "hybrid": 1, "hybrid_dp_first": 2, "dp": 3, "auto": 4, "cluster": 5, "gemv": 6}
FIXUPS = {"atomic": 0, "block_reduce": 1}
SK_FLAG_PDL = 1
SK_FLAG_NO_TABLE = 2
SK_FLAG_BF16 = 4
SK_FLAG_Q4_GROUP = {128: 0, 32: 0x100, 64: 0x200, 0: 0x300}   # group size -> sk_problem.flags bits (0 = per-channel)


class SkProblem(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "M", "N", "K", "lda", "ldb", "ldc", "layout", "schedule", "fixup", "tile_m", "tile_n", "num_sms",
        "group_m", "fixup_timeout_us", "test_drop_flag_cta", "flags")]


class SkScheduleInfo(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "tile_m", "tile_n", "tile_k", "tiles_m", "tiles_n", "total_tiles", "iters_per_tile",
        "sk_tiles", "dp_tiles", "grid", "sk_iters_per_cta", "sk_iters_rem", "dp_waves",
        "dp_first", "group_m", "swap_ab", "schedule", "cluster", "wide_units")]

    def as_dict(self) -> dict:
        return {n: getattr(self, n) for n, _ in self._fields_}


class SkDeviceInfo(C.Structure):
    _fields_ = [("cc_major", C.c_int32), ("cc_minor", C.c_int32), ("num_sms", C.c_int32),
                ("max_smem_optin", C.c_int32), ("l2_bytes", C.c_int64), ("total_mem", C.c_int64)]


class SkStatus(C.Structure):
    _fields_ = [("code", C.c_uint32), ("cta", C.c_uint32), ("detail0", C.c_uint32),
                ("detail1", C.c_uint32)]


# Every exported symbol with its (restype, argtypes); used by load() and by the
# CPU-side test that the library exports what the header declares.
_P = C.c_void_p
SIGNATURES = {
    "sk_version": (C.c_char_p, []),
    "sk_status_string": (C.c_char_p, [C.c_int]),
    "sk_last_cuda_error": (C.c_int, []),
    "sk_query": (C.c_int, [C.c_int, C.POINTER(SkDeviceInfo)]),
    "sk_debug_set_trace": (C.c_int, [_P]),
    "sk_schedule": (C.c_int, [C.POINTER(SkProblem), C.c_int, C.c_int, C.POINTER(SkScheduleInfo)]),
    "sk_schedule_gather": (C.c_int, [C.POINTER(SkProblem), C.c_int, C.c_int, C.POINTER(SkScheduleInfo)]),
    "sk_cta_interval": (C.c_int, [C.POINTER(SkScheduleInfo), C.c_int, C.POINTER(C.c_int64),
                                  C.POINTER(C.c_int64)]),
    "sk_tile_coords": (C.c_int, [C.POINTER(SkScheduleInfo), C.c_int, C.POINTER(C.c_int),
                                 C.POINTER(C.c_int)]),
    "sk_memcpy2d_async": (C.c_int, [_P, C.c_size_t, _P, C.c_size_t, C.c_size_t, C.c_size_t, _P]),
    "sk_workspace_bytes": (C.c_size_t, [C.c_int]),
    "sk_workspace_init": (C.c_int, [_P, C.c_size_t, _P]),
    "sk_poll_status": (C.c_int, [_P, C.POINTER(SkStatus), _P]),
    "sk_gemm_f32": (C.c_int, [C.POINTER(SkProblem), _P, _P, _P, _P, C.c_size_t, _P]),
    "sk_gemm_f32_noalloc": (C.c_int, [C.POINTER(SkProblem), _P, _P, _P, C.POINTER(SkStatus), _P]),
    "sk_gemm_f16": (C.c_int, [C.POINTER(SkProblem), _P, _P, _P, _P, C.c_size_t, _P]),
    "sk_gemm_f16_gather": (C.c_int, [C.POINTER(SkProblem), _P, _P, _P, C.POINTER(_P), C.c_int, _P,
                                     C.c_size_t, _P]),
    "sk_gemm_f16_scatter": (C.c_int, [C.POINTER(SkProblem), _P, _P, C.POINTER(_P), C.c_int, _P, C.c_size_t, _P]),
    "sk_reduce_partials": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, _P, C.c_int, C.c_int, _P]),
    "sk_peer_alloc": (C.c_int, [C.c_size_t, C.POINTER(_P), _P]),
    "sk_peer_open": (C.c_int, [_P, C.POINTER(_P)]),
    "sk_peer_close": (C.c_int, [_P]),
    "sk_peer_free": (C.c_int, [_P]),
    "sk_ladder_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "sk_prepack_ladder": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, _P, C.c_size_t, _P]),
    "sk_q4_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "sk_prepack_q4": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, _P, C.c_size_t, _P]),
    "sk_dequant_q4": (C.c_int, [_P, C.c_int, C.c_int, _P, C.c_int, _P]),
    "sk_q4_bytes_ex": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "sk_prepack_q4_ex": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P, C.c_size_t, _P]),
    "sk_dequant_q4_ex": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, _P, C.c_int, _P]),
    "sk_gemm_w4a16": (C.c_int, [C.POINTER(SkProblem), _P, _P, _P, _P, C.c_size_t, _P]),
}

_lib = None


class StreamKError(RuntimeError):
    def __init__(self, status: int, where: str, extra: str = ""):
        self.status = status
        msg = f"{where}: status {status}"
        if _lib is not None:
            msg += f" ({_lib.sk_status_string(status).decode()})"
            if status == SK_ERR_LAUNCH:
                msg += f", cudaError {_lib.sk_last_cuda_error()}"
        if extra:
            msg += f" {extra}"
        super().__init__(msg)


def load(path: str | None = None):
    """Load the in-tree shared library (building it first when STREAMK_B200_BUILD=1)."""
    global _lib
    if _lib is not None:
        return _lib
    explicit = path or os.environ.get("STREAMK_B200_LIB")
    if explicit:
        path = explicit   # a named library that is absent is an error (CDLL raises OSError)
    else:
        path = _build.lib_path()
        if os.environ.get("STREAMK_B200_BUILD") == "1" or not os.path.exists(path):
            path = _build.build()   # compiles the CUDA sources; raises if nvcc fails
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing: fail loudly
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, where: str) -> None:
    if status != SK_OK:
        raise StreamKError(status, where)
