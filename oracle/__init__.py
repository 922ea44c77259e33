"""CPU oracle for the Stream-K GEMM path.  TEST INFRASTRUCTURE ONLY.

This package restates, on the CPU, what the reference (LeiWang1999/Stream-k.tvm)
computes on its hot path, so that the CUDA library can be checked against it.
Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm
may import it; the product (the streamk_b200 package and its shared library)
never does.

Parity status
-------------
* End-to-end results are pinned: the reference's own check of every kernel is
  `torch.testing.assert_close(torch.matmul(A, B[.T]), C, rtol=1e-2, atol=1e-2)`
  (streamk_fp32.py:204-208, streamk_fp16.py:389-399, …_q4.py:545-557,601-606);
  gemm_ref / unpack_u4 / w4a16_ref below are those same expressions.
* The host scheduler is pinned against the reference's own lines, executed
  verbatim by tests/golden/make_golden.py (streamk_fp16.py:83-113) into
  tests/golden/sched_golden.json.
* The reference's internal layouts (mma fragments, swizzle, ladder permutation,
  LOP3 nibble interleave) live in BitBLAS (unpinned `pip install git+…`,
  README.md:8), are absent from the reference tree and have no golden vectors:
  parity unpinned for those; the library uses its own layouts.
* Group scales / zero-points are not in the reference (its q4 kernels apply
  none); W = (q - z) * s is defined here and is anchored to the reference by the
  s = 1, z = 0 case.
"""
from .gemm_ref import gemm_ref, unpack_u4, pack_u4_int32, dequant_ref, w4a16_ref, rel_err  # noqa: F401
from .sched_ref import reference_schedule, cta_segments, cluster_segments, coverage, tile_coords  # noqa: F401
from .inputs import make_case, CONFIGS  # noqa: F401


def load_triton_ref():
    """The reference's own Triton Stream-K kernel (oracle/_ref/triton_streamk.py, generated from a
    reference checkout by oracle/make_triton_ref.py), or None when the file or triton is absent.
    A GPU comparator for tests/ and bench.py's sweep; importing it compiles nothing yet."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "triton_streamk.py")
    if not os.path.exists(path):
        return None
    try:
        import triton  # noqa: F401
    except Exception:
        return None
    spec = importlib.util.spec_from_file_location("oracle_ref_triton_streamk", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
