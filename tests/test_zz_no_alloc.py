"""sk_gemm_f32_noalloc: the entry point for callers that must not allocate (fixed memory
budgets, regions where cudaMalloc is forbidden, operand-only plugin interfaces).  Its fixup
scratch is a fixed array inside the library, so nothing is passed but the operands.

Called through the C ABI twice in a row (the second call reuses the array the first one
left behind) and compared with sk_gemm_f32, which gets an ordinary caller-owned workspace.
Collected last on purpose: a run that stops at the first failure has then already run every
other test.  Works alone in a fresh process as well: it does its own set-up.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL32 = 1e-4   # the fp32 bar of the other GPU tests


def _problem(L, M, N, K, fixup, num_sms):
    return L.SkProblem(M=M, N=N, K=K, lda=K, ldb=N, ldc=N, layout=L.LAYOUTS["nn"],
                       schedule=L.SCHEDULES["streamk"], fixup=L.FIXUPS[fixup], num_sms=num_sms)


@pytest.mark.parametrize("fixup", ["atomic", "block_reduce"])
def test_noalloc_matches_workspace_entry_point_twice(fixup):
    import streamk_b200  # noqa: F401
    from streamk_b200 import _lib as L
    lib = L.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    nbytes = int(lib.sk_workspace_bytes(sms))
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    status = (L.SkStatus * 1)()
    g = torch.Generator().manual_seed(123)
    for (M, N, K) in ((256, 256, 1024), (100, 90, 700)):      # two calls in a row
        A = (torch.rand(M, K, generator=g) * 2 - 1).to(dev)
        B = (torch.rand(K, N, generator=g) * 2 - 1).to(dev)
        want = torch.empty(M, N, device=dev)
        got = torch.full((M, N), float("nan"), device=dev)
        prob = _problem(L, M, N, K, fixup, 16)
        st = lib.sk_gemm_f32(C.byref(prob), A.data_ptr(), B.data_ptr(), want.data_ptr(),
                             ws.data_ptr(), nbytes, stream)
        assert st == 0, lib.sk_status_string(st)
        prob0 = _problem(L, M, N, K, fixup, 0)                  # 0 = the maximum (16 CTAs)
        st = lib.sk_gemm_f32_noalloc(C.byref(prob0), A.data_ptr(), B.data_ptr(), got.data_ptr(),
                                     status, stream)
        assert st == 0, lib.sk_status_string(st)
        torch.cuda.synchronize()
        assert status[0].code == 0
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= TOL32 * scale
        ref = A.double() @ B.double()
        assert float((got.double() - ref).abs().max()) <= TOL32 * float(ref.abs().max())


def test_noalloc_rejects_more_ctas_than_the_scratch_holds():
    import streamk_b200  # noqa: F401
    from streamk_b200 import _lib as L
    lib = L.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    A = torch.zeros(64, 64, device=dev)
    prob = _problem(L, 64, 64, 64, "atomic", 17)
    st = lib.sk_gemm_f32_noalloc(C.byref(prob), A.data_ptr(), A.data_ptr(), A.data_ptr(), None,
                                 C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == L.SK_ERR_LIMIT
    assert b"maximum" in lib.sk_status_string(st)
