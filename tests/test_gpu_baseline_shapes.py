"""GPU parity on EVERY shape of the benchmark configurations 3 (24 fp16 NT shapes) and 4 (9
W4A16 shapes), through the C ABI, against the CPU oracle on the same seeded inputs.

The library's default schedule (`auto`) picks a different kernel path per shape -- cluster
split-K of 2, 4 or 8, operands swapped with a fitted weight-tile height, CTA pairs with a
fitted tile width, plain Stream-K -- so a sample of the shapes would leave paths unchecked.
Every shape runs with `auto` and with the explicit schedules of the configuration
(streamk / hybrid / dp) under the deterministic fixup, and with the atomic fixup under
Stream-K; the device status word is read after each launch.

Tolerance: max|C - C_ref| <= 1e-2 * max|C_ref| (the configurations' bar; the reference checks
its kernels with rtol = atol = 1e-2, streamk_fp16.py:389-399, ..._q4.py:552-557,601).
"""
import pytest
import torch

import oracle
import streamk_b200 as sk

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL16 = 1e-2

CFG3 = list(range(len(oracle.CONFIGS[3]["shapes"])))
CFG4 = list(range(len(oracle.CONFIGS[4]["shapes"])))


def _id3(i):
    return "x".join(map(str, oracle.CONFIGS[3]["shapes"][i]))


def _id4(i):
    return "x".join(map(str, oracle.CONFIGS[4]["shapes"][i]))


def _check(C, ref, what):
    sk.check_status()
    err = oracle.rel_err(C, ref)
    assert err <= TOL16, (what, err)


@pytest.mark.parametrize("case", CFG3, ids=_id3)
def test_fp16_config3_every_shape(case):
    c = oracle.make_case(3, case)
    ref = oracle.gemm_ref(c["A"], c["B"], "nt")
    A, B = c["A"].to(DEV), c["B"].to(DEV)
    first = sk.streamk_fp16_nt(A, B)                         # auto, block_reduce: the default call
    _check(first, ref, "auto")
    assert torch.equal(sk.streamk_fp16_nt(A, B), first)     # deterministic fixup: same bits again
    for schedule in ("streamk", "hybrid", "dp"):
        _check(sk.streamk_fp16_nt(A, B, schedule=schedule, fixup="block_reduce"), ref, schedule)
    _check(sk.streamk_fp16_nt(A, B, schedule="streamk", fixup="atomic"), ref, "streamk/atomic")
    _check(sk.streamk_fp16_nt(A, B, pdl=True), ref, "auto+pdl")


@pytest.mark.parametrize("case", CFG4, ids=_id4)
def test_w4a16_config4_every_shape(case):
    c = oracle.make_case(4, case)
    ref = oracle.w4a16_ref(c["A"], c["q"], c["scales"], c["zeros"])
    P = sk.q4_prepack(c["qweight"].to(DEV), c["scales"].to(DEV), c["zeros"].to(DEV))
    # int4 unpack / dequantisation bit-exact on the full-size weight
    W = sk.dequant_w4(P).cpu()
    assert torch.equal(W.view(torch.int16),
                       oracle.dequant_ref(c["q"], c["scales"], c["zeros"]).view(torch.int16))
    A = c["A"].to(DEV)
    first = sk.streamk_fp16_ladder_block_reduce_q4(A, P)     # auto, block_reduce
    _check(first, ref, "auto")
    assert torch.equal(sk.streamk_fp16_ladder_block_reduce_q4(A, P), first)
    for schedule in ("streamk", "hybrid", "dp"):
        _check(sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule=schedule, fixup="block_reduce"),
               ref, schedule)
    _check(sk.streamk_fp16_ladder_block_reduce_q4(A, P, schedule="streamk", fixup="atomic"), ref,
           "streamk/atomic")


def test_config1_and_config2_default_calls():
    c = oracle.make_case(1)
    C = sk.streamk_fp32(c["A"].to(DEV), c["B"].to(DEV))
    sk.check_status()
    assert oracle.rel_err(C, oracle.gemm_ref(c["A"], c["B"], "nn")) <= 1e-4
    c = oracle.make_case(2)
    ref = oracle.gemm_ref(c["A"], c["B"], "nt")
    for fixup in ("atomic", "block_reduce"):
        _check(sk.streamk_fp16_nt(c["A"].to(DEV), c["B"].to(DEV), fixup=fixup), ref, fixup)
        _check(sk.streamk_fp16_nt(c["A"].to(DEV), c["B"].to(DEV), fixup=fixup, schedule="streamk",
                                  tile_n=128), ref, "streamk " + fixup)


def test_zero_initialised_problem_means_no_test_hook():
    """A C caller that memsets sk_problem to zero and fills in the shape gets an ordinary
    launch: the flag-dropping test hook is off at 0 (it used to be off at -1 only)."""
    import ctypes as C
    from streamk_b200 import _lib as L
    from streamk_b200 import ops as _ops
    lib = L.load()
    A = torch.randn(128, 1024).half().to(DEV)
    B = (torch.randn(128, 1024) / 32).half().to(DEV)
    out = torch.empty(128, 128, dtype=torch.float16, device=DEV)
    prob = L.SkProblem()                       # all zero
    prob.M, prob.N, prob.K, prob.lda, prob.ldb, prob.ldc = 128, 128, 1024, 1024, 1024, 128
    prob.layout, prob.schedule, prob.fixup = L.LAYOUTS["nt"], L.SCHEDULES["streamk"], L.FIXUPS["block_reduce"]
    prob.num_sms, prob.fixup_timeout_us = 2, 2000      # two CTAs share the one tile
    dev = torch.device("cuda", torch.cuda.current_device())
    ws = _ops._workspace(dev)
    st = lib.sk_gemm_f16(C.byref(prob), A.data_ptr(), B.data_ptr(), out.data_ptr(), ws.buf.data_ptr(),
                         ws.nbytes, _ops._stream_ptr(dev))
    assert st == 0
    sk.check_status()                          # no SK_ERR_FIXUP_TIMEOUT
    assert oracle.rel_err(out, oracle.gemm_ref(A.cpu(), B.cpu(), "nt")) <= TOL16


def test_tabled_shapes_in_the_other_layouts():
    """The tuned table holds choices for the NT entry point; the NN and ladder entry points (whose
    weights come in 128-row units) must not inherit tile widths they cannot run."""
    c = oracle.make_case(3, 20)                      # 256 x 4096 x 4096: in the table with 64-wide tiles
    ref = oracle.gemm_ref(c["A"], c["B"], "nt")
    A, B = c["A"].to(DEV), c["B"].to(DEV)
    _check(sk.streamk_fp16_nn(A, B.t().contiguous()), ref, "nn")
    _check(sk.streamk_fp16_ladder(A, sk.ladder_prepack(B)), ref, "ladder")
    _check(sk.streamk_fp16_nt(A, B, no_table=True), ref, "nt, rules only")
