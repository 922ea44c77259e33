"""The CPU oracle against the fixtures generated from the reference's own lines
(tests/golden/make_golden.py) and against independent scalar models."""
import json
import os

import numpy as np
import pytest
import torch

import oracle

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_scheduler_matches_reference_host_block():
    cases = json.load(open(os.path.join(GOLD, "sched_golden.json")))["cases"]
    assert len(cases) > 40
    for c in cases:
        r = oracle.reference_schedule(c["M"], c["N"], c["K"], c["BM"], c["BN"], c["BK"], c["P"])
        for key in ("total_tiles", "iters_per_tile", "streamk_tiles", "blocking_tiles",
                    "streamk_full_tiles", "streamk_partial_tiles"):
            assert r[key] == c[key], (c, key)


def test_unpack_matches_reference_expression():
    g = json.load(open(os.path.join(GOLD, "q4_unpack_golden.json")))
    qB = torch.tensor(g["qB"], dtype=torch.int8)
    exp = torch.tensor(g["expanded"], dtype=torch.uint8)
    assert torch.equal(oracle.unpack_u4(qB), exp)
    # int32 packing is byte-identical to the int8 low-nibble-first storage
    assert torch.equal(oracle.pack_u4_int32(exp).view(torch.int8).reshape(qB.shape), qB)


def test_gemm_ref_matches_golden():
    z = np.load(os.path.join(GOLD, "gemm_golden.npz"))
    for tag, layout in (("nt", "nt"), ("nn32", "nn"), ("nn", "nn")):
        C = oracle.gemm_ref(torch.from_numpy(z[f"{tag}_A"]), torch.from_numpy(z[f"{tag}_B"]), layout)
        assert torch.allclose(C, torch.from_numpy(z[f"{tag}_C"]), rtol=1e-6, atol=1e-6)


def test_gemm_ref_against_float64():
    torch.manual_seed(1)
    A = torch.randn(37, 300).half()
    B = torch.randn(29, 300).half()
    ref64 = (A.double() @ B.double().t())
    assert oracle.rel_err(oracle.gemm_ref(A, B, "nt"), ref64.float()) < 1e-6


def _half_bits(x: float) -> int:
    return int(np.array([x], dtype=np.float16).view(np.uint16)[0])


def test_dequant_ref_scalar_model_all_qz_pairs():
    """(q - z) is exact in fp16, the product is rounded once: check every (q, z) pair
    against numpy float16 arithmetic done element by element."""
    torch.manual_seed(2)
    scales = (0.002 + 0.018 * torch.rand(16)).half()
    for si in range(16):
        s = scales[si]
        q = torch.arange(16, dtype=torch.uint8).repeat(16, 8)          # [16, 128]
        z = torch.arange(16, dtype=torch.uint8).view(16, 1)            # one group per row
        W = oracle.dequant_ref(q, s.expand(16, 1).contiguous(), z)
        for zi in range(16):
            for qi in range(16):
                want = np.float16(np.float16(qi) - np.float16(zi)) * np.float16(float(s))
                assert _half_bits(float(W[zi, qi])) == _half_bits(float(np.float16(want)))


def test_dequant_ref_reference_semantics():
    q = torch.randint(0, 16, (8, 256), dtype=torch.uint8)
    assert torch.equal(oracle.dequant_ref(q, None, None), q.half())


def test_input_generators_are_deterministic_and_shaped():
    a = oracle.make_case(2, shape=(8, 16, 64))
    b = oracle.make_case(2, shape=(8, 16, 64))
    assert torch.equal(a["A"], b["A"]) and torch.equal(a["B"], b["B"])
    c = oracle.make_case(4, shape=(2, 128, 256))
    assert c["qweight"].shape == (128, 32) and c["zeros"].shape == (128, 2)
    assert c["scales"].dtype == torch.float16 and float(c["scales"].min()) >= 0.0019
    assert int(c["q"].max()) <= 15
    assert len(oracle.CONFIGS[3]["shapes"]) == 24 and len(oracle.CONFIGS[4]["shapes"]) == 9


@pytest.mark.parametrize("P", [1, 2, 3, 5, 108, 132, 148])
def test_reference_walk_covers_streamk_tiles_once(P):
    """The interval walk (streamk_fp16.py:176-193) covers every (tile, k) of the Stream-K
    tiles exactly once and the DP formula covers the rest."""
    import random
    rnd = random.Random(P)
    for _ in range(20):
        M, N, K = rnd.randint(1, 700), rnd.randint(1, 3000), rnd.randint(1, 2000)
        BM, BN, BK = rnd.choice([16, 64, 128]), rnd.choice([64, 128, 256]), rnd.choice([16, 32, 64])
        r = oracle.reference_schedule(M, N, K, BM, BN, BK, P)
        sched = dict(grid=P, sk_tiles=r["streamk_tiles"], total_tiles=r["total_tiles"],
                     iters_per_tile=r["iters_per_tile"], sk_iters_per_cta=r["streamk_full_tiles"],
                     sk_iters_rem=r["streamk_partial_tiles"], dp_first=0)
        cov = oracle.coverage(sched)
        assert len(cov) == r["total_tiles"] * r["iters_per_tile"]
        assert set(cov.values()) == {1}
