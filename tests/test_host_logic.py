"""Argument checking of the Python entry points (no GPU needed: everything is rejected
before a kernel would launch)."""
import pytest
import torch

import streamk_b200 as sk


def test_cpu_tensors_are_rejected_not_computed():
    A = torch.zeros(4, 8, dtype=torch.float16)
    B = torch.zeros(4, 8, dtype=torch.float16)
    with pytest.raises(ValueError, match="no CPU path"):
        sk.streamk_fp16_nt(A, B)
    with pytest.raises(ValueError, match="no CPU path"):
        sk.streamk_fp32(A.float(), B.float().t().contiguous())
    with pytest.raises(ValueError, match="no CPU path"):
        sk.q4_prepack(torch.zeros(128, 16, dtype=torch.int32))


def test_entry_points_exist_with_reference_names():
    for name in ("streamk_fp32", "streamk_fp16_nn", "streamk_fp16_nt", "streamk_fp16_atomic",
                 "streamk_fp16_block_reduce", "ladder_prepack", "streamk_fp16_ladder",
                 "streamk_fp16_ladder_block_reduce", "q4_prepack", "dequant_w4",
                 "streamk_fp16_ladder_block_reduce_q4"):
        assert callable(getattr(sk, name))


def test_schedule_info_needs_no_gpu():
    d = sk.schedule_info(384, 384, 8192, schedule="hybrid", tile_n=128)
    assert (d["total_tiles"], d["sk_tiles"], d["sk_iters_per_cta"], d["sk_iters_rem"]) == (9, 9, 7, 116)
    with pytest.raises(ValueError):
        sk.schedule_info(4, 4, 4, schedule="nope")


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from streamk_b200 import _lib as L
    monkeypatch.setattr(L, "_lib", None)
    with pytest.raises(OSError):
        L.load(str(tmp_path / "absent.so"))
