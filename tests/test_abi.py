"""The shared library loads without a GPU and exports every symbol the header declares."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    txt = open(os.path.join(ROOT, "include", "streamk_b200.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(sk_[a-z0-9_]+)\s*\(", txt)))


def test_header_symbols_are_exported(lib):
    names = _declared()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/streamk_b200.h but not exported"


def test_binding_table_matches_header():
    from streamk_b200 import _lib as L
    assert sorted(L.SIGNATURES) == _declared()


def test_struct_sizes(lib):
    from streamk_b200 import _lib as L
    assert C.sizeof(L.SkProblem) == 16 * 4
    assert C.sizeof(L.SkScheduleInfo) == 19 * 4
    assert C.sizeof(L.SkStatus) == 16


def test_host_only_calls(lib):
    assert b"sm_100a" in lib.sk_version()
    assert lib.sk_status_string(0) == b"ok"
    assert lib.sk_workspace_bytes(148) > 2 * 148 * 128 * 256 * 4
    assert lib.sk_workspace_bytes(0) == 0
    assert lib.sk_ladder_bytes(100, 100) == 2 * 2 * 16384      # one 256-row tile, two K blocks
    assert lib.sk_q4_bytes(128, 256) == 2 * 4 * 4096 + 2 * 2 * 384
    assert lib.sk_q4_bytes(128, 100) == 0                       # K must be a multiple of 128


def test_the_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "stream-k.tvm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src, f
