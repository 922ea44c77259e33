"""Build recipe: compiles csrc/*.cu for sm_100a into lib/libstreamk_b200.so.

The library is a plain C-ABI shared object (no torch, no pybind): nvcc only.
Objects are rebuilt when a source or header is newer than the object.

STREAMK_B200_TRACE=1 builds a second library, lib/libstreamk_b200_trace.so, compiled with
-DSK_TRACE: its kernels record per-CTA timestamps while sk_debug_set_trace() names a buffer.
The ordinary library carries no tracing code.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
LIBNAME = "libstreamk_b200.so"
TRACE_LIBNAME = "libstreamk_b200_trace.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def trace_build() -> bool:
    return os.environ.get("STREAMK_B200_TRACE") == "1"


def lib_path() -> str:
    return os.path.join(LIBDIR, TRACE_LIBNAME if trace_build() else LIBNAME)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".inc"))]
    hs.append(os.path.join(HERE, "..", "include", "streamk_b200.h"))
    return hs


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile (if needed) and return the path of the shared library."""
    objdir = OBJDIR + ("_trace" if trace_build() else "")
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    headers = _headers()
    common = [nvcc, "-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS, "-Xcompiler", "-fPIC",
              "-Xptxas", "-v"]
    if trace_build():
        common.append("-DSK_TRACE")
    jobs = []
    objs = []
    for src in _sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src, *headers]):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        r = subprocess.run([*common, "-c", src, "-o", obj], capture_output=True, text=True)
        return src, r

    with ThreadPoolExecutor(max_workers=max(1, min(8, len(jobs) or 1))) as ex:
        for src, r in ex.map(compile_one, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(f"--- {os.path.basename(src)}\n{r.stdout}{r.stderr}\n")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
    out = lib_path()
    if force or jobs or _stale(out, objs):
        r = subprocess.run([nvcc, "-shared", *ARCH_FLAGS, "-o", out, *objs],
                           capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
