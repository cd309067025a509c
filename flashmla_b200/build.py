"""Builds libflashmla_b200.so (sm_100a only) in-tree with nvcc.

    python -m flashmla_b200.build [--force]

One object file per .cu source, rebuilt when the source or a header is newer, then linked into
flashmla_b200/lib/libflashmla_b200.so.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libflashmla_b200.so")
OBJ_DIR = os.path.join(PKG, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-Xptxas", "--warn-on-spills",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_header() -> float:
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(ROOT, "include", "flashmla_b200.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    hdr_time = _newest_header()
    jobs = []
    objs = []
    for src in sources():
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        r = subprocess.run([_nvcc(), *NVCC_FLAGS, "-c", s, "-o", o], capture_output=True, text=True)
        return s, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for s, r in pool.map(compile_one, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {s}")
    if jobs or not os.path.exists(LIB_PATH):
        r = subprocess.run([_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-lcuda"], capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB_PATH


def build_test_helper(force: bool = False) -> str:
    """Compiles tests/wait_timeout/wait_timeout.cu (a test-only kernel whose bounded wait runs out) into a shared
    object beside its source, so that the GPU test finds it prebuilt."""
    src = os.path.join(ROOT, "tests", "wait_timeout", "wait_timeout.cu")
    out = os.path.join(ROOT, "tests", "wait_timeout", "libwait_timeout.so")
    newest = max(os.path.getmtime(src), os.path.getmtime(os.path.join(CSRC, "sm100_ptx.cuh")))
    if force or not os.path.exists(out) or os.path.getmtime(out) < newest:
        r = subprocess.run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-lineinfo",
                            "-Xcompiler", "-fPIC", "-shared", "-o", out, src], capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("nvcc failed on the wait_timeout test helper")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
    print(build_test_helper(force="--force" in sys.argv))
