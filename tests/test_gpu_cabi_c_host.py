"""Hosts written in plain C (tests/cabi_host/decode_from_c.c, dense_decode_from_c.c) drive the library through
include/flashmla_b200.h alone: plan, tile scheduler and decode, checked against a closed-form answer.  Shows that the
boundary is the C ABI and not the Python layer."""
import os
import shutil
import subprocess

import pytest

from flashmla_b200 import _lib

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build_host(tmp_path, source):
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler on this machine")
    _lib.load()          # builds the library if it is missing
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = str(tmp_path / source[:-2])
    libdir = os.path.dirname(_lib.LIB_PATH)
    subprocess.run(["gcc", "-O1", "-std=c99", os.path.join(ROOT, "tests", "cabi_host", source), "-o", exe,
                    "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"), "-L", libdir,
                    "-L", os.path.join(cuda, "lib64"), "-lflashmla_b200", "-lcudart", "-lm",
                    "-Wl,-rpath," + libdir, "-Wl,-rpath," + os.path.join(cuda, "lib64")], check=True)
    return exe


@pytest.mark.parametrize("h_q", [128, 16])
def test_plain_c_host_runs_decode(tmp_path, h_q):
    exe = _build_host(tmp_path, "decode_from_c.c")
    run = subprocess.run([exe, str(h_q)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stderr + run.stdout
    assert run.stdout.startswith("OK")


def test_plain_c_host_runs_dense_decode(tmp_path):
    """tests/cabi_host/dense_decode_from_c.c: plan, tile scheduler over cache_seqlens and fmla_dense_decode (causal, a
    block-table entry outside the cache) against a closed-form answer."""
    exe = _build_host(tmp_path, "dense_decode_from_c.c")
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stderr + run.stdout
    assert run.stdout.startswith("OK dense")
