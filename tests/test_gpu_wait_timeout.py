"""The device-side waits of the kernels are bounded: a wait that runs out makes the kernel record a code in a status
word and return, instead of spinning or trapping.  A small test-only kernel (tests/wait_timeout/wait_timeout.cu)
drives the library's own wait helper to its limit on a barrier that nobody arrives at; the status must come back
through ``flashmla_b200.kernel_status`` and the device must stay usable for the next ordinary call."""
import ctypes as C
import os

import pytest
import torch

import flashmla_b200
from flashmla_b200 import interface, workloads as wl
from gpu_utils import DEV, run_decode, oracle_decode, check_decode

pytestmark = pytest.mark.gpu
HELPER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "wait_timeout", "libwait_timeout.so")


def _helper():
    if not os.path.exists(HELPER):
        from flashmla_b200 import build
        build.build_test_helper()
    lib = C.CDLL(HELPER)
    lib.wait_timeout_probe.restype = C.c_int
    lib.wait_timeout_probe.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
    lib.wait_timeout_code.restype = C.c_int
    return lib


def test_a_wait_that_runs_out_sets_the_status_word_and_the_next_call_works():
    lib = _helper()
    dev = torch.device(DEV)
    status = interface._status(dev)                      # the word the library's own kernels report to
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert flashmla_b200.kernel_status(dev) == 0
    # control: the barrier completes, the wait succeeds, nothing is reported
    assert lib.wait_timeout_probe(status.data_ptr(), 1, stream) == 0
    assert flashmla_b200.kernel_status(dev) == 0
    # nobody arrives: the wait gives up after its poll limit and the kernel returns with the code
    assert lib.wait_timeout_probe(status.data_ptr(), 0, stream) == 0
    assert flashmla_b200.kernel_status(dev) == lib.wait_timeout_code()
    assert flashmla_b200.kernel_status(dev) == 0         # reading clears the word
    # the context is intact: an ordinary decode call runs and matches the oracle
    w = wl.make_decode_workload(3, 2, 128, 256, 300, 900, seed=41, invalid_frac=0.03, q_std=1.0, kv_std=0.1, clamp=1.0,
                                sm_scale=576 ** -0.55)
    out, lse, _ = run_decode(w)
    ref_out, ref_lse = oracle_decode(w)
    check_decode(out, lse, ref_out, ref_lse)
