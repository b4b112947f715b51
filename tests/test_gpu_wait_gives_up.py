"""The give-up path of the library's bounded in-kernel waits, executed once, safely.

A test-only library (``tests/wait_probe.cu``, not linked into ``libpalimpsa_b200.so``) launches one 32-thread CTA
that waits with the product kernels' ``tc::mbar_wait`` on an mbarrier nobody arrives at, with a poll limit of a
few thousand: the wait runs out by construction, the kernel records its code, frees the TMEM it allocated and
returns.  The test checks the code, that the same kernel succeeds when somebody does arrive, and that the
device keeps working (a normal forward/backward right after)."""
import ctypes as C
import os

import pytest
import torch

from oracle import palimpsa_oracle as orc
from tests import wait_probe
from tests.gpu_util import compare, run_cuda, run_oracle
from tests.helpers import TOL_FP32

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_the_device_stays_usable():
    if not os.path.exists(wait_probe.LIB):
        wait_probe.build()
    lib = C.CDLL(wait_probe.LIB)
    lib.palimpsa_test_wait_probe.argtypes = [C.c_int, C.c_uint, C.c_void_p, C.c_void_p]
    status = torch.full((1,), -5, dtype=torch.int32, device="cuda:0")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.palimpsa_test_wait_probe(0, 4000, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert status.item() == 7                      # nobody arrived: the wait gave up after 4000 polls and said so
    assert lib.palimpsa_test_wait_probe(1, 4000, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert status.item() == 0                      # with an arrival the same wait completes
    assert lib.palimpsa_test_wait_probe(0, 100, status.data_ptr(), stream) == 0   # TMEM was freed: allocate again
    torch.cuda.synchronize()
    assert status.item() == 7
    inp = orc.make_inputs(3, B=1, T=40, H=2, K=32, V=16)
    compare(run_cuda(inp, "chunk"), run_oracle(inp), TOL_FP32, what="after the probe")
    from palimpsa_b200 import _lib
    assert _lib.lib().palimpsa_tensor_core_status() == 0     # the probe's own status word is not the library's
