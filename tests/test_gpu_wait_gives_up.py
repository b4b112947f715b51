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


def test_peer_wait_runs_out_records_its_code_and_poisons_the_buffer():
    """The stream-ordered wait on a peer's flag (used by the context-parallel hops) on ONE GPU: a flag nobody sets
    makes it run out after its wall-clock limit (5 ms here); it records code 7, writes a NaN into the buffer it
    guards and lets the stream go on.  After a signal the same wait passes."""
    from palimpsa_b200 import _lib
    lib = _lib.lib()
    lib.palimpsa_tensor_core_status()                                   # clear whatever earlier tests left
    flag = torch.zeros(1, dtype=torch.int64, device="cuda:0")
    guarded = torch.ones(4, dtype=torch.float32, device="cuda:0")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.palimpsa_peer_wait(flag.data_ptr(), 1, 5, guarded.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert lib.palimpsa_tensor_core_status() == 7
    assert torch.isnan(guarded[0]) and bool((guarded[1:] == 1).all())
    assert lib.palimpsa_tensor_core_status() == 0                       # reading cleared it
    guarded.fill_(1.0)
    assert lib.palimpsa_peer_signal(flag.data_ptr(), 3, stream) == 0    # sequence numbers only grow: 3 >= 1 and >= 2
    assert lib.palimpsa_peer_wait(flag.data_ptr(), 1, 5, guarded.data_ptr(), stream) == 0
    assert lib.palimpsa_peer_wait(flag.data_ptr(), 2, 5, guarded.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert flag.item() == 3 and lib.palimpsa_tensor_core_status() == 0 and bool((guarded == 1).all())
    assert lib.palimpsa_peer_wait(None, 1, 5, None, stream) == _lib.E_NULL
    assert lib.palimpsa_peer_signal(flag.data_ptr() + 4, 1, stream) == _lib.E_ALIGN   # flags are 8-byte aligned
