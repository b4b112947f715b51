"""Collected last: after every other GPU test of the session has run in this process, no bounded in-kernel
wait (tensor-core kernels' mbarriers, the backward's split-phase barriers) may have given up."""
import pytest

pytestmark = pytest.mark.gpu


def test_no_bounded_wait_gave_up():
    from palimpsa_b200 import _lib
    import torch
    torch.cuda.synchronize()
    assert _lib.lib().palimpsa_tensor_core_status() == 0
