"""Host-buffer pipeline: slicing the batch across copy/compute streams must not change any result."""
import pytest
import torch

from oracle import palimpsa_oracle as orc
from tests.gpu_util import DEV, run_cuda

pytestmark = pytest.mark.gpu


def test_host_pipeline_equals_plain_call():
    from palimpsa_b200.host_pipeline import fwd_bwd_from_host
    inp = orc.make_inputs(6, B=5, T=130, H=2, K=64, V=64, dtype=torch.bfloat16)
    host = {n: inp[n].pin_memory() for n in ("q", "k", "v", "b", "gt", "g", "Ip", "do")}
    ref = run_cuda(inp, "chunk")
    for slices in (1, 3, 5, (1, 3, 1)):
        got = fwd_bwd_from_host(host, DEV, slices=slices)
        got = {n: x.clone() for n, x in got.items()}
        for n in ("o", "dq", "dk", "dv", "db", "dgt"):
            assert torch.equal(got[n], ref[n]), (slices, n)
        assert orc.rel_err(got["dg"], ref["dg"]) < 1e-5 and orc.rel_err(got["dIp"], ref["dIp"]) < 1e-5


def test_ramped_widths_cover_the_batch():
    from palimpsa_b200.host_pipeline import HostPipeline, ramped_widths
    assert ramped_widths(8) == [1, 2, 2, 2, 1] and ramped_widths(5) == [1, 2, 1, 1] and ramped_widths(1) == [1]
    for b in range(1, 12):
        assert sum(ramped_widths(b)) == b
    inp = orc.make_inputs(6, B=3, T=32, H=1, K=32, V=32, dtype=torch.bfloat16)
    host = {n: inp[n].pin_memory() for n in ("q", "k", "v", "b", "gt", "g", "Ip", "do")}
    with pytest.raises(ValueError):
        HostPipeline(host, DEV, slices=(1, 1))
