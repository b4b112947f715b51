"""Segment summaries through the C ABI against the float64 identity: the tensor-core (tcgen05/TMEM) kernel, which the
library picks for bf16 heads of at least 8192 state elements, and the element-wise kernel it picks below that."""
import ctypes as C

import pytest
import torch

from oracle import palimpsa_oracle as orc
from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu


def _summaries(inp, G, env_simt):
    from palimpsa_b200 import _lib as L
    from palimpsa_b200.ops.palimpsa import _core
    lib = L.lib()
    d = {n: inp[n].to(DEV).contiguous() for n in ("q", "k", "v", "b", "gt", "g", "Ip")}
    N, T, H, K = d["q"].shape
    V = d["v"].shape[-1]
    sg, bufs = _core.make_segments(N, G, _core.segment_len(T, G), H, V, K, d["q"].device, True)
    prob = _core._problem(d["q"], d["k"], d["v"], d["b"], d["gt"], d["g"], d["Ip"], None, None, None, None, 1.0, 0)
    for t in bufs.values():
        t.fill_(float("nan"))
    rc = lib.palimpsa_segment_summary(C.byref(prob), C.byref(sg), None)
    assert rc == 0
    torch.cuda.synchronize()
    return bufs, _core.segment_len(T, G)


@pytest.mark.parametrize("K,V,T,G", [(128, 128, 500, 3), (64, 128, 200, 2), (128, 64, 130, 1), (96, 96, 150, 2),   # tensor cores
                                     (32, 48, 70, 2), (48, 48, 200, 3)])                                          # element-wise
def test_segment_summary_matches_identity(K, V, T, G):
    from palimpsa_b200 import _lib as L
    inp = orc.make_inputs(K + T, B=2, T=T, H=2, K=K, V=V, dtype=torch.bfloat16)
    inp["gt"] = inp["gt"] * 0.1
    bufs, seg_len = _summaries(inp, G, False)
    assert L.lib().palimpsa_tensor_core_status() == 0
    for g in range(G):
        lo, hi = min(T, g * seg_len), min(T, (g + 1) * seg_len)
        SM, SJ, P = orc.segment_summary(inp["k"][:, lo:hi], inp["v"][:, lo:hi], inp["b"][:, lo:hi], inp["gt"][:, lo:hi],
                                        inp["g"])
        assert orc.rel_err(bufs["sum_M"][:, g, :, :, :K], SM) < 1e-2, (g, "M")
        assert orc.rel_err(bufs["sum_J"][:, g, :, :, :K], SJ) < 1e-2, (g, "J")
        assert orc.rel_err(bufs["decay"][:, g], P) < 1e-5
