"""Decode path: the dedicated single-token kernel (in-place state cache) against the float64 oracle."""
import pytest
import torch

from oracle import palimpsa_oracle as orc
from tests.gpu_util import DEV
from tests.helpers import TOL_BF16, TOL_FP32

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K,V,dtype", [(128, 128, torch.bfloat16), (64, 40, torch.float32), (16, 32, torch.float32),
                                       (32, 8, torch.float16), (48, 48, torch.float32)])
def test_decode_steps_match_oracle(K, V, dtype):
    from palimpsa_b200.ops import decode_step, fused_recurrent_palimpsa
    N, H, T0, steps = 3, 2, 20, 6
    inp = orc.make_inputs(K + V, B=N, T=T0 + steps, H=H, K=K, V=V, dtype=dtype)
    d = {n: inp[n].to(DEV) for n in ("q", "k", "v", "b", "gt", "g", "Ip")}
    sl = lambda a, b: {n: (x[:, a:b] if x.dim() >= 3 else x) for n, x in d.items()}
    # prefill with the recurrent op, then decode token by token on the cache, in place
    _, mu, I = fused_recurrent_palimpsa(**sl(0, T0), output_final_state=True)
    ref_o, ref_ov, ref_mu, ref_I = orc.oracle_forward(inp["q"], inp["k"], inp["v"], inp["b"], inp["gt"], inp["g"],
                                                      inp["Ip"], output_uncertainty=True)
    tol = TOL_FP32 if dtype == torch.float32 else TOL_BF16
    outs, outvs = [], []
    mu_ptr = mu.data_ptr()
    for t in range(T0, T0 + steps):
        o, ov = decode_step(**sl(t, t + 1), mu_state=mu, I_state=I, output_uncertainty=True)
        outs.append(o)
        outvs.append(ov)
    assert mu.data_ptr() == mu_ptr
    assert orc.rel_err(torch.cat(outs, 1), ref_o[:, T0:]) <= tol
    assert orc.rel_err(torch.cat(outvs, 1), ref_ov[:, T0:]) <= tol
    assert orc.rel_err(mu, ref_mu) <= tol and orc.rel_err(I, ref_I) <= tol
    # the reference-style call (new state tensors per step) gives the same numbers
    _, mu2, I2 = fused_recurrent_palimpsa(**sl(0, T0), output_final_state=True)
    for t in range(T0, T0 + steps):
        o2, mu2, I2 = fused_recurrent_palimpsa(**sl(t, t + 1), initial_mu_state=mu2, initial_I_state=I2,
                                               output_final_state=True)
    assert torch.equal(o2, outs[-1])
    assert torch.equal(mu2, mu) and torch.equal(I2, I)


def test_graph_replay_equals_eager_decode():
    """The step captured in a CUDA graph: same outputs and same cache as step-by-step launches, bit for bit."""
    from palimpsa_b200.ops import DecodeGraph, decode_step, fused_recurrent_palimpsa
    N, H, K, V, T0, steps = 4, 3, 64, 64, 12, 8
    inp = orc.make_inputs(77, B=N, T=T0 + steps, H=H, K=K, V=V, dtype=torch.bfloat16)
    d = {n: inp[n].to(DEV) for n in ("q", "k", "v", "b", "gt", "g", "Ip")}
    sl = lambda a, b: {n: (x[:, a:b] if x.dim() >= 3 else x) for n, x in d.items()}
    _, mu, I = fused_recurrent_palimpsa(**sl(0, T0), output_final_state=True)
    mu_g, I_g = mu.clone(), I.clone()
    dec = DecodeGraph(d["g"], d["Ip"], mu_g, I_g, dtype=torch.bfloat16, output_uncertainty=True)
    assert torch.equal(mu_g, mu) and torch.equal(I_g, I)          # building the graph leaves the cache alone
    for t in range(T0, T0 + steps):
        o, ov = decode_step(**sl(t, t + 1), mu_state=mu, I_state=I, output_uncertainty=True)
        tok = sl(t, t + 1)
        og, ovg = dec.step(tok["q"], tok["k"], tok["v"], tok["b"], tok["gt"])
        assert torch.equal(og, o) and torch.equal(ovg, ov), t
    assert torch.equal(mu_g, mu) and torch.equal(I_g, I)
