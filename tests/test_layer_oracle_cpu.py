"""CPU checks of the layer-side oracle: independent torch functions and finite differences."""
import torch
import torch.nn.functional as F

from oracle import layer_oracle as lo


def test_epilogue_oracle_against_torch_rms_norm():
    d = lo.make_layer_inputs(0, B=2, T=5, H=3, Hq=3, K=8, V=20)
    z = d["o"].double() + d["x"].double() * d["D"].double().view(-1, 1)
    want = F.rms_norm(z, (20,), d["weight"].double(), eps=1e-5)
    got = lo.layer_epilogue_ref(d["o"], d["x"], d["D"], d["weight"], None, 1e-5)
    assert torch.allclose(got, want, rtol=1e-12, atol=1e-12)
    got_g = lo.layer_epilogue_ref(d["o"], d["x"], d["D"], d["weight"], d["gate"], 1e-5)
    assert torch.allclose(got_g, want * F.silu(d["gate"].double()), rtol=1e-12, atol=1e-12)
    plain = lo.layer_epilogue_ref(d["o"], None, None, d["weight"], None, 1e-5)
    assert torch.allclose(plain, F.rms_norm(d["o"].double(), (20,), d["weight"].double(), eps=1e-5), rtol=1e-12,
                          atol=1e-12)


def test_prologue_oracle_shapes_and_rounding_point():
    d = lo.make_layer_inputs(1, B=2, T=4, H=4, Hq=2, K=6, V=5, dtype=torch.bfloat16)
    args = [d[n] for n in ("q_raw", "k_raw", "x", "b_raw", "dt_raw", "bs_raw", "dt_bias", "b_scale")]
    q, k, v, b, dt = lo.layer_prologue_ref(*args, act_dtype=torch.bfloat16)
    assert q.shape == (2, 4, 4, 6) and v.shape == (2, 4, 4, 5) and dt.shape == (2, 4, 4)
    assert torch.allclose(q.norm(dim=-1), torch.ones(2, 4, 4, dtype=torch.float64))
    assert torch.equal(q[:, :, 0], q[:, :, 1]) and torch.equal(q[:, :, 2], q[:, :, 3])   # heads repeat in groups
    bs = torch.sigmoid(d["bs_raw"].float()).to(torch.bfloat16)                           # the layer's rounding point
    assert torch.equal(v, d["x"].double() * bs.double().unsqueeze(-1))
    # the layer's own expressions in its activation dtype agree to bf16 accuracy
    ql, kl, vl, bl, dtl = lo.layer_prologue_ref(*args, compute=torch.float32, act_dtype=torch.bfloat16)
    assert (bl.double() - b).abs().max() < 1e-5 and (dtl.double() - dt).abs().max() < 1e-5


def test_oracle_gradients_by_finite_differences():
    d = lo.make_layer_inputs(2, B=1, T=3, H=2, Hq=1, K=4, V=3)
    names = ("q_raw", "k_raw", "x", "b_raw", "dt_raw", "bs_raw", "dt_bias", "b_scale")
    args = [d[n].double().requires_grad_(True) for n in names]
    assert torch.autograd.gradcheck(lambda *a: lo.layer_prologue_ref(*a), args, eps=1e-6, atol=1e-6)
    eargs = [d[n].double().requires_grad_(True) for n in ("o", "x", "D", "weight", "gate")]
    assert torch.autograd.gradcheck(lambda *a: lo.layer_epilogue_ref(*a), eargs, eps=1e-6, atol=1e-6)


def test_epilogue_oracle_against_the_gated_norm_fixture():
    """The fixture holds outputs and gradients of flash-linear-attention's own FusedRMSNormGated (generated on a GPU
    by tests/golden/make_gated_norm_golden.py); the oracle's restatement must reproduce them."""
    import os

    import numpy as np
    import pytest
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gated_norm.npz")
    if not os.path.exists(path):
        pytest.skip("tests/golden/gated_norm.npz has not been generated yet")
    z = np.load(path)
    eps = float(z["meta_eps"])
    for tag, tol in (("f32", 2e-6), ("f32_v48", 2e-6), ("bf16", 1e-2)):
        zz = torch.from_numpy(z[f"{tag}_z"]).double().requires_grad_(True)
        gate = torch.from_numpy(z[f"{tag}_gate"]).double().requires_grad_(True)
        w = torch.from_numpy(z[f"{tag}_weight"]).double().requires_grad_(True)
        y = lo.layer_epilogue_ref(zz, None, None, w, gate, eps)
        y.backward(torch.from_numpy(z[f"{tag}_dy"]).double())
        for name, got in (("y", y.detach()), ("dz", zz.grad), ("dgate", gate.grad), ("dweight", w.grad)):
            ref = torch.from_numpy(z[f"{tag}_{name}"]).double()
            err = (got - ref).abs().max().item() / ref.abs().max().item()
            assert err <= tol, (tag, name, err)
