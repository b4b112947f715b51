"""Fused layer prologue / epilogue kernels against the torch restatement of the layer's lines."""
import pytest
import torch

from oracle import layer_oracle as lo
from oracle.palimpsa_oracle import rel_err
from tests.gpu_util import DEV, tol_for

pytestmark = pytest.mark.gpu

PRO_IN = ("q_raw", "k_raw", "x", "b_raw", "dt_raw", "bs_raw", "dt_bias", "b_scale")
PRO_OUT = ("q", "k", "v", "b", "gt")
PRO_COT = ("dq", "dk", "dv", "db", "dgt")


def _check(got, ref, tol, what):
    errs = {n: rel_err(got[n], ref[n]) for n in ref}
    bad = {n: e for n, e in errs.items() if not e <= tol}
    assert not bad, f"{what} tol={tol:g} FAILED {bad} | all: " + " ".join(f"{n}={e:.2e}" for n, e in errs.items())


def _prologue_pair(d, dtype):
    from palimpsa_b200.layers import layer_prologue
    act = None if dtype == torch.float32 else dtype
    ref_in = [d[n].double().requires_grad_(True) for n in PRO_IN]
    ref_out = lo.layer_prologue_ref(*ref_in, act_dtype=act)
    sum((o * d[c].double()).sum() for o, c in zip(ref_out, PRO_COT)).backward()
    ref = dict(zip(PRO_OUT, ref_out))
    ref.update({"d_" + n: t.grad for n, t in zip(PRO_IN, ref_in)})
    cu_in = [d[n].to(DEV).requires_grad_(True) for n in PRO_IN]
    cu_out = layer_prologue(*cu_in)
    assert all(o.dtype == dtype for o in cu_out[:4]) and cu_out[4].dtype == torch.float32
    sum((o.float() * d[c].to(DEV).float()).sum() for o, c in zip(cu_out, PRO_COT)).backward()
    torch.cuda.synchronize()
    got = dict(zip(PRO_OUT, cu_out))
    got.update({"d_" + n: t.grad for n, t in zip(PRO_IN, cu_in)})
    return got, ref


@pytest.mark.parametrize("shape", [(2, 37, 4, 2, 48, 40), (1, 5, 3, 3, 31, 65), (1, 9, 2, 1, 256, 200),
                                   (2, 16, 6, 6, 128, 128), (1, 1, 1, 1, 16, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prologue_matches_the_layer(shape, dtype):
    B, T, H, Hq, K, V = shape
    d = lo.make_layer_inputs(3, B, T, H, Hq, K, V, dtype)
    got, ref = _prologue_pair(d, dtype)
    _check(got, ref, tol_for(dtype), f"prologue {shape} {dtype}")


def _epilogue_pair(d, dtype, residual, gated):
    from palimpsa_b200.layers import layer_epilogue
    names = ("o", "x", "D", "weight", "gate")
    use = {"o": True, "x": residual, "D": residual, "weight": True, "gate": gated}
    ref_in = {n: d[n].double().requires_grad_(True) if use[n] else None for n in names}
    y = lo.layer_epilogue_ref(*[ref_in[n] for n in names], eps=1e-5)
    (y * d["dy"].double()).sum().backward()
    ref = {"y": y}
    ref.update({"d_" + n: t.grad for n, t in ref_in.items() if t is not None})
    cu_in = {n: d[n].to(DEV).requires_grad_(True) if use[n] else None for n in names}
    yc = layer_epilogue(*[cu_in[n] for n in names], eps=1e-5)
    assert yc.dtype == dtype
    (yc.float() * d["dy"].to(DEV).float()).sum().backward()
    torch.cuda.synchronize()
    got = {"y": yc}
    got.update({"d_" + n: t.grad for n, t in cu_in.items() if t is not None})
    return got, ref


@pytest.mark.parametrize("shape", [(2, 37, 4, 40), (1, 5, 3, 65), (2, 16, 6, 128), (1, 7, 2, 640), (1, 3, 1, 1024),
                                   (2, 300, 6, 128)])
@pytest.mark.parametrize("dtype,residual,gated", [(torch.float32, True, True), (torch.float32, False, False),
                                                  (torch.bfloat16, True, True), (torch.float16, True, False)])
def test_epilogue_matches_the_layer(shape, dtype, residual, gated):
    B, T, H, V = shape
    d = lo.make_layer_inputs(4, B, T, H, H, 16, V, dtype)
    got, ref = _epilogue_pair(d, dtype, residual, gated)
    _check(got, ref, tol_for(dtype), f"epilogue {shape} {dtype} residual={residual} gated={gated}")


def test_repeat_runs_are_bitwise_equal_and_empty_batches_pass():
    from palimpsa_b200.layers import layer_epilogue, layer_prologue
    d = lo.make_layer_inputs(5, 2, 200, 6, 3, 64, 64, torch.bfloat16)
    a, _ = _epilogue_pair(d, torch.bfloat16, True, True)
    b, _ = _epilogue_pair(d, torch.bfloat16, True, True)
    for n in a:
        assert torch.equal(a[n], b[n]), n
    p1, _ = _prologue_pair(d, torch.bfloat16)
    p2, _ = _prologue_pair(d, torch.bfloat16)
    for n in p1:
        assert torch.equal(p1[n], p2[n]), n
    e = lo.make_layer_inputs(5, 0, 4, 2, 2, 16, 16, torch.bfloat16)
    out = layer_prologue(*[e[n].to(DEV) for n in PRO_IN])
    assert out[0].shape == (0, 4, 2, 16)
    y = layer_epilogue(e["o"].to(DEV), e["x"].to(DEV), e["D"].to(DEV), e["weight"].to(DEV), e["gate"].to(DEV))
    assert y.shape == (0, 4, 2, 16)


def test_argument_errors():
    from palimpsa_b200.layers import layer_epilogue, layer_prologue
    d = lo.make_layer_inputs(6, 1, 2, 4, 2, 16, 16)
    g = {n: t.to(DEV) for n, t in d.items()}
    with pytest.raises(ValueError):
        layer_prologue(g["q_raw"][..., :1, :].expand(1, 2, 3, 16), g["k_raw"], g["x"], g["b_raw"], g["dt_raw"],
                       g["bs_raw"], g["dt_bias"], g["b_scale"])
    with pytest.raises(ValueError):
        layer_epilogue(g["o"], g["x"], None, g["weight"])
    with pytest.raises(RuntimeError):
        layer_epilogue(d["o"], d["x"], d["D"], d["weight"])           # CPU tensors: no CPU path
    wide = torch.zeros(1, 1, 1, 1028, device=DEV)
    with pytest.raises(RuntimeError):
        layer_epilogue(wide, None, None, torch.ones(1028, device=DEV))   # V above the kernels' maximum
