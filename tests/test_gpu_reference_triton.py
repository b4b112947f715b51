"""The CUDA ops beside the reference's own Triton ops on the same device and the same seeded inputs.

Both are compared with the float64 oracle; the test prints the two error tables, requires the CUDA ops to be
within the operator's stated tolerance (1e-5 fp32, 2e-2 bf16; max|x-ref| / max|ref| per tensor) and the two
implementations to agree with each other.  The reference's kernels are only REPORTED against the tolerance:
chunk_palimpsa_bwd_kernel rebuilds M_{t-1} by a division (chunk_palimpsa_forgetting_scalar.py:409-410), which
costs it accuracy the CUDA kernels do not lose.  Needs the unmodified working copy under ``oracle/_ref/``.
"""
import pytest
import torch

from oracle import palimpsa_oracle as orc
from tests import reference_ops as R
from tests.gpu_util import DEV, compare, run_cuda, run_oracle
from tests.helpers import GRADS, TOL_BF16, TOL_FP32

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.available(), reason=R.SKIP_REASON)]
NAMES = ("q", "k", "v", "b", "gt", "g", "Ip")


def run_triton(inp, op="chunk", unc=False, scale=None, mu0=None, I0=None, cu=None, grads=True, chunk_size=16):
    """Same protocol as tests.gpu_util.run_cuda, through the reference's wrappers."""
    leaves = {n: inp[n].to(DEV).clone().requires_grad_(grads and op == "chunk") for n in NAMES}
    kw = dict(scale=scale, output_final_state=True, output_uncertainty=unc)
    if mu0 is not None:
        kw.update(initial_mu_state=mu0.to(DEV), initial_I_state=I0.to(DEV))
    if cu is not None:
        kw["cu_seqlens"] = torch.as_tensor(cu, dtype=torch.int32, device=DEV)
    if op == "chunk":
        out, fmu, fI = R.triton_chunk_palimpsa()(*[leaves[n] for n in NAMES], chunk_size=chunk_size, **kw)
    else:
        with torch.no_grad():                             # the reference's fused op has no backward (:250-253)
            out, fmu, fI = R.triton_fused_recurrent_palimpsa()(*[leaves[n] for n in NAMES], **kw)
    res = {"final_mu": fmu, "final_I": fI}
    if unc:
        res["o"], res["o_var"] = out
    else:
        res["o"] = out
    if grads and op == "chunk":
        loss = (res["o"].float() * inp["do"].to(DEV).float()).sum()
        if unc:
            loss = loss + (res["o_var"].float() * inp["do_var"].to(DEV).float()).sum()
        loss.backward()
        for n in NAMES:
            res["d" + n] = leaves[n].grad
    torch.cuda.synchronize()
    return {k: v.detach().float().cpu() for k, v in res.items()}


def _table(title, errs):
    print(f"  {title:<22}" + " ".join(f"{n}={e:.1e}" for n, e in errs.items()))


def _three_way(inp, tol, agree, what, op="chunk", **kw):
    ref = run_oracle(inp, **kw)
    got = run_cuda(inp, op, **kw)
    tri = run_triton(inp, op, **kw)
    names = [n for n in ("o", "o_var", "final_mu", "final_I") + GRADS if n in tri and n in ref]
    e_cuda = compare(got, ref, tol, names=names, what=f"{what}: CUDA vs float64 oracle")
    e_tri = {n: orc.rel_err(tri[n], ref[n]) for n in names}
    e_mut = {n: orc.rel_err(got[n], tri[n]) for n in names}
    print(f"\n{what} ({op})")
    _table("CUDA   vs oracle", e_cuda)
    _table("Triton vs oracle", e_tri)
    _table("CUDA   vs Triton", e_mut)
    bad = {n: e for n, e in e_mut.items() if not e <= agree}
    assert not bad, f"{what}: CUDA and the reference's Triton op disagree beyond {agree:g}: {bad}"
    return e_cuda, e_tri


def test_config1_fp32_three_way():
    """B=2, T=512, H=4, d_k=d_v=64, fp32, benchmark distributions."""
    inp = orc.make_inputs(0, B=2, T=512, H=4, K=64, V=64)
    _three_way(inp, TOL_FP32, 1e-3, "config 1")


def test_check_script_shape_three_way():
    """The reference check script's shape (check_palimpsa.py:46): B,L,H,D,N = 4,511,4,65,31, raw q/k, scale 1,
    both outputs in the loss."""
    inp = orc.make_inputs(42, B=4, T=511, H=4, K=31, V=65, check_style=True)
    _three_way(inp, TOL_FP32, 1e-3, "check-script shape", unc=True, scale=1.0)


def test_varlen_and_initial_state_three_way():
    """check_palimpsa.py's packed case [128, 64, rest] with an explicit initial state.  dIp is left out of the
    mutual comparison: with an initial state the reference kernel drops a term of it (:418)."""
    inp = orc.make_inputs(43, B=1, T=700, H=3, K=31, V=65, check_style=True)
    cu = [0, 128, 192, 700]
    mu0, I0 = orc.make_states(5, 3, 3, 65, 31, inp["Ip"])
    ref = run_oracle(inp, unc=True, scale=1.0, cu=cu, mu0=mu0, I0=I0)
    got = run_cuda(inp, "chunk", unc=True, scale=1.0, cu=cu, mu0=mu0, I0=I0)
    tri = run_triton(inp, "chunk", unc=True, scale=1.0, cu=cu, mu0=mu0, I0=I0)
    compare(got, ref, TOL_FP32, what="varlen + initial state: CUDA vs oracle")
    names = [n for n in got if n != "dIp"]
    e_tri = {n: orc.rel_err(tri[n], ref[n]) for n in names}
    e_mut = {n: orc.rel_err(got[n], tri[n]) for n in names}
    print("\nvarlen + initial state")
    _table("Triton vs oracle", e_tri)
    _table("CUDA   vs Triton", e_mut)
    assert all(e <= 1e-3 for e in e_mut.values()), e_mut


def test_bf16_c2_head_shape_three_way():
    """bf16 io at the benchmark's head shape (H=6, d_k=d_v=128), shortened to T=256."""
    inp = orc.make_inputs(7, B=2, T=256, H=6, K=128, V=128, dtype=torch.bfloat16)
    _three_way(inp, TOL_BF16, 4e-2, "bf16 d=128")


@pytest.mark.parametrize("T", [1, 17, 64])
def test_fused_recurrent_three_way(T):
    """Forward only: the reference's fused-recurrent op (what its layers call for q_len <= 64 at inference)."""
    inp = orc.make_inputs(T, B=3, T=T, H=4, K=64, V=64)
    mu0, I0 = orc.make_states(T + 1, 3, 4, 64, 64, inp["Ip"])
    _three_way(inp, TOL_FP32, 1e-4, f"fused T={T}", op="fused", unc=True, scale=1.0, mu0=mu0, I0=I0)
