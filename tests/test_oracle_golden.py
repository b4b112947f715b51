"""Pins the float64 oracle to outputs of the reference's own ``palimpsa_ref`` (tests/golden)."""
import pytest
import torch

from oracle import palimpsa_oracle as orc
from tests.helpers import GOLDEN_CASES, GOLDEN_TOL, GRADS, load_golden


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_oracle_matches_reference_fixture(case):
    inp, out, meta = load_golden(case)
    unc = bool(meta["unc"])
    cu = inp["cu_seqlens"].tolist() if "cu_seqlens" in inp else None
    res = orc.oracle_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["b"], inp["gt"], inp["g"], inp["Ip"], inp["do"],
                             inp["do_var"] if unc else None, inp.get("mu0"), inp.get("I0"),
                             scale=meta["scale"], cu_seqlens=cu)
    names = ["o", "final_mu", "final_I"] + (["o_var"] if unc else []) + list(GRADS)
    if "mu0" in inp:
        names += ["dmu0", "dI0"]
    for n in names:
        e = orc.rel_err(res[n], out[n])
        assert e < GOLDEN_TOL, f"{case}:{n} rel err {e:.3e}"


@pytest.mark.parametrize("case", ["check_style_unc", "bench_style", "initial_state"])
def test_explicit_backward_matches_autograd(case):
    """The hand-derived reverse recurrence (what the CUDA backward implements) equals autograd."""
    inp, out, meta = load_golden(case)
    unc = bool(meta["unc"])
    args = (inp["q"], inp["k"], inp["v"], inp["b"], inp["gt"], inp["g"], inp["Ip"], inp["do"],
            inp["do_var"] if unc else None, inp.get("mu0"), inp.get("I0"))
    ref = orc.oracle_fwd_bwd(*args, scale=meta["scale"])
    got = orc.oracle_backward_explicit(*args, scale=meta["scale"])
    for n in GRADS:
        e = orc.rel_err(got[n], ref[n])
        assert e < 1e-12, f"{case}:{n} rel err {e:.3e}"
    if "mu0" in inp:
        # (M, I) form -> (mu, I) form: dmu0 = dM0 * I0 ; dI0_api = dI0 + dM0 * mu0
        I0, mu0 = inp["I0"].double(), inp["mu0"].double()
        assert orc.rel_err(got["dM0"] * I0, ref["dmu0"]) < 1e-12
        assert orc.rel_err(got["dI0"] + got["dM0"] * mu0, ref["dI0"]) < 1e-12


def test_segment_identities():
    """Summaries + exclusive scan over segments reproduce the sequential end state and outputs."""
    d = orc.make_inputs(5, B=2, T=40, H=2, K=4, V=6, dtype=torch.float64)
    cuts = [0, 16, 32, 40]
    o_ref, _, mu_ref, I_ref = orc.oracle_forward(d["q"], d["k"], d["v"], d["b"], d["gt"], d["g"], d["Ip"])
    SM, SJ, P = [], [], []
    for s, e in zip(cuts[:-1], cuts[1:]):
        sm, sj, p = orc.segment_summary(d["k"][:, s:e], d["v"][:, s:e], d["b"][:, s:e], d["gt"][:, s:e], d["g"])
        SM.append(sm), SJ.append(sj), P.append(p)
    z = torch.zeros_like(SM[0])
    M_in, J_in, (M_end, J_end) = orc.combine_segments(SM, SJ, P, z, z)
    ipb = d["Ip"].double().view(1, -1, 1, 1)
    assert orc.rel_err(M_end / (J_end + ipb), mu_ref) < 1e-12
    assert orc.rel_err(J_end + ipb, I_ref) < 1e-12
    outs = []
    for (s, e), m, j in zip(zip(cuts[:-1], cuts[1:]), M_in, J_in):
        I0 = j + ipb
        o, _, _, _ = orc.oracle_forward(d["q"][:, s:e], d["k"][:, s:e], d["v"][:, s:e], d["b"][:, s:e],
                                        d["gt"][:, s:e], d["g"], d["Ip"], m / I0, I0)
        outs.append(o)
    assert orc.rel_err(torch.cat(outs, 1), o_ref) < 1e-12


def test_naive_fp32_port_matches_fixture():
    """The float32 port used as the CPU baseline reproduces the reference's numbers."""
    inp, out, meta = load_golden("bench_style")
    o, mu, I = orc.naive_recurrence_fp32(inp["q"], inp["k"], inp["v"], inp["b"], inp["gt"], inp["g"], inp["Ip"],
                                         output_final_state=True)
    assert orc.rel_err(o, out["o"]) < 1e-6
    assert orc.rel_err(mu, out["final_mu"]) < 1e-6
    assert orc.rel_err(I, out["final_I"]) < 1e-6
