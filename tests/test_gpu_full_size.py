"""Properties that hold at any size, checked at the benchmark's FULL sizes (where the float64 oracle is out of
reach): the 170M-shaped batch (B=8 T=4096 H=6 d=128 bf16), a long sequence cut into segments, and the decode
configuration.  Exactness claims are bitwise: scaling by 2 and permuting the batch are exact in floating point."""
import pytest
import torch

from oracle.palimpsa_oracle import rel_err
from tests.gpu_util import DEV
from tests.helpers import TOL_BF16

pytestmark = pytest.mark.gpu
NAMES = ("q", "k", "v", "b", "gt", "g", "Ip")


def _inputs(B, T, H, K, V, seed=0):
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen)
    d = {"q": torch.nn.functional.normalize(rn(B, T, H, K), dim=-1).bfloat16(),
         "k": torch.nn.functional.normalize(rn(B, T, H, K), dim=-1).bfloat16(),
         "v": rn(B, T, H, V).bfloat16(), "b": torch.sigmoid(rn(B, T, H, V)).bfloat16(),
         "gt": torch.nn.functional.softplus(rn(B, T, H)), "g": torch.nn.functional.softplus(rn(H)),
         "Ip": torch.ones(H), "do": rn(B, T, H, V).bfloat16()}
    return {n: x.to(DEV) for n, x in d.items()}


def _fwd_bwd(d, **kw):
    from palimpsa_b200.ops import chunk_palimpsa
    leaves = {n: d[n].detach().clone().requires_grad_(True) for n in NAMES}
    out = chunk_palimpsa(*[leaves[n] for n in NAMES], output_final_state=True, **kw)
    o, mu, I = out
    o.backward(d["do"])
    res = {"o": o.detach(), "mu": mu, "I": I}
    res.update({"d" + n: leaves[n].grad for n in NAMES})
    return res


@pytest.fixture(scope="module")
def c2():
    d = _inputs(8, 4096, 6, 128, 128)
    return d, _fwd_bwd(d)


def test_full_size_results_are_finite_and_reproducible(c2):
    d, a = c2
    b = _fwd_bwd(d)
    for n in a:
        assert torch.isfinite(a[n].float()).all(), n
        assert torch.equal(a[n], b[n]), n


def test_full_size_linearity_in_v_and_in_the_output_gradient(c2):
    d, a = c2
    d2 = dict(d, v=d["v"] * 2)                       # M, and so o and every gradient but dv, doubles exactly
    r = _fwd_bwd(d2)
    assert torch.equal(r["o"], a["o"] * 2) and torch.equal(r["I"], a["I"]) and torch.equal(r["mu"], a["mu"] * 2)
    for n in ("dq", "dk", "db", "dgt", "dg", "dIp"):
        assert torch.equal(r[n], a[n] * 2), n
    assert torch.equal(r["dv"], a["dv"])
    d3 = dict(d, do=d["do"] * 2)                     # every gradient is linear in the output gradient
    r = _fwd_bwd(d3)
    for n in ("dq", "dk", "dv", "db", "dgt", "dg", "dIp"):
        assert torch.equal(r[n], a[n] * 2), n


def test_full_size_batch_permutation(c2):
    d, a = c2
    perm = torch.tensor([3, 0, 7, 1, 6, 2, 5, 4], device=DEV)
    dp = {n: (x[perm] if x.dim() >= 3 else x) for n, x in d.items()}
    r = _fwd_bwd(dp)
    for n in ("o", "mu", "I", "dq", "dk", "dv", "db", "dgt"):
        assert torch.equal(r[n], a[n][perm]), n
    for n in ("dg", "dIp"):                          # sums over the batch in another order
        assert rel_err(r[n], a[n]) < 1e-5, n


def test_full_size_state_passing_and_parameter_gradient_identity(c2):
    from palimpsa_b200.ops import chunk_palimpsa
    d, a = c2
    with torch.no_grad():
        h1 = {n: (x[:, :2048] if x.dim() >= 3 else x) for n, x in d.items()}
        h2 = {n: (x[:, 2048:] if x.dim() >= 3 else x) for n, x in d.items()}
        o1, mu1, I1 = chunk_palimpsa(*[h1[n] for n in NAMES], output_final_state=True)
        o2, mu2, I2 = chunk_palimpsa(*[h2[n] for n in NAMES], initial_mu_state=mu1, initial_I_state=I1,
                                     output_final_state=True)
    assert torch.equal(o1, a["o"][:, :2048])
    assert rel_err(o2, a["o"][:, 2048:]) < 1e-2 and rel_err(mu2, a["mu"]) < 1e-5 and rel_err(I2, a["I"]) < 1e-5
    # dgt = -g f df and dg = sum -gt f df share df:  dg[h] = sum_{b,t} gt * dgt / g
    dg_from_dgt = (d["gt"].double() * a["dgt"].double()).sum((0, 1)) / d["g"].double()
    assert rel_err(a["dg"], dg_from_dgt) < 1e-4


def test_long_sequence_segments_agree_with_the_serial_walk():
    d = _inputs(1, 32768, 12, 128, 128, seed=3)
    d["gt"] = d["gt"] * 0.05                         # slow decay: the boundary states matter over the whole sequence
    a = _fwd_bwd(d, num_segments=1)
    b = _fwd_bwd(d, num_segments=32)
    for n in a:
        assert rel_err(b[n], a[n]) <= TOL_BF16, (n, rel_err(b[n], a[n]))


def test_decode_configuration_matches_the_chunk_op():
    from palimpsa_b200.ops import chunk_palimpsa, decode_step
    B, H, K, V, T0, steps = 256, 12, 128, 128, 64, 16
    d = _inputs(B, T0 + steps, H, K, V, seed=5)
    with torch.no_grad():
        o_all, mu_all, I_all = chunk_palimpsa(*[d[n] for n in NAMES], output_final_state=True)
        pre = {n: (x[:, :T0] if x.dim() >= 3 else x) for n, x in d.items()}
        _, mu, I = chunk_palimpsa(*[pre[n] for n in NAMES], output_final_state=True)
        outs = []
        for t in range(T0, T0 + steps):
            tok = {n: (x[:, t:t + 1] if x.dim() >= 3 else x) for n, x in d.items()}
            outs.append(decode_step(*[tok[n] for n in NAMES], mu, I))
    assert rel_err(torch.cat(outs, 1), o_all[:, T0:]) < 1e-2
    assert rel_err(mu, mu_all) < 1e-5 and rel_err(I, I_all) < 1e-5
