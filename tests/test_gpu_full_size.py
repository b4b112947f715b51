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


# ------------------------------------------------------------------------------------------------------------
# The float64 oracle AT the benchmark's sizes.  The property tests above compare the CUDA path with itself; these
# compare it with the independent CPU recurrence on whole benchmark-length sequences (one sequence and one or
# two heads at a time is what the oracle finishes in seconds).  Bound: 2e-2 (bf16), max|x-ref| / max|ref|.
# ------------------------------------------------------------------------------------------------------------
from oracle import palimpsa_oracle as orc  # noqa: E402

PER_TOKEN = ("dq", "dk", "dv", "db", "dgt")


def _cpu_slice(d, seq, heads, lo=None, hi=None):
    """Sequence ``seq``, heads ``heads`` and tokens [lo, hi) of the device dict ``d`` as CPU tensors."""
    out = {}
    for n, x in d.items():
        x = x.detach().cpu()
        if x.dim() >= 3:
            x = x[seq:seq + 1, lo:hi][:, :, heads]
        else:
            x = x[heads]
        out[n] = x
    return out


def _explicit(sl, **kw):
    return orc.oracle_backward_explicit(*[sl[n] for n in NAMES], sl["do"], block=256, **kw)


def _check(got, ref, names, what, tol=TOL_BF16):
    errs = {n: rel_err(got[n], ref[n]) for n in names}
    print(f"\n{what}: " + " ".join(f"{n}={e:.1e}" for n, e in errs.items()))
    bad = {n: e for n, e in errs.items() if not e <= tol}
    assert not bad, (what, bad)


def test_c2_sequence_matches_the_float64_oracle(c2):
    """One whole sequence of the 170M-shaped batch (T = 4096): outputs and final states on all 6 heads, the seven
    gradients on two heads (dg / dIp are sums over the batch, so they come from a call on that slice alone)."""
    d, a = c2
    seq = 5
    sl = _cpu_slice(d, seq, slice(0, 6))
    with torch.no_grad():
        o, _, mu, I = orc.oracle_forward(*[sl[n] for n in NAMES])
    got = {"o": a["o"][seq:seq + 1], "mu": a["mu"][seq:seq + 1], "I": a["I"][seq:seq + 1]}
    _check(got, {"o": o, "mu": mu, "I": I}, ("o", "mu", "I"), "C2 sequence, forward, 6 heads")
    heads = slice(2, 4)
    sl2 = _cpu_slice(d, seq, heads)
    ref = _explicit(sl2)
    got = {n: a[n][seq:seq + 1][:, :, heads] for n in PER_TOKEN}
    got["o"] = a["o"][seq:seq + 1][:, :, heads]
    _check(got, ref, ("o",) + PER_TOKEN, "C2 sequence, gradients, heads 2-3")
    alone = _fwd_bwd({n: x.to(DEV) for n, x in sl2.items()})
    _check(alone, ref, ("dg", "dIp") + PER_TOKEN, "C2 sequence alone (parameter gradients)")


def test_packed_batch_documents_match_the_float64_oracle():
    """The packed training batch (32 768 tokens, documents of seeded random length in [128, 4096], states reset at
    every boundary): the longest and the shortest document against the oracle run on that document alone."""
    T, H = 32768, 6
    gen = torch.Generator().manual_seed(0)
    lens, tot = [], 0
    while tot < T:
        n = min(int(torch.randint(128, 4097, (1,), generator=gen).item()), T - tot)
        lens.append(n)
        tot += n
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    d = _inputs(1, T, H, 128, 128, seed=0)
    a = _fwd_bwd(d, cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=DEV))
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    heads = slice(0, 2)
    for doc in (order[-1], order[0]):
        lo, hi = cu[doc], cu[doc + 1]
        ref = _explicit(_cpu_slice(d, 0, heads, lo, hi))
        got = {n: a[n][:, lo:hi][:, :, heads] for n in ("o",) + PER_TOKEN}
        got["final_mu"], got["final_I"] = a["mu"][doc:doc + 1, heads], a["I"][doc:doc + 1, heads]
        _check(got, ref, ("o", "final_mu", "final_I") + PER_TOKEN, f"packed batch, document {doc} ({hi - lo} tokens)")


def test_long_segmented_sequence_matches_the_float64_oracle():
    """One 32 768-token sequence cut into 32 segments (tensor-core summaries, boundary scans, carried-gradient
    terms): every token's output and gradients, the final state and the parameter gradients of one head against a
    float64 walk of the whole sequence (which also supplies the true boundary states and carried gradients)."""
    d = _inputs(1, 32768, 2, 128, 128, seed=11)
    d["gt"] = d["gt"] * 0.05                         # slow decay: early tokens reach the end of the sequence
    a = _fwd_bwd(d, num_segments=32)
    head = slice(1, 2)
    ref = _explicit(_cpu_slice(d, 0, head))
    got = {n: a[n][:, :, head] for n in ("o",) + PER_TOKEN}
    got.update(final_mu=a["mu"][:, head], final_I=a["I"][:, head], dg=a["dg"][head], dIp=a["dIp"][head])
    names = ("o", "final_mu", "final_I", "dg", "dIp") + PER_TOKEN
    _check(got, ref, names, "32 segments x 1024 tokens, all tokens")
    for lo, hi, tag in ((0, 2048, "first"), (32768 - 2048, 32768, "last")):
        win = {n: got[n][:, lo:hi] for n in ("o",) + PER_TOKEN}
        _check(win, {n: ref[n][:, lo:hi] for n in win}, tuple(win), f"{tag} 2048 tokens")


def test_small_head_batch_matches_the_float64_oracle():
    """The reference's 170M configuration (16 heads of d_k = d_v = 48) at the benchmark's length: B = 8, T = 4096,
    bf16, through the 48-row tiles (3 forward / 6 backward warps per CTA).  One whole sequence: outputs and final
    states on four heads, the per-token gradients on two; parameter gradients from a call on that slice alone."""
    d = _inputs(8, 4096, 16, 48, 48)
    a = _fwd_bwd(d)
    seq = 3
    sl = _cpu_slice(d, seq, slice(4, 8))
    with torch.no_grad():
        o, _, mu, I = orc.oracle_forward(*[sl[n] for n in NAMES])
    got = {"o": a["o"][seq:seq + 1][:, :, 4:8], "mu": a["mu"][seq:seq + 1][:, 4:8], "I": a["I"][seq:seq + 1][:, 4:8]}
    _check(got, {"o": o, "mu": mu, "I": I}, ("o", "mu", "I"), "170M heads, forward, heads 4-7")
    heads = slice(9, 11)
    sl2 = _cpu_slice(d, seq, heads)
    ref = _explicit(sl2)
    got = {n: a[n][seq:seq + 1][:, :, heads] for n in PER_TOKEN}
    _check(got, ref, PER_TOKEN, "170M heads, gradients, heads 9-10")
    alone = _fwd_bwd({n: x.to(DEV) for n, x in sl2.items()})
    _check(alone, ref, ("dg", "dIp") + PER_TOKEN, "170M heads, slice alone (parameter gradients)")
