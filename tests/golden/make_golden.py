"""Generate the golden fixtures in this folder from the REFERENCE's own naive recurrence.

Run once, in a container where the reference checkout is available:

    PALIMPSA_REFERENCE=/path/to/Palimpsa python tests/golden/make_golden.py

It imports ``palimpsa_ref`` (palimpsa/ops/palimpsa/chunk_palimpsa_forgetting_scalar.py:669-725)
unmodified, runs it in float32 under autograd on small seeded inputs and stores inputs, outputs,
final states and all gradients as ``.npz``.  The tests never import the reference; they read
these files.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.palimpsa_oracle import make_inputs, make_states  # noqa: E402


def _ref():
    root = os.environ.get("PALIMPSA_REFERENCE")
    if not root or not os.path.isdir(os.path.join(root, "palimpsa")):
        raise SystemExit("set PALIMPSA_REFERENCE to the root of a checkout of the reference project")
    sys.path.insert(0, root)
    from palimpsa.ops.palimpsa import palimpsa_ref
    return palimpsa_ref


def _run(palimpsa_ref, inp, scale, unc, mu0=None, I0=None):
    leaves = {n: inp[n].clone().float().requires_grad_(True) for n in ("q", "k", "v", "b", "gt", "g", "Ip")}
    extra = {}
    if mu0 is not None:
        extra = {"initial_mu_state": mu0.clone().requires_grad_(True),
                 "initial_I_state": I0.clone().requires_grad_(True)}
    out, fmu, fI = palimpsa_ref(*[leaves[n] for n in ("q", "k", "v", "b", "gt", "g", "Ip")], scale=scale,
                                output_final_state=True, output_uncertainty=unc, **extra)
    if unc:
        o, o_var = out
        loss = (o * inp["do"]).sum() + (o_var * inp["do_var"]).sum()
    else:
        o, o_var = out, None
        loss = (o * inp["do"]).sum()
    loss.backward()
    res = {"o": o.detach(), "final_mu": fmu.detach(), "final_I": fI.detach()}
    if unc:
        res["o_var"] = o_var.detach()
    for n in leaves:
        res["d" + n] = leaves[n].grad
    if mu0 is not None:
        res["dmu0"] = extra["initial_mu_state"].grad
        res["dI0"] = extra["initial_I_state"].grad
    return res


def _save(name, inp, res, meta, **more):
    arrs = {"in_" + n: x.numpy() for n, x in inp.items()}
    arrs.update({"out_" + n: x.numpy() for n, x in res.items()})
    arrs.update({"meta_" + n: np.asarray(x) for n, x in meta.items()})
    arrs.update({n: x.numpy() for n, x in more.items()})
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrs)
    print(name, {n: tuple(x.shape) for n, x in res.items()})


def main():
    torch.manual_seed(0)
    palimpsa_ref = _ref()

    # 1. the manual check's distributions and odd, non-power-of-two dims (check_palimpsa.py:46-59),
    #    scaled down; scale=1 so that both o_var conventions agree; loss uses o and o_var.
    inp = make_inputs(42, B=2, T=37, H=2, K=7, V=9, check_style=True)
    _save("check_style_unc", inp, _run(palimpsa_ref, inp, 1.0, True), {"scale": 1.0, "unc": 1})

    # 2. benchmark distributions, default scale, no uncertainty output.
    inp = make_inputs(0, B=2, T=48, H=2, K=16, V=16)
    _save("bench_style", inp, _run(palimpsa_ref, inp, None, False), {"scale": 16 ** -0.5, "unc": 0})

    # 3. explicit initial state with I0 > Ip (check_palimpsa.py:197-205); autograd gives the exact dIp.
    inp = make_inputs(7, B=2, T=21, H=3, K=8, V=12, check_style=True)
    mu0, I0 = make_states(8, 2, 3, 12, 8, inp["Ip"])
    _save("initial_state", inp, _run(palimpsa_ref, inp, 1.0, True, mu0, I0), {"scale": 1.0, "unc": 1},
          in_mu0=mu0, in_I0=I0)

    # 4. packed variable-length batch, ground truth = per-segment loop (check_palimpsa.py:157-179).
    inp = make_inputs(3, B=1, T=45, H=2, K=8, V=8, check_style=True)
    cu = [0, 20, 27, 45]
    acc = None
    for n in range(len(cu) - 1):
        sl = {x: (inp[x][:, cu[n]:cu[n + 1]] if inp[x].dim() >= 3 else inp[x]) for x in inp}
        r = _run(palimpsa_ref, sl, 1.0, True)
        if acc is None:
            acc = {x: [y] for x, y in r.items()}
        else:
            for x, y in r.items():
                acc[x].append(y)
    res = {}
    for x, ys in acc.items():
        if x in ("dg", "dIp"):
            res[x] = torch.stack(ys).sum(0)
        elif x in ("final_mu", "final_I"):
            res[x] = torch.cat(ys, 0)
        else:
            res[x] = torch.cat(ys, 1)
    _save("varlen", inp, res, {"scale": 1.0, "unc": 1}, in_cu_seqlens=torch.tensor(cu, dtype=torch.int32))


if __name__ == "__main__":
    main()
