"""Helpers for the GPU parity tests: run the CUDA ops and the float64 oracle on the same inputs."""
import torch

from oracle import palimpsa_oracle as orc
from tests.helpers import GRADS, TOL_BF16, TOL_FP32

DEV = "cuda:0"


def run_cuda(inp, op="chunk", unc=False, scale=None, mu0=None, I0=None, cu=None, grads=True):
    from palimpsa_b200.ops import chunk_palimpsa, fused_recurrent_palimpsa
    fn = chunk_palimpsa if op == "chunk" else fused_recurrent_palimpsa
    names = ("q", "k", "v", "b", "gt", "g", "Ip")
    leaves = {n: inp[n].to(DEV).clone().requires_grad_(grads) for n in names}
    kw = dict(scale=scale, output_final_state=True, output_uncertainty=unc)
    if mu0 is not None:
        kw.update(initial_mu_state=mu0.to(DEV), initial_I_state=I0.to(DEV))
    if cu is not None:
        kw["cu_seqlens"] = torch.as_tensor(cu, dtype=torch.int32, device=DEV)
    out, fmu, fI = fn(*[leaves[n] for n in names], **kw)
    res = {"final_mu": fmu, "final_I": fI}
    if unc:
        res["o"], res["o_var"] = out
    else:
        res["o"] = out
    if grads:
        loss = (res["o"].float() * inp["do"].to(DEV).float()).sum()
        if unc:
            loss = loss + (res["o_var"].float() * inp["do_var"].to(DEV).float()).sum()
        loss.backward()
        for n in names:
            res["d" + n] = leaves[n].grad
    torch.cuda.synchronize()
    return {k: v.detach().cpu() for k, v in res.items()}


def run_oracle(inp, unc=False, scale=None, mu0=None, I0=None, cu=None):
    return orc.oracle_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["b"], inp["gt"], inp["g"], inp["Ip"], inp["do"],
                              inp["do_var"] if unc else None, mu0, I0, scale=scale, cu_seqlens=cu)


def compare(got, ref, tol, names=None, what=""):
    names = names or [n for n in ("o", "o_var", "final_mu", "final_I") + GRADS if n in got and n in ref]
    errs = {n: orc.rel_err(got[n], ref[n]) for n in names}
    bad = {n: e for n, e in errs.items() if not (e <= tol)}
    report = " ".join(f"{n}={e:.2e}" for n, e in errs.items())
    assert not bad, f"{what} tol={tol:g} FAILED {bad} | all: {report}"
    return errs


def tol_for(dtype):
    return TOL_FP32 if dtype == torch.float32 else TOL_BF16
