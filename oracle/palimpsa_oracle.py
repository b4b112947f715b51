"""CPU oracle for the Palimpsa operator -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

This module restates, in float64 on the CPU, the algorithm that the reference
defines in ``palimpsa/ops/palimpsa/chunk_palimpsa_forgetting_scalar.py:669-725``
(``palimpsa_ref``, the per-timestep recurrence) and the gradient algebra that
its backward kernel implements at ``:334-434`` of the same file.  It exists so
that the CUDA kernels can be checked against something independent of them.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import it.  The shipped operator never does: it has no CPU path at all.

Parity pin: ``tests/golden/*.npz`` hold outputs of the reference's own
``palimpsa_ref`` (float32, run under autograd) on seeded inputs; the generating
script sits beside them.  ``tests/test_oracle_golden.py`` checks this oracle
against every one of those fixtures.

Conventions
-----------
* shapes: ``q,k [B,T,H,K]``, ``v,b [B,T,H,V]``, ``gt [B,T,H]``, ``g,Ip [H]``,
  states ``[N,H,V,K]`` (V-major, K contiguous) exactly as the reference
  (``chunk_palimpsa_forgetting_scalar.py:475-476``).
* the uncertainty output follows the shipped kernels
  (``chunk_palimpsa_forgetting_scalar.py:204``, ``fused_recurrent_palimpsa.py:136``):
  ``o_var = scale * sum_k q^2 / I``.  ``palimpsa_ref`` itself uses ``scale**2``
  (``:709,718``); pass ``var_scale_power=2`` to reproduce that.
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch

F64 = torch.float64


def _f64(x):
    return None if x is None else x.detach().to("cpu", F64)


def oracle_forward(q, k, v, b, gt, g, Ip, initial_mu_state=None, initial_I_state=None,
                   scale=None, output_uncertainty=False, var_scale_power=1, dtype=F64):
    """Differentiable per-timestep recurrence (``palimpsa_ref`` without the fp32 casts).

    Follows chunk_palimpsa_forgetting_scalar.py:697-725 line by line, but in the
    (M, I) form the fused kernel uses (fused_recurrent_palimpsa.py:99-125):
    ``M = f*M + v k^T``, ``I = f*I + (1-f)*Ip + b (k*k)^T``, ``mu = M/I``.
    Returns ``(o, o_var or None, final_mu, final_I)`` in ``dtype``.
    """
    q, k, v, b, gt, g, Ip = [x.to(dtype) for x in (q, k, v, b, gt, g, Ip)]
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    ipb = Ip.view(1, H, 1, 1)
    if initial_mu_state is None:
        mu = torch.zeros(B, H, V, K, dtype=dtype)
        I = ipb.expand(B, H, V, K)
    else:
        mu = initial_mu_state.to(dtype)
        I = initial_I_state.to(dtype)
    M = mu * I
    ys, yvs = [], []
    for t in range(T):
        f = torch.exp(-gt[:, t] * g.view(1, H)).view(B, H, 1, 1)
        M = f * M + v[:, t, :, :, None] * k[:, t, :, None, :]
        I = f * I + (1.0 - f) * ipb + b[:, t, :, :, None] * (k[:, t, :, None, :] ** 2)
        mu = M / I
        ys.append(scale * torch.einsum("bhvk,bhk->bhv", mu, q[:, t]))
        if output_uncertainty:
            yvs.append((scale ** var_scale_power) * torch.einsum("bhvk,bhk->bhv", 1.0 / I, q[:, t] ** 2))
    if T > 0:
        o = torch.stack(ys, dim=1)
        o_var = torch.stack(yvs, dim=1) if output_uncertainty else None
    else:
        o = torch.zeros(B, 0, H, V, dtype=dtype)
        o_var = torch.zeros(B, 0, H, V, dtype=dtype) if output_uncertainty else None
    return o, o_var, mu, I


def oracle_forward_varlen(q, k, v, b, gt, g, Ip, cu_seqlens: Sequence[int], initial_mu_state=None,
                          initial_I_state=None, scale=None, output_uncertainty=False,
                          var_scale_power=1, dtype=F64):
    """Packed variant: batch 1, one independent recurrence per ``cu_seqlens`` segment.

    Mirrors the per-segment loop the reference's check script uses as ground
    truth (palimpsa/check_palimpsa.py:157-179).
    """
    cu = [int(x) for x in cu_seqlens]
    outs, outvs, mus, Is = [], [], [], []
    for n in range(len(cu) - 1):
        s, e = cu[n], cu[n + 1]
        mu0 = None if initial_mu_state is None else initial_mu_state[n:n + 1]
        I0 = None if initial_I_state is None else initial_I_state[n:n + 1]
        o, ov, mu, I = oracle_forward(q[:, s:e], k[:, s:e], v[:, s:e], b[:, s:e], gt[:, s:e], g, Ip,
                                      mu0, I0, scale, output_uncertainty, var_scale_power, dtype)
        outs.append(o)
        outvs.append(ov)
        mus.append(mu)
        Is.append(I)
    o = torch.cat(outs, dim=1)
    o_var = torch.cat(outvs, dim=1) if output_uncertainty else None
    return o, o_var, torch.cat(mus, 0), torch.cat(Is, 0)


def oracle_fwd_bwd(q, k, v, b, gt, g, Ip, do, do_var=None, initial_mu_state=None, initial_I_state=None,
                   scale=None, cu_seqlens=None, var_scale_power=1) -> Dict[str, torch.Tensor]:
    """Forward + autograd backward in float64.  Returns outputs, final states and the 7 gradients
    (plus the gradients of explicit initial states, which the reference op does not return).
    """
    leaves = [_f64(x).requires_grad_(True) for x in (q, k, v, b, gt, g, Ip)]
    mu0 = I0 = None
    if initial_mu_state is not None:
        mu0 = _f64(initial_mu_state).requires_grad_(True)
        I0 = _f64(initial_I_state).requires_grad_(True)
    unc = do_var is not None
    if cu_seqlens is None:
        o, o_var, fmu, fI = oracle_forward(*leaves, mu0, I0, scale, unc, var_scale_power)
    else:
        o, o_var, fmu, fI = oracle_forward_varlen(*leaves, cu_seqlens, mu0, I0, scale, unc, var_scale_power)
    loss = (o * _f64(do)).sum()
    if unc:
        loss = loss + (o_var * _f64(do_var)).sum()
    inputs = leaves + ([mu0, I0] if mu0 is not None else [])
    if o.numel() > 0:
        grads = torch.autograd.grad(loss, inputs, allow_unused=True)
        grads = [torch.zeros_like(x) if gr is None else gr for gr, x in zip(grads, inputs)]
    else:
        grads = [torch.zeros_like(x) for x in inputs]
    out = {"o": o.detach(), "final_mu": fmu.detach(), "final_I": fI.detach()}
    if unc:
        out["o_var"] = o_var.detach()
    for name, gr in zip(("dq", "dk", "dv", "db", "dgt", "dg", "dIp", "dmu0", "dI0"), grads):
        out[name] = gr
    return out


def oracle_backward_explicit(q, k, v, b, gt, g, Ip, do, do_var=None, initial_mu_state=None,
                             initial_I_state=None, scale=None, carry_M=None, carry_I=None, block=None):
    """Hand-derived backward of one batch of equal-length sequences, float64, no autograd.

    This is the recurrence the CUDA backward kernels implement; the reference's version of the same
    algebra is chunk_palimpsa_forgetting_scalar.py:343-434 (recompute forward, local terms
    ``dM_loc = dmu/I``, ``dI_loc = -dmu*M/I^2``, reverse scan with the NEXT token's decay, then
    ``dk, dv, db`` contractions and the decay gradient).  Differences, on purpose:
    the previous-token state is carried forward instead of being rebuilt by dividing by the decay
    (``:409-410``), and the prior-precision gradient is exact when an explicit initial precision
    is supplied (the kernel's ``:418`` omits that term).

    ``carry_M/carry_I`` are optional gradients w.r.t. the END state in (M, I) form (used by the
    segment / context-parallel identities).  ``block``: keep the per-token states of only that many
    tokens at a time (states at block starts are kept, each block is walked forward again when the
    reverse walk reaches it), which bounds the memory for long sequences; the result is the same.
    Returns a dict with the 7 gradients plus ``dM0, dI0`` (gradients w.r.t. the start state in (M, I)
    form), ``df`` and the forward's ``o`` and final ``(mu, I)``.
    """
    q, k, v, b, gt, g, Ip, do = [_f64(x) for x in (q, k, v, b, gt, g, Ip, do)]
    do_var = _f64(do_var)
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    if block is None or block <= 0:
        block = max(T, 1)
    ipb = Ip.view(1, H, 1, 1)
    if initial_mu_state is None:
        I = ipb.expand(B, H, V, K).clone()
        M = torch.zeros(B, H, V, K, dtype=F64)
    else:
        I = _f64(initial_I_state).clone()
        M = _f64(initial_mu_state) * I
    f_all = torch.exp(-gt * g.view(1, 1, H))                      # [B,T,H]

    def step(M, I, t):
        f = f_all[:, t].view(B, H, 1, 1)
        M = f * M + v[:, t, :, :, None] * k[:, t, :, None, :]
        I = f * I + (1.0 - f) * ipb + b[:, t, :, :, None] * (k[:, t, :, None, :] ** 2)
        return M, I

    o = torch.zeros_like(v)
    starts = []                                                    # state before the first token of every block
    for t in range(T):
        if t % block == 0:
            starts.append((M, I))
        M, I = step(M, I, t)
        o[:, t] = ((M / I) * (q[:, t] * scale)[:, :, None, :]).sum(-1)
    final_mu, final_I = M / I, I
    dq = torch.zeros_like(q)
    dk = torch.zeros_like(k)
    dv = torch.zeros_like(v)
    db = torch.zeros_like(b)
    df = torch.zeros_like(gt)
    s2 = torch.zeros_like(gt)                                     # sum_{v,k} GI_t
    GM = torch.zeros(B, H, V, K, dtype=F64) if carry_M is None else _f64(carry_M).clone()
    GI = torch.zeros(B, H, V, K, dtype=F64) if carry_I is None else _f64(carry_I).clone()
    for blk in range(len(starts) - 1, -1, -1):
        t_lo, t_hi = blk * block, min(T, (blk + 1) * block)
        Ms, Is = [starts[blk][0]], [starts[blk][1]]               # Ms[j] = state before token t_lo + j
        for t in range(t_lo, t_hi):
            Mn, In = step(Ms[-1], Is[-1], t)
            Ms.append(Mn)
            Is.append(In)
        for t in range(t_hi - 1, t_lo - 1, -1):
            Mt, It, Mp, Ipv = Ms[t - t_lo + 1], Is[t - t_lo + 1], Ms[t - t_lo], Is[t - t_lo]
            r = 1.0 / It
            mu = Mt * r
            qs = (q[:, t] * scale)[:, :, None, :]                     # [B,H,1,K]
            dy = do[:, t][:, :, :, None]                              # [B,H,V,1]
            dMl = dy * qs * r
            dIl = -dMl * mu
            dq[:, t] = scale * (dy * mu).sum(2)
            if do_var is not None:
                dyv = do_var[:, t][:, :, :, None]
                qq = (scale * q[:, t] ** 2)[:, :, None, :]
                dIl = dIl - dyv * qq * r * r
                dq[:, t] += 2.0 * scale * q[:, t] * (dyv * r).sum(2)
            # GM/GI hold f_{t+1} * (total gradient at t+1) when entering the iteration
            GM = dMl + GM
            GI = dIl + GI
            kt = k[:, t][:, :, None, :]
            vt = v[:, t][:, :, :, None]
            bt = b[:, t][:, :, :, None]
            dk[:, t] = (GM * vt).sum(2) + 2.0 * k[:, t] * (GI * bt).sum(2)
            dv[:, t] = (GM * kt).sum(3)
            db[:, t] = (GI * kt * kt).sum(3)
            df[:, t] = (GM * Mp).sum((2, 3)) + (GI * (Ipv - ipb)).sum((2, 3))
            s2[:, t] = GI.sum((2, 3))
            f = f_all[:, t].view(B, H, 1, 1)
            GM = f * GM
            GI = f * GI
        del Ms, Is
    dgt = -g.view(1, 1, H) * f_all * df
    dg = (-gt * f_all * df).sum((0, 1))
    dIp = ((1.0 - f_all) * s2).sum((0, 1))
    if initial_mu_state is None:
        dIp = dIp + GI.sum((0, 2, 3))        # I_0 = Ip: the start-state gradient flows into Ip
    return {"dq": dq, "dk": dk, "dv": dv, "db": db, "dgt": dgt, "dg": dg, "dIp": dIp,
            "dM0": GM, "dI0": GI, "df": df, "o": o, "final_mu": final_mu, "final_I": final_I}


# --------------------------------------------------------------------------------------------
# Segment (chunk-boundary / context-parallel) identities, float64.  They restate what the
# reference's forward kernel does when it closes a chunk (chunk_palimpsa_forgetting_scalar.py:
# 209-212: decayed sums of the chunk's inputs plus the decayed carried state) for a segment of any
# length, which is what lets segments of one sequence be processed by different CTAs or ranks.
# --------------------------------------------------------------------------------------------
def segment_summary(k, v, b, gt, g):
    """End state of a segment started from ZERO, in (M, J) form, and its total decay P.

    ``M_end = sum_t a_t v_t k_t^T``, ``J_end = sum_t a_t b_t (k_t*k_t)^T`` with
    ``a_t = prod_{s>t} f_s``; ``P = prod_t f_t``.  Shapes as the operator's; returns
    ``(S_M [B,H,V,K], S_J [B,H,V,K], P [B,H])``.
    """
    k, v, b, gt, g = [_f64(x) for x in (k, v, b, gt, g)]
    B, T, H, K = k.shape
    lf = -gt * g.view(1, 1, H)                                     # log f
    rev = torch.flip(torch.cumsum(torch.flip(lf, [1]), 1), [1])    # sum_{s>=t} log f_s
    a = torch.exp(rev - lf)                                        # prod_{s>t} f_s
    S_M = torch.einsum("bth,bthv,bthk->bhvk", a, v, k)
    S_J = torch.einsum("bth,bthv,bthk->bhvk", a, b, k * k)
    P = torch.exp(lf.sum(1))
    return S_M, S_J, P


def combine_segments(S_M, S_J, P, M0, J0):
    """Exclusive scan over segments: start state of every segment from the local summaries.

    ``S_*`` are lists (one per segment) from :func:`segment_summary`; ``M0, J0`` the start state of
    segment 0 in (M, J) form.  Returns lists ``(M_in, J_in)`` and the final state.
    """
    M_in, J_in = [], []
    M, J = M0, J0
    for sm, sj, p in zip(S_M, S_J, P):
        M_in.append(M)
        J_in.append(J)
        pb = p.view(*p.shape, 1, 1)
        M = pb * M + sm
        J = pb * J + sj
    return M_in, J_in, (M, J)


def make_inputs(seed, B, T, H, K, V, dtype=torch.float32, normalize_qk=True, check_style=False):
    """Seeded synthetic inputs.  Default distributions are the benchmark's (q,k L2-normalised
    N(0,1); v ~ N(0,1); b = sigmoid(N); gt = softplus(N); g = softplus(N); Ip = 1; dO ~ N(0,1)).
    ``check_style=True`` reproduces the distributions of the reference's manual check
    (palimpsa/check_palimpsa.py:52-59: raw q,k; gt = sigmoid(N); g = |N|*10+1; Ip = |N|+0.1).
    Values are drawn in float32 on the CPU generator in a fixed order, then q,k,v,b,dO are rounded
    to ``dtype``; gt, g, Ip stay float32.
    """
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32)
    if check_style:
        v = rn(B, T, H, V)
        q = rn(B, T, H, K)
        k = rn(B, T, H, K)
        b = torch.sigmoid(rn(B, T, H, V))
        gt = torch.sigmoid(rn(B, T, H))
        g = rn(H).abs() * 10 + 1
        Ip = rn(H).abs() + 0.1
    else:
        q = rn(B, T, H, K)
        k = rn(B, T, H, K)
        if normalize_qk:
            q = torch.nn.functional.normalize(q, dim=-1)
            k = torch.nn.functional.normalize(k, dim=-1)
        v = rn(B, T, H, V)
        b = torch.sigmoid(rn(B, T, H, V))
        gt = torch.nn.functional.softplus(rn(B, T, H))
        g = torch.nn.functional.softplus(rn(H))
        Ip = torch.ones(H)
    do = rn(B, T, H, V)
    do_var = rn(B, T, H, V)
    return {"q": q.to(dtype), "k": k.to(dtype), "v": v.to(dtype), "b": b.to(dtype), "gt": gt, "g": g,
            "Ip": Ip, "do": do.to(dtype), "do_var": do_var.to(dtype)}


def make_states(seed, N, H, V, K, Ip):
    """Random explicit initial state as in palimpsa/check_palimpsa.py:197-205 (I0 > Ip)."""
    gen = torch.Generator().manual_seed(seed)
    mu0 = torch.randn(N, H, V, K, generator=gen, dtype=torch.float32)
    I0 = Ip.view(1, H, 1, 1) + torch.relu(torch.randn(N, H, V, K, generator=gen, dtype=torch.float32)) + 1.0
    return mu0, I0


def rel_err(x, ref) -> float:
    """max|x-ref| / max|ref| (the error metric every parity test uses)."""
    x = x.detach().to("cpu", F64)
    ref = ref.detach().to("cpu", F64)
    if ref.numel() == 0:
        return 0.0
    den = ref.abs().max().item()
    return (x - ref).abs().max().item() / (den if den > 0 else 1.0)


def naive_recurrence_fp32(q, k, v, b, gt, g, Ip, initial_mu_state=None, initial_I_state=None, scale=None,
                          output_final_state=False, output_uncertainty=False):
    """float32 port of ``palimpsa_ref`` as written (chunk_palimpsa_forgetting_scalar.py:684-725:
    (mu, I) carried, ``mu*I`` re-multiplied each step, fp32 casts, ``scale**2`` on the variance).
    This is the CPU baseline the benchmark times; it is differentiable through autograd.
    """
    dtype_in = v.dtype
    q, k, v, b, gt, g, Ip = [x.float() for x in (q, k, v, b, gt, g, Ip)]
    if scale is None:
        scale = q.shape[-1] ** -0.5
    B, T, H, V = b.shape
    K = k.shape[-1]
    ipb = Ip[None, :, None, None]
    if initial_mu_state is None:
        mu = torch.zeros(B, H, V, K)
        I = ipb
    else:
        mu, I = initial_mu_state, initial_I_state
    q = q * scale
    ys, yvs = [], []
    for t in range(T):
        f = torch.exp(-gt[:, t, :, None, None] * g[None, :, None, None])
        M = v[:, t, :, :, None] * k[:, t, :, None, :] + f * mu * I
        I = b[:, t, :, :, None] * (k[:, t, :, None, :] ** 2) + (1 - f) * ipb + f * I
        mu = M / I
        ys.append(torch.einsum("bhdn,bhn->bhd", mu, q[:, t]))
        if output_uncertainty:
            yvs.append(torch.einsum("bhdn,bhn->bhd", 1 / I, q[:, t] ** 2))
    y = torch.stack(ys, 1).to(dtype_in)
    out = (y, torch.stack(yvs, 1).to(dtype_in)) if output_uncertainty else y
    return (out, mu, I) if output_final_state else out
