"""``palimpsa_ref``: the naive per-timestep definition of the operator, kept because the reference
exports it next to the two ops (palimpsa/ops/palimpsa/__init__.py:4; definition at
chunk_palimpsa_forgetting_scalar.py:669-725).  Plain PyTorch on whatever device the inputs are on;
never called by the CUDA ops."""
from __future__ import annotations

import torch


def palimpsa_ref(q, k, v, b, gt, g, Ip, initial_mu_state=None, initial_I_state=None, scale=None,
                 output_final_state=False, output_uncertainty=False):
    dtype_in = v.dtype
    q, k, v, b, gt, g, Ip = [x.float() for x in (q, k, v, b, gt, g, Ip)]
    if scale is None:
        scale = q.shape[-1] ** -0.5
    B, T, H, V = b.shape
    K = k.shape[-1]
    dev = q.device
    ip = Ip.view(1, H, 1, 1)
    if initial_mu_state is None:
        mu = torch.zeros(B, H, V, K, device=dev)
        prec = ip.expand(B, H, V, K)
    else:
        mu, prec = initial_mu_state, initial_I_state
    qs = q * scale
    ys, yvs = [], []
    for t in range(T):
        f = torch.exp(-gt[:, t] * g.view(1, H)).view(B, H, 1, 1)
        num = f * (mu * prec) + v[:, t].unsqueeze(-1) * k[:, t].unsqueeze(-2)
        prec = f * prec + (1 - f) * ip + b[:, t].unsqueeze(-1) * (k[:, t] ** 2).unsqueeze(-2)
        mu = num / prec
        ys.append((mu * qs[:, t].unsqueeze(-2)).sum(-1))
        if output_uncertainty:
            yvs.append(((qs[:, t] ** 2).unsqueeze(-2) / prec).sum(-1))
    y = torch.stack(ys, 1).to(dtype_in) if T else torch.zeros(B, 0, H, V, dtype=dtype_in, device=dev)
    if output_uncertainty:
        yv = torch.stack(yvs, 1).to(dtype_in) if T else torch.zeros(B, 0, H, V, dtype=dtype_in, device=dev)
        out = (y, yv)
    else:
        out = y
    return (out, mu, prec) if output_final_state else out
