"""CPU oracle for the layer-side element-wise work -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Restates, with plain torch functions on the CPU, what the reference layer computes around the operator:

* prologue: ``palimpsa/layers/palimpsa.py:266-281`` (repeat of q/k over value heads, ``softplus(dt+bias)``,
  ``F.normalize`` of q and k, ``bs = sigmoid(...)`` cast to the activation dtype, ``v = x*bs``,
  ``b = sigmoid(b_raw) * softplus(b_scale) * bs`` cast to the activation dtype);
* epilogue: ``:337-343`` (``o + x*D``, then the gated RMS norm).  The norm is ``FusedRMSNormGated`` of the
  pinned third-party dependency flash-linear-attention 0.5.1 (``fla/modules/fused_norm_gate.py``), whose
  published algorithm is ``y = x / sqrt(mean(x^2) + eps) * weight * gate * sigmoid(gate)`` in float32.

Gradients come from autograd through these expressions.  ``compute`` is the dtype the arithmetic runs in
(float64 for the exact answer; pass the activation dtype itself to get the layer's own rounding points).

Parity pin: the prologue is made of the same torch functions, in the same order, as the layer's lines and
needs no further pin.  The gated norm is pinned against flash-linear-attention's own ``FusedRMSNormGated``:
``tests/golden/gated_norm.npz`` holds that module's outputs and gradients (float32 and bfloat16), generated on a
GPU by ``tests/golden/make_gated_norm_golden.py`` (its kernels are Triton and cannot run on a CPU), and
``tests/test_layer_oracle_cpu.py`` checks this restatement against the file.

Only the tests may import this module.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


def layer_prologue_ref(q_raw, k_raw, x, b_raw, dt_raw, bs_raw, dt_bias, b_scale, compute=torch.float64,
                       act_dtype: Optional[torch.dtype] = None):
    """``act_dtype``: dtype ``bs`` is rounded to before use (the layer's activation dtype; None = no rounding)."""
    H, Hq = x.shape[-2], q_raw.shape[-2]
    c = lambda t: t.to(compute)
    q = c(q_raw).repeat_interleave(H // Hq, dim=-2)       # einops repeat '... h d -> ... (h g) d'  (:266)
    k = c(k_raw).repeat_interleave(H // Hq, dim=-2)
    dt = F.softplus(c(dt_raw) + c(dt_bias))               # :269
    q, k = F.normalize(q, p=2, dim=-1), F.normalize(k, p=2, dim=-1)   # :271
    bs = torch.sigmoid(c(bs_raw))                         # :272
    if act_dtype is not None:
        bs = bs.detach().to(act_dtype).to(compute) + (bs - bs.detach())   # rounded value, identity gradient
    v = c(x) * bs.unsqueeze(-1)                           # :273
    b = torch.sigmoid(c(b_raw)) * F.softplus(c(b_scale).view(-1, 1))  # :276-278
    b = b * bs.unsqueeze(-1)                              # :279
    return q, k, v, b, dt


def layer_epilogue_ref(o, x, D, weight, gate=None, eps=1e-5, compute=torch.float64):
    c = lambda t: t.to(compute)
    z = c(o)
    if x is not None:
        z = z + c(x) * c(D).view(-1, 1)                   # :338
    y = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + eps) * c(weight)
    if gate is not None:
        g = c(gate)
        y = y * g * torch.sigmoid(g)
    return y


def make_layer_inputs(seed, B, T, H, Hq, K, V, dtype=torch.float32):
    """Seeded stand-ins for the projections' outputs and the layer's parameters."""
    gen = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=gen)
    d = {
        "q_raw": r(B, T, Hq, K), "k_raw": r(B, T, Hq, K), "x": r(B, T, H, V), "b_raw": r(B, T, H, V),
        "dt_raw": r(B, T, H), "bs_raw": r(B, T, H), "gate": r(B, T, H, V), "o": r(B, T, H, V),
        "dt_bias": r(H), "b_scale": 1.0 + 0.3 * r(H), "D": 1.0 + 0.2 * r(H), "weight": 1.0 + 0.2 * r(V),
    }
    # cotangents
    d.update({"dq": r(B, T, H, K), "dk": r(B, T, H, K), "dv": r(B, T, H, V), "db": r(B, T, H, V), "dgt": r(B, T, H),
              "dy": r(B, T, H, V)})
    acts = ("q_raw", "k_raw", "x", "b_raw", "dt_raw", "bs_raw", "gate", "o", "dq", "dk", "dv", "db", "dy")
    for n in acts:
        d[n] = d[n].to(dtype)
    return d
