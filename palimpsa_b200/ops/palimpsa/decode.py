"""In-place single-token decode over a persistent state cache.

The reference's layer keeps the pair ``(final_mu, final_I)`` returned by ``fused_recurrent_palimpsa``
in its cache and passes it back as the next call's initial state, allocating two new state tensors
per layer and token (palimpsa/layers/palimpsa.py:317-331).  ``decode_step`` does the same update on
the cache tensors themselves.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ... import _lib as L
from . import _core


def decode_step(q, k, v, b, gt, g, Ip, mu_state: torch.Tensor, I_state: torch.Tensor, scale: Optional[float] = None,
                output_uncertainty: bool = False):
    """One token for each of N sequences: ``q,k [N,1,H,K]`` (or ``[N,H,K]``), ``v,b [N,1,H,V]``,
    ``gt [N,1,H]``, ``g,Ip [H]``; ``mu_state, I_state [N,H,V,K]`` float32 contiguous CUDA tensors that
    are UPDATED IN PLACE.  Returns ``o [N,1,H,V]`` (and ``o_var`` with ``output_uncertainty``).
    Not differentiable (inference only)."""
    if q.dim() == 3:
        q, k, v, b, gt = q.unsqueeze(1), k.unsqueeze(1), v.unsqueeze(1), b.unsqueeze(1), gt.unsqueeze(1)
    N, T, H, K = q.shape
    V = v.shape[-1]
    if T != 1:
        raise ValueError("decode_step takes exactly one token per sequence")
    _core._require_cuda(q, k, v, b, gt, g, Ip, mu_state, I_state)
    for s in (mu_state, I_state):
        if s.dtype != torch.float32 or not s.is_contiguous() or tuple(s.shape) != (N, H, V, K):
            raise ValueError(f"state cache tensors must be contiguous float32 of shape {(N, H, V, K)}")
    if scale is None:
        scale = K ** -0.5
    io = q.dtype
    q, k, v, b = [x.detach().to(io).contiguous() for x in (q, k, v, b)]
    gt, g, Ip = [x.detach().float().contiguous() for x in (gt, g, Ip)]
    lib = L.lib()
    with torch.cuda.device(q.device):
        o = torch.empty(N, 1, H, V, dtype=io, device=q.device)
        o_var = torch.empty(N, 1, H, V, dtype=io, device=q.device) if output_uncertainty else None
        prm = L.FwdParams()
        prm.struct_size = C.sizeof(L.FwdParams)
        prm.p = _core._problem(q, k, v, b, gt, g, Ip, None, None, mu_state, I_state, scale,
                               L.FLAG_UNCERTAINTY if output_uncertainty else 0)
        prm.o, prm.o_var = _core._ptr(o), _core._ptr(o_var)
        prm.final_mu, prm.final_I = mu_state.data_ptr(), I_state.data_ptr()
        L.check(lib.palimpsa_decode_step(C.byref(prm), _core._stream(q)), "palimpsa decode step")
    return (o, o_var) if output_uncertainty else o
