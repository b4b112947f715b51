"""In-place single-token decode over a persistent state cache.

The reference's layer keeps the pair ``(final_mu, final_I)`` returned by ``fused_recurrent_palimpsa``
in its cache and passes it back as the next call's initial state, allocating two new state tensors
per layer and token (palimpsa/layers/palimpsa.py:317-331).  ``decode_step`` does the same update on
the cache tensors themselves.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
from torch import Tensor

from ... import _lib as L
from . import _core


@torch.library.custom_op("palimpsa_b200::decode_step", mutates_args=("mu_state", "I_state"), device_types="cuda")
def decode_step_op(q: Tensor, k: Tensor, v: Tensor, b: Tensor, gt: Tensor, g: Tensor, Ip: Tensor, mu_state: Tensor,
                   I_state: Tensor, scale: float, uncertainty: bool) -> Tuple[Tensor, Tensor]:
    """The registered op: contiguous ``[N,1,H,*]`` inputs of one io dtype, float32 ``gt, g, Ip`` and state cache;
    returns ``(o, o_var)`` (``o_var`` empty without ``uncertainty``) and updates the two cache tensors in place."""
    N, _, H, K = q.shape
    V = v.shape[-1]
    lib = L.lib()
    with torch.cuda.device(q.device):
        o = torch.empty(N, 1, H, V, dtype=q.dtype, device=q.device)
        o_var = torch.empty(N, 1, H, V, dtype=q.dtype, device=q.device) if uncertainty else q.new_empty(0)
        prm = L.FwdParams()
        prm.struct_size = C.sizeof(L.FwdParams)
        prm.p = _core._problem(q, k, v, b, gt, g, Ip, None, None, mu_state, I_state, scale,
                               L.FLAG_UNCERTAINTY if uncertainty else 0)
        prm.o, prm.o_var = _core._ptr(o), _core._ptr(o_var)
        prm.final_mu, prm.final_I = mu_state.data_ptr(), I_state.data_ptr()
        L.check(lib.palimpsa_decode_step(C.byref(prm), _core._stream(q)), "palimpsa decode step")
    return o, o_var


@decode_step_op.register_fake
def _(q, k, v, b, gt, g, Ip, mu_state, I_state, scale, uncertainty):
    N, _, H, _ = q.shape
    V = v.shape[-1]
    return q.new_empty(N, 1, H, V), (q.new_empty(N, 1, H, V) if uncertainty else q.new_empty(0))


def decode_step(q, k, v, b, gt, g, Ip, mu_state: torch.Tensor, I_state: torch.Tensor, scale: Optional[float] = None,
                output_uncertainty: bool = False):
    """One token for each of N sequences: ``q,k [N,1,H,K]`` (or ``[N,H,K]``), ``v,b [N,1,H,V]``,
    ``gt [N,1,H]``, ``g,Ip [H]``; ``mu_state, I_state [N,H,V,K]`` float32 contiguous CUDA tensors that
    are UPDATED IN PLACE.  Returns ``o [N,1,H,V]`` (and ``o_var`` with ``output_uncertainty``).
    Not differentiable (inference only).  The work is done by the registered op
    ``torch.ops.palimpsa_b200.decode_step`` (declared as mutating the two cache tensors), so the call can sit
    inside a ``torch.compile``d decode loop."""
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
    o, o_var = decode_step_op(q, k, v, b, gt, g, Ip, mu_state, I_state, float(scale), bool(output_uncertainty))
    return (o, o_var) if output_uncertainty else o


class DecodeGraph:
    """``decode_step`` captured once in a CUDA graph and replayed per token: the step then costs one graph
    launch instead of the Python-side argument handling and kernel launch.  The graph reads its inputs from
    static buffers (``self.q, k, v, b, gt``: fill them, or pass tensors to :meth:`step`, which copies) and
    updates ``mu_state`` / ``I_state`` in place; ``self.o`` (and ``self.o_var``) hold the latest outputs and
    are overwritten by the next replay."""

    def __init__(self, g, Ip, mu_state: torch.Tensor, I_state: torch.Tensor, dtype=torch.bfloat16,
                 scale: Optional[float] = None, output_uncertainty: bool = False):
        N, H, V, K = mu_state.shape
        dev = mu_state.device
        _core._require_cuda(g, Ip, mu_state, I_state)
        self.q = torch.zeros(N, 1, H, K, dtype=dtype, device=dev)
        self.k = torch.zeros_like(self.q)
        self.v = torch.zeros(N, 1, H, V, dtype=dtype, device=dev)
        self.b = torch.zeros_like(self.v)
        self.gt = torch.zeros(N, 1, H, dtype=torch.float32, device=dev)
        self.g, self.Ip = g.detach().float().contiguous(), Ip.detach().float().contiguous()
        self.mu_state, self.I_state = mu_state, I_state
        self.unc = output_uncertainty
        L.lib()                                        # load (and fail) outside the capture
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            # zero inputs are an identity update only for f = 1, so the warm-up runs on copies of the cache
            mu_tmp, I_tmp = mu_state.clone(), I_state.clone()
            decode_step(self.q, self.k, self.v, self.b, self.gt, self.g, self.Ip, mu_tmp, I_tmp, scale,
                        output_uncertainty)
        torch.cuda.current_stream(dev).wait_stream(side)
        with torch.cuda.graph(self.graph):
            out = decode_step(self.q, self.k, self.v, self.b, self.gt, self.g, self.Ip, mu_state, I_state, scale,
                              output_uncertainty)
        self.o, self.o_var = out if output_uncertainty else (out, None)

    def step(self, q=None, k=None, v=None, b=None, gt=None):
        """Copies the given tensors into the static input buffers (those left ``None`` keep their content) and
        replays the graph on the current stream.  Returns ``self.o`` (and ``self.o_var``)."""
        for dst, src in ((self.q, q), (self.k, k), (self.v, v), (self.b, b), (self.gt, gt)):
            if src is not None:
                dst.copy_(src.reshape(dst.shape), non_blocking=True)
        self.graph.replay()
        return (self.o, self.o_var) if self.unc else self.o
