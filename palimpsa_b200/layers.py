"""Fused element-wise sides of the Palimpsa layer (one CUDA pass each, forward and backward).

The reference layer prepares the operator's inputs and post-processes its output with separate PyTorch
element-wise passes (palimpsa/layers/palimpsa.py:266-281 and :337-343).  :func:`layer_prologue` and
:func:`layer_epilogue` compute the same quantities, so the layer's ``forward`` can read::

    q, k, v, b, dt = layer_prologue(q, k, x, b_raw, self.dt_proj(h), self.bs_proj(h), self.dt_bias, self.b_scale)
    o = chunk_palimpsa(q, k, v, b, dt, A, Ip, ...)
    o = layer_epilogue(o, x, self.D, self.o_norm.weight, gate, eps=self.o_norm.eps)

Both are differentiable (``torch.autograd.Function`` over the C ABI) and run on CUDA only.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
from torch import Tensor

from . import _lib as L
from .ops.palimpsa._core import _DT, _ptr, _require_cuda, _stream


def _workspace(tokens: int, H: int, V: int, dev) -> Tensor:
    need = L.lib().palimpsa_layer_workspace_bytes(tokens, H, V)
    return torch.empty(max(int(need), 256), dtype=torch.uint8, device=dev)


def _prologue_struct(q_raw, k_raw, x, b_raw, dt_raw, bs_raw, dt_bias, b_scale) -> L.LayerPrologue:
    a = L.LayerPrologue()
    a.struct_size = C.sizeof(L.LayerPrologue)
    a.io_dtype = _DT[x.dtype]
    a.H, a.Hq, a.K, a.V = x.shape[-2], q_raw.shape[-2], q_raw.shape[-1], x.shape[-1]
    a.tokens = x.numel() // (x.shape[-1] * x.shape[-2]) if x.numel() else 0
    a.q_raw, a.k_raw, a.x, a.b_raw = _ptr(q_raw), _ptr(k_raw), _ptr(x), _ptr(b_raw)
    a.dt_raw, a.bs_raw, a.dt_bias, a.b_scale = _ptr(dt_raw), _ptr(bs_raw), _ptr(dt_bias), _ptr(b_scale)
    return a


class _Prologue(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q_raw, k_raw, x, b_raw, dt_raw, bs_raw, dt_bias, b_scale):
        io = x.dtype
        ts = [t.to(io).contiguous() for t in (q_raw, k_raw, x, b_raw, dt_raw, bs_raw)]
        ps = [t.detach().float().contiguous() for t in (dt_bias, b_scale)]
        q_raw_, k_raw_, x_, b_raw_, dt_raw_, bs_raw_ = ts
        H, V, K = x_.shape[-2], x_.shape[-1], q_raw_.shape[-1]
        lead = x_.shape[:-2]
        q = torch.empty(*lead, H, K, dtype=io, device=x.device)
        k = torch.empty_like(q)
        v, b = torch.empty_like(x_), torch.empty_like(x_)
        gt = torch.empty(*lead, H, dtype=torch.float32, device=x.device)
        a = _prologue_struct(*ts, *ps)
        a.q, a.k, a.v, a.b, a.gt = _ptr(q), _ptr(k), _ptr(v), _ptr(b), _ptr(gt)
        if a.tokens > 0:                              # an empty batch has nothing to launch (and no pointers)
            with torch.cuda.device(x.device):
                L.check(L.lib().palimpsa_layer_prologue_fwd(C.byref(a), _stream(x)), "layer prologue")
        ctx.save_for_backward(*ts, *ps)
        ctx.dtypes = (q_raw.dtype, k_raw.dtype, x.dtype, b_raw.dtype, dt_raw.dtype, bs_raw.dtype, dt_bias.dtype,
                      b_scale.dtype)
        return q, k, v, b, gt

    @staticmethod
    def backward(ctx, dq, dk, dv, db, dgt):
        q_raw, k_raw, x, b_raw, dt_raw, bs_raw, dt_bias, b_scale = ctx.saved_tensors
        io, dev = x.dtype, x.device
        H, V = x.shape[-2], x.shape[-1]

        def grad(g, like, dtype):
            return torch.zeros_like(like, dtype=dtype) if g is None else g.to(dtype).contiguous()

        q_like = torch.empty(*x.shape[:-1], q_raw.shape[-1], dtype=io, device=dev)
        dq, dk = grad(dq, q_like, io), grad(dk, q_like, io)
        dv, db = grad(dv, x, io), grad(db, x, io)
        dgt = grad(dgt, dt_raw, torch.float32)
        a = _prologue_struct(q_raw, k_raw, x, b_raw, dt_raw, bs_raw, dt_bias, b_scale)
        a.dq, a.dk, a.dv, a.db, a.dgt = _ptr(dq), _ptr(dk), _ptr(dv), _ptr(db), _ptr(dgt)
        outs = [torch.empty_like(q_raw), torch.empty_like(k_raw), torch.empty_like(x), torch.empty_like(b_raw),
                torch.empty_like(dt_raw), torch.empty_like(bs_raw),
                torch.empty(H, dtype=torch.float32, device=dev), torch.empty(H, dtype=torch.float32, device=dev)]
        (a.dq_raw, a.dk_raw, a.dx, a.db_raw, a.ddt_raw, a.dbs_raw, a.d_dt_bias, a.d_b_scale) = [_ptr(t) for t in outs]
        ws = _workspace(a.tokens, H, V, dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        if a.tokens > 0:
            with torch.cuda.device(dev):
                L.check(L.lib().palimpsa_layer_prologue_bwd(C.byref(a), _stream(x)), "layer prologue backward")
        else:
            outs[6].zero_()
            outs[7].zero_()
        return tuple(t.to(dt) for t, dt in zip(outs, ctx.dtypes))


def layer_prologue(q_raw: Tensor, k_raw: Tensor, x: Tensor, b_raw: Tensor, dt_raw: Tensor, bs_raw: Tensor,
                   dt_bias: Tensor, b_scale: Tensor):
    """Inputs of the operator from the layer's projections (palimpsa/layers/palimpsa.py:266-281).

    ``q_raw, k_raw [..., Hq, K]`` (after the short convolution / SiLU), ``x, b_raw [..., H, V]``,
    ``dt_raw, bs_raw [..., H]`` (outputs of ``dt_proj`` / ``bs_proj``), ``dt_bias, b_scale [H]``.
    Returns ``q, k [..., H, K]`` (L2-normalised, repeated over ``H // Hq`` value heads), ``v = x*bs``,
    ``b = sigmoid(b_raw) * softplus(b_scale) * bs`` in ``x.dtype`` and ``dt = softplus(dt_raw + dt_bias)`` in
    float32, where ``bs = sigmoid(bs_raw)`` rounded to ``x.dtype`` as in the layer."""
    _require_cuda(q_raw, k_raw, x, b_raw, dt_raw, bs_raw, dt_bias, b_scale)
    if x.dtype not in _DT:
        raise TypeError(f"unsupported dtype {x.dtype}: use float32, bfloat16 or float16")
    H, Hq = x.shape[-2], q_raw.shape[-2]
    if H % Hq or q_raw.shape != k_raw.shape or b_raw.shape != x.shape or q_raw.shape[:-2] != x.shape[:-2]:
        raise ValueError("layer_prologue: q_raw/k_raw [...,Hq,K], x/b_raw [...,H,V] with H a multiple of Hq")
    if dt_raw.shape != x.shape[:-1] or bs_raw.shape != x.shape[:-1] or dt_bias.numel() != H or b_scale.numel() != H:
        raise ValueError("layer_prologue: dt_raw/bs_raw [...,H], dt_bias/b_scale [H]")
    return _Prologue.apply(q_raw, k_raw, x, b_raw, dt_raw, bs_raw, dt_bias, b_scale)


class _Epilogue(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, x, D, weight, gate, eps):
        io = o.dtype
        o_ = o.contiguous()
        x_ = None if x is None else x.to(io).contiguous()
        g_ = None if gate is None else gate.to(io).contiguous()
        D_ = None if D is None else D.detach().float().contiguous()
        w_ = weight.detach().float().contiguous()
        y = torch.empty_like(o_)
        a = _Epilogue._struct(o_, x_, D_, w_, g_, eps)
        a.y = _ptr(y)
        if a.tokens > 0:
            with torch.cuda.device(o.device):
                L.check(L.lib().palimpsa_layer_epilogue_fwd(C.byref(a), _stream(o)), "layer epilogue")
        ctx.save_for_backward(o_, x_, D_, w_, g_)
        ctx.eps = eps
        ctx.dtypes = (None if x is None else x.dtype, None if D is None else D.dtype, weight.dtype,
                      None if gate is None else gate.dtype)
        return y

    @staticmethod
    def _struct(o, x, D, w, g, eps) -> L.LayerEpilogue:
        a = L.LayerEpilogue()
        a.struct_size = C.sizeof(L.LayerEpilogue)
        a.io_dtype = _DT[o.dtype]
        a.H, a.V = o.shape[-2], o.shape[-1]
        a.flags = (L.LAYER_RESIDUAL if x is not None else 0) | (L.LAYER_GATE if g is not None else 0)
        a.eps = float(eps)
        a.tokens = o.numel() // (o.shape[-1] * o.shape[-2]) if o.numel() else 0
        a.o, a.x, a.gate, a.D, a.weight = _ptr(o), _ptr(x), _ptr(g), _ptr(D), _ptr(w)
        return a

    @staticmethod
    def backward(ctx, dy):
        o, x, D, w, g = ctx.saved_tensors
        dev = o.device
        H, V = o.shape[-2], o.shape[-1]
        a = _Epilogue._struct(o, x, D, w, g, ctx.eps)
        dy = dy.to(o.dtype).contiguous()
        d_o = torch.empty_like(o)
        dx = None if x is None else torch.empty_like(o)
        dgate = None if g is None else torch.empty_like(o)
        dD = None if x is None else torch.empty(H, dtype=torch.float32, device=dev)
        dw = torch.empty(V, dtype=torch.float32, device=dev)
        a.dy, a.d_o, a.dx, a.dgate, a.dD, a.dweight = _ptr(dy), _ptr(d_o), _ptr(dx), _ptr(dgate), _ptr(dD), _ptr(dw)
        ws = _workspace(a.tokens, H, V, dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        if a.tokens > 0:
            with torch.cuda.device(dev):
                L.check(L.lib().palimpsa_layer_epilogue_bwd(C.byref(a), _stream(o)), "layer epilogue backward")
        else:
            dw.zero_()
            if dD is not None:
                dD.zero_()
        xd, Dd, wd, gd = ctx.dtypes
        return (d_o, None if dx is None else dx.to(xd), None if dD is None else dD.to(Dd), dw.to(wd),
                None if dgate is None else dgate.to(gd), None)


def layer_epilogue(o: Tensor, x: Optional[Tensor], D: Optional[Tensor], weight: Tensor,
                   gate: Optional[Tensor] = None, eps: float = 1e-5) -> Tensor:
    """Output side of the layer (palimpsa/layers/palimpsa.py:337-343): ``z = o + x * D[h]`` (skipped when
    ``x`` / ``D`` are ``None``: ``use_residual=False``), then the RMS norm over the last axis with
    ``weight [V]``, multiplied by ``gate * sigmoid(gate)`` when ``gate [..., H, V]`` is given (the gated
    norm of flash-linear-attention's ``FusedRMSNormGated``, activation "swish").  float32 arithmetic, result
    in ``o.dtype``."""
    _require_cuda(o, x, D, weight, gate)
    if o.dtype not in _DT:
        raise TypeError(f"unsupported dtype {o.dtype}: use float32, bfloat16 or float16")
    if (x is None) != (D is None):
        raise ValueError("layer_epilogue: pass both x and D (residual) or neither")
    if x is not None and (x.shape != o.shape or D.numel() != o.shape[-2]):
        raise ValueError("layer_epilogue: x like o, D [H]")
    if gate is not None and gate.shape != o.shape:
        raise ValueError("layer_epilogue: gate like o")
    if weight.numel() != o.shape[-1]:
        raise ValueError("layer_epilogue: weight [V]")
    return _Epilogue.apply(o, x, D, weight, gate, float(eps))
