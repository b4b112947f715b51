"""torch custom ops ``palimpsa_b200::fwd`` / ``palimpsa_b200::bwd`` over the C ABI.

The op bodies only allocate outputs with torch, fill the parameter structs of
include/palimpsa_b200.h with raw device pointers and call the shared library on the current CUDA
stream.  There is no fallback: CPU tensors are rejected and a missing library raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
from torch import Tensor

from ... import _lib as L

_DT = {torch.float32: L.F32, torch.bfloat16: L.BF16, torch.float16: L.F16}

# Segmented backward: take the tensor-core route for the carried-gradient terms wherever the library supports
# the problem (bf16, d_v <= 128, padded d_k in {32,48,64,96,128}).  Tests set this to False to exercise the
# two-pass CUDA-core route on the same problems.
carry_on_tensor_cores = True


def _ptr(t: Optional[Tensor]):
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _problem(q, k, v, b, gt, g, Ip, cu_seqlens, chunk_offsets, init_mu, init_I, scale, flags, seq_order=None) -> L.Problem:
    B, T, H, K = q.shape
    V = v.shape[-1]
    p = L.Problem()
    p.num_seqs = B if cu_seqlens is None else cu_seqlens.numel() - 1
    p.seq_len = T if cu_seqlens is None else 0
    p.total_tokens = B * T
    p.H, p.K, p.V = H, K, V
    p.io_dtype = _DT[q.dtype]
    p.flags = flags
    p.scale = float(scale)
    p.q, p.k, p.v, p.b = _ptr(q), _ptr(k), _ptr(v), _ptr(b)
    p.gt, p.g, p.Ip = _ptr(gt), _ptr(g), _ptr(Ip)
    p.cu_seqlens = _ptr(cu_seqlens)
    p.chunk_offsets = _ptr(chunk_offsets)
    p.init_mu, p.init_I = _ptr(init_mu), _ptr(init_I)
    p.seq_order = _ptr(seq_order)
    return p


def _stream(t: Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "palimpsa_b200 runs on CUDA (sm_100a) only and has no CPU path; "
                "for CPU tensors use palimpsa_b200.ops.palimpsa_ref (naive recurrence).")


def padded_k(K: int) -> int:
    for s in (16, 32, 48, 64, 96, 128, 192, 256):
        if K <= s:
            return s
    raise ValueError(f"d_k = {K} is above the supported maximum of 256")


def _ckpt_slots(total_tokens: int, num_seqs: int) -> int:
    return (total_tokens + L.CKPT_INTERVAL - 1) // L.CKPT_INTERVAL + num_seqs


def _longest_first(cu_seqlens: Tensor) -> Tensor:
    """Sequences of a packed batch by decreasing length (device-side, no host sync): the order in which the
    main kernels start them, so that the longest documents are not the tail of the launch."""
    lens = cu_seqlens[1:] - cu_seqlens[:-1]
    return torch.argsort(lens, descending=True, stable=True).to(torch.int32)


def _chunk_offsets(cu_seqlens: Tensor) -> Tensor:
    lens = cu_seqlens[1:] - cu_seqlens[:-1]
    nblk = (lens + (L.CKPT_INTERVAL - 1)) // L.CKPT_INTERVAL
    return (torch.cumsum(nblk, 0) - nblk).to(torch.int32)


B200_SM_COUNT = 148     # used only when no CUDA device is visible (planning on a build machine)
_sm_count_cache = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current CUDA device)."""
    if not torch.cuda.is_available():
        return B200_SM_COUNT
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _sm_count_cache:
        _sm_count_cache[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count_cache[idx]


@torch.compiler.assume_constant_result        # ints in, int out: evaluated once when a caller is traced by torch.compile
def plan_segments(N: int, T: int, H: int, K: int, V: int, device=None, backward: bool = False,
                  io_dtype: int = L.BF16, uncertainty: bool = False, packed: bool = False) -> int:
    """How many segments to cut every sequence into on one GPU.  Segments cost an extra summary pass
    (and the carried-gradient terms in backward: about a fifth of a step), so they are only used when the grid of
    (sequence, head, row-tile) CTAs would leave SMs idle, e.g. one very long sequence or a narrow batch slice.

    Forward only: the forward grid has fewer CTAs than the device has SMs.  With a backward to follow
    (``backward=True``) the backward kernel decides, since it is 3/4 of the step and keeps one CTA of up to 12 warps
    per SM: segments when its grid fills less than 80 % of the waves it occupies (72 CTAs on 148 SMs, or 192 CTAs =
    1.3 waves; not 128 CTAs = 0.86 of a wave, nor 288 = 1.95 waves).  Tile heights come from the library, the SM
    count from the device.

    ``packed``: N documents of unequal length in one row of T tokens (``cu_seqlens``).  Only N and T are known
    without a host synchronisation.  With more CTAs than SMs the documents, started longest first, fill the waves by
    themselves (14 or 19 documents in 32 768 tokens: 4.3 ms unsegmented, 5.0-6.0 ms segmented); with fewer, the
    longest document is the critical path and segments of T / G tokens shorten it (7 documents x 16 heads in
    16 384 tokens: 4.16 -> 2.79 ms)."""
    if T < 2048:
        return 1
    lib = L.lib()
    sms = sm_count(device)
    rows = lib.palimpsa_fwd_tile_rows(int(K), int(V))
    if rows <= 0:
        raise ValueError(f"d_k = {K} is above the supported maximum of 256")
    if backward:
        brow = lib.palimpsa_bwd_tile_rows(int(K), int(V), int(io_dtype), int(bool(uncertainty)))
        if brow <= 0:
            raise ValueError(f"no backward tiling for d_k = {K}, d_v = {V}")
        ctas = N * H * ((V + brow - 1) // brow)
        waves = (ctas + sms - 1) // sms
        if ctas >= (sms if packed else 0.8 * waves * sms):
            return 1
    elif N * H * ((V + rows - 1) // rows) >= sms:
        return 1
    # The boundary passes' total work does not depend on the number of segments, and their own grids
    # (one CTA per sequence x head x segment) want many of them: cut down to 256 tokens, at most 32 pieces
    # (measured flat from 16 to 128 pieces on T = 4096 .. 32768).
    return max(1, min(32, T // 256))


def segment_len(T: int, G: int) -> int:
    per = (T + G - 1) // G
    return max(L.CKPT_INTERVAL, (per + L.CKPT_INTERVAL - 1) // L.CKPT_INTERVAL * L.CKPT_INTERVAL)


def make_segments(N, G, seg_len, H, V, K, dev, fwd: bool, with_rloc=True):
    """Allocates the [N,G,H,V,KP] boundary buffers and returns (ctypes struct, dict of tensors)."""
    KP = padded_k(K)
    f32 = dict(dtype=torch.float32, device=dev)
    sg = L.Segments()
    sg.num_segments, sg.seg_len = G, seg_len
    t = {}
    names = ("sum_M", "sum_J", "start_M", "start_I") if fwd else ("carry_M", "carry_I", "rloc_M", "rloc_I")
    for n in names:
        t[n] = torch.empty(N, G, H, V, KP, **f32)
        setattr(sg, n, t[n].data_ptr())
    if fwd:
        t["decay"] = torch.empty(N, G, H, **f32)
        sg.decay = t["decay"].data_ptr()
    return sg, t


@torch.library.custom_op("palimpsa_b200::fwd", mutates_args=(), device_types="cuda")
def fwd_op(q: Tensor, k: Tensor, v: Tensor, b: Tensor, gt: Tensor, g: Tensor, Ip: Tensor,
           init_mu: Optional[Tensor], init_I: Optional[Tensor], cu_seqlens: Optional[Tensor],
           scale: float, uncertainty: bool, save_ckpt: bool, want_final: bool, recurrent: bool,
           num_segments: int) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    _require_cuda(q, k, v, b, gt, g, Ip, init_mu, init_I, cu_seqlens)
    lib = L.lib()
    B, T, H, K = q.shape
    V = v.shape[-1]
    N = B if cu_seqlens is None else cu_seqlens.numel() - 1
    dev = q.device
    with torch.cuda.device(dev):
        o = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
        o_var = torch.empty(B, T, H, V, dtype=q.dtype, device=dev) if uncertainty else q.new_empty(0)
        if want_final:
            fmu = torch.empty(N, H, V, K, dtype=torch.float32, device=dev)
            fI = torch.empty(N, H, V, K, dtype=torch.float32, device=dev)
        else:
            fmu = fI = None
        coff = _chunk_offsets(cu_seqlens) if cu_seqlens is not None else None
        order = _longest_first(cu_seqlens) if cu_seqlens is not None and N > 1 else None
        if save_ckpt:
            slots = _ckpt_slots(B * T, N)
            ckM = torch.empty(slots, H, V, padded_k(K), dtype=torch.float32, device=dev)
            ckI = torch.empty(slots, H, V, padded_k(K), dtype=torch.float32, device=dev)
        else:
            ckM = ckI = None
        prm = L.FwdParams()
        prm.struct_size = C.sizeof(L.FwdParams)
        prm.p = _problem(q, k, v, b, gt, g, Ip, cu_seqlens, coff, init_mu, init_I, scale,
                         L.FLAG_UNCERTAINTY if uncertainty else 0, order)
        prm.o, prm.o_var = _ptr(o), _ptr(o_var)
        prm.final_mu, prm.final_I = _ptr(fmu), _ptr(fI)
        prm.ckpt_M, prm.ckpt_I = _ptr(ckM), _ptr(ckI)
        decay = None
        if num_segments > 1 and T > 0:
            # summaries of every segment -> boundary scan -> all segments run side by side; in a packed batch
            # (T = all tokens) a segment index beyond a sequence's end is an empty segment
            sg, bufs = make_segments(N, num_segments, segment_len(T, num_segments), H, V, K, dev, fwd=True)
            st = _stream(q)
            L.check(lib.palimpsa_segment_summary(C.byref(prm.p), C.byref(sg), st), "palimpsa segment summary")
            L.check(lib.palimpsa_cp_combine(C.byref(prm.p), C.byref(sg), None, None, None, None, st),
                    "palimpsa boundary scan")
            L.check(lib.palimpsa_chunk_fwd_segments(C.byref(prm), C.byref(sg), st), "palimpsa forward (segments)")
            decay = bufs["decay"]
        else:
            fn = lib.palimpsa_recurrent_fwd if recurrent else lib.palimpsa_chunk_fwd
            L.check(fn(C.byref(prm), _stream(q)), "palimpsa forward")
    e = q.new_empty(0, dtype=torch.float32)
    return (o, o_var, fmu if want_final else e, fI if want_final else e.clone(),
            ckM if save_ckpt else e.clone(), ckI if save_ckpt else e.clone(),
            coff if coff is not None else q.new_empty(0, dtype=torch.int32),
            decay if decay is not None else e.clone())


@fwd_op.register_fake
def _(q, k, v, b, gt, g, Ip, init_mu, init_I, cu_seqlens, scale, uncertainty, save_ckpt, want_final, recurrent,
      num_segments):
    B, T, H, K = q.shape
    V = v.shape[-1]
    N = B if cu_seqlens is None else cu_seqlens.numel() - 1
    f32 = dict(dtype=torch.float32, device=q.device)
    o = q.new_empty(B, T, H, V)
    o_var = q.new_empty(B, T, H, V) if uncertainty else q.new_empty(0)
    fmu = q.new_empty((N, H, V, K) if want_final else (0,), **f32)
    fI = q.new_empty((N, H, V, K) if want_final else (0,), **f32)
    cs = (_ckpt_slots(B * T, N), H, V, padded_k(K)) if save_ckpt else (0,)
    coff = q.new_empty((N,) if cu_seqlens is not None else (0,), dtype=torch.int32)
    seg = num_segments > 1 and T > 0
    decay = q.new_empty((N, num_segments, H) if seg else (0,), **f32)
    return o, o_var, fmu, fI, q.new_empty(cs, **f32), q.new_empty(cs, **f32), coff, decay


@torch.library.custom_op("palimpsa_b200::bwd", mutates_args=(), device_types="cuda")
def bwd_op(do: Tensor, do_var: Optional[Tensor], q: Tensor, k: Tensor, v: Tensor, b: Tensor, gt: Tensor, g: Tensor,
           Ip: Tensor, cu_seqlens: Optional[Tensor], chunk_offsets: Optional[Tensor], ckpt_M: Tensor, ckpt_I: Tensor,
           scale: float, explicit_init: bool, recurrent: bool,
           seg_decay: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    _require_cuda(do, do_var, q, k, v, b, gt, g, Ip, cu_seqlens, ckpt_M, ckpt_I)
    lib = L.lib()
    B, T, H, K = q.shape
    dev = q.device
    with torch.cuda.device(dev):
        dq, dk, dv, db = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(b)
        dgt = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        dg = torch.empty(H, dtype=torch.float32, device=dev)
        dIp = torch.empty(H, dtype=torch.float32, device=dev)
        flags = (L.FLAG_UNCERTAINTY if do_var is not None else 0) | (L.FLAG_EXPLICIT_INIT if explicit_init else 0)
        prm = L.BwdParams()
        prm.struct_size = C.sizeof(L.BwdParams)
        order = _longest_first(cu_seqlens) if cu_seqlens is not None and cu_seqlens.numel() > 2 else None
        prm.p = _problem(q, k, v, b, gt, g, Ip, cu_seqlens, chunk_offsets, None, None, scale, flags, order)
        need = lib.palimpsa_bwd_workspace_bytes(C.byref(prm.p))
        ws = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
        prm.d_o, prm.d_o_var = _ptr(do), _ptr(do_var)
        prm.ckpt_M, prm.ckpt_I = _ptr(ckpt_M), _ptr(ckpt_I)
        prm.dq, prm.dk, prm.dv, prm.db = _ptr(dq), _ptr(dk), _ptr(dv), _ptr(db)
        prm.dgt, prm.dg, prm.dIp = _ptr(dgt), _ptr(dg), _ptr(dIp)
        prm.workspace, prm.workspace_bytes = ws.data_ptr(), ws.numel()
        if seg_decay is not None and seg_decay.numel() > 0:
            # state-gradient pass per segment -> reverse boundary scan -> full backward per segment
            G = seg_decay.shape[1]
            V = v.shape[-1]
            N = B if cu_seqlens is None else cu_seqlens.numel() - 1
            sg, bufs = make_segments(N, G, segment_len(T, G), H, V, K, dev, fwd=False)
            sg.decay = seg_decay.data_ptr()
            st = _stream(q)
            if carry_on_tensor_cores and lib.palimpsa_carry_apply_supported(C.byref(prm.p)):
                # zero-carry backward of every segment -> reverse boundary scan -> carried terms on the tensor
                # cores -> finishing kernels
                L.check(lib.palimpsa_chunk_bwd_segments(C.byref(prm), C.byref(sg), 2, st), "palimpsa backward (main)")
                L.check(lib.palimpsa_cp_combine_bwd(C.byref(prm.p), C.byref(sg), None, None, None, None, st),
                        "palimpsa boundary scan (backward)")
                L.check(lib.palimpsa_carry_apply(C.byref(prm), C.byref(sg), st), "palimpsa carried-gradient terms")
                L.check(lib.palimpsa_chunk_bwd_segments(C.byref(prm), C.byref(sg), 3, st), "palimpsa backward (finish)")
            else:
                # state-gradient pass per segment -> reverse boundary scan -> full backward per segment
                L.check(lib.palimpsa_chunk_bwd_segments(C.byref(prm), C.byref(sg), 1, st),
                        "palimpsa backward (carry pass)")
                L.check(lib.palimpsa_cp_combine_bwd(C.byref(prm.p), C.byref(sg), None, None, None, None, st),
                        "palimpsa boundary scan (backward)")
                sg.rloc_M = sg.rloc_I = None
                L.check(lib.palimpsa_chunk_bwd_segments(C.byref(prm), C.byref(sg), 0, st),
                        "palimpsa backward (segments)")
        else:
            fn = lib.palimpsa_recurrent_bwd if recurrent else lib.palimpsa_chunk_bwd
            L.check(fn(C.byref(prm), _stream(q)), "palimpsa backward")
    return dq, dk, dv, db, dgt, dg, dIp


@bwd_op.register_fake
def _(do, do_var, q, k, v, b, gt, g, Ip, cu_seqlens, chunk_offsets, ckpt_M, ckpt_I, scale, explicit_init, recurrent,
      seg_decay):
    B, T, H, K = q.shape
    f32 = dict(dtype=torch.float32, device=q.device)
    return (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(b),
            q.new_empty(B, T, H, **f32), q.new_empty(H, **f32), q.new_empty(H, **f32))


def _setup_context(ctx, inputs, output):
    (q, k, v, b, gt, g, Ip, init_mu, init_I, cu_seqlens, scale, uncertainty, save_ckpt, want_final, recurrent,
     num_segments) = inputs
    o, o_var, fmu, fI, ckM, ckI, coff, decay = output
    ctx.scale, ctx.uncertainty, ctx.recurrent = scale, uncertainty, recurrent
    ctx.explicit_init = init_mu is not None
    ctx.has_ckpt = save_ckpt
    ctx.varlen = cu_seqlens is not None
    ctx.save_for_backward(q, k, v, b, gt, g, Ip, cu_seqlens, coff, ckM, ckI, decay)
    # Only `o` (and `o_var`) ever receive a gradient.  Without this, autograd hands the backward a ZERO tensor for
    # every other float output -- including the two checkpoint buffers, i.e. 1.6 GB of fills per step at the
    # benchmark's size.
    ctx.set_materialize_grads(False)


def _backward(ctx, do, do_var, dfmu, dfI, _dckM, _dckI, _dcoff, _ddecay):
    # Gradients reaching the final states are ignored and initial states get none, as in the
    # reference (chunk_palimpsa_forgetting_scalar.py:522, :617-620: truncated BPTT across calls).
    q, k, v, b, gt, g, Ip, cu_seqlens, coff, ckM, ckI, decay = ctx.saved_tensors
    if not ctx.has_ckpt:
        raise RuntimeError("palimpsa_b200: backward needs the forward's checkpoints (forward ran with save_ckpt=False)")
    if do is None:
        do = torch.zeros(v.shape, dtype=q.dtype, device=q.device)
    do = do.to(q.dtype).contiguous()
    if do_var is not None:
        do_var = do_var.to(q.dtype)
    if ctx.uncertainty:
        do_var = torch.zeros_like(do) if do_var is None else do_var.contiguous()
    else:
        do_var = None
    dq, dk, dv, db, dgt, dg, dIp = bwd_op(do, do_var, q, k, v, b, gt, g, Ip, cu_seqlens if ctx.varlen else None,
                                          coff if ctx.varlen else None, ckM, ckI, ctx.scale, ctx.explicit_init,
                                          ctx.recurrent, decay if decay.numel() > 0 else None)
    return dq, dk, dv, db, dgt, dg, dIp, None, None, None, None, None, None, None, None, None


fwd_op.register_autograd(_backward, setup_context=_setup_context)


def run(q, k, v, b, gt, g, Ip, initial_mu_state, initial_I_state, scale, output_final_state, output_uncertainty,
        cu_seqlens, recurrent: bool, out_dtype, num_segments: Optional[int] = None, var_dtype=None):
    """Shared body of chunk_palimpsa / fused_recurrent_palimpsa: checks, dtype policy, op call, packing."""
    if q.dim() != 4 or k.shape != q.shape or v.dim() != 4 or b.shape != v.shape or v.shape[:3] != q.shape[:3]:
        raise ValueError("expected q,k [B,T,H,K] and v,b [B,T,H,V]")
    B, T, H, K = q.shape
    V = v.shape[-1]
    if tuple(gt.shape) != (B, T, H) or tuple(g.shape) != (H,) or tuple(Ip.shape) != (H,):
        raise ValueError("expected gt [B,T,H] and g, Ip [H]")
    _require_cuda(q, k, v, b, gt, g, Ip, initial_mu_state, initial_I_state, cu_seqlens)
    if q.dtype not in _DT:
        raise TypeError(f"unsupported dtype {q.dtype}; use float32, bfloat16 or float16")
    if cu_seqlens is not None:
        cu_seqlens = cu_seqlens.to(torch.int32).contiguous()
        N = cu_seqlens.numel() - 1
    else:
        N = B
    if (initial_mu_state is None) != (initial_I_state is None):
        raise ValueError("initial_mu_state and initial_I_state must be given together")
    if initial_mu_state is not None:
        if tuple(initial_mu_state.shape) != (N, H, V, K) or tuple(initial_I_state.shape) != (N, H, V, K):
            raise ValueError(f"initial states must have shape {(N, H, V, K)}")
        initial_mu_state = initial_mu_state.detach().float().contiguous()
        initial_I_state = initial_I_state.detach().float().contiguous()
    # One io dtype per call: the widest of the four token tensors (the reference's kernels read each tensor in its
    # own dtype and compute in fp32, so a narrower choice would round an input the reference does not round;
    # under autocast its layers do pass fp32 q/k next to bf16 v).
    io = q.dtype
    for x in (k, v, b):
        io = torch.promote_types(io, x.dtype)
    if io not in _DT:
        raise TypeError(f"unsupported dtype combination {[x.dtype for x in (q, k, v, b)]}")
    q, k, v, b = [x.to(io).contiguous() for x in (q, k, v, b)]
    gt, g, Ip = [x.float().contiguous() for x in (gt, g, Ip)]
    save_ckpt = torch.is_grad_enabled() and any(x.requires_grad for x in (q, k, v, b, gt, g, Ip))
    if num_segments is None:
        num_segments = plan_segments(N, T, H, K, V, q.device, backward=bool(save_ckpt), io_dtype=_DT[io],
                                     uncertainty=bool(output_uncertainty), packed=cu_seqlens is not None)
    o, o_var, fmu, fI, _, _, _, _ = fwd_op(q, k, v, b, gt, g, Ip, initial_mu_state, initial_I_state, cu_seqlens,
                                           float(scale), bool(output_uncertainty), save_ckpt, bool(output_final_state),
                                           recurrent, int(num_segments))
    if out_dtype is not None and out_dtype != o.dtype:
        o = o.to(out_dtype)
    if output_uncertainty and var_dtype is not None and var_dtype != o_var.dtype:
        o_var = o_var.to(var_dtype)
    out = (o, o_var) if output_uncertainty else o
    if output_final_state:
        return out, fmu, fI
    return out
