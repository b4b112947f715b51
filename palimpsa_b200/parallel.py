"""Multi-GPU use of the Palimpsa operator: one process per GPU, ``torch.distributed`` for the plumbing.

Two modes, neither of which exists in the reference (it has no collective at all; its multi-GPU runs
come from the external trainer):

* **batch x head sharding** -- the operator is independent per (sequence, head), so every rank simply
  runs the single-GPU op on its slice (:func:`shard_batch`, :func:`shard_heads`).  No communication;
  ``dg`` / ``dIp`` come out as per-rank partial sums, exactly like data-parallel parameter gradients.

* **context parallelism** (:func:`cp_chunk_palimpsa`) -- one long sequence split contiguously over the
  ranks of a group.  The recurrence is linear in the state pair (M, J = I - Ip) with a scalar decay per
  head, so every rank first summarises its own tokens (end state from a zero start + total decay)
  without waiting for anybody; the true boundary states then travel down the ranks as ONE small
  point-to-point message per hop (2 x N x H x V x KP floats: 1.5 MB at H=12, d=128), and all ranks run
  their heavy pass side by side.  Backward mirrors this with the state gradients travelling up.

The hop logic is written against a small backend interface so that the protocol can be exercised with
CPU ranks (gloo) and a float64 stand-in for the kernels; the product backend below drives the CUDA
library through its C ABI.

Two transports for the hop.  ``"nccl"``: ``torch.distributed`` send / recv of the state.  ``"peer"`` (default on one
node when the ranks' buffers can be mapped into each other's address space): the boundary-scan kernel stores its
result straight into the next rank's buffer over NVLink and two one-thread kernels of the library order the
hand-over on the stream (:class:`PeerLink`); no host round trip and no library call per hop.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import _lib as L


# --------------------------------------------------------------------------------------------------
# batch x head sharding (no communication)
# --------------------------------------------------------------------------------------------------
def shard_bounds(n: int, rank: int, world: int):
    """Contiguous, balanced split of ``n`` units: the first ``n % world`` ranks get one extra."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    lo, hi = shard_bounds(x.shape[0], rank, world)
    return x[lo:hi]


def shard_heads(x: torch.Tensor, rank: int, world: int, head_dim: int = 2) -> torch.Tensor:
    """Slice of the head axis (dim 2 of ``[B,T,H,*]`` tensors, dim 0 of ``g`` / ``Ip``)."""
    lo, hi = shard_bounds(x.shape[head_dim], rank, world)
    return x.narrow(head_dim, lo, hi - lo)


# --------------------------------------------------------------------------------------------------
# boundary-state hops
# --------------------------------------------------------------------------------------------------
def _peer(group, r: int) -> int:
    return r if group is None else dist.get_global_rank(group, r)


def chain_down(rank: int, world: int, group, local: Callable[[Optional[torch.Tensor]], torch.Tensor],
               like: torch.Tensor) -> None:
    """Forward hop: rank r receives the boundary state from rank r-1 (rank 0 gets ``None``), runs
    ``local(state)`` which must return the state after its own tokens, and sends that to rank r+1.
    A peer that died or raised before sending surfaces here as the process group's timeout error."""
    inc = None
    if rank > 0:
        inc = torch.empty_like(like)
        dist.recv(inc, src=_peer(group, rank - 1), group=group)
    out = local(inc)
    if rank < world - 1:
        dist.send(out.contiguous(), dst=_peer(group, rank + 1), group=group)


def chain_up(rank: int, world: int, group, local: Callable[[Optional[torch.Tensor]], torch.Tensor],
             like: torch.Tensor) -> None:
    """Backward hop: the mirror image, state gradients travel from rank r+1 to rank r."""
    inc = None
    if rank < world - 1:
        inc = torch.empty_like(like)
        dist.recv(inc, src=_peer(group, rank + 1), group=group)
    out = local(inc)
    if rank > 0:
        dist.send(out.contiguous(), dst=_peer(group, rank - 1), group=group)


class PeerLink:
    """Exchange buffers of the ranks of one node, mapped into each other's address space (torch symmetric memory:
    CUDA virtual-memory handles exchanged through the process group's store).  Every rank owns::

        [ready_down, ack_down, ready_up, ack_up : uint64, 64 bytes in all][inbox_down : n floats][inbox_up : n floats]

    Direction 0 ("down") carries the boundary state from rank r to r+1, direction 1 ("up") the state gradient from
    r+1 to r.  The producer's kernel writes into the consumer's inbox through the mapped pointer, then publishes the
    sequence number of the call in the consumer's ``ready`` flag; the consumer, once its kernels have read the inbox,
    publishes the same number in the producer's ``ack`` flag, and the producer waits for the previous number there
    before it overwrites the inbox.  Sequence numbers only grow, so nothing is ever reset.  Every rank must make the
    same sequence of calls (as with any collective), and a rank must enqueue the calls of one group on one stream
    (the hand-over is ordered by stream order).  All waits are the library's bounded ones."""

    FLAG_FLOATS = 16                                        # 64 bytes of flags in front of the inboxes
    _links = {}                                             # (group id, numel) -> PeerLink, or None if unavailable

    def __init__(self, group, numel: int, device, timeout_ms: int = 20000):
        import os
        # Only plain peer loads and stores are used here: ask torch not to bind the buffers to an NVLink multicast
        # object as well (it reads the variable when its symmetric-memory code is first used).
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.n, self.timeout_ms = int(numel), int(timeout_ms)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.buf = symm.empty(self.FLAG_FLOATS + 2 * self.n, dtype=torch.float32, device=device)
        self.buf.zero_()
        self.hdl = symm.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
        self.ptrs = [int(x) for x in self.hdl.buffer_ptrs]
        if len(self.ptrs) != self.world or self.ptrs[self.rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric memory returned an unexpected set of buffers")
        self.epoch = [0, 0]
        torch.cuda.synchronize(device)

    def inbox(self, d: int) -> torch.Tensor:
        lo = self.FLAG_FLOATS + d * self.n
        return self.buf[lo:lo + self.n]

    def inbox_ptr(self, rank: int, d: int) -> int:
        return self.ptrs[rank] + 4 * (self.FLAG_FLOATS + d * self.n)

    def flag_ptr(self, rank: int, d: int, ack: bool) -> int:
        return self.ptrs[rank] + 16 * d + (8 if ack else 0)

    @classmethod
    def get(cls, group, numel: int, device):
        """The link of this group for states of ``numel`` floats, built on first use (a collective: every rank of
        the group comes here in the same call).  ``None`` when the ranks are not on one node or the mapping cannot
        be set up; all ranks then agree on that and use send / recv."""
        pg = group if group is not None else dist.group.WORLD
        key = (getattr(pg, "group_name", None) or id(pg), int(numel))
        if key not in cls._links:
            cls._links[key] = cls._build(group, numel, device)
        return cls._links[key]

    @classmethod
    def _build(cls, group, numel, device):
        import socket

        def all_agree(ok: bool) -> bool:
            t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
            return bool(t.item())

        world = dist.get_world_size(group)
        names = [None] * world
        dist.all_gather_object(names, socket.gethostname(), group=group)
        ok = len(set(names)) == 1 and "nccl" in str(dist.get_backend(group))
        try:
            import torch.distributed._symmetric_memory  # noqa: F401
        except Exception:                                   # noqa: BLE001
            ok = False
        if not all_agree(ok):
            return None
        link = None
        try:
            link = cls(group, numel, device)
        except Exception:                                   # noqa: BLE001  (no peer access, old driver, ...)
            link = None
        if not all_agree(link is not None):
            return None
        dist.barrier(group)                                 # every rank's flags are zero before anybody signals
        return link


def chain_peer(link: PeerLink, d: int, rank: int, world: int, local, stream, prepare=None, relay=None) -> None:
    """One hop of direction ``d`` (0: down, 1: up) over a :class:`PeerLink`.  ``local(inc, out_ptr, want_out)``
    enqueues the boundary scan: ``inc`` is the incoming state (a view of this rank's inbox, ``None`` at the start of
    the chain) and ``out_ptr`` the address in the NEXT rank's inbox where the outgoing state goes (``None`` at the
    end).  A rank in the middle shortens the chain's critical path with ``prepare() -> total`` (enqueued before the
    wait: what its own segments add, independent of the incoming state) and ``relay(inc, total, out_ptr)``
    (``out = decay * inc + total``): the next rank is signalled right after the relay, the full scan follows."""
    lib = L.lib()
    src, dst = (rank - 1, rank + 1) if d == 0 else (rank + 1, rank - 1)
    has_src, has_dst = 0 <= src < world, 0 <= dst < world
    link.epoch[d] += 1
    e = link.epoch[d]
    inc = out_ptr = None
    middle = has_src and has_dst and prepare is not None and relay is not None
    total = prepare() if middle else None
    if has_src:
        inbox = link.inbox(d)
        L.check(lib.palimpsa_peer_wait(link.flag_ptr(rank, d, False), e, link.timeout_ms, inbox.data_ptr(), stream),
                "wait for the previous rank's boundary state")
        inc = inbox
    if has_dst:
        L.check(lib.palimpsa_peer_wait(link.flag_ptr(rank, d, True), e - 1, link.timeout_ms, None, stream),
                "wait for the next rank to have read the previous state")
        out_ptr = link.inbox_ptr(dst, d)
    if middle:
        relay(inc, total, out_ptr)
        L.check(lib.palimpsa_peer_signal(link.flag_ptr(dst, d, False), e, stream), "publish the boundary state")
        local(inc, None, False)
    else:
        local(inc, out_ptr, has_dst)
        if has_dst:
            L.check(lib.palimpsa_peer_signal(link.flag_ptr(dst, d, False), e, stream), "publish the boundary state")
    if has_src:
        L.check(lib.palimpsa_peer_signal(link.flag_ptr(src, d, True), e, stream), "release the previous rank's buffer")


# --------------------------------------------------------------------------------------------------
# CUDA backend of the context-parallel op
# --------------------------------------------------------------------------------------------------
class _CudaLocal:
    """One rank's share of the sequence, driven through the C ABI (segment entry points)."""

    def __init__(self, q, k, v, b, gt, g, Ip, scale, num_segments, first_rank: bool, init_mu=None, init_I=None,
                 uncertainty: bool = False):
        from .ops.palimpsa import _core
        self.core = _core
        self.lib = L.lib()
        self.t = (q, k, v, b, gt, g, Ip)
        self.N, self.T, self.H, self.K = q.shape
        self.V = v.shape[-1]
        self.KP = _core.padded_k(self.K)
        self.scale = float(scale)
        self.G = max(1, int(num_segments))
        self.seg_len = _core.segment_len(max(self.T, 1), self.G)
        self.first = first_rank
        self.dev = q.device
        self.stream = _core._stream(q)
        self.do_var = None                               # gradient of the uncertainty output, set by backward
        self.sg, self.bufs = _core.make_segments(self.N, self.G, self.seg_len, self.H, self.V, self.K, self.dev, True)
        self.unc = uncertainty
        # only the rank that holds the start of the sequence knows an explicit initial state
        self.init = (init_mu, init_I) if first_rank and init_mu is not None else (None, None)
        self.prob = _core._problem(q, k, v, b, gt, g, Ip, None, None, self.init[0], self.init[1], self.scale,
                                   L.FLAG_UNCERTAINTY if uncertainty else 0)

    def state_like(self):
        return torch.empty(2, self.N, self.H, self.V, self.KP, dtype=torch.float32, device=self.dev)

    def summary(self):
        L.check(self.lib.palimpsa_segment_summary(C.byref(self.prob), C.byref(self.sg), self.stream), "segment summary")

    def _halves(self, inc, out_ptr, want_out=True):
        """(in_M, in_J, out_M, out_J, out tensor): ``inc`` a [2,N,H,V,KP] tensor (or its flat view) or None;
        ``out_ptr`` a raw address to write the outgoing pair to (a peer's inbox) or None for a fresh local tensor;
        ``want_out=False``: the scan writes no outgoing state at all."""
        half = 4 * self.N * self.H * self.V * self.KP
        a, bb = (None, None) if inc is None else (inc.data_ptr(), inc.data_ptr() + half)
        if not want_out:
            return a, bb, None, None, None
        out = None
        if out_ptr is None:
            out = self.state_like()
            out_ptr = out.data_ptr()
        return a, bb, out_ptr, out_ptr + half, out

    def relay_prepare(self, sg, backward: bool):
        tot = self.state_like()
        L.check(self.lib.palimpsa_cp_relay_prepare(C.byref(self.prob), C.byref(sg), int(backward), tot[0].data_ptr(),
                                                   tot[1].data_ptr(), self.stream), "relay total")
        return tot

    def relay(self, sg, inc, tot, out_ptr):
        a, bb, oa, ob, _ = self._halves(inc, out_ptr)
        L.check(self.lib.palimpsa_cp_relay(C.byref(self.prob), C.byref(sg), a, bb, tot[0].data_ptr(), tot[1].data_ptr(),
                                           oa, ob, self.stream), "relay")

    def combine(self, inc, out_ptr=None, want_out=True):
        a, bb, om, oj, out = self._halves(inc, out_ptr, want_out)
        L.check(self.lib.palimpsa_cp_combine(C.byref(self.prob), C.byref(self.sg), a, bb, om, oj, self.stream),
                "boundary scan")
        return out

    def forward(self, save_ckpt: bool):
        q, k, v, b, gt, g, Ip = self.t
        core = self.core
        o = torch.empty(self.N, self.T, self.H, self.V, dtype=q.dtype, device=self.dev)
        o_var = torch.empty_like(o) if self.unc else None
        fmu = torch.empty(self.N, self.H, self.V, self.K, dtype=torch.float32, device=self.dev)
        fI = torch.empty_like(fmu)
        ckM = ckI = None
        if save_ckpt:
            slots = core._ckpt_slots(self.N * self.T, self.N)
            ckM = torch.empty(slots, self.H, self.V, self.KP, dtype=torch.float32, device=self.dev)
            ckI = torch.empty_like(ckM)
        prm = L.FwdParams()
        prm.struct_size = C.sizeof(L.FwdParams)
        prm.p = self.prob
        prm.o, prm.o_var = core._ptr(o), core._ptr(o_var)
        prm.final_mu, prm.final_I = fmu.data_ptr(), fI.data_ptr()
        prm.ckpt_M, prm.ckpt_I = core._ptr(ckM), core._ptr(ckI)
        L.check(self.lib.palimpsa_chunk_fwd_segments(C.byref(prm), C.byref(self.sg), self.stream), "forward (segments)")
        return o, o_var, fmu, fI, ckM, ckI

    # ---- backward ----
    def _bwd_params(self, do, ckM, ckI, outs=None, ws=None):
        core = self.core
        prm = L.BwdParams()
        prm.struct_size = C.sizeof(L.BwdParams)
        prm.p = self.prob
        if not self.first:
            prm.p.flags |= L.FLAG_EXPLICIT_INIT      # this rank starts from a received state, not from the prior
        prm.d_o, prm.d_o_var = core._ptr(do), core._ptr(self.do_var)
        prm.ckpt_M, prm.ckpt_I = ckM.data_ptr(), ckI.data_ptr()
        if outs is not None:
            prm.dq, prm.dk, prm.dv, prm.db, prm.dgt, prm.dg, prm.dIp = [core._ptr(x) for x in outs]
            prm.workspace, prm.workspace_bytes = ws.data_ptr(), ws.numel()
        return prm

    def bwd_segments(self, decay):
        sg, bufs = self.core.make_segments(self.N, self.G, self.seg_len, self.H, self.V, self.K, self.dev, False)
        sg.decay = decay.data_ptr()
        return sg, bufs

    def bwd_carry(self, do, ckM, ckI, sg):
        prm = self._bwd_params(do, ckM, ckI)
        L.check(self.lib.palimpsa_chunk_bwd_segments(C.byref(prm), C.byref(sg), 1, self.stream), "backward carry pass")

    def combine_bwd(self, sg, inc, out_ptr=None, want_out=True):
        a, bb, om, oi, out = self._halves(inc, out_ptr, want_out)
        L.check(self.lib.palimpsa_cp_combine_bwd(C.byref(self.prob), C.byref(sg), a, bb, om, oi, self.stream),
                "boundary scan (backward)")
        return out

    def _outs(self, do, ckM, ckI):
        q, k, v, b, gt, g, Ip = self.t
        outs = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(b),
                torch.empty(self.N, self.T, self.H, dtype=torch.float32, device=self.dev),
                torch.empty(self.H, dtype=torch.float32, device=self.dev),
                torch.empty(self.H, dtype=torch.float32, device=self.dev)]
        prm = self._bwd_params(do, ckM, ckI)
        need = self.lib.palimpsa_bwd_workspace_bytes(C.byref(prm.p))
        ws = torch.empty(max(need, 256), dtype=torch.uint8, device=self.dev)
        return outs, ws, self._bwd_params(do, ckM, ckI, outs, ws)

    def tensor_core_carry(self) -> bool:
        return self.core.carry_on_tensor_cores and bool(self.lib.palimpsa_carry_apply_supported(C.byref(self.prob)))

    def backward(self, do, ckM, ckI, sg):
        """Full backward of every local segment with the end-state gradients in sg.carry_*."""
        outs, ws, prm = self._outs(do, ckM, ckI)
        sg.rloc_M = sg.rloc_I = None
        L.check(self.lib.palimpsa_chunk_bwd_segments(C.byref(prm), C.byref(sg), 0, self.stream), "backward (segments)")
        return outs

    def backward_main(self, do, ckM, ckI, sg):
        """Tensor-core path, step 1: zero-carry backward of every local segment (+ start-state gradients)."""
        outs, ws, prm = self._outs(do, ckM, ckI)
        L.check(self.lib.palimpsa_chunk_bwd_segments(C.byref(prm), C.byref(sg), 2, self.stream), "backward (main)")
        return outs, ws, prm

    def backward_finish(self, prm, sg):
        """Tensor-core path, step 2 (after the chain): carried terms as GEMMs, then the finishing kernels."""
        L.check(self.lib.palimpsa_carry_apply(C.byref(prm), C.byref(sg), self.stream), "carried-gradient terms")
        L.check(self.lib.palimpsa_chunk_bwd_segments(C.byref(prm), C.byref(sg), 3, self.stream), "backward (finish)")


class _CpChunkPalimpsa(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, b, gt, g, Ip, scale, group, num_segments, reduce_param_grads, init_mu, init_I,
                uncertainty, link):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        loc = _CudaLocal(q, k, v, b, gt, g, Ip, scale, num_segments, first_rank=(rank == 0), init_mu=init_mu,
                         init_I=init_I, uncertainty=uncertainty)
        need_grad = any(ctx.needs_input_grad[:7])
        with torch.cuda.device(q.device):
            loc.summary()                                    # no dependence on other ranks
            if link is not None:
                chain_peer(link, 0, rank, world, loc.combine, loc.stream,
                           prepare=lambda: loc.relay_prepare(loc.sg, False),
                           relay=lambda inc, tot, out: loc.relay(loc.sg, inc, tot, out))
            else:
                chain_down(rank, world, group, loc.combine, loc.state_like())
            o, o_var, fmu, fI, ckM, ckI = loc.forward(save_ckpt=need_grad)
        ctx.loc, ctx.group, ctx.reduce, ctx.link = loc, group, reduce_param_grads, link
        ctx.set_materialize_grads(False)                 # no zero tensors for outputs that received no gradient
        ctx.rank, ctx.world = rank, world
        if need_grad:
            # the inputs go through save_for_backward as well, so that an in-place change between forward and
            # backward is detected (the C structs of `loc` hold their raw addresses)
            ctx.save_for_backward(q, k, v, b, gt, g, Ip, ckM, ckI, loc.bufs["decay"])
        # ONE call with every non-differentiable output (a second call would replace the first): the final
        # states never carry a graph, like the reference's (chunk_palimpsa_forgetting_scalar.py:522)
        if o_var is None:
            o_var = o.new_empty(0)
            ctx.mark_non_differentiable(fmu, fI, o_var)
        else:
            ctx.mark_non_differentiable(fmu, fI)
        return o, o_var, fmu, fI

    @staticmethod
    def backward(ctx, do, do_var, _dmu, _dI):
        loc = ctx.loc
        *inputs, ckM, ckI, decay = ctx.saved_tensors       # raises if an input was modified in place meanwhile
        assert all(x.data_ptr() == y.data_ptr() for x, y in zip(inputs, loc.t))
        io = loc.t[0].dtype
        do = torch.zeros_like(loc.t[2]) if do is None else do.to(io).contiguous()
        if loc.unc:
            loc.do_var = torch.zeros_like(do) if do_var is None else do_var.to(io).contiguous()
        with torch.cuda.device(do.device):
            sg, bufs = loc.bwd_segments(decay)

            def hop_up():
                if ctx.link is not None:
                    chain_peer(ctx.link, 1, ctx.rank, ctx.world,
                               lambda inc, out, want: loc.combine_bwd(sg, inc, out, want), loc.stream,
                               prepare=lambda: loc.relay_prepare(sg, True),
                               relay=lambda inc, tot, out: loc.relay(sg, inc, tot, out))
                else:
                    chain_up(ctx.rank, ctx.world, ctx.group, lambda inc: loc.combine_bwd(sg, inc), loc.state_like())

            if loc.tensor_core_carry():
                # the heavy pass needs no remote data: it runs BEFORE the chain, on all ranks at once
                outs, ws, prm = loc.backward_main(do, ckM, ckI, sg)
                hop_up()
                loc.backward_finish(prm, sg)
                dq, dk, dv, db, dgt, dg, dIp = outs
            else:
                loc.bwd_carry(do, ckM, ckI, sg)              # zero-carry state gradients of every segment
                hop_up()
                dq, dk, dv, db, dgt, dg, dIp = loc.backward(do, ckM, ckI, sg)
            if ctx.reduce and ctx.world > 1:
                pg = torch.stack([dg, dIp])
                dist.all_reduce(pg, group=ctx.group)
                dg, dIp = pg[0], pg[1]
        return dq, dk, dv, db, dgt, dg, dIp, None, None, None, None, None, None, None, None


def cp_chunk_palimpsa(q, k, v, b, gt, g, Ip, group=None, scale=None, output_final_state=False, num_segments=None,
                      reduce_param_grads=True, initial_mu_state=None, initial_I_state=None,
                      output_uncertainty=False, transport: str = "auto"):
    """Context-parallel ``chunk_palimpsa``: every rank of ``group`` passes ITS contiguous share of the
    sequence (``q,k [B,T_local,H,K]`` ...; shares in rank order; lengths may differ) and gets its share of
    ``o`` and of the gradients.  With ``output_final_state`` also returns the state after this rank's
    last token (the sequence's final state on the last rank).  ``dg`` / ``dIp`` are summed over the group
    unless ``reduce_param_grads=False``.  ``initial_mu_state`` / ``initial_I_state`` ``[B,H,V,K]`` (both or
    neither) are the state before the sequence's first token: only the first rank's are used, and they get
    no gradient, as in ``chunk_palimpsa``.  ``output_uncertainty`` returns ``(o, o_var)`` in place of ``o``.
    ``transport``: ``"nccl"`` (send / recv), ``"peer"`` (stores into the next rank's mapped buffer, :class:`PeerLink`;
    an error if it cannot be set up) or ``"auto"`` (peer where available, else nccl); the same on every rank."""
    from .ops.palimpsa import _core
    _core._require_cuda(q, k, v, b, gt, g, Ip)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    io = q.dtype
    q, k, v, b = [x.to(io).contiguous() for x in (q, k, v, b)]
    gt, g, Ip = [x.float().contiguous() for x in (gt, g, Ip)]
    B, T, H, K = q.shape
    if num_segments is None:
        num_segments = _core.plan_segments(B, T, H, K, v.shape[-1], q.device, backward=torch.is_grad_enabled(),
                                            io_dtype=_core._DT.get(q.dtype, L.BF16))
    if (initial_mu_state is None) != (initial_I_state is None):
        raise ValueError("pass both initial_mu_state and initial_I_state, or neither")
    if initial_mu_state is not None:
        _core._require_cuda(initial_mu_state, initial_I_state)
        shape = (B, H, v.shape[-1], K)
        if tuple(initial_mu_state.shape) != shape or tuple(initial_I_state.shape) != shape:
            raise ValueError(f"initial states must have shape {shape}")
        initial_mu_state = initial_mu_state.detach().float().contiguous()
        initial_I_state = initial_I_state.detach().float().contiguous()
    if transport not in ("auto", "nccl", "peer"):
        raise ValueError(f"transport must be 'auto', 'nccl' or 'peer', got {transport!r}")
    link = None
    if transport != "nccl" and dist.get_world_size(group) > 1:
        with torch.cuda.device(q.device):                  # the set-up's collectives run on this rank's GPU
            link = PeerLink.get(group, 2 * B * H * v.shape[-1] * _core.padded_k(K), q.device)
        if link is None and transport == "peer":
            raise RuntimeError("palimpsa_b200: the ranks' buffers cannot be mapped into each other's address space "
                               "(not one node, no peer access, or no symmetric-memory support); use transport='nccl'")
    o, o_var, fmu, fI = _CpChunkPalimpsa.apply(q, k, v, b, gt, g, Ip, float(scale), group, int(num_segments),
                                               bool(reduce_param_grads), initial_mu_state, initial_I_state,
                                               bool(output_uncertainty), link)
    out = (o, o_var) if output_uncertainty else o
    return (out, fmu, fI) if output_final_state else out
