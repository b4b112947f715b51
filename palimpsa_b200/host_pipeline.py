"""Forward + backward of ``chunk_palimpsa`` for data that lives in HOST memory.

The op is independent per sequence, so a batch held in pinned host buffers can be processed in slices:
while slice i computes, slice i+1 is on its way to the device and the results of slice i-1 are on their
way back (three CUDA streams; PCIe is full duplex).  Device staging buffers are allocated once and
reused, so that a step makes no allocator round trip on the copy streams.  ``dg`` / ``dIp`` (sums over
the batch) are accumulated on the device and returned once.  Not part of the reference, whose ops only
see device tensors; it exists because end-to-end throughput from host buffers is copy-bound otherwise.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Union

import torch

from . import _lib as L
from .ops import chunk_palimpsa

_IN_BATCHED = ("q", "k", "v", "b", "gt", "do")
_OUT_BATCHED = ("o", "dq", "dk", "dv", "db", "dgt")


def ramped_widths(batch: int, middle: int = 2):
    """Slice widths ``1, middle, ..., middle, 1`` covering ``batch`` sequences (fewer, wider slices keep
    the kernels' grids full; the single-sequence slices at both ends keep the exposed copies short)."""
    if batch <= 2:
        return [1] * batch
    inner, widths = batch - 2, [1]
    while inner > 0:
        w = min(middle, inner)
        widths.append(w)
        inner -= w
    return widths + [1]


class HostPipeline:
    """Reusable pipeline for one problem shape.  ``run(host)`` takes pinned CPU tensors ``q,k,v,b,do``
    ``[B,T,H,*]``, ``gt [B,T,H]``, ``g,Ip [H]`` and returns pinned CPU tensors ``o, dq, dk, dv, db, dgt,
    dg, dIp``; it returns after everything has landed on the host.  The returned pinned tensors belong to the
    pipeline and are overwritten by the next ``run``: copy what must outlive it."""

    def __init__(self, host: Dict[str, torch.Tensor], device, slices: Union[int, Sequence[int]] = 4):
        """``slices``: a count (even split of the batch) or the slice widths themselves, e.g. ``(1, 2, 2,
        2, 1)``: a narrow first slice starts the compute early and a narrow last one shortens the final
        download, which is all of the copy time that cannot hide behind compute."""
        self.dev = torch.device(device)
        B = host["q"].shape[0]
        if isinstance(slices, int):
            n = max(1, min(slices, B))
            widths = [(i + 1) * B // n - i * B // n for i in range(n)]
        else:
            widths = [int(w) for w in slices]
            if not widths or min(widths) < 1 or sum(widths) != B:
                raise ValueError(f"slice widths {widths} must be positive and sum to the batch size {B}")
        self.slices = len(widths)
        self.bounds, lo = [], 0
        for w in widths:
            self.bounds.append((lo, lo + w))
            lo += w
        width = max(hi - lo for lo, hi in self.bounds)
        # two staging slots: slice i+1 uploads while slice i computes
        self.slots = [{n: torch.empty((width,) + tuple(host[n].shape[1:]), dtype=host[n].dtype, device=self.dev)
                       for n in _IN_BATCHED} for _ in range(2)]
        self.out = {}
        self.s_in, self.s_out = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        self.free = [None, None]   # event after which a slot may be overwritten

    def run(self, host: Dict[str, torch.Tensor], scale=None) -> Dict[str, torch.Tensor]:
        dev, cur = self.dev, torch.cuda.current_stream(self.dev)
        s_in, s_out = self.s_in, self.s_out
        B = host["q"].shape[0]
        s_in.wait_stream(cur)
        with torch.cuda.stream(s_in):
            g = host["g"].to(dev, non_blocking=True)
            Ip = host["Ip"].to(dev, non_blocking=True)
        g.record_stream(cur)
        Ip.record_stream(cur)

        def upload(i):
            lo, hi = self.bounds[i]
            slot = self.slots[i % 2]
            with torch.cuda.stream(s_in):
                if self.free[i % 2] is not None:
                    s_in.wait_event(self.free[i % 2])
                for n in _IN_BATCHED:
                    slot[n][: hi - lo].copy_(host[n][lo:hi], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
            return ev

        ready = {0: upload(0)}
        dg_acc = dIp_acc = None
        pending = []
        for i, (lo, hi) in enumerate(self.bounds):
            if i + 1 < self.slices:
                ready[i + 1] = upload(i + 1)
            cur.wait_event(ready.pop(i))
            slot = self.slots[i % 2]
            leaves = [slot[n][: hi - lo].detach().requires_grad_(True) for n in ("q", "k", "v", "b", "gt")]
            gl, ipl = g.detach().requires_grad_(True), Ip.detach().requires_grad_(True)
            o = chunk_palimpsa(*leaves, gl, ipl, scale=scale)
            o.backward(slot["do"][: hi - lo])
            res = dict(zip(_OUT_BATCHED, [o.detach()] + [x.grad for x in leaves]))
            dg_acc = gl.grad if dg_acc is None else dg_acc + gl.grad
            dIp_acc = ipl.grad if dIp_acc is None else dIp_acc + ipl.grad
            done = torch.cuda.Event()
            done.record(cur)
            self.free[i % 2] = done
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                for n, x in res.items():
                    if n not in self.out:
                        self.out[n] = torch.empty((B,) + tuple(x.shape[1:]), dtype=x.dtype, pin_memory=True)
                    self.out[n][lo:hi].copy_(x, non_blocking=True)
            pending.append(res)          # keep the device results alive until their copies are done
        for n, x in (("dg", dg_acc), ("dIp", dIp_acc)):
            if n not in self.out:
                self.out[n] = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
            self.out[n].copy_(x, non_blocking=True)
        cur.synchronize()
        s_out.synchronize()
        pending.clear()
        code = L.lib().palimpsa_tensor_core_status()     # everything has finished: did a bounded in-kernel wait give up?
        if code:
            raise RuntimeError(f"palimpsa_b200: a bounded wait inside a kernel gave up (code {code}); "
                               "the results of this run are invalid")
        return self.out


def fwd_bwd_from_host(host: Dict[str, torch.Tensor], device, slices: Union[int, Sequence[int]] = 4, scale=None,
                      pipeline: Optional[HostPipeline] = None) -> Dict[str, torch.Tensor]:
    """One-shot convenience wrapper; pass ``pipeline`` to reuse staging buffers across calls."""
    pipe = pipeline or HostPipeline(host, device, slices)
    return pipe.run(host, scale=scale)
