"""The allocation-free backward (``palimpsa_chunk_bwd_static``) against the regular backward.

Some hosts of this library may not allocate GPU memory once they are running: a plugin inside a
serving process whose memory pool was carved up at start-up, or a latency-critical thread for which
an allocation (which synchronises the device) is not acceptable.  For them the library carries its
own fixed scratch array.  This test drives both entry points through the C ABI on the same inputs,
twice in a row with different data, and expects identical gradients: the second call must not be
disturbed by what the first one left in the shared scratch.  Collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from oracle import palimpsa_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bwd_both(seed, B, T, H, K, V, dtype, unc):
    from palimpsa_b200 import _lib as L
    from palimpsa_b200.ops.palimpsa import _core
    lib = L.lib()
    inp = orc.make_inputs(seed, B=B, T=T, H=H, K=K, V=V, dtype=dtype)
    d = {n: x.to(DEV) for n, x in inp.items()}
    scale = K ** -0.5
    with torch.no_grad():
        _, _, _, _, ckM, ckI, _, _ = _core.fwd_op(d["q"], d["k"], d["v"], d["b"], d["gt"], d["g"], d["Ip"], None, None,
                                                  None, scale, unc, True, False, False, 1)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    results = []
    for static in (False, True):
        out = {n: torch.full_like(d[n], float("nan")) for n in ("q", "k", "v", "b")}
        dgt = torch.full((B, T, H), float("nan"), device=DEV)
        dg = torch.full((H,), float("nan"), device=DEV)
        dIp = torch.full((H,), float("nan"), device=DEV)
        prm = L.BwdParams()
        prm.struct_size = C.sizeof(L.BwdParams)
        prm.p = _core._problem(d["q"], d["k"], d["v"], d["b"], d["gt"], d["g"], d["Ip"], None, None, None, None, scale,
                               L.FLAG_UNCERTAINTY if unc else 0)
        prm.d_o = d["do"].data_ptr()
        prm.d_o_var = d["do_var"].data_ptr() if unc else None
        prm.ckpt_M, prm.ckpt_I = ckM.data_ptr(), ckI.data_ptr()
        prm.dq, prm.dk, prm.dv, prm.db = [out[n].data_ptr() for n in ("q", "k", "v", "b")]
        prm.dgt, prm.dg, prm.dIp = dgt.data_ptr(), dg.data_ptr(), dIp.data_ptr()
        need = lib.palimpsa_bwd_workspace_bytes(C.byref(prm.p))
        assert 0 < need <= L.STATIC_SCRATCH_BYTES
        if static:
            rc = lib.palimpsa_chunk_bwd_static(C.byref(prm), stream)
        else:
            ws = torch.empty(need, dtype=torch.uint8, device=DEV)
            prm.workspace, prm.workspace_bytes = ws.data_ptr(), need
            rc = lib.palimpsa_chunk_bwd(C.byref(prm), stream)
        assert rc == 0, lib.palimpsa_last_error_string(rc)
        torch.cuda.synchronize()
        results.append({"dq": out["q"], "dk": out["k"], "dv": out["v"], "db": out["b"], "dgt": dgt, "dg": dg,
                        "dIp": dIp})
    return results


def test_static_scratch_backward_matches_regular_backward_twice():
    for seed, shape in ((1, (2, 100, 2, 64, 64)), (2, (1, 333, 3, 128, 128))):
        ref, got = _bwd_both(seed, *shape, dtype=torch.bfloat16, unc=(seed == 2))
        for n in ref:
            assert torch.isfinite(got[n].float()).all(), n
            assert orc.rel_err(got[n], ref[n]) <= 1e-6, (seed, n)
            assert torch.equal(got[n], ref[n]), (seed, n)


def test_static_scratch_rejects_oversized_problem():
    from palimpsa_b200 import _lib as L
    lib = L.lib()
    prm = L.BwdParams()
    prm.struct_size = C.sizeof(L.BwdParams)
    one = torch.zeros(16, device=DEV)
    p = prm.p
    p.num_seqs, p.seq_len, p.total_tokens, p.H, p.K, p.V = 8, 4096, 8 * 4096, 6, 128, 128
    p.io_dtype = L.BF16
    p.scale = 1.0
    for f in ("q", "k", "v", "b", "gt", "g", "Ip"):
        setattr(p, f, one.data_ptr())
    for f in ("d_o", "ckpt_M", "ckpt_I", "dq", "dk", "dv", "db", "dgt", "dg", "dIp"):
        setattr(prm, f, one.data_ptr())
    assert lib.palimpsa_bwd_workspace_bytes(C.byref(p)) > L.STATIC_SCRATCH_BYTES
    assert lib.palimpsa_chunk_bwd_static(C.byref(prm), None) == -9      # PALIMPSA_E_LIMIT, nothing launched
    assert b"capacity" in lib.palimpsa_last_error_string(-9)
