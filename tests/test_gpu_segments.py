"""Segment-parallel execution on one GPU: sequences cut into segments that run side by side must give
the same outputs, final states and gradients as the float64 oracle (and as the unsegmented op)."""
import pytest
import torch

from oracle import palimpsa_oracle as orc
from tests.gpu_util import DEV, compare, run_oracle
from tests.helpers import TOL_BF16, TOL_FP32

pytestmark = pytest.mark.gpu


def _run(inp, G, unc=False, mu0=None, I0=None, cu=None):
    from palimpsa_b200.ops import chunk_palimpsa
    names = ("q", "k", "v", "b", "gt", "g", "Ip")
    leaves = {n: inp[n].to(DEV).clone().requires_grad_(True) for n in names}
    kw = dict(output_final_state=True, output_uncertainty=unc, num_segments=G)
    if mu0 is not None:
        kw.update(initial_mu_state=mu0.to(DEV), initial_I_state=I0.to(DEV))
    if cu is not None:
        kw["cu_seqlens"] = torch.as_tensor(cu, dtype=torch.int32, device=DEV)
    out, fmu, fI = chunk_palimpsa(*[leaves[n] for n in names], **kw)
    res = {"final_mu": fmu, "final_I": fI}
    if unc:
        res["o"], res["o_var"] = out
    else:
        res["o"] = out
    loss = (res["o"].float() * inp["do"].to(DEV).float()).sum()
    if unc:
        loss = loss + (res["o_var"].float() * inp["do_var"].to(DEV).float()).sum()
    loss.backward()
    for n in names:
        res["d" + n] = leaves[n].grad
    torch.cuda.synchronize()
    return {k: v.detach().cpu() for k, v in res.items()}


@pytest.mark.parametrize("T,G", [(200, 3), (64, 4), (131, 2), (50, 7)])
def test_segments_fp32(T, G):
    inp = orc.make_inputs(T + G, B=2, T=T, H=2, K=64, V=40)
    got = _run(inp, G, unc=True)
    ref = run_oracle(inp, unc=True)
    compare(got, ref, TOL_FP32, what=f"segments T={T} G={G}")


def test_segments_with_initial_state_and_slow_decay():
    inp = orc.make_inputs(3, B=1, T=300, H=3, K=32, V=32)
    inp["gt"] = inp["gt"] * 0.02            # decays 0.95 .. 0.9998: boundary states matter over long ranges
    mu0, I0 = orc.make_states(4, 1, 3, 32, 32, inp["Ip"])
    got = _run(inp, 5, mu0=mu0, I0=I0)
    ref = run_oracle(inp, mu0=mu0, I0=I0)
    compare(got, ref, TOL_FP32, what="segments + init")


@pytest.mark.parametrize("dtype,G", [(torch.float32, 4), (torch.float32, 9), (torch.bfloat16, 4)])
def test_segments_in_a_packed_batch(dtype, G):
    """Packed sequences of very different lengths (one empty): a segment index past a sequence's end is an
    empty segment; every sequence still starts from the prior / its own initial state."""
    cu = [0, 40, 41, 300, 300, 811, 1024]
    inp = orc.make_inputs(21, B=1, T=1024, H=2, K=64, V=64, dtype=dtype)
    inp["gt"] = inp["gt"] * 0.1
    mu0, I0 = orc.make_states(5, len(cu) - 1, 2, 64, 64, inp["Ip"])
    got = _run(inp, G, unc=(dtype == torch.float32), mu0=mu0, I0=I0, cu=cu)
    ref = run_oracle(inp, unc=(dtype == torch.float32), mu0=mu0, I0=I0, cu=cu)
    compare(got, ref, TOL_FP32 if dtype == torch.float32 else TOL_BF16, what=f"packed + segments {dtype} G={G}")


def test_packed_batch_with_few_documents_is_segmented_by_default():
    """Three documents x two heads cannot fill the GPU: the planner cuts the packed axis (T / 256 = 10 segments of
    ~256 tokens) without being asked, and the results still match the float64 oracle."""
    from palimpsa_b200.ops.palimpsa._core import plan_segments
    cu = [0, 1500, 1700, 2560]
    assert plan_segments(3, 2560, 2, 64, 64, backward=True, packed=True) == 10
    inp = orc.make_inputs(33, B=1, T=2560, H=2, K=64, V=64, dtype=torch.float32)
    inp["gt"] = inp["gt"] * 0.1
    got = _run(inp, None, cu=cu)
    ref = run_oracle(inp, cu=cu)
    compare(got, ref, TOL_FP32, what="packed batch, planner's segments")


def test_segments_bf16_match_unsegmented():
    inp = orc.make_inputs(9, B=1, T=2048, H=2, K=128, V=128, dtype=torch.bfloat16)
    inp["gt"] = inp["gt"] * 0.05
    a = _run(inp, 1)
    b = _run(inp, 4)
    for n in a:
        assert orc.rel_err(b[n], a[n]) <= TOL_BF16, n


def test_auto_plan_uses_segments_only_when_starved():
    from palimpsa_b200.ops.palimpsa._core import plan_segments
    assert plan_segments(8, 4096, 6, 128, 128) == 1       # 170M-shaped batch: the grid already fills the GPU
    assert plan_segments(1, 131072, 12, 128, 128) == 32   # one long sequence: 96 CTAs -> 32 segments of 4096
    assert plan_segments(1, 4096, 6, 128, 128) == 16      # a one-sequence slice: 256-token segments
    assert plan_segments(1, 512, 2, 64, 64) == 1


def test_tensor_core_carry_terms_match_oracle_and_cuda_core_path(monkeypatch):
    """bf16: the carried-gradient terms computed with tcgen05 GEMMs equal the two-pass CUDA-core path and the
    float64 oracle within the bf16 bound; no bounded wait gave up."""
    from palimpsa_b200 import _lib as L
    inp = orc.make_inputs(17, B=2, T=700, H=2, K=128, V=128, dtype=torch.bfloat16)
    inp["gt"] = inp["gt"] * 0.05            # slow decay (0.9 .. 0.99): the carried terms are large
    ref = run_oracle(inp)
    tc_path = _run(inp, 5)
    assert L.lib().palimpsa_tensor_core_status() == 0
    from palimpsa_b200.ops.palimpsa import _core
    monkeypatch.setattr(_core, "carry_on_tensor_cores", False)
    simt = _run(inp, 5)
    compare(tc_path, ref, TOL_BF16, what="tensor-core carry vs oracle")
    compare(simt, ref, TOL_BF16, what="CUDA-core carry vs oracle")
    for n in ("dk", "dv", "db", "dgt", "dg", "dIp"):
        assert orc.rel_err(tc_path[n], simt[n]) < 1e-2, n


@pytest.mark.parametrize("K,V,T,G", [(64, 128, 300, 3), (128, 64, 260, 2), (32, 48, 130, 2), (48, 48, 300, 3), (48, 96, 260, 2),
                                     (96, 96, 200, 2)])
def test_tensor_core_carry_other_shapes(K, V, T, G):
    inp = orc.make_inputs(K + V + T, B=1, T=T, H=2, K=K, V=V, dtype=torch.bfloat16)
    inp["gt"] = inp["gt"] * 0.05
    got = _run(inp, G)
    ref = run_oracle(inp)
    compare(got, ref, TOL_BF16, what=f"tensor-core carry K={K} V={V}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_relay_of_a_passing_state_equals_the_full_boundary_scan(dtype):
    """A rank in the middle of a context-parallel chain forwards ``decay * in + total`` (total computed before the
    state arrives) instead of waiting for its full boundary scan: both must give the same outgoing state, forward
    (boundary state) and backward (state gradient).  One GPU: the rank's local machinery needs no process group."""
    from palimpsa_b200.parallel import _CudaLocal
    inp = orc.make_inputs(41, B=2, T=700, H=3, K=64, V=48, dtype=dtype)
    inp["gt"] = inp["gt"] * 0.05
    t = [inp[n].to(DEV).contiguous() for n in ("q", "k", "v", "b", "gt", "g", "Ip")]
    loc = _CudaLocal(*t, 64 ** -0.5, 5, first_rank=False)
    gen = torch.Generator().manual_seed(7)
    loc.summary()
    inc = torch.randn(loc.state_like().shape, generator=gen).to(DEV)
    full = loc.combine(inc)
    tot = loc.relay_prepare(loc.sg, False)
    out = torch.full_like(full, float("nan"))
    loc.relay(loc.sg, inc, tot, out.data_ptr())
    torch.cuda.synchronize()
    assert orc.rel_err(out, full) <= 2e-6
    # backward: start-state gradients of the segments from a zero end-state gradient, then the two routes
    o, _, _, _, ckM, ckI = loc.forward(save_ckpt=True)
    sg, bufs = loc.bwd_segments(loc.bufs["decay"])
    loc.bwd_carry(inp["do"].to(DEV).to(o.dtype).contiguous(), ckM, ckI, sg)
    inc = torch.randn(loc.state_like().shape, generator=gen).to(DEV)
    full = loc.combine_bwd(sg, inc)
    tot = loc.relay_prepare(sg, True)
    out = torch.full_like(full, float("nan"))
    loc.relay(sg, inc, tot, out.data_ptr())
    torch.cuda.synchronize()
    assert orc.rel_err(out, full) <= 2e-6
