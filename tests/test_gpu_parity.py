"""GPU parity: the CUDA ops, called through the Python wrappers over the C ABI, against the
float64 oracle and against the fixtures produced by the reference's own ``palimpsa_ref``.
Error metric: max|x-ref| / max|ref| per tensor; bounds: 1e-5 (fp32), 2e-2 (bf16/fp16)."""
import pytest
import torch

from oracle import palimpsa_oracle as orc
from tests.gpu_util import DEV, compare, run_cuda, run_oracle, tol_for
from tests.helpers import GOLDEN_CASES, GOLDEN_TOL, TOL_BF16, TOL_FP32, load_golden

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", GOLDEN_CASES)
@pytest.mark.parametrize("op", ["chunk", "fused"])
def test_reference_fixtures(case, op):
    inp, out, meta = load_golden(case)
    unc = bool(meta["unc"])
    cu = inp["cu_seqlens"].tolist() if "cu_seqlens" in inp else None
    got = run_cuda(inp, op, unc, meta["scale"], inp.get("mu0"), inp.get("I0"), cu)
    compare(got, out, GOLDEN_TOL, what=f"{case}/{op} vs reference fixture")
    ref = run_oracle(inp, unc, meta["scale"], inp.get("mu0"), inp.get("I0"), cu)
    compare(got, ref, TOL_FP32, what=f"{case}/{op} vs oracle")


def test_config1_fp32():
    """B=2, T=512, H=4, d_k=d_v=64, fp32, benchmark distributions: outputs, states, 7 gradients."""
    inp = orc.make_inputs(0, B=2, T=512, H=4, K=64, V=64)
    got = run_cuda(inp, "chunk")
    ref = run_oracle(inp)
    compare(got, ref, TOL_FP32, what="config 1")


def test_check_script_shape_fp32():
    """The reference's manual check: B,L,H,D,N = 4,511,4,65,31, raw q/k, o and o_var in the loss."""
    inp = orc.make_inputs(42, B=4, T=511, H=4, K=31, V=65, check_style=True)
    got = run_cuda(inp, "chunk", unc=True, scale=1.0)
    ref = run_oracle(inp, unc=True, scale=1.0)
    compare(got, ref, TOL_FP32, what="check shape")


def test_check_script_varlen_and_initial_state():
    inp = orc.make_inputs(43, B=1, T=700, H=3, K=31, V=65, check_style=True)
    cu = [0, 128, 192, 700]
    got = run_cuda(inp, "chunk", unc=True, scale=1.0, cu=cu)
    ref = run_oracle(inp, unc=True, scale=1.0, cu=cu)
    compare(got, ref, TOL_FP32, what="varlen")
    mu0, I0 = orc.make_states(5, 3, 3, 65, 31, inp["Ip"])
    got = run_cuda(inp, "chunk", unc=True, scale=1.0, cu=cu, mu0=mu0, I0=I0)
    ref = run_oracle(inp, unc=True, scale=1.0, cu=cu, mu0=mu0, I0=I0)
    compare(got, ref, TOL_FP32, what="varlen+init")


@pytest.mark.parametrize("K,V", [(16, 32), (48, 48), (48, 96), (96, 192), (128, 128), (192, 64), (64, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_shipped_head_shapes(K, V, dtype):
    inp = orc.make_inputs(K + V, B=2, T=83, H=2, K=K, V=V, dtype=dtype)
    got = run_cuda(inp, "chunk")
    ref = run_oracle(inp)
    compare(got, ref, tol_for(dtype), what=f"K={K} V={V} {dtype}")


@pytest.mark.parametrize("V", [64, 108, 128, 130, 136, 200])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_tiling_at_dk128(V, dtype):
    """d_k = 128 picks 22- or 24-row tiles by padding; 22-row tiles start off the 16-byte grid of the rows
    (staged supersets), and d_v that is not a multiple of 8 takes the unstaged path."""
    inp = orc.make_inputs(V, B=2, T=50, H=2, K=128, V=V, dtype=dtype)
    got = run_cuda(inp, "chunk", unc=True)
    ref = run_oracle(inp, unc=True)
    compare(got, ref, tol_for(dtype), what=f"K=128 V={V} {dtype}")


@pytest.mark.parametrize("dtype,unc", [(torch.float32, False), (torch.float32, True), (torch.bfloat16, True)])
def test_k256(dtype, unc):
    """The widest supported d_k: one state row per thread column group, 8-row tiles in the backward."""
    inp = orc.make_inputs(1, B=2, T=70, H=2, K=256, V=24, dtype=dtype)
    got = run_cuda(inp, "chunk", unc=unc)
    ref = run_oracle(inp, unc=unc)
    compare(got, ref, tol_for(dtype), what=f"K=256 {dtype} unc={unc}")
    inp = orc.make_inputs(2, B=1, T=33, H=1, K=200, V=5, dtype=dtype)
    got = run_cuda(inp, "chunk", unc=unc)
    ref = run_oracle(inp, unc=unc)
    compare(got, ref, tol_for(dtype), what=f"K=200 {dtype} unc={unc}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_half_precision_io(dtype):
    inp = orc.make_inputs(11, B=2, T=300, H=3, K=128, V=128, dtype=dtype)
    got = run_cuda(inp, "chunk", unc=True)
    ref = run_oracle(inp, unc=True)
    compare(got, ref, TOL_BF16, what=str(dtype))


@pytest.mark.parametrize("T", [1, 3, 15, 16, 17, 33])
def test_short_sequences(T):
    inp = orc.make_inputs(T, B=3, T=T, H=2, K=32, V=24)
    for op in ("chunk", "fused"):
        got = run_cuda(inp, op, unc=True)
        ref = run_oracle(inp, unc=True)
        compare(got, ref, TOL_FP32, what=f"T={T} {op}")


def test_varlen_with_empty_sequence():
    inp = orc.make_inputs(9, B=1, T=50, H=2, K=16, V=16)
    cu = [0, 0, 20, 20, 50]
    got = run_cuda(inp, "chunk", cu=cu)
    ref = run_oracle(inp, cu=cu)
    compare(got, ref, TOL_FP32, what="varlen with empty sequences")


def test_state_passing_equals_one_pass():
    """Forward over [0,T) equals forward over [0,S) then [S,T) started from the first call's final state."""
    from palimpsa_b200.ops import chunk_palimpsa, fused_recurrent_palimpsa
    inp = orc.make_inputs(21, B=2, T=100, H=2, K=64, V=64)
    d = {n: inp[n].to(DEV) for n in ("q", "k", "v", "b", "gt", "g", "Ip")}
    full, mu, I = chunk_palimpsa(**d, output_final_state=True)
    S = 37
    sl = lambda a, b: {n: (x[:, a:b] if x.dim() >= 3 else x) for n, x in d.items()}
    o1, mu1, I1 = chunk_palimpsa(**sl(0, S), output_final_state=True)
    o2, mu2, I2 = fused_recurrent_palimpsa(**sl(S, 100), initial_mu_state=mu1, initial_I_state=I1,
                                           output_final_state=True)
    assert orc.rel_err(torch.cat([o1, o2], 1), full) < TOL_FP32
    assert orc.rel_err(mu2, mu) < TOL_FP32 and orc.rel_err(I2, I) < TOL_FP32


def test_bitwise_reproducible():
    inp = orc.make_inputs(2, B=2, T=70, H=2, K=128, V=128, dtype=torch.bfloat16)
    a = run_cuda(inp, "chunk", unc=True)
    b = run_cuda(inp, "chunk", unc=True)
    for n in a:
        assert torch.equal(a[n], b[n]), n


def test_non_contiguous_and_mixed_dtype_inputs():
    from palimpsa_b200.ops import chunk_palimpsa
    inp = orc.make_inputs(4, B=2, T=40, H=2, K=32, V=32)
    d = {n: inp[n].to(DEV) for n in ("q", "k", "v", "b", "gt", "g", "Ip")}
    ref = chunk_palimpsa(**d)
    qk = torch.stack([d["q"], d["k"]], dim=-1)          # strided views
    got = chunk_palimpsa(qk[..., 0], qk[..., 1], d["v"], d["b"], d["gt"].double(), d["g"], d["Ip"])
    assert torch.equal(ref, got)
