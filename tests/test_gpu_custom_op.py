"""The torch custom-op registrations (schema, fake/meta kernels, autograd wiring) as torch.compile and
activation checkpointing need them (the reference's blocks are GradientCheckpointingLayers,
palimpsa/models/palimpsa/modeling_palimpsa.py:34)."""
import pytest
import torch

from oracle import palimpsa_oracle as orc
from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu


def _args(T=40, dtype=torch.float32, grad=True):
    inp = orc.make_inputs(1, B=2, T=T, H=2, K=32, V=16, dtype=dtype)
    return [inp[n].to(DEV).requires_grad_(grad) for n in ("q", "k", "v", "b", "gt", "g", "Ip")]


def test_opcheck_forward_op():
    from palimpsa_b200.ops.palimpsa import _core
    q, k, v, b, gt, g, Ip = _args()
    args = (q, k, v, b, gt, g, Ip, None, None, None, 0.25, False, True, True, False, 1)
    torch.library.opcheck(_core.fwd_op, args, test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


def test_activation_checkpointing_recomputes_consistently():
    from torch.utils.checkpoint import checkpoint
    from palimpsa_b200.ops import chunk_palimpsa
    a1, a2 = _args(), _args()
    o1 = chunk_palimpsa(*a1)
    o2 = checkpoint(lambda *xs: chunk_palimpsa(*xs), *a2, use_reentrant=False)
    w = torch.randn_like(o1)
    (o1 * w).sum().backward()
    (o2 * w).sum().backward()
    assert torch.equal(o1, o2)
    for x, y in zip(a1, a2):
        assert torch.equal(x.grad, y.grad)


def test_torch_compile_traces_through_the_op():
    from palimpsa_b200.ops import chunk_palimpsa
    args = _args(grad=False)

    def f(q, k, v, b, gt, g, Ip):
        return chunk_palimpsa(q * 1.0, k, v, b, gt, g, Ip) + 1.0

    ref = f(*args)
    out = torch.compile(f, backend="aot_eager", fullgraph=True)(*args)
    assert torch.allclose(ref, out)


def _decode_args(dtype=torch.bfloat16):
    N, H, K, V = 3, 2, 32, 16
    inp = orc.make_inputs(3, B=N, T=1, H=H, K=K, V=V, dtype=dtype)
    mu, I = orc.make_states(4, N, H, V, K, inp["Ip"])
    return [inp[n].to(DEV) for n in ("q", "k", "v", "b", "gt", "g", "Ip")] + [mu.to(DEV), I.to(DEV)]


def test_opcheck_decode_step_op():
    """``palimpsa_b200::decode_step`` declares that it mutates the two cache tensors; schema and fake kernel agree."""
    from palimpsa_b200.ops.palimpsa import decode as D
    args = (*_decode_args(), 0.25, True)
    torch.library.opcheck(D.decode_step_op, args, test_utils=("test_schema", "test_faketensor"))


def test_torch_compile_decode_loop_updates_the_cache_in_place():
    from palimpsa_b200.ops import decode_step
    args = _decode_args()
    ref_args = [x.clone() for x in args]

    def loop(q, k, v, b, gt, g, Ip, mu, I):
        o = None
        for _ in range(3):
            o = decode_step(q, k, v, b, gt, g, Ip, mu, I)
        return o + 0.0

    ref = loop(*ref_args)
    out = torch.compile(loop, backend="aot_eager", fullgraph=True)(*args)
    assert torch.equal(ref, out)
    assert torch.equal(args[7], ref_args[7]) and torch.equal(args[8], ref_args[8])      # caches advanced identically
    assert not torch.equal(args[7], _decode_args()[7])
