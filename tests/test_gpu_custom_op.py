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
