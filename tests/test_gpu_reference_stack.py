"""The reference's own layer and trainer on top of the CUDA ops, against the same stack on its Triton ops.

Two child processes run ``tests/reference_stack_arm.py`` on cuda:0, one after the other: one leaves the
reference untouched (Triton ops), the other calls ``palimpsa_b200.install_as_palimpsa_ops()`` first, so that
``from palimpsa.ops.palimpsa import chunk_palimpsa, fused_recurrent_palimpsa`` in the reference's layer
(palimpsa/layers/palimpsa.py:17) binds the CUDA ops.  Compared:

* the ``Palimpsa`` layer in training mode (chunk call, palimpsa/layers/palimpsa.py:309): output, input
  gradient, parameter gradients;
* the ``MetaMamba2`` layer in training mode (raw q/k, ``scale=1.0``, palimpsa/layers/meta_mamba2.py:333);
* prefill + cached single-token steps in eval mode (fused-recurrent call with cached states, :317-331);
* a packed variable-length training step of the 170M-shaped ``PalimpsaForCausalLM`` (``cu_seqlens`` through the
  model's kwargs, as the Flame recipe README.md:135-158 does): loss, gradients, step time;
* ``train_nano.py`` (train_nano.py:163-185) for 100 iterations from the same seed: the evaluation losses at
  step 0 and the training losses it prints at iterations 0, 50 and 100.

Tolerances are those of bf16 autocast stacks that differ in rounding only (the projections, convolutions and
norms around the op run in bf16 in both arms).  Needs ``oracle/_ref/``.
"""
import os
import subprocess
import sys

import pytest
import torch

from oracle import palimpsa_oracle as orc
from tests import reference_ops as R

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.available(), reason=R.SKIP_REASON)]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def arms(tmp_path_factory):
    out = {}
    tmp = tmp_path_factory.mktemp("stack")
    for ops in ("triton", "cuda"):
        path = str(tmp / f"{ops}.pt")
        r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "reference_stack_arm.py"), "--ops", ops,
                            "--out", path], capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, f"{ops} arm failed:\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
        out[ops] = torch.load(path)
    return out


def test_layer_binds_the_cuda_ops(arms):
    assert arms["cuda"]["chunk_op_module"].startswith("palimpsa_b200.")
    assert arms["cuda"]["fused_op_module"].startswith("palimpsa_b200.")
    assert not arms["triton"]["chunk_op_module"].startswith("palimpsa_b200.")


def test_reference_layer_training_step(arms):
    a, b = arms["cuda"], arms["triton"]
    errs = {n: orc.rel_err(a[n], b[n]) for n in a if n.startswith("train_")}
    print("\nreference layer, training mode, CUDA ops vs Triton ops:", {n: f"{e:.1e}" for n, e in errs.items()})
    assert all(torch.isfinite(a[n]).all() for n in errs)
    assert max(errs.values()) <= 3e-2, errs


def test_reference_meta_mamba2_layer_training_step(arms):
    """The reference's second caller: raw q/k, ``scale=1.0``, d_k = 32, d_v = 128 (palimpsa/layers/meta_mamba2.py:333)."""
    a, b = arms["cuda"], arms["triton"]
    assert a["mm2_chunk_op_module"].startswith("palimpsa_b200.")
    names = [n for n in a if n.startswith("mm2_") and torch.is_tensor(a[n])]
    errs = {n: orc.rel_err(a[n], b[n]) for n in names}
    print("\nreference MetaMamba2 layer, training mode, CUDA ops vs Triton ops:", {n: f"{e:.1e}" for n, e in errs.items()})
    assert len(names) >= 6 and all(torch.isfinite(a[n]).all() for n in names)
    assert max(errs.values()) <= 3e-2, errs


def test_reference_layer_cached_decode(arms):
    a, b = arms["cuda"], arms["triton"]
    errs = {n: orc.rel_err(a[n], b[n]) for n in ("decode_out", "decode_final_mu", "decode_final_I")}
    print("\nreference layer, prefill + 3 cached steps, CUDA ops vs Triton ops:", {n: f"{e:.1e}" for n, e in errs.items()})
    assert max(errs.values()) <= 2e-2, errs


def test_train_nano_loss_curve(arms):
    a, b = arms["cuda"], arms["triton"]
    assert set(a["nano_iter_loss"]) == set(b["nano_iter_loss"]) and len(a["nano_iter_loss"]) >= 3, \
        (a["nano_stdout"][-1500:], b["nano_stdout"][-1500:])
    print("\ntrain_nano.py losses (iteration: CUDA ops / Triton ops):",
          {i: (a["nano_iter_loss"][i], b["nano_iter_loss"][i]) for i in sorted(a["nano_iter_loss"])},
          "| evaluation at step 0 (train, val):", a["nano_eval"].get(0), b["nano_eval"].get(0),
          "| ms per 50 iterations:", a["nano_iter_ms"], b["nano_iter_ms"])
    # before any update both arms evaluate the same weights: only the ops' rounding differs
    for x, y in zip(a["nano_eval"][0], b["nano_eval"][0]):
        assert abs(x - y) <= 2e-3 * abs(y), (a["nano_eval"], b["nano_eval"])
    assert abs(a["nano_iter_loss"][0] - b["nano_iter_loss"][0]) <= 2e-3 * b["nano_iter_loss"][0]
    # after 50 and 100 AdamW steps in bf16 the curves have drifted by rounding only; both must have learned
    last = max(a["nano_iter_loss"])
    for i in sorted(a["nano_iter_loss"])[1:]:
        x, y = a["nano_iter_loss"][i], b["nano_iter_loss"][i]
        assert abs(x - y) <= 5e-2 * y, (i, x, y)
    assert a["nano_iter_loss"][last] < 0.8 * a["nano_iter_loss"][0]


def test_packed_variable_length_model_step(arms):
    """The 170M-shaped ``PalimpsaForCausalLM`` (4 of its layers) on one packed row with ``cu_seqlens``, forward +
    backward, the way the reference's Flame recipe drives it: same loss and gradients on both op sets."""
    a, b = arms["cuda"], arms["triton"]
    if "varlen_error" in b:
        pytest.skip("the reference stack itself could not run the packed step here: " + b["varlen_error"][-300:])
    assert "varlen_error" not in a, a.get("varlen_error")
    names = [n for n in a if n.startswith("varlen_grad_")]
    errs = {n[12:]: orc.rel_err(a[n], b[n]) for n in names}
    print(f"\npacked 170M-shaped model step ({a['varlen_documents']} documents, 16 384 tokens): loss {a['varlen_loss']:.4f} "
          f"(CUDA ops) vs {b['varlen_loss']:.4f} (Triton ops); step {a['varlen_step_ms']:.1f} ms vs {b['varlen_step_ms']:.1f} ms;",
          {n: f"{e:.1e}" for n, e in errs.items()})
    assert abs(a["varlen_loss"] - b["varlen_loss"]) <= 2e-3 * abs(b["varlen_loss"])
    assert len(names) >= 4 and max(errs.values()) <= 5e-2, errs
