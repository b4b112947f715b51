"""Generate ``tests/golden/gated_norm.npz`` from flash-linear-attention's own ``FusedRMSNormGated`` (0.5.1), the
module the reference layer applies after the operator (palimpsa/layers/palimpsa.py:138, :341).

Its kernels are Triton, so this runs where a CUDA device is available:

    python tests/golden/make_gated_norm_golden.py [--out tests/golden/gated_norm.npz]

Seeded float32 and bfloat16 inputs (o + x*D as the layer forms it at :338, a gate, a non-trivial weight) go
through the unmodified module, forward and backward; inputs, output and the three gradients are stored.  The CPU
test ``tests/test_layer_oracle_cpu.py`` checks ``oracle/layer_oracle.py``'s restatement against this file: that
is what pins the gated-norm oracle to the third-party code instead of to its published formula alone.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.layer_oracle import make_layer_inputs  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "gated_norm.npz"))
    a = ap.parse_args()
    import fla
    from fla.modules import FusedRMSNormGated
    dev = torch.device("cuda", 0)
    arrs = {"meta_fla_version": np.array(fla.__version__), "meta_eps": np.array(1e-5)}
    for tag, dtype, V in (("f32", torch.float32, 128), ("bf16", torch.bfloat16, 128), ("f32_v48", torch.float32, 48)):
        d = make_layer_inputs(11, B=1, T=13, H=3, Hq=3, K=8, V=V, dtype=dtype)
        norm = FusedRMSNormGated(V, eps=1e-5).to(dev)
        with torch.no_grad():
            norm.weight.copy_(d["weight"].to(dev))
        # the layer's own line :338 in the activation dtype, then the module as the layer calls it (:341)
        z = (d["o"].to(dev) + d["x"].to(dev) * d["D"].to(dev).to(dtype)[None, None, :, None]).detach().requires_grad_(True)
        gate = d["gate"].to(dev).detach().requires_grad_(True)
        y = norm(z, gate)
        y.backward(d["dy"].to(dev))
        arrs.update({f"{tag}_z": z.detach().float().cpu().numpy(), f"{tag}_gate": gate.detach().float().cpu().numpy(),
                     f"{tag}_weight": d["weight"].numpy(), f"{tag}_dy": d["dy"].float().numpy(),
                     f"{tag}_y": y.detach().float().cpu().numpy(), f"{tag}_dz": z.grad.float().cpu().numpy(),
                     f"{tag}_dgate": gate.grad.float().cpu().numpy(),
                     f"{tag}_dweight": norm.weight.grad.float().cpu().numpy()})
    np.savez_compressed(a.out, **arrs)
    print("wrote", a.out, {k: v.shape for k, v in arrs.items() if k.endswith("_y")})


if __name__ == "__main__":
    main()
