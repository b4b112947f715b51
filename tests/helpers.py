"""Shared helpers for the test-suite (fixtures loading, tolerances)."""
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GOLDEN_CASES = ("check_style_unc", "bench_style", "initial_state", "varlen")
GRADS = ("dq", "dk", "dv", "db", "dgt", "dg", "dIp")

# max|x-ref| / max|ref| bounds.  fp32 and bf16 are the operator's stated tolerances against a
# float64 recurrence; GOLDEN_TOL bounds float64-oracle vs the reference's float32 run.
TOL_FP32 = 1e-5
TOL_BF16 = 2e-2
GOLDEN_TOL = 2e-5


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    inp = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    out = {k[4:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("out_")}
    meta = {k[5:]: z[k].item() for k in z.files if k.startswith("meta_")}
    return inp, out, meta
