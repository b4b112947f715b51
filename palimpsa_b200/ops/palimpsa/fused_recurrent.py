"""``fused_recurrent_palimpsa``: same signature as the reference's
palimpsa/ops/palimpsa/fused_recurrent_palimpsa.py:258-272 (note: ``scale`` precedes the states)."""
from __future__ import annotations

from typing import Optional

import torch

from . import _core


def fused_recurrent_palimpsa(q, k, v, b, gt, g, Ip, scale: Optional[float] = None,
                             initial_mu_state: Optional[torch.Tensor] = None,
                             initial_I_state: Optional[torch.Tensor] = None, output_final_state: bool = False,
                             output_uncertainty: bool = False, cu_seqlens: Optional[torch.Tensor] = None):
    """Token-by-token form of the operator, used by the layers for decode and short evaluation
    sequences (palimpsa/layers/palimpsa.py:221,317).  ``o`` comes back in ``v``'s dtype and ``o_var`` in
    float32, as in the reference (:247-248); with 16-bit inputs the kernel writes ``o_var`` in that dtype first,
    so its float32 values carry that rounding.  Unlike the reference (:250-253) it is differentiable."""
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`.")
        if initial_mu_state is not None and initial_mu_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError("Initial states mismatch sequence length.")
    if scale is None:
        scale = k.shape[-1] ** -0.5
    return _core.run(q, k, v, b, gt, g, Ip, initial_mu_state, initial_I_state, scale, output_final_state,
                     output_uncertainty, cu_seqlens, recurrent=True, out_dtype=v.dtype, var_dtype=torch.float32)
