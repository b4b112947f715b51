"""``chunk_palimpsa``: same signature as the reference's
palimpsa/ops/palimpsa/chunk_palimpsa_forgetting_scalar.py:623."""
from __future__ import annotations

from . import _core


def chunk_palimpsa(q, k, v, b, gt, g, Ip, initial_mu_state=None, initial_I_state=None, scale=None, chunk_size=16,
                   output_final_state=False, output_uncertainty=False, cu_seqlens=None, *, num_segments=None):
    """Palimpsa operator for training and prefill; differentiable w.r.t. q, k, v, b, gt, g, Ip.

    Arguments and return value follow the reference: ``q,k [B,T,H,K]``, ``v,b [B,T,H,V]``,
    ``gt [B,T,H]``, ``g,Ip [H]``, states ``[N,H,V,K]`` float32; returns ``o`` (dtype of ``q``),
    or ``(o, o_var)`` with ``output_uncertainty``, followed by ``final_mu, final_I`` with
    ``output_final_state``.  With ``cu_seqlens`` the batch must be 1 and states are per sequence.

    ``chunk_size`` is accepted for compatibility and does not change the result: the kernels
    checkpoint the state every 16 tokens (the value the reference's layers pass,
    palimpsa/layers/palimpsa.py:309) whatever is asked.  The uncertainty output uses ``scale`` to
    the first power like the reference's kernels (:204), not ``scale**2`` like ``palimpsa_ref``.
    Unlike the reference kernel (:418), ``dIp`` is exact when an initial state is given.

    ``num_segments`` (keyword-only, not in the reference): cut every sequence into that many segments
    that run side by side (boundary states from a summary pass and a scan); default: chosen from the
    problem size, 1 unless the grid would leave SMs idle.  With ``cu_seqlens`` the packed token axis is what is
    cut (segments of ``T / num_segments`` tokens; those past a sequence's end are empty), and the default only does
    so when there are too few documents to fill one wave of CTAs.
    """
    if scale is None:
        scale = q.shape[-1] ** -0.5
    if cu_seqlens is not None and q.shape[0] != 1:
        raise ValueError(f"Batch size must be 1 for Varlen, got {q.shape[0]}")
    return _core.run(q, k, v, b, gt, g, Ip, initial_mu_state, initial_I_state, scale, output_final_state,
                     output_uncertainty, cu_seqlens, recurrent=False, out_dtype=q.dtype, num_segments=num_segments,
                     var_dtype=q.dtype)
