"""palimpsa_b200: the Palimpsa operator (Bayesian-metaplastic linear attention) as hand-written
sm_100a CUDA behind the reference's ``palimpsa.ops`` Python interface."""
from .ops import chunk_palimpsa, decode_step, fused_recurrent_palimpsa, palimpsa_ref

__all__ = ["chunk_palimpsa", "fused_recurrent_palimpsa", "palimpsa_ref", "decode_step", "install_as_palimpsa_ops"]


def install_as_palimpsa_ops():
    """Make ``palimpsa.ops`` and ``palimpsa.ops.palimpsa`` resolve to this package, so that the
    reference's layers (``from palimpsa.ops.palimpsa import chunk_palimpsa, ...``,
    palimpsa/layers/palimpsa.py:17) and its check script (``from palimpsa.ops import ...``,
    palimpsa/check_palimpsa.py:6) pick up these ops unchanged.  Call before importing them."""
    import sys

    from . import ops
    from .ops import palimpsa as ops_palimpsa
    sys.modules["palimpsa.ops"] = ops
    sys.modules["palimpsa.ops.palimpsa"] = ops_palimpsa
    parent = sys.modules.get("palimpsa")
    if parent is not None:
        parent.ops = ops
