"""Loader for the reference's own ops from the unmodified working copy under ``oracle/_ref/`` (placed there by
``oracle/fetch_reference.py``).  The two op files are loaded by path under private module names, so the result
does not depend on what ``palimpsa.ops`` currently resolves to in ``sys.modules``."""
import importlib.util
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")
OPS = os.path.join(REF, "palimpsa", "ops", "palimpsa")
_cache = {}


def available() -> bool:
    return os.path.exists(os.path.join(OPS, "chunk_palimpsa_forgetting_scalar.py")) and \
        os.path.exists(os.path.join(OPS, "fused_recurrent_palimpsa.py"))


SKIP_REASON = "oracle/_ref is absent: run `python oracle/fetch_reference.py` where the reference checkout is mounted"


def _load(name, fname):
    if name not in _cache:
        spec = importlib.util.spec_from_file_location(name, os.path.join(OPS, fname))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        _cache[name] = mod
    return _cache[name]


def triton_chunk_palimpsa():
    """The reference's ``chunk_palimpsa`` (chunk_palimpsa_forgetting_scalar.py:623-667; Triton kernels :66-434)."""
    return _load("_reference_chunk_palimpsa", "chunk_palimpsa_forgetting_scalar.py").chunk_palimpsa


def reference_palimpsa_ref():
    """The reference's naive recurrence ``palimpsa_ref`` (chunk_palimpsa_forgetting_scalar.py:669-725)."""
    return _load("_reference_chunk_palimpsa", "chunk_palimpsa_forgetting_scalar.py").palimpsa_ref


def triton_fused_recurrent_palimpsa():
    """The reference's ``fused_recurrent_palimpsa`` (fused_recurrent_palimpsa.py:258-297; Triton kernel :24-154)."""
    return _load("_reference_fused_recurrent_palimpsa", "fused_recurrent_palimpsa.py").fused_recurrent_palimpsa
