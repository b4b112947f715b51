"""ctypes binding of libpalimpsa_b200.so (the C ABI declared in include/palimpsa_b200.h)."""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libpalimpsa_b200.so")

ABI_VERSION = 11
F32, BF16, F16 = 0, 1, 2
FLAG_UNCERTAINTY = 1
FLAG_EXPLICIT_INIT = 2
CKPT_INTERVAL = 16
STATIC_SCRATCH_BYTES = 64 << 20
E_NULL, E_ALIGN, E_LIMIT, E_SYMBOL = -1, -7, -9, -10


class Problem(C.Structure):
    _fields_ = [
        ("num_seqs", C.c_int32), ("seq_len", C.c_int32), ("total_tokens", C.c_int32),
        ("H", C.c_int32), ("K", C.c_int32), ("V", C.c_int32),
        ("io_dtype", C.c_int32), ("flags", C.c_int32),
        ("scale", C.c_float), ("reserved0", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("b", C.c_void_p),
        ("gt", C.c_void_p), ("g", C.c_void_p), ("Ip", C.c_void_p),
        ("cu_seqlens", C.c_void_p), ("chunk_offsets", C.c_void_p),
        ("init_mu", C.c_void_p), ("init_I", C.c_void_p), ("seq_order", C.c_void_p),
    ]


class FwdParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t), ("p", Problem),
        ("o", C.c_void_p), ("o_var", C.c_void_p),
        ("final_mu", C.c_void_p), ("final_I", C.c_void_p),
        ("ckpt_M", C.c_void_p), ("ckpt_I", C.c_void_p),
    ]


class BwdParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t), ("p", Problem),
        ("d_o", C.c_void_p), ("d_o_var", C.c_void_p),
        ("ckpt_M", C.c_void_p), ("ckpt_I", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("db", C.c_void_p),
        ("dgt", C.c_void_p), ("dg", C.c_void_p), ("dIp", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class Segments(C.Structure):
    _fields_ = [
        ("num_segments", C.c_int32), ("seg_len", C.c_int32),
        ("sum_M", C.c_void_p), ("sum_J", C.c_void_p), ("decay", C.c_void_p),
        ("start_M", C.c_void_p), ("start_I", C.c_void_p),
        ("carry_M", C.c_void_p), ("carry_I", C.c_void_p),
        ("rloc_M", C.c_void_p), ("rloc_I", C.c_void_p),
    ]


LAYER_RESIDUAL, LAYER_GATE = 1, 2


class LayerPrologue(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t), ("io_dtype", C.c_int32),
        ("H", C.c_int32), ("Hq", C.c_int32), ("K", C.c_int32), ("V", C.c_int32),
        ("tokens", C.c_int64),
        ("q_raw", C.c_void_p), ("k_raw", C.c_void_p), ("x", C.c_void_p), ("b_raw", C.c_void_p),
        ("dt_raw", C.c_void_p), ("bs_raw", C.c_void_p), ("dt_bias", C.c_void_p), ("b_scale", C.c_void_p),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("b", C.c_void_p), ("gt", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("db", C.c_void_p), ("dgt", C.c_void_p),
        ("dq_raw", C.c_void_p), ("dk_raw", C.c_void_p), ("dx", C.c_void_p), ("db_raw", C.c_void_p),
        ("ddt_raw", C.c_void_p), ("dbs_raw", C.c_void_p), ("d_dt_bias", C.c_void_p), ("d_b_scale", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class LayerEpilogue(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t), ("io_dtype", C.c_int32),
        ("H", C.c_int32), ("V", C.c_int32), ("flags", C.c_uint32), ("eps", C.c_float),
        ("tokens", C.c_int64),
        ("o", C.c_void_p), ("x", C.c_void_p), ("gate", C.c_void_p), ("D", C.c_void_p), ("weight", C.c_void_p),
        ("y", C.c_void_p),
        ("dy", C.c_void_p), ("d_o", C.c_void_p), ("dx", C.c_void_p), ("dgate", C.c_void_p),
        ("dD", C.c_void_p), ("dweight", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


# every symbol include/palimpsa_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "palimpsa_abi_version": (C.c_int, []),
    "palimpsa_last_error_string": (C.c_char_p, [C.c_int]),
    "palimpsa_padded_k": (C.c_int, [C.c_int]),
    "palimpsa_fwd_tile_rows": (C.c_int, [C.c_int, C.c_int]),
    "palimpsa_bwd_tile_rows": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "palimpsa_peer_wait": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p, C.c_void_p]),
    "palimpsa_peer_signal": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "palimpsa_ckpt_slots": (C.c_longlong, [C.POINTER(Problem)]),
    "palimpsa_segment_summary": (C.c_int, [C.POINTER(Problem), C.POINTER(Segments), C.c_void_p]),
    "palimpsa_tensor_core_status": (C.c_int, []),
    "palimpsa_cp_combine": (C.c_int, [C.POINTER(Problem), C.POINTER(Segments), C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p]),
    "palimpsa_cp_combine_bwd": (C.c_int, [C.POINTER(Problem), C.POINTER(Segments), C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p]),
    "palimpsa_cp_relay_prepare": (C.c_int, [C.POINTER(Problem), C.POINTER(Segments), C.c_int, C.c_void_p, C.c_void_p,
                                            C.c_void_p]),
    "palimpsa_cp_relay": (C.c_int, [C.POINTER(Problem), C.POINTER(Segments), C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "palimpsa_chunk_fwd_segments": (C.c_int, [C.POINTER(FwdParams), C.POINTER(Segments), C.c_void_p]),
    "palimpsa_chunk_bwd_segments": (C.c_int, [C.POINTER(BwdParams), C.POINTER(Segments), C.c_int, C.c_void_p]),
    "palimpsa_carry_apply_supported": (C.c_int, [C.POINTER(Problem)]),
    "palimpsa_carry_apply": (C.c_int, [C.POINTER(BwdParams), C.POINTER(Segments), C.c_void_p]),
    "palimpsa_chunk_fwd": (C.c_int, [C.POINTER(FwdParams), C.c_void_p]),
    "palimpsa_recurrent_fwd": (C.c_int, [C.POINTER(FwdParams), C.c_void_p]),
    "palimpsa_decode_step": (C.c_int, [C.POINTER(FwdParams), C.c_void_p]),
    "palimpsa_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(Problem)]),
    "palimpsa_chunk_bwd": (C.c_int, [C.POINTER(BwdParams), C.c_void_p]),
    "palimpsa_chunk_bwd_stages": (C.c_int, [C.POINTER(BwdParams), C.c_void_p, C.c_int]),
    "palimpsa_chunk_bwd_static": (C.c_int, [C.POINTER(BwdParams), C.c_void_p]),
    "palimpsa_recurrent_bwd": (C.c_int, [C.POINTER(BwdParams), C.c_void_p]),
    "palimpsa_layer_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32, C.c_int32]),
    "palimpsa_layer_prologue_fwd": (C.c_int, [C.POINTER(LayerPrologue), C.c_void_p]),
    "palimpsa_layer_prologue_bwd": (C.c_int, [C.POINTER(LayerPrologue), C.c_void_p]),
    "palimpsa_layer_epilogue_fwd": (C.c_int, [C.POINTER(LayerEpilogue), C.c_void_p]),
    "palimpsa_layer_epilogue_bwd": (C.c_int, [C.POINTER(LayerEpilogue), C.c_void_p]),
}

_lib = None


class PalimpsaLibraryError(RuntimeError):
    pass


def lib():
    """The loaded library.  There is no fallback: a missing or stale library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise PalimpsaLibraryError(
            f"{LIB_PATH} is missing. Build it with `python -m palimpsa_b200.build` (needs nvcc). "
            "palimpsa_b200 has no CPU or PyTorch fallback.")
    h = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        try:
            fn = getattr(h, name)
        except AttributeError as e:
            raise PalimpsaLibraryError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype = res
        fn.argtypes = args
    v = h.palimpsa_abi_version()
    if v != ABI_VERSION:
        raise PalimpsaLibraryError(f"{LIB_PATH} has ABI version {v}, Python side expects {ABI_VERSION}; rebuild it")
    _lib = h
    return h


def check(rc: int, what: str):
    if rc != 0:
        msg = lib().palimpsa_last_error_string(rc).decode()
        raise RuntimeError(f"{what} failed with code {rc}: {msg}")
