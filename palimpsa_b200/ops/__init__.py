from .palimpsa import DecodeGraph, chunk_palimpsa, decode_step, fused_recurrent_palimpsa, palimpsa_ref

__all__ = ["palimpsa_ref", "chunk_palimpsa", "fused_recurrent_palimpsa", "decode_step", "DecodeGraph"]
