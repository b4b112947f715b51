from .chunk import chunk_palimpsa
from .decode import DecodeGraph, decode_step
from .fused_recurrent import fused_recurrent_palimpsa
from .naive import palimpsa_ref

__all__ = ["palimpsa_ref", "chunk_palimpsa", "fused_recurrent_palimpsa", "decode_step", "DecodeGraph"]
