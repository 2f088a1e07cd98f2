"""E8 lattice, codecs and layer factory (mirror of coset/core/e8/__init__.py:20-38)."""
from .lattice import E8Lattice
from .codecs import (
    e8_encode,
    e8_decode,
    e8_quantize,
    e8_encode_packed,
    e8_decode_packed,
    e8_quant_stats,
    E8Decoder,
    DecodingMethod,
)
from .layers import create_e8_hnlq_linear

__all__ = [
    "E8Lattice",
    "e8_encode",
    "e8_decode",
    "e8_quantize",
    "e8_encode_packed",
    "e8_decode_packed",
    "e8_quant_stats",
    "E8Decoder",
    "DecodingMethod",
    "create_e8_hnlq_linear",
]
