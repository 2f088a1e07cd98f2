"""D4 lattice and layer factory (mirror of coset/core/d4/__init__.py)."""
from .lattice import D4Lattice
from .layers import create_d4_hnlq_linear, d4_quantize

__all__ = ["D4Lattice", "create_d4_hnlq_linear", "d4_quantize"]
