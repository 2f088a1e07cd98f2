"""Paper-faithful hierarchical nested-lattice quantiser (mirror of the reference's `ref` package,
E8 only): float64, tie dither, re-quantising recurrence, overload loop.  Parity path, not tuned."""
from .hnlq import HNLQ, HNLQConfig, TIE_DITHER_E8  # noqa: F401
