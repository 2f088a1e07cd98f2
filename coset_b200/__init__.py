"""coset_b200: the E8 hierarchical nested-lattice quantisation hot path of coset on B200 GPUs.

The module layout mirrors the reference so that imports translate one to one:
    coset.core.base        -> coset_b200.core.base        (LatticeConfig)
    coset.core.e8          -> coset_b200.core.e8          (E8Lattice, e8_encode, e8_decode, ...)
    coset.core.e8.layers   -> coset_b200.core.e8.layers   (create_e8_hnlq_linear)
    coset.core.layers      -> coset_b200.core.layers      (HNLQLinearQAT, ste_quantize)
"""
__version__ = "0.1.0"
