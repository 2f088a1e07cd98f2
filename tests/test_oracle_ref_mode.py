"""The float64 "ref" restatement (ref/hnlq.py semantics) against fixtures from the reference."""
import os

import numpy as np
import pytest

from oracle import oracle as O

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_mode.npz"))
CASES = ["b1", "b025", "b025_noover", "b01", "q3m3", "b4"]


def test_tie_dither_constants():
    assert np.array_equal(O.TIE_DITHER, G["tie_dither"])


@pytest.mark.parametrize("tag", CASES)
def test_ref_encode_decode(tag):
    beta, alpha, q, M, over = G[f"{tag}_params"]
    digits, T = O.ref_encode(G["x"], beta=beta, alpha=alpha, q=int(q), M=int(M), overload=bool(over))
    assert np.array_equal(digits, G[f"{tag}_digits"])
    assert np.array_equal(T, G[f"{tag}_T"])
    xh = O.ref_decode(digits, T, beta=beta, alpha=alpha, q=int(q))
    assert np.array_equal(xh, G[f"{tag}_xhat"])


GC = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_coarse.npz"))


@pytest.mark.parametrize("tag", ["b025", "b01", "q3m3"])
def test_ref_coarse_to_fine_decode(tag):
    """decode_coarse_to_fine / decode_progressive of the reference, every depth 1 .. M."""
    beta, alpha, q, M, _ = G[f"{tag}_params"]
    want = GC[f"{tag}_by_depth"]
    n = want.shape[1]
    digits, T = G[f"{tag}_digits"][:n], G[f"{tag}_T"][:n]
    for depth in range(1, int(M) + 1):
        got = O.ref_decode(digits, T, beta=beta, alpha=alpha, q=int(q), depth=depth)
        assert np.array_equal(got, want[depth - 1]), depth
