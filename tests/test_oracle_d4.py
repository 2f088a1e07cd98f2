"""The D4 / Babai restatement (oracle/d4_oracle.c) against fixtures produced by the reference."""
import os

import numpy as np
import pytest

from conftest import bits
from oracle import oracle as O

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "d4.npz"))


def test_d4_projection_and_g_x():
    x = G["x"]
    assert np.array_equal(bits(O.d4_projection(x)), bits(G["projection"]))
    assert np.array_equal(bits(O.d4_g_x(x)), bits(G["g_x"]))


@pytest.mark.parametrize("tag", ["small", "big", "mid"])
def test_d4_layer_weight_path(tag):
    W = G[f"{tag}_W"]
    o, i = W.shape
    wq, _ = O.d4_fake_quant(W.reshape(-1, 4), G[f"{tag}_beta"], i // 4, 2.0)
    assert np.array_equal(bits(wq.reshape(o, i)), bits(G[f"{tag}_Wq"]))
    wqb, _ = O.d4_fake_quant(W.reshape(-1, 4), G[f"{tag}_blk_beta"].reshape(-1), 1, 2.0)
    assert np.array_equal(bits(wqb.reshape(o, i)), bits(G[f"{tag}_blk_Wq"]))


@pytest.mark.parametrize("name", ["e8", "d4"])
@pytest.mark.parametrize("step", [1.0, 0.25])
def test_babai(name, step):
    from oracle.oracle import generators
    if name == "e8":
        Gm, Gi = generators()
    else:
        Gm, Gi = G["G"], G["G_inv"]
    x = G[f"babai_{name}_x"]
    safe = G[f"babai_{name}_step{step}_safe"]
    want = G[f"babai_{name}_step{step}_y"]
    got = O.babai(x, Gm, Gi, step)
    assert safe.mean() > 0.99
    # float32 evaluation against the float64 fixture: identical integers away from rounding
    # boundaries, so only representation error of the final products remains
    assert np.abs(got[safe] - want[safe]).max() <= 1e-5
