"""GPU "ref" semantics (float64, ref/hnlq.py) against fixtures produced by the reference."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_mode.npz"))


@pytest.mark.parametrize("tag", ["b1", "b025", "b025_noover", "b01", "q3m3", "b4"])
def test_ref_mode_matches_reference(tag):
    from coset_b200.ref import HNLQ
    beta, alpha, q, M, over = G[f"{tag}_params"]
    h = HNLQ.create_e8_quantizer(q=int(q), M=int(M), beta=float(beta), alpha=float(alpha), overload=bool(over))
    digits, T = h.encode(torch.from_numpy(G["x"]))
    assert np.array_equal(digits.cpu().numpy(), G[f"{tag}_digits"])
    assert np.array_equal(T.cpu().numpy(), G[f"{tag}_T"])
    xh = h.decode(digits, T)
    assert np.array_equal(xh.cpu().numpy(), G[f"{tag}_xhat"])
    # single-vector form returns what the reference returns
    b_list, t = h.encode(G["x"][3])
    assert len(b_list) == int(M) and t == int(G[f"{tag}_T"][3])
    assert np.array_equal(np.stack(b_list), G[f"{tag}_digits"][3])
    assert np.array_equal(h.decode(b_list, t), G[f"{tag}_xhat"][3])
    assert np.array_equal(h.quantize(G["x"][3]), G[f"{tag}_xhat"][3])


def test_core_and_ref_modes_disagree_as_in_the_reference():
    """The two reference codecs differ on a large share of rows; one kernel cannot serve both."""
    from coset_b200.core.base import LatticeConfig
    from coset_b200.core.e8 import e8_encode
    from coset_b200.ref import HNLQ
    x = torch.from_numpy(G["x"])
    core, _ = e8_encode(x.float().cuda(), LatticeConfig(lattice_type="E8", q=4, M=2, beta=1.0))
    ref, _ = HNLQ.create_e8_quantizer(q=4, M=2, beta=1.0, overload=False).encode(x)
    differ = (core.long() != ref.long()).any(dim=2).any(dim=1).float().mean()
    assert 0.1 < float(differ) < 0.7


GC = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_coarse.npz"))


@pytest.mark.parametrize("tag", ["b025", "b01", "q3m3"])
def test_ref_coarse_to_fine_and_progressive_decode(tag):
    from coset_b200.ref import HNLQ
    beta, alpha, q, M, over = G[f"{tag}_params"]
    M = int(M)
    want = GC[f"{tag}_by_depth"]
    n = want.shape[1]
    digits = torch.from_numpy(G[f"{tag}_digits"][:n])
    T = torch.from_numpy(G[f"{tag}_T"][:n])
    h = HNLQ.create_e8_quantizer(q=int(q), M=M, beta=float(beta), alpha=float(alpha), overload=bool(over),
                                 decoding="progressive")
    prog = h.get_default_decoding(digits, T)
    assert len(prog) == M
    for depth in range(1, M + 1):
        assert np.array_equal(prog[depth - 1].cpu().numpy(), want[depth - 1]), depth
        assert np.array_equal(h.decode_with_depth(digits, T, depth).cpu().numpy(), want[depth - 1])
    assert np.array_equal(h.decode_coarse_to_fine(digits, T).cpu().numpy(), want[M - 1])  # depth=None: full decode
    # single-vector form
    b_list = tuple(G[f"{tag}_digits"][5, m] for m in range(M))
    assert np.array_equal(h.decode_coarse_to_fine(b_list, int(G[f"{tag}_T"][5]), depth=1), want[0][5])
    with pytest.raises(ValueError):
        h.decode_coarse_to_fine(digits, T, depth=M + 1)
    with pytest.raises(ValueError):
        h.decode_with_depth(digits, T, 0)
