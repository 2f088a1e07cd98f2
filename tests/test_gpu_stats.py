"""Quantisation statistics kernel (two-stage reduction through scratch memory) against the CPU
restatement: counts exact, sums to double-precision accumulation of the same float32 terms."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def cpu_stats(x):
    digits = O.encode(x, threads=8)
    xh = O.decode(digits, threads=8)
    err2 = float(((xh.astype(np.float64) - x.astype(np.float64)) ** 2).sum())
    sig2 = float((x.astype(np.float64) ** 2).sum())
    over = int((O.projection((x / np.float32(16.0)).astype(np.float32)) != 0).any(axis=1).sum())
    nonzero = int((digits.reshape(len(x), -1) != 0).any(axis=1).sum())
    return err2, over, nonzero, sig2


@pytest.mark.parametrize("n,scale", [(1, 1.0), (300, 0.5), (8192, 0.5), (8193, 3.0), (50000, 9.0)])
def test_stats_match_cpu(n, scale):
    from coset_b200.core.e8 import e8_quant_stats
    rng = np.random.default_rng(n)
    x = (rng.standard_normal((n, 8)) * scale).astype(np.float32)
    got = e8_quant_stats(torch.from_numpy(x).cuda())
    err2, over, nonzero, sig2 = cpu_stats(x)
    assert got["overloaded_blocks"] == over and got["nonzero_blocks"] == nonzero and got["n_blocks"] == n
    assert abs(got["squared_error"] - err2) <= 1e-5 * max(err2, 1e-12)
    assert abs(got["signal_energy"] - sig2) <= 1e-5 * sig2
    if scale >= 9:
        assert over > 0


def test_stats_with_per_block_scale_and_rejects_small_scratch():
    from coset_b200 import _lib
    from coset_b200.core.e8 import e8_quant_stats
    x = torch.randn(20000, 8, device="cuda") * 0.02
    beta = torch.full((20000,), 25.0, device="cuda")
    a = e8_quant_stats(x, scale=beta, scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=1)
    b = e8_quant_stats((x * 25.0).contiguous())
    assert a["nonzero_blocks"] == b["nonzero_blocks"] and a["overloaded_blocks"] == b["overloaded_blocks"]
    assert abs(a["squared_error"] - b["squared_error"]) < 1e-9 * b["squared_error"]
    out = torch.empty(4, dtype=torch.float64, device="cuda")
    scratch = torch.empty(16, dtype=torch.uint8, device="cuda")
    rc = _lib.lib().coset_e8_quant_stats(_lib.ptr(x), 0, None, 0, 20000, 1, _lib.ptr(scratch), 16, _lib.ptr(out), _lib.stream())
    assert rc < 0
