"""The allocation-free statistics entry point against the regular one.

Some callers of this library cannot allocate device memory: code running inside another
framework's fixed memory pool, a plugin that is only ever handed its input and output buffers, a
thread that must not touch the allocator.  coset_e8_quant_stats_static serves them by keeping its
per-CTA partial records in an array built into the library.  This test drives it through the C
ABI exactly as such a caller would (raw pointers, no scratch argument) and checks, twice in a row
because the array is shared and keeps the previous call's contents, that it returns what
coset_e8_quant_stats returns with caller-provided scratch.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(L, _lib, x, n, scale, mode, bpt):
    nbytes = L.coset_e8_quant_stats_scratch_bytes(n)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = torch.full((4,), -1.0, dtype=torch.float64, device="cuda")
    rc = L.coset_e8_quant_stats(_lib.ptr(x), _lib.dtype_code(x, "x"), _lib.ptr(scale), mode, n, bpt, _lib.ptr(scratch), nbytes,
                                _lib.ptr(out), _lib.stream())
    assert rc == 0, L.coset_last_error_string()
    return out.cpu().numpy()


def _static(L, _lib, x, n, scale, mode, bpt):
    out = torch.full((4,), -1.0, dtype=torch.float64, device="cuda")
    rc = L.coset_e8_quant_stats_static(_lib.ptr(x), _lib.dtype_code(x, "x"), _lib.ptr(scale), mode, n, bpt, _lib.ptr(out),
                                       _lib.stream())
    assert rc == 0, L.coset_last_error_string()
    return out.cpu().numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_static_scratch_matches_regular_entry_point_twice(dtype, mode):
    """Every input type and scale convention of the allocation-free entry point (no scale, one scalar
    divisor, one multiplier per tile of 64 blocks).  The first size needs more than 256 partial records,
    so the final reduction strides over the built-in array more than once."""
    from coset_b200 import _lib
    L = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    # two different sizes, the larger first: the second call must not be disturbed by the
    # records the first one left in the shared array
    for n, spread in ((2_400_000, 0.5), (70_001, 4.0)):
        x = (torch.randn(n, 8, device="cuda", generator=g) * spread).to(dtype).contiguous()
        bpt = 64
        if mode == 0:
            scale = None
        elif mode == 1:
            scale = torch.tensor([0.8], device="cuda")
        else:
            scale = 0.5 + torch.rand((n + bpt - 1) // bpt, device="cuda", generator=g)
        want = _regular(L, _lib, x, n, scale, mode, bpt)
        got = _static(L, _lib, x, n, scale, mode, bpt)
        torch.cuda.synchronize()
        assert got[1] == want[1] and got[2] == want[2]                    # counts: exact
        assert np.allclose(got[[0, 3]], want[[0, 3]], rtol=1e-5, atol=0)  # sums: tolerance of the stats tests
        assert want[2] > 0 and want[0] > 0


def test_static_scratch_rejects_oversized_input():
    from coset_b200 import _lib
    L = _lib.lib()
    limit = L.coset_e8_quant_stats_static_max_blocks()
    assert limit == 1 << 25
    x = torch.zeros(8, 8, device="cuda")
    out = torch.zeros(4, dtype=torch.float64, device="cuda")
    rc = L.coset_e8_quant_stats_static(_lib.ptr(x), 0, None, 0, limit + 1, 1, _lib.ptr(out), _lib.stream())
    assert rc < 0
    assert b"exceeds" in L.coset_last_error_string()
