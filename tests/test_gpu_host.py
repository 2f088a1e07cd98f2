"""Host-array codec (coset_e8_encode_host / decode_host / quantize_host): pinned and pageable inputs,
several chunks per call, ragged last chunk, tiles that span chunk boundaries -- against the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import bits
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hc():
    from coset_b200.host import HostCodec
    c = HostCodec(chunk_blocks=1000, n_slots=3)  # small chunks: every call below spans several
    yield c
    c.close()


@pytest.mark.parametrize("n", [0, 1, 999, 1000, 1001, 7777])
@pytest.mark.parametrize("pinned", [True, False])
def test_encode_decode_host_vs_oracle(hc, n, pinned):
    rng = np.random.default_rng(n + 1)
    x = torch.from_numpy((rng.standard_normal((n, 8)) * 0.6).astype(np.float32))
    if pinned and n:
        x = x.pin_memory()
    codes = hc.encode(x)
    want = O.encode(x.numpy()) if n else np.zeros((0, 2, 8), np.float32)
    assert np.array_equal(codes.numpy().view(np.uint32).reshape(-1), O.pack_q4(want))
    xh = hc.decode(codes)
    if n:
        assert np.array_equal(bits(xh.numpy()), bits(O.decode(want)))
    assert xh.shape == (n, 8)


@pytest.mark.parametrize("bpt", [1, 7, 96])
def test_per_tile_scales_across_chunks(hc, bpt):
    from coset_b200 import _lib
    rng = np.random.default_rng(bpt)
    n = 96 * 40 + 13
    x = torch.from_numpy((rng.standard_normal((n, 8)) * 0.05).astype(np.float32)).pin_memory()
    tiles = (n + bpt - 1) // bpt
    beta = torch.from_numpy((rng.random(tiles) * 40 + 1).astype(np.float32)).pin_memory()
    want = O.encode(x.numpy(), beta=beta.numpy(), scale_mode=2, blocks_per_tile=bpt)
    codes = hc.encode(x, scale=beta, scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=bpt)
    assert np.array_equal(codes.numpy().view(np.uint32).reshape(-1), O.pack_q4(want))
    xh = hc.decode(codes, scale=beta, scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=bpt)
    want_xh = O.decode(want, beta=beta.numpy(), scale_mode=2, blocks_per_tile=bpt)
    assert np.array_equal(bits(xh.numpy()), bits(want_xh))
    # the one-pass round trip returns the same reconstruction and the same codes
    xh2, codes2 = hc.quantize(x, scale=beta, scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=bpt, return_codes=True)
    assert np.array_equal(bits(xh2.numpy()), bits(want_xh))
    assert torch.equal(codes2, codes)
    # with the layer's clamp, and without asking for the codes
    wq, _ = O.fake_quant(x.numpy(), beta.numpy(), bpt, 4, 0.04)
    xh3 = hc.quantize(x, scale=beta, scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=bpt, clip=0.04)
    assert np.array_equal(bits(xh3.numpy()), bits(wq))


def test_quantize_host_plain_and_bf16(hc):
    rng = np.random.default_rng(9)
    x = torch.from_numpy((rng.standard_normal((4321, 8)) * 1.3).astype(np.float32)).pin_memory()
    assert np.array_equal(bits(hc.quantize(x).numpy()), bits(O.quantize(x.numpy())))
    xb = x.to(torch.bfloat16)
    got = hc.quantize(xb, dtype=torch.bfloat16)
    want = torch.from_numpy(O.quantize(xb.float().numpy())).to(torch.bfloat16)
    assert torch.equal(got, want)


def test_host_errors(hc):
    with pytest.raises(ValueError):
        hc.encode(torch.zeros(4, 8, device="cuda"))
    with pytest.raises(Exception):
        hc.encode(torch.zeros(4, 8), q=99)
