"""CUDA codec against the golden vectors of the reference and against the CPU oracle.

Everything here goes through the C ABI (ctypes) exactly as a user of coset_b200.core.e8 does.
Integer codes and float32 reconstructions must be BIT-EXACT.
"""
import numpy as np
import pytest
import torch

from conftest import bits
from oracle import oracle as O

pytestmark = pytest.mark.gpu

BETA_MID = 0.021440971642732620


@pytest.fixture(scope="module")
def e8():
    from coset_b200.core import e8 as mod
    return mod


@pytest.fixture(scope="module")
def cfgcls():
    from coset_b200.core.base import LatticeConfig
    return LatticeConfig


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dtype)


def cfg(cls, q=4, M=2, beta=1.0):
    return cls(lattice_type="E8", q=q, M=M, beta=beta)


def test_library_is_loaded():
    from coset_b200 import _lib
    assert _lib.lib().coset_version() >= 100


def test_projection_golden(e8, golden_codec):
    x = golden_codec["proj_in"]
    y = e8.E8Lattice().projection(dev(x)).cpu().numpy()
    assert np.array_equal(bits(y), bits(golden_codec["proj_out"]))
    # single vector form
    y1 = e8.E8Lattice().projection(dev(x[5])).cpu().numpy()
    assert np.array_equal(bits(y1), bits(golden_codec["proj_out"][5]))


def test_lattice_helpers_golden(e8, golden_codec):
    L = e8.E8Lattice()
    x = dev(golden_codec["proj_in"])
    assert np.array_equal(bits(L.g_x(x).cpu().numpy()), bits(golden_codec["gx_out"]))
    cr = L.custom_round(dev(golden_codec["cr_in"])).cpu().numpy()
    assert np.array_equal(bits(cr), bits(golden_codec["cr_out"]))
    G, Gi = L.get_generators()
    assert np.array_equal(G.cpu().numpy(), golden_codec["G"]) and np.array_equal(Gi.cpu().numpy(), golden_codec["Ginv"])
    p = dev(golden_codec["proj_out"][:4096])
    b = L.encode_coords(p, 4)
    back = L.decode_coords(b, 4)
    assert torch.equal(L.encode_coords(back, 4).long(), b.long())


@pytest.mark.parametrize("name,s", [("s0p25", 0.25), ("s0p5", 0.5), ("s1", 1.0), ("s2", 2.0), ("s4", 4.0), ("s8", 8.0)])
def test_encode_decode_scale_sweep(e8, cfgcls, golden_codec, name, s):
    x = dev(golden_codec["cfg1_x"] * np.float32(s))
    c = cfg(cfgcls)
    digits, t = e8.e8_encode(x, c)
    assert t == 0 and digits.shape == (x.shape[0], 2, 8) and digits.dtype == torch.float32
    assert np.array_equal(digits.cpu().numpy().astype(np.int64), golden_codec[f"cfg1_codesA_{name}"].astype(np.int64))
    xh = e8.e8_decode(digits, c)
    assert np.array_equal(bits(xh.cpu().numpy()), bits(golden_codec[f"cfg1_xhatA_{name}"]))
    # packed format == oracle packing of the reference digits
    packed = e8.e8_encode_packed(x).view(torch.int32).view(-1).cpu().numpy().view(np.uint32)
    assert np.array_equal(packed, O.pack_q4(golden_codec[f"cfg1_codesA_{name}"].astype(np.float32)))


@pytest.mark.parametrize("name,b", [("mid", BETA_MID), ("0p3", 0.3), ("1p7", 1.7)])
def test_codec_convention(e8, cfgcls, golden_codec, name, b):
    x = dev(golden_codec["cfg1_x"])
    c = cfg(cfgcls, beta=b)
    digits, _ = e8.e8_encode(x, c)
    assert np.array_equal(digits.cpu().numpy().astype(np.int64), golden_codec[f"cfg1_codesB_{name}"].astype(np.int64))
    xh = e8.e8_decode(digits, c)
    assert np.array_equal(bits(xh.cpu().numpy()), bits(golden_codec[f"cfg1_xhatB_{name}"]))


def test_layer_convention_literal_is_all_zero(e8, golden_codec):
    from coset_b200 import _lib
    x = dev(golden_codec["cfg1_x"])
    beta = torch.full((x.shape[0],), BETA_MID, device="cuda")
    packed = e8.e8_encode_packed(x, scale=beta, scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=1)
    assert not packed.any()
    xh = e8.e8_decode_packed(packed, scale=beta, scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=1)
    assert np.array_equal(bits(xh.cpu().numpy()), bits(golden_codec["cfg1_xhatA_lit"]))


@pytest.mark.parametrize("q,M", [(2, 1), (3, 2), (4, 1), (4, 3), (5, 2), (8, 2), (16, 2)])
def test_other_q_m(e8, cfgcls, golden_codec, q, M):
    x = dev(golden_codec["cfg1_x"][:2048] * np.float32(3.0))
    c = cfg(cfgcls, q=q, M=M, beta=0.7)
    digits, _ = e8.e8_encode(x, c)
    assert np.array_equal(digits.cpu().numpy().astype(np.int64), golden_codec[f"qm_codes_{q}_{M}"].astype(np.int64))
    xh = e8.e8_decode(digits, c)
    assert np.array_equal(bits(xh.cpu().numpy()), bits(golden_codec[f"qm_xhat_{q}_{M}"]))


def test_adversarial_rows(e8, cfgcls, golden_codec):
    x = dev(golden_codec["adv_x"])
    c = cfg(cfgcls)
    digits, _ = e8.e8_encode(x, c)
    assert np.array_equal(digits.cpu().numpy().astype(np.int64), golden_codec["adv_codes"].astype(np.int64))
    assert np.array_equal(bits(e8.e8_decode(digits, c).cpu().numpy()), bits(golden_codec["adv_xhat"]))
    assert np.array_equal(bits(e8.e8_quantize(x, 4).cpu().numpy()), bits(golden_codec["adv_quant"]))


def test_quantize_golden(e8, golden_codec):
    x = golden_codec["cfg1_x"]
    assert np.array_equal(bits(e8.e8_quantize(dev(x), 4).cpu().numpy()), bits(golden_codec["cfg1_quant_s1"]))
    assert np.array_equal(bits(e8.e8_quantize(dev(x * np.float32(4)), 4).cpu().numpy()), bits(golden_codec["cfg1_quant_s4"]))
    v = e8.e8_quantize(dev(x[3]), 4)
    assert v.shape == (8,) and np.array_equal(bits(v.cpu().numpy()), bits(golden_codec["cfg1_quant_s1"][3]))


def test_exhaustive_single_level_decode(e8, cfgcls, golden_decode_table):
    idx = np.arange(65536)
    digits = np.stack([(idx >> (2 * j)) & 3 for j in range(8)], axis=1).astype(np.float32)
    # through the reference-shaped API (M = 1 -> generic kernel) ...
    res = e8.e8_decode(dev(digits[:, None, :]), cfg(cfgcls, M=1)).cpu().numpy()
    assert np.array_equal((res * 2).astype(np.int8), golden_decode_table)
    # ... and through the table-driven q=4, M=2 kernel, level 0 and level 1 separately
    lo = torch.from_numpy(idx.astype(np.int32)).cuda()
    r0 = e8.e8_decode_packed(lo).cpu().numpy()
    assert np.array_equal((r0 * 2).astype(np.int8), golden_decode_table)
    hi = torch.from_numpy((idx.astype(np.int64) << 16).astype(np.uint32).view(np.int32)).cuda()
    r1 = e8.e8_decode_packed(hi).cpu().numpy()
    assert np.array_equal((r1 / 2).astype(np.int8), golden_decode_table)


@pytest.mark.parametrize("scale", [0.02, 0.5, 1.0, 3.0, 17.0])
def test_config1_full_vs_oracle(e8, scale):
    """BASELINE config 1: [65536, 8] N(0,1) seed 0 clipped to +-2 (the scale sweeps coverage)."""
    torch.manual_seed(0)
    x = torch.randn(65536, 8).clamp_(-2, 2) * scale
    xn = x.numpy()
    want = O.pack_q4(O.encode(xn, threads=8))
    got = e8.e8_encode_packed(x.cuda()).view(torch.int32).view(-1)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want)
    xh = e8.e8_decode_packed(got).cpu().numpy()
    assert np.array_equal(bits(xh), bits(O.quantize(xn)))
    assert np.array_equal(bits(e8.e8_quantize(x.cuda(), 4).cpu().numpy()), bits(xh))


def test_per_tile_scales_vs_oracle(e8):
    from coset_b200 import _lib
    rng = np.random.default_rng(3)
    n, bpt = 96 * 50 + 17, 96
    x = (rng.standard_normal((n, 8)) * 0.05).astype(np.float32)
    for blocks_per_tile in (1, bpt, 7):
        tiles = (n + blocks_per_tile - 1) // blocks_per_tile
        beta = (rng.random(tiles) * 40 + 1).astype(np.float32)
        want = O.encode(x, beta=beta, scale_mode=2, blocks_per_tile=blocks_per_tile)
        got = e8.e8_encode_packed(dev(x), scale=dev(beta), scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=blocks_per_tile)
        assert np.array_equal(got.view(torch.int32).view(-1).cpu().numpy().view(np.uint32), O.pack_q4(want))
        xh = e8.e8_decode_packed(got, scale=dev(beta), scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=blocks_per_tile)
        want_xh = O.decode(want, beta=beta, scale_mode=2, blocks_per_tile=blocks_per_tile)
        assert np.array_equal(bits(xh.cpu().numpy()), bits(want_xh))


@pytest.mark.parametrize("q,M", [(4, 2), (3, 3), (8, 2)])
def test_coarse_to_fine_packed_decode(e8, q, M):
    """depth = d keeps the d coarsest levels: equal to decoding digits whose finer levels are zero."""
    rng = np.random.default_rng(8)
    x = (rng.standard_normal((5000, 8)) * (q ** M) / 8).astype(np.float32)
    digits = O.encode(x, q=q, M=M)
    codes = e8.e8_encode_packed(dev(x), q, M)
    for depth in range(1, M + 1):
        kept = digits.copy()
        kept[:, :M - depth] = 0
        want = O.decode(kept, q=q)
        got = e8.e8_decode_packed(codes, q, M, depth=depth).cpu().numpy()
        assert np.array_equal(bits(got), bits(want)), depth
    assert np.array_equal(bits(e8.e8_decode_packed(codes, q, M, depth=M).cpu().numpy()),
                          bits(e8.e8_decode_packed(codes, q, M).cpu().numpy()))
    with pytest.raises(ValueError):
        e8.e8_decode_packed(codes, q, M, depth=0)


def test_bf16_in_and_out(e8):
    """bf16 oracle = widen to float32, run the reference arithmetic, round the result to bf16."""
    torch.manual_seed(5)
    xb = (torch.randn(40000, 8) * 0.7).to(torch.bfloat16)
    xn = xb.float().numpy()
    want = O.pack_q4(O.encode(xn, threads=4))
    got = e8.e8_encode_packed(xb.cuda()).view(torch.int32).view(-1)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want)
    out = e8.e8_decode_packed(got, dtype=torch.bfloat16)
    want_out = torch.from_numpy(O.quantize(xn)).to(torch.bfloat16)
    assert torch.equal(out.cpu(), want_out)


@pytest.mark.parametrize("n", [0, 1, 7, 31, 32, 33, 255, 256, 257])
def test_ragged_sizes(e8, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal((n, 8)).astype(np.float32)
    got = e8.e8_encode_packed(dev(x).reshape(n, 8))
    assert got.shape == (n, 4)
    if n:
        assert np.array_equal(got.view(torch.int32).view(-1).cpu().numpy().view(np.uint32), O.pack_q4(O.encode(x)))
    xh = e8.e8_decode_packed(got)
    assert xh.shape == (n, 8)


def test_non_finite_inputs_do_not_fault(e8):
    x = torch.tensor([[float("nan")] * 8, [float("inf")] * 8, [-float("inf"), 1, 2, 3, 4, 5, 6, 7], [1e30] * 8],
                     device="cuda")
    codes = e8.e8_encode_packed(x)
    out = e8.e8_decode_packed(codes)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()  # any code decodes to a finite lattice point


def test_errors(e8, cfgcls):
    c = cfg(cfgcls)
    with pytest.raises(ValueError):
        e8.e8_encode(torch.zeros(4, 7, device="cuda"), c)
    with pytest.raises(ValueError):
        e8.e8_encode(torch.zeros(2, 3, 8, device="cuda"), c)
    with pytest.raises(ValueError):
        e8.e8_encode(torch.zeros(4, 8), c)  # CPU tensor: no fallback
    with pytest.raises(ValueError):
        e8.e8_decode(torch.zeros(4, 2, 8, device="cuda"), c, method="progressive")
    with pytest.raises(ValueError):
        e8.e8_encode(torch.zeros(4, 8, device="cuda"), cfg(cfgcls, q=64))
    from coset_b200 import _lib
    rc = _lib.lib().coset_e8_encode(None, 0, None, 0, 5, 1, 4, 2, 0, None, None)
    assert rc < 0 and b"null" in _lib.lib().coset_last_error_string()


def test_dither_path(e8, cfgcls):
    torch.manual_seed(9)
    x = torch.randn(2000, 8)
    d = torch.rand(8) - 0.5
    c = cfgcls(lattice_type="E8", q=4, M=2, beta=0.3, with_dither=True)
    digits, _ = e8.e8_encode(x.cuda(), c, dither=d.cuda())
    xs = (x.numpy() / np.float32(0.3) + d.numpy()[None]).astype(np.float32)
    assert np.array_equal(digits.cpu().numpy().astype(np.int64), O.codes_to_int(O.encode(xs)))


# ---------------------------------------------------------------------------------------------
# Full-size properties: inputs far too large for the CPU oracle are cross-checked between the
# guarded fast path and the op-by-op search (two independent evaluations inside the library;
# the op-by-op one is what the golden / oracle tests above pin).
@pytest.mark.parametrize("scale", [0.02, 0.125, 0.5, 1.0, 3.0, 20.0, 200.0])
def test_fast_path_equals_literal_at_full_size(e8, scale):
    g = torch.Generator(device="cuda").manual_seed(int(scale * 1000))
    n = 1 << 24
    x = torch.randn(n, 8, device="cuda", generator=g) * scale
    fast = e8.e8_encode_packed(x).view(torch.int32)
    lit = e8.e8_encode_packed(x, literal=True).view(torch.int32)
    assert torch.equal(fast, lit), int((fast != lit).sum())
    if 0.4 < scale < 5:
        assert (fast != 0).float().mean() > 0.5  # not the degenerate all-zero regime


def test_fast_path_equals_literal_on_structured_inputs(e8):
    g = torch.Generator(device="cuda").manual_seed(77)
    n = 1 << 22
    cases = []
    cases.append(torch.randint(-16, 17, (n, 8), device="cuda", generator=g).float() / 8)        # decoder-like ties
    cases.append(torch.randint(-6, 7, (n, 8), device="cuda", generator=g).float() / 2)          # lattice points
    x = torch.randn(n, 8, device="cuda", generator=g)
    x[torch.rand(n, 8, device="cuda", generator=g) < 0.3] = 0.0                                  # sparse
    cases.append(x)
    x = torch.randn(n, 8, device="cuda", generator=g) * 2
    k = torch.randint(0, 8, (n,), device="cuda", generator=g)
    near = torch.randint(-4, 5, (n,), device="cuda", generator=g).float() + 0.5
    near = near + torch.randint(-3, 4, (n,), device="cuda", generator=g).float() * 2.0 ** -23    # a few ulps around a tie
    x[torch.arange(n, device="cuda"), k] = near
    cases.append(x)
    cases.append(torch.zeros(n, 8, device="cuda"))
    for x in cases:
        fast = e8.e8_encode_packed(x).view(torch.int32)
        lit = e8.e8_encode_packed(x, literal=True).view(torch.int32)
        assert torch.equal(fast, lit), int((fast != lit).sum())


def test_bulk_config_properties(e8):
    """BASELINE bulk config at full size (2^25 blocks): fused round trip == decode(encode), the
    reconstruction error is within the covering radius for the blocks the reference itself
    reconstructs to the projection, and re-quantising a reconstruction is idempotent for the inner level."""
    from coset_b200 import _lib
    g = torch.Generator(device="cuda").manual_seed(0)
    n = 1 << 25
    x = torch.randn(n, 8, device="cuda", generator=g) * 0.02
    beta = torch.full((n,), 25.0, device="cuda")
    MT = _lib.SCALE_MUL_TILE
    codes = e8.e8_encode_packed(x, scale=beta, scale_mode=MT)
    xh = e8.e8_decode_packed(codes, scale=beta, scale_mode=MT)
    fused = torch.empty_like(x)
    rc = _lib.lib().coset_e8_quantize(_lib.ptr(x), 0, _lib.ptr(beta), MT, n, 1, 4, 2, 0.0, _lib.ptr(fused), 0, None,
                                      _lib.stream())
    assert rc == 0
    assert torch.equal(fused, xh)
    err = ((xh - x) * 25.0).norm(dim=1)
    inside = (x * 25.0).abs().amax(dim=1) < 3.0
    # core semantics do not re-quantise between levels, so only ~79 % of the blocks decode to the
    # projection of the input (error <= covering radius sqrt(2)/2); the rest land on another coset
    assert 0.6 < float(err[inside].median()) < 0.9  # CPU restatement of the reference: 0.78 on this distribution
    codes2 = e8.e8_encode_packed(xh, scale=beta, scale_mode=MT)
    same = (codes2.view(torch.int32) == codes.view(torch.int32)).float().mean()
    assert same > 0.99  # re-encoding a reconstruction returns the same code (CPU restatement: 99.87 %)


def test_encode_on_concurrent_streams_and_growing_sizes(e8):
    """The codes-only encoder keeps library-owned scratch per (device, stream): calls issued on several
    streams at once must not disturb each other, a larger tensor on the same stream grows the scratch,
    and an overloaded tensor (most blocks deferred: the fix-up kernel's sweep) leaves the scratch clean
    for the next call."""
    g = torch.Generator(device="cuda").manual_seed(5)
    sizes = [4096, 300_000, 70_001, 1_200_000]
    xs = [torch.randn(n, 8, device="cuda", generator=g) * (0.5 if i != 2 else 6.0) for i, n in enumerate(sizes)]
    xs[1][::97, 3] = 5.0  # exact integers: deferred blocks in an otherwise easy tensor
    want = [e8.e8_encode_packed(x, literal=True).view(torch.int32).clone() for x in xs]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in range(3)]
    got = {}
    for rep in range(3):
        for i, x in enumerate(xs):
            st = streams[(i + rep) % 3]
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                got[(rep, i)] = e8.e8_encode_packed(x).view(torch.int32)
    torch.cuda.synchronize()
    for (rep, i), c in got.items():
        assert torch.equal(c, want[i]), (rep, i, int((c != want[i]).sum()))
