"""D4 lattice path and Babai projection on the GPU against fixtures produced by the reference
(tests/golden/d4.npz) and against the CPU oracle on larger seeded inputs."""
import os

import numpy as np
import pytest
import torch

from conftest import bits
from oracle import oracle as O

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "d4.npz"))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def test_lattice_constants_and_helpers():
    from coset_b200.core.d4 import D4Lattice
    lat = D4Lattice(device="cuda")
    assert np.array_equal(lat.G.cpu().numpy(), G["G"])
    assert np.array_equal(lat.G_inv.cpu().numpy(), G["G_inv"])
    assert lat.r_pack == float(G["r_pack"]) and lat.r_cov == float(G["r_cov"])
    assert lat.compute_delta0(4, 2) == float(G["delta0_q4_M2"])
    x = dev(G["x"])
    assert np.array_equal(bits(lat.custom_round(x).cpu().numpy()), bits(G["custom_round"]))
    assert np.array_equal(bits(lat.g_x(x).cpu().numpy()), bits(G["g_x"]))
    assert str(lat) == "D4Lattice(d=4)"


def test_projection_golden():
    from coset_b200.core.d4 import D4Lattice, d4_quantize
    lat = D4Lattice(device="cuda")
    x = dev(G["x"])
    assert np.array_equal(bits(lat.projection(x).cpu().numpy()), bits(G["projection"]))
    assert np.array_equal(bits(lat.projection(x[7]).cpu().numpy()), bits(G["projection"][7]))
    assert np.array_equal(bits(d4_quantize(x, 4).cpu().numpy()), bits(G["projection"]))
    with pytest.raises(ValueError):
        lat.projection(torch.zeros(3, 8, device="cuda"))
    with pytest.raises(ValueError):
        lat.projection(torch.zeros(3, 4))


@pytest.mark.parametrize("n", [0, 1, 2, 3, 255, 256, 257, 100001])
def test_quantize_ragged_sizes_vs_oracle(n):
    """Odd block counts exercise the single-block tail; per-tile scales with ragged tiles."""
    from coset_b200 import _lib
    rng = np.random.default_rng(n)
    x = (rng.standard_normal((n, 4)) * 0.05).astype(np.float32)
    for bpt in (1, 7, 48):
        tiles = max((n + bpt - 1) // bpt, 1)
        beta = (rng.random(tiles) * 40 + 1).astype(np.float32)
        want, _ = O.d4_fake_quant(x, beta, bpt, 2.0) if n else (x, None)
        out = torch.empty((n, 4), dtype=torch.float32, device="cuda")
        xd, bd = dev(x), dev(beta)
        rc = _lib.lib().coset_d4_quantize(_lib.ptr(xd), 0, _lib.ptr(bd), _lib.SCALE_MUL_TILE, n, bpt, 2.0, _lib.ptr(out), 0,
                                          _lib.stream())
        assert rc == 0
        assert np.array_equal(bits(out.cpu().numpy()), bits(want))


def test_quantize_full_size_properties():
    """2^24 blocks: every output is a D4 point (integers, even sum), idempotent, and within the
    covering radius of the reference rule (one coordinate may move away by the -1 rule)."""
    from coset_b200 import _lib
    n = 1 << 24
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(n, 4, device="cuda", generator=g) * 3.0
    out = torch.empty_like(x)
    L = _lib.lib()
    assert L.coset_d4_quantize(_lib.ptr(x), 0, None, _lib.SCALE_NONE, n, 1, 0.0, _lib.ptr(out), 0, _lib.stream()) == 0
    assert bool((out == out.round()).all())
    assert bool((out.sum(dim=1) % 2 == 0).all())
    again = torch.empty_like(x)
    assert L.coset_d4_quantize(_lib.ptr(out), 0, None, _lib.SCALE_NONE, n, 1, 0.0, _lib.ptr(again), 0, _lib.stream()) == 0
    assert torch.equal(again, out)
    assert float((out - x).abs().max()) <= 1.5 + 1e-6
    sub = slice(0, 200000)
    assert np.array_equal(bits(out[sub].cpu().numpy()), bits(O.d4_projection(x[sub].cpu().numpy())))


def test_bf16_in_and_out():
    from coset_b200 import _lib
    rng = np.random.default_rng(5)
    n = 4099
    x = torch.from_numpy((rng.standard_normal((n, 4)) * 0.05).astype(np.float32)).to(torch.bfloat16)
    beta = (rng.random(n) * 40 + 1).astype(np.float32)
    want, _ = O.d4_fake_quant(x.float().numpy(), beta, 1, 2.0)
    want_bf = torch.from_numpy(want).to(torch.bfloat16)
    xd, bd = x.cuda(), dev(beta)
    out = torch.empty((n, 4), dtype=torch.bfloat16, device="cuda")
    assert _lib.lib().coset_d4_quantize(_lib.ptr(xd), 1, _lib.ptr(bd), _lib.SCALE_MUL_TILE, n, 1, 2.0, _lib.ptr(out), 1,
                                        _lib.stream()) == 0
    assert torch.equal(out.cpu(), want_bf)


def make_layer(tag, tiling="row"):
    from coset_b200.core.d4 import create_d4_hnlq_linear
    W = G[f"{tag}_W"]
    o, i = W.shape
    layer = create_d4_hnlq_linear(i, o, q=4, M=2, tiling=tiling, device="cuda")
    with torch.no_grad():
        layer.weight.copy_(dev(W))
        layer.bias.copy_(dev(G[f"{tag}_bias"]))
        if tiling == "row":
            layer.theta_beta.copy_(dev(G[f"{tag}_theta"]))
            layer.sigma_ema.copy_(dev(G[f"{tag}_sigma"]))
            layer.xmax_ema.copy_(dev(G[f"{tag}_xmax"]))
    return layer


@pytest.mark.parametrize("tag", ["small", "big", "mid"])
def test_fake_quant_kernel_bit_exact(tag):
    from coset_b200.core.d4.layers import d4_fake_quantize
    W = dev(G[f"{tag}_W"])
    o, i = W.shape
    wq = d4_fake_quantize(W, dev(G[f"{tag}_beta"]), i // 4, 2.0)
    assert np.array_equal(bits(wq.cpu().numpy()), bits(G[f"{tag}_Wq"]))
    wqb = d4_fake_quantize(W, dev(G[f"{tag}_blk_beta"]).reshape(-1), 1, 2.0)
    assert np.array_equal(bits(wqb.cpu().numpy()), bits(G[f"{tag}_blk_Wq"]))


@pytest.mark.parametrize("tag", ["small", "big", "mid"])
def test_layer_forward_backward_row_tiling(tag):
    """The reference layer (row tiling) end to end: the device sigmoid may differ from the CPU's in
    the last bit of beta, which moves whole rows by one ulp -- hence tolerances, not bits."""
    layer = make_layer(tag)
    assert layer._fused_d4 and not layer._fused
    assert abs(layer.Delta0 - float(G[f"{tag}_Delta0"])) < 1e-12
    assert float(layer.gamma_inv) == float(G[f"{tag}_gamma_inv"])
    x = dev(G[f"{tag}_x"]).requires_grad_(True)
    y = layer(x)
    ((y - dev(G[f"{tag}_t"])) ** 2).mean().backward()
    assert rel(y.detach().cpu().numpy(), G[f"{tag}_y"]) < 1e-5
    assert rel(layer.weight.grad.cpu().numpy(), G[f"{tag}_dW"]) < 1e-5
    assert rel(layer.bias.grad.cpu().numpy(), G[f"{tag}_dbias"]) < 1e-5
    assert rel(x.grad.cpu().numpy(), G[f"{tag}_dx"]) < 1e-5
    want = G[f"{tag}_dtheta"]
    assert np.abs(layer.theta_beta.grad.cpu().numpy() - want).max() <= 1e-4 * max(np.abs(want).max(), 1e-12) + 1e-12


@pytest.mark.parametrize("tag", ["small", "big", "mid"])
def test_block_tiling_gradients(tag):
    from coset_b200.core.d4.layers import d4_fake_quantize
    W = dev(G[f"{tag}_W"]).requires_grad_(True)
    beta = dev(G[f"{tag}_blk_beta"]).reshape(-1).requires_grad_(True)
    wq = d4_fake_quantize(W, beta, 1, 2.0)
    y = torch.nn.functional.linear(dev(G[f"{tag}_x"]), wq, dev(G[f"{tag}_bias"]))
    ((y - dev(G[f"{tag}_t"])) ** 2).mean().backward()
    assert rel(W.grad.cpu().numpy(), G[f"{tag}_blk_dW"]) < 1e-5
    want = G[f"{tag}_blk_dbeta"].reshape(-1)
    assert np.abs(beta.grad.cpu().numpy() - want).max() <= 1e-5 * max(np.abs(want).max(), 1e-12) + 1e-12


def test_layer_errors():
    from coset_b200.core.d4 import create_d4_hnlq_linear
    with pytest.raises(ValueError):
        create_d4_hnlq_linear(30, 8)
    layer = create_d4_hnlq_linear(32, 8, device="cuda", tiling="block")  # the reference raises for 'block'
    assert layer(torch.randn(5, 32, device="cuda")).shape == (5, 8)


@pytest.mark.parametrize("name", ["e8", "d4"])
@pytest.mark.parametrize("step", [1.0, 0.25])
def test_babai(name, step):
    from coset_b200.core.babai import babai_project, babai_quantize_ste
    from coset_b200.core.d4 import D4Lattice
    from coset_b200.core.e8 import E8Lattice
    lat = (E8Lattice if name == "e8" else D4Lattice)(device="cuda")
    x = G[f"babai_{name}_x"]
    safe = G[f"babai_{name}_step{step}_safe"]
    want = G[f"babai_{name}_step{step}_y"]
    got = babai_project(dev(x), lat, step).cpu().numpy()
    assert np.abs(got[safe] - want[safe]).max() <= 1e-5       # float64 evaluation of the reference formula
    oracle = O.babai(x, lat.G.cpu().numpy(), lat.G_inv.cpu().numpy(), step)
    assert np.array_equal(bits(got), bits(oracle))            # same float32 operation order: every row
    # the result is a lattice point of step * L: its basis coordinates are multiples of step
    z = got.astype(np.float64) @ lat.G_inv.cpu().numpy().astype(np.float64).T / step
    assert np.abs(z - np.round(z)).max() < 1e-4
    xg = dev(x).requires_grad_(True)
    babai_quantize_ste(xg, lat, step).sum().backward()
    assert torch.equal(xg.grad, torch.ones_like(xg))
    with pytest.raises(ValueError):
        babai_project(torch.zeros(2, 5, device="cuda"), lat, step)


def test_babai_non_power_of_two_step_vs_oracle():
    """A step that is not a power of two takes the IEEE division, like the CPU restatement."""
    from coset_b200.core.babai import babai_project
    from coset_b200.core.e8 import E8Lattice
    lat = E8Lattice(device="cuda")
    x = G["babai_e8_x"]
    for step in (0.3, 0.0059375):
        got = babai_project(dev(x), lat, step).cpu().numpy()
        want = O.babai(x, lat.G.cpu().numpy(), lat.G_inv.cpu().numpy(), step)
        assert np.array_equal(bits(got), bits(want))
