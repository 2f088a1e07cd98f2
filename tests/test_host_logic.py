"""CPU-only checks: host-side mirrors, and that the C-ABI library loads and exports every
symbol the public header declares (no compute calls: there is no GPU here)."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from coset_b200 import _lib, build
    build.build()
    header = open(os.path.join(ROOT, "include", "coset_b200.h")).read()
    declared = set(re.findall(r"\b(coset_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    L = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(L, name), f"{name} declared in include/coset_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert _lib.lib().coset_version() >= 100
    assert _lib.lib().coset_e8_code_bytes(4, 2) == 4
    assert _lib.lib().coset_e8_code_bytes(16, 3) == 12
    assert _lib.lib().coset_e8_code_bytes(64, 2) == 0


def test_bad_arguments_are_rejected_without_a_gpu():
    from coset_b200 import _lib
    L = _lib.lib()
    assert L.coset_e8_encode(None, 0, None, 0, -1, 1, 4, 2, 0, None, None) < 0
    assert L.coset_e8_encode(None, 0, None, 0, 8, 1, 4, 2, 0, None, None) < 0
    assert b"null" in L.coset_last_error_string()
    assert L.coset_e8_encode(None, 0, None, 0, 0, 1, 99, 2, 0, None, None) < 0
    assert L.coset_e8_decode(None, None, 7, 0, 1, 4, 2, 0, None, 0, None) < 0
    assert L.coset_e8_encode(None, 0, None, 0, 0, 1, 4, 2, 0, None, None) == 0  # empty input is fine


def test_lattice_config_mirror():
    from coset_b200.core.base import LatticeConfig
    c = LatticeConfig(lattice_type="E8", q=4, M=2)
    assert (c.beta, c.alpha, c.decoding, c.with_dither, c.max_scaling_iterations) == (1.0, 1.0, "full", False, 10)
    assert LatticeConfig.from_dict(c.to_dict()) == c
    with pytest.raises(TypeError):
        LatticeConfig(q=4, M=2)
    with pytest.raises(TypeError):
        LatticeConfig(lattice_type="E8", q=4, M=2, bogus=1)


def test_cpu_tensors_are_refused():
    from coset_b200.core.e8 import e8_encode, e8_quantize, E8Lattice
    from coset_b200.core.base import LatticeConfig
    c = LatticeConfig(lattice_type="E8", q=4, M=2)
    with pytest.raises(ValueError, match="CUDA"):
        e8_encode(torch.zeros(4, 8), c)
    with pytest.raises(ValueError, match="CUDA"):
        e8_quantize(torch.zeros(4, 8), 4)
    with pytest.raises(ValueError, match="CUDA"):
        E8Lattice(device="cpu").projection(torch.zeros(4, 8))


def test_lattice_constants_and_helpers_on_cpu():
    from coset_b200.core.e8 import E8Lattice
    L = E8Lattice(device="cpu")
    assert L.name == "E8" and L.d == 8 and L.r_pack == 0.5 and abs(L.r_cov - 2 ** 0.5 / 2) < 1e-12
    assert abs(L.compute_delta0(4, 2, 0.95) - 2 * 0.95 * 0.5 / 15) < 1e-15
    assert torch.equal(L.G @ L.G_inv, torch.eye(8))
    assert L.custom_round(torch.tensor([0.5, -0.5, 1.5, 2.5, -2.5])).tolist() == [0.0, 0.0, 1.0, 3.0, -2.0]
    z = torch.randint(0, 4, (100, 8)).float()
    assert torch.equal(L.encode_coords(L.decode_coords(z, 4), 4), z)


def test_layer_bounds_and_state_on_cpu(golden_layer):
    """_bounds / beta reproduce the reference's numbers; construction works without a GPU."""
    import numpy as np
    from coset_b200.core.e8 import create_e8_hnlq_linear
    g = golden_layer
    layer = create_e8_hnlq_linear(64, 48, device="cpu")
    with torch.no_grad():
        layer.theta_beta.copy_(torch.from_numpy(g["small_theta"]))
        layer.sigma_ema.copy_(torch.from_numpy(g["small_sigma"]))
        layer.xmax_ema.copy_(torch.from_numpy(g["small_xmax"]))
    bmin, bmax = layer._bounds()
    assert np.array_equal(bmin.numpy(), g["small_bmin"]) and np.array_equal(bmax.numpy(), g["small_bmax"])
    assert np.allclose(layer._beta().detach().numpy(), g["small_beta"], rtol=1e-6)
    assert abs(layer.Delta0 - float(g["small_Delta0"])) < 1e-15
    assert float(layer.gamma_inv) == float(g["small_gamma_inv"]) == 12.0
    fresh = create_e8_hnlq_linear(768, 3072, device="cpu")
    assert abs(float(fresh._beta()[0]) - 0.021440971642732620) < 1e-9
    with pytest.raises(ValueError, match="CUDA"):
        layer(torch.zeros(2, 64))
    layer.disable_quantization()
    assert layer(torch.zeros(2, 64)).shape == (2, 48)


def test_scale_bounds_cache_follows_the_statistics():
    """The cached (beta_min, beta_max) are recomputed after any write to the statistics buffers and
    after a hyper-parameter change, and equal the reference formula (coset/core/layers.py:381-396)."""
    import torch
    from coset_b200.core.e8 import create_e8_hnlq_linear
    layer = create_e8_hnlq_linear(64, 8, device="cpu")

    def formula():
        qM = float(layer.q ** layer.M)
        g = float(layer.gamma_inv)
        bmin = (layer.Delta0 / qM) / (layer.eta * g * layer.sigma_ema)
        bmax = torch.minimum((layer.Delta0 * (qM - 1)) / (2 * g * layer.xmax_ema),
                             (layer.Delta0 * (qM - 1)) / (2 * layer.eta * g * layer.sigma_ema))
        return torch.minimum(bmin, bmax * 0.9), bmax

    for mutate in (lambda: None, lambda: layer.sigma_ema.mul_(3.0), lambda: layer.xmax_ema.add_(0.5),
                   lambda: layer.sigma_ema.copy_(torch.rand(8) + 0.1), lambda: setattr(layer, "eta", 0.2)):
        mutate()
        got = layer._bounds()
        again = layer._bounds()
        assert got[0] is again[0]  # served from the cache while nothing changes
        want = formula()
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    beta = layer._beta()
    assert torch.equal(beta, want[0] + torch.sigmoid(layer.theta_beta) * (want[1] - want[0]))
    layer.load_state_dict({k: (v * 2 if k == "xmax_ema" else v) for k, v in layer.state_dict().items()})
    assert torch.equal(layer._bounds()[1], formula()[1])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float64])
def test_low_precision_parameters_are_refused_before_any_launch(dtype):
    """The fused weight kernels read float32 rows; a layer converted with .bfloat16() / .half() /
    .double() must be refused on the host, not misread on the device."""
    from coset_b200.core.layers import e8_fake_quantize
    from coset_b200.core.d4.layers import d4_fake_quantize, d4_quantize
    w8 = torch.zeros(4, 16, dtype=dtype)
    beta = torch.ones(4)
    with pytest.raises(TypeError, match="float32"):
        e8_fake_quantize(w8, beta, 2)
    with pytest.raises(TypeError, match="float32"):
        d4_fake_quantize(w8, beta, 4)
    with pytest.raises(TypeError, match="float32"):
        d4_quantize(torch.zeros(4, 4, dtype=dtype))
