"""The rest of the layer / codec API surface against outputs of the unmodified reference
(tests/golden/api.npz, written by tests/golden/make_golden_api.py): the EMA statistics update
(coset/core/layers.py:366-379, 409-413), activation quantisation (:117-137, 481-482), the get_*
diagnostics and the dense export (:509-650), load_from_linear, E8Decoder / DecodingMethod
(coset/core/e8/codecs.py:99-180), plus the packed export -> E8CodeLinear round trip."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    return np.load(os.path.join(GOLDEN, "api.npz"))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def test_ema_statistics_after_256_and_512_forwards(api):
    from coset_b200.core.e8 import create_e8_hnlq_linear
    layer = create_e8_hnlq_linear(32, 24, q=4, M=2, device="cuda")
    with torch.no_grad():
        layer.weight.copy_(dev(api["ema_W0"]))
    x = dev(api["ema_x"])
    with torch.no_grad():
        for step in range(1, 513):
            y = layer(x)
            if step == 300:
                layer.weight.add_(dev(api["ema_delta"]))
            if step in (256, 512):
                bmin, bmax = layer._bounds()
                assert np.allclose(layer.sigma_ema.cpu().numpy(), api[f"ema_sigma_{step}"], rtol=2e-6, atol=0)
                assert np.allclose(layer.xmax_ema.cpu().numpy(), api[f"ema_xmax_{step}"], rtol=2e-6, atol=0)
                assert np.allclose(bmin.cpu().numpy(), api[f"ema_bmin_{step}"], rtol=5e-6, atol=0)
                assert np.allclose(bmax.cpu().numpy(), api[f"ema_bmax_{step}"], rtol=5e-6, atol=0)
                assert rel(y.cpu().numpy(), api[f"ema_y_{step}"]) < 1e-5 or np.abs(api[f"ema_y_{step}"]).max() == 0
    assert int(layer.step_count) == int(api["ema_step_count"]) == 512
    # the statistics moved away from their initial value 1 only at the two update steps
    assert not np.allclose(api["ema_sigma_256"], 1.0) and not np.allclose(api["ema_sigma_512"], api["ema_sigma_256"])


def test_layer_with_activation_quantisation(api):
    from coset_b200.core.e8 import create_e8_hnlq_linear
    layer = create_e8_hnlq_linear(32, 16, q=4, M=2, quantize_activations=True, act_bit_width=6, act_init_alpha=2.5, device="cuda")
    with torch.no_grad():
        layer.weight.copy_(dev(api["qa_W"]))
    y = layer(dev(api["qa_x"]))
    ((y - dev(api["qa_t"])) ** 2).mean().backward()
    assert rel(y.detach().cpu().numpy(), api["qa_y"]) < 1e-5
    assert rel(layer.weight.grad.cpu().numpy(), api["qa_dW"]) < 1e-5
    assert abs(float(layer.actq.alpha.grad) - float(api["qa_dalpha"])) <= 1e-5 * abs(float(api["qa_dalpha"])) + 1e-9
    want = api["qa_dtheta"]
    assert np.abs(layer.theta_beta.grad.cpu().numpy() - want).max() <= 2e-4 * np.abs(want).max() + 1e-9


def test_diagnostics_export_and_load_from_linear(api):
    from coset_b200.core.e8 import create_e8_hnlq_linear
    layer = create_e8_hnlq_linear(64, 24, q=4, M=2, enable_diagnostics=True, device="cuda")
    with torch.no_grad():
        layer.weight.copy_(dev(api["diag_W"]))
    stats = layer.get_weight_statistics()
    for k, v in stats.items():
        assert abs(v - float(api[f"diag_stat_{k}"])) <= 1e-5 * abs(float(api[f"diag_stat_{k}"])) + 1e-7, k
    assert np.allclose(layer.get_weight_quantiles().cpu().numpy(), api["diag_quantiles"], rtol=1e-5, atol=1e-6)
    assert abs(layer.get_quantization_error() - float(api["diag_qerr"])) <= 1e-5 * float(api["diag_qerr"])
    assert abs(layer.get_effective_bits() - float(api["diag_bits"])) < 1e-6
    assert abs(layer.get_sparsity_ratio() - float(api["diag_sparsity"])) < 1e-9
    for k, v in layer.compare_weights().items():
        assert abs(v - float(api[f"diag_cmp_{k}"])) <= 1e-5 * abs(float(api[f"diag_cmp_{k}"])) + 1e-7, k
    for k, v in layer.get_weight_clipping_stats().items():
        assert abs(v - float(api[f"diag_clip_{k}"])) <= 1e-6 * abs(float(api[f"diag_clip_{k}"])) + 1e-9, k
    hist, edges = layer.get_quantization_histogram(bins=20)
    assert np.array_equal(hist.numpy(), api["diag_hist"]) and np.allclose(edges.numpy(), api["diag_edges"], rtol=1e-6)
    summary = layer.get_diagnostic_summary()
    assert summary["quantization_enabled"] and "weight_comparison" in summary
    ex = layer.export_quantized()
    assert np.array_equal(bits(ex["weight"].cpu().numpy()), bits(api["diag_export_weight"]))
    assert ex["metadata"]["q"] == int(api["diag_export_meta_q"]) and ex["metadata"]["lattice_type"] == "E8"
    assert torch.equal(layer.get_scaling_factors(), layer.theta_beta.detach())
    lin = torch.nn.Linear(64, 24)
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(api["diag_lin_W"]))
        lin.bias.copy_(torch.from_numpy(api["diag_lin_b"]))
    layer.load_from_linear(lin)
    assert layer.weight.is_cuda and np.array_equal(layer.weight.detach().cpu().numpy(), api["diag_lin_W"])
    assert np.array_equal(bits(layer._quantize_weights().detach().cpu().numpy()), bits(api["diag_after_load_Wq"]))
    with pytest.raises(ValueError):
        layer.load_from_linear(torch.nn.Linear(32, 24))


def test_decoder_class_and_method_enum(api):
    from coset_b200.core.base import LatticeConfig
    from coset_b200.core.e8 import DecodingMethod, E8Decoder, e8_decode
    c = LatticeConfig(lattice_type="E8", q=4, M=2, beta=0.5)
    codes = dev(api["dec_codes"])
    dec = E8Decoder(torch.device("cuda"))
    got = dec.decode(codes, c, method=DecodingMethod.FULL)
    assert np.array_equal(bits(got.cpu().numpy()), bits(api["dec_xhat"]))
    assert torch.equal(got, e8_decode(codes, c, method="full"))
    assert DecodingMethod.FULL.value == "full"
    with pytest.raises(ValueError):
        dec.decode(codes, c, method="progressive")


@pytest.mark.parametrize("tiling", ["row", "block"])
def test_packed_export_round_trip_with_default_clip(tiling):
    """A trained layer with the default weight_clip_value = 2.0 and N(0, 20) weights (the clamp is active
    on most weights): the exported E8CodeLinear, also after a trip through a state_dict, computes what the
    layer computes, for every kernel that can serve it."""
    from coset_b200.core.e8 import create_e8_hnlq_linear
    from coset_b200.vlut import E8CodeLinear, e8_dequant_gemm
    torch.manual_seed(0)
    layer = create_e8_hnlq_linear(128, 64, q=4, M=2, tiling=tiling, init_kwargs={"std": 20.0}, device="cuda")
    assert layer.weight_clip_value == 2.0
    ex = layer.export_quantized(packed=True)
    assert ex["codes"].dtype == torch.int32 and tuple(ex["codes"].shape) == (64, 16)
    assert ex["metadata"]["weight_clip_value"] == 2.0 and ex["blocks_per_tile"] == (16 if tiling == "row" else 1)
    lin = E8CodeLinear.from_exported(ex, small_t_max=64)
    with torch.no_grad():
        wq = layer._quantize_weights()
        assert float((wq.abs() == 2.0).float().mean()) > 0.2  # the clamp really is active
        assert torch.equal(lin.dense_weight(), wq)
        for T in (1, 5, 40, 200):
            x = torch.randn(T, 128, device="cuda")
            assert rel(lin(x).cpu().numpy(), layer(x).cpu().numpy()) < 1e-5, T
        xb = torch.randn(96, 128, device="cuda").to(torch.bfloat16)
        want = (xb.float() @ wq.t() + layer.bias).cpu().numpy()
        got = e8_dequant_gemm(lin.codes, lin.beta, lin.blocks_per_tile, xb, lin.bias, check=True, clip=lin.weight_clip_value)
        assert rel(got.cpu().numpy(), want) < 1e-2
    # a checkpoint alone rebuilds the layer
    sd = {k: v.clone() for k, v in lin.state_dict().items()}
    again = E8CodeLinear.from_state_dict(sd)
    assert again.blocks_per_tile == lin.blocks_per_tile and again.weight_clip_value == 2.0
    x = torch.randn(7, 128, device="cuda")
    assert torch.equal(again(x), lin(x))
    # load_state_dict into an existing instance refreshes the cached dense copy used for many tokens
    other = E8CodeLinear.from_weight(torch.randn(64, 128, device="cuda"), torch.full((lin.beta.numel(),), 3.0, device="cuda"),
                                     lin.blocks_per_tile, torch.zeros(64, device="cuda"))
    xl = torch.randn(100, 128, device="cuda").to(torch.bfloat16)
    other(xl)
    other.load_state_dict(sd)
    assert torch.equal(other(xl), lin(xl))
    with pytest.raises(ValueError):
        create_e8_hnlq_linear(64, 8, q=3, device="cuda").export_quantized(packed=True)
