"""HNLQLinearQAT on the GPU against golden outputs of the reference layer (row tiling) and of
the function-assembled expectation for block tiling (the reference layer raises there)."""
import numpy as np
import pytest
import torch

from conftest import bits

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def make_layer(g, tag, tiling="row"):
    from coset_b200.core.e8 import create_e8_hnlq_linear
    W = g[f"{tag}_W"]
    o, i = W.shape
    layer = create_e8_hnlq_linear(i, o, q=4, M=2, tiling=tiling, device="cuda")
    with torch.no_grad():
        layer.weight.copy_(dev(W))
        layer.bias.copy_(dev(g[f"{tag}_bias"]))
        if tiling == "row":
            layer.theta_beta.copy_(dev(g[f"{tag}_theta"]))
            layer.sigma_ema.copy_(dev(g[f"{tag}_sigma"]))
            layer.xmax_ema.copy_(dev(g[f"{tag}_xmax"]))
    return layer


@pytest.mark.parametrize("tag", ["small", "big", "mid"])
def test_fake_quant_kernel_bit_exact(golden_layer, tag):
    from coset_b200.core.layers import e8_fake_quantize
    g = golden_layer
    W = dev(g[f"{tag}_W"])
    o, i = W.shape
    wq = e8_fake_quantize(W, dev(g[f"{tag}_beta"]), i // 8, 4, 2.0)
    assert np.array_equal(bits(wq.cpu().numpy()), bits(g[f"{tag}_Wq"]))
    wqb = e8_fake_quantize(W, dev(g[f"{tag}_blk_beta"]).reshape(-1), 1, 4, 2.0)
    assert np.array_equal(bits(wqb.cpu().numpy()), bits(g[f"{tag}_blk_Wq"]))


@pytest.mark.parametrize("tag", ["small", "big", "mid"])
def test_block_tiling_gradients(golden_layer, tag):
    from coset_b200.core.layers import e8_fake_quantize
    g = golden_layer
    W = dev(g[f"{tag}_W"]).requires_grad_(True)
    o, i = W.shape
    beta = dev(g[f"{tag}_blk_beta"]).reshape(-1).requires_grad_(True)
    wq = e8_fake_quantize(W, beta, 1, 4, 2.0)
    y = torch.nn.functional.linear(dev(g[f"{tag}_x"]), wq, dev(g[f"{tag}_bias"]))
    ((y - dev(g[f"{tag}_t"])) ** 2).mean().backward()
    assert rel(W.grad.cpu().numpy(), g[f"{tag}_blk_dW"]) < 1e-5
    want = g[f"{tag}_blk_dbeta"].reshape(-1)
    assert np.abs(beta.grad.cpu().numpy() - want).max() <= 1e-5 * max(np.abs(want).max(), 1e-12) + 1e-12


@pytest.mark.parametrize("tag", ["small", "big", "mid"])
def test_layer_forward_backward_row_tiling(golden_layer, tag):
    g = golden_layer
    layer = make_layer(g, tag)
    # beta is computed with device sigmoid; it may differ from the CPU value in the last bit
    beta = layer._beta().detach().cpu().numpy()
    assert rel(beta, g[f"{tag}_beta"]) < 1e-6
    x = dev(g[f"{tag}_x"]).requires_grad_(True)
    y = layer(x)
    ((y - dev(g[f"{tag}_t"])) ** 2).mean().backward()
    wq = layer._quantize_weights().detach().cpu().numpy()
    # A row whose beta differs from the CPU value in the last bit rescales by that bit; a changed
    # code would show as an O(1) jump, which must stay a rare boundary event.
    want_wq = g[f"{tag}_Wq"]
    jumps = (np.abs(wq - want_wq) > 1e-4 * np.maximum(np.abs(want_wq), 1e-3)).mean()
    assert jumps < 2e-3, jumps
    if jumps == 0:
        assert rel(wq, want_wq) < 1e-6
        assert rel(y.detach().cpu().numpy(), g[f"{tag}_y"]) < 1e-5
        assert rel(layer.weight.grad.cpu().numpy(), g[f"{tag}_dW"]) < 1e-5
        assert rel(x.grad.cpu().numpy(), g[f"{tag}_dx"]) < 1e-5
        assert rel(layer.bias.grad.cpu().numpy(), g[f"{tag}_dbias"]) < 1e-5
        want = g[f"{tag}_dtheta"]
        got = layer.theta_beta.grad.cpu().numpy()
        assert np.abs(got - want).max() <= 2e-4 * np.abs(want).max() + 1e-9


def test_state_dict_keys_and_warmup(golden_layer):
    from coset_b200.core.e8 import create_e8_hnlq_linear
    layer = create_e8_hnlq_linear(64, 48, warmup_epochs=2, device="cuda")
    assert set(layer.state_dict().keys()) == {"weight", "bias", "theta_beta", "G", "Ginv", "sigma_ema", "xmax_ema",
                                              "step_count", "gamma_inv"}
    assert not layer.is_quantization_enabled()
    x = torch.randn(4, 64, device="cuda")
    y0 = layer(x)
    assert torch.allclose(y0, torch.nn.functional.linear(x, layer.weight, layer.bias))
    layer.update_epoch(1)
    assert not layer.is_quantization_enabled()
    layer.update_epoch(2)
    assert layer.is_quantization_enabled()
    layer(x)
    assert int(layer.step_count) == 1
    other = create_e8_hnlq_linear(64, 48, device="cuda")
    other.load_state_dict(layer.state_dict())
    assert other._step_host == 1
    with pytest.raises(ValueError):
        create_e8_hnlq_linear(60, 48)
    with pytest.raises(ValueError):
        layer.load_weights(torch.zeros(3, 3))


def test_bf16_activations(golden_layer):
    g = golden_layer
    layer = make_layer(g, "mid")
    x = dev(g["mid_x"])
    y32 = layer(x)
    y16 = layer(x.to(torch.bfloat16))
    assert y16.dtype == torch.bfloat16
    assert rel(y16.detach().float().cpu().numpy(), y32.detach().cpu().numpy()) < 1e-2
    y16.float().sum().backward()
    assert layer.weight.grad is not None and layer.theta_beta.grad is not None


def test_training_step_is_graph_capturable():
    """Forward + backward of the layer enqueue work only on the current stream: one CUDA graph replays
    the step and yields the gradients of the eager step."""
    import warnings
    from coset_b200.core.e8 import create_e8_hnlq_linear
    torch.manual_seed(0)
    layer = create_e8_hnlq_linear(64, 48, q=4, M=2, init_kwargs={"std": 20.0}, device="cuda")
    x = torch.randn(32, 64, device="cuda")
    t = torch.randn(32, 48, device="cuda")

    def step():
        ((layer(x) - t) ** 2).mean().backward()

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            layer.zero_grad(set_to_none=True)
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    layer.zero_grad(set_to_none=True)
    g = torch.cuda.CUDAGraph()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with torch.cuda.graph(g):
            step()
    g.replay()
    torch.cuda.synchronize()
    gw, gt = layer.weight.grad.clone(), layer.theta_beta.grad.clone()
    layer.zero_grad(set_to_none=True)
    step()
    torch.cuda.synchronize()
    assert torch.equal(gw, layer.weight.grad)
    assert torch.allclose(gt, layer.theta_beta.grad, rtol=1e-6, atol=0)
