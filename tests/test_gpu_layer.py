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


def expected_from_oracle(W, beta, theta, bmin, bmax, bias, x, t, blocks_per_tile, clip=2.0):
    """Forward and backward of the reference graph clamp(ste(e8_quantize(W beta)) / beta) evaluated on
    the CPU in float64 around the oracle's quantised weights (coset/core/layers.py:415-470, 472-484):
    the straight-through estimator passes dWq where the clamp is inactive, dbeta collects
    dWq * (W - Wq_unclipped) / beta per tile and dtheta = dbeta * sigmoid'(theta) * (bmax - bmin)."""
    from oracle import oracle as O
    o, i = W.shape
    wq, un = O.fake_quant(W.reshape(-1, 8), beta.reshape(-1), blocks_per_tile, 4, clip)
    wq64 = torch.from_numpy(wq.reshape(o, i).astype(np.float64)).requires_grad_(True)
    x64 = torch.from_numpy(x.astype(np.float64)).requires_grad_(True)
    b64 = torch.from_numpy(bias.astype(np.float64)).requires_grad_(True)
    y = torch.nn.functional.linear(x64, wq64, b64)
    ((y - torch.from_numpy(t.astype(np.float64))) ** 2).mean().backward()
    g = wq64.grad.numpy().reshape(-1, 8)
    inside = (np.abs(un.astype(np.float64)) <= clip)  # clamp passes the gradient on the closed interval
    dW = (g * inside).reshape(o, i)
    beta_blocks = np.repeat(beta.reshape(-1).astype(np.float64), blocks_per_tile)[:, None]
    per_block = (g * inside * (W.reshape(-1, 8).astype(np.float64) - un.astype(np.float64)) / beta_blocks).sum(axis=1)
    dbeta = per_block.reshape(-1, blocks_per_tile).sum(axis=1)
    sg = 1.0 / (1.0 + np.exp(-theta.astype(np.float64)))
    dtheta = dbeta * sg * (1.0 - sg) * (bmax.astype(np.float64) - bmin.astype(np.float64))
    return {"Wq": wq.reshape(o, i), "y": y.detach().numpy(), "dW": dW, "dx": x64.grad.numpy(), "dbias": b64.grad.numpy(),
            "dtheta": dtheta}


@pytest.mark.parametrize("tag", ["small", "big", "mid"])
def test_layer_forward_backward_row_tiling(golden_layer, tag):
    """Every assertion always runs.  The layer's scale comes from the device sigmoid and may differ
    from the fixture's CPU value in the last bit, so the expectation is (1) the oracle evaluated with
    the layer's own scales, bit for bit for the weights and to 1e-5 for outputs and gradients, and
    (2) the reference layer's fixture on every row whose codes are the fixture's (a last-bit change of
    the scale rescales a row by that bit; a changed code is an O(1) jump), which must be nearly all rows."""
    g = golden_layer
    layer = make_layer(g, tag)
    beta = layer._beta().detach().cpu().numpy()
    assert rel(beta, g[f"{tag}_beta"]) < 1e-6
    x = dev(g[f"{tag}_x"]).requires_grad_(True)
    y = layer(x)
    ((y - dev(g[f"{tag}_t"])) ** 2).mean().backward()
    wq = layer._quantize_weights().detach().cpu().numpy()
    o, i = wq.shape
    want = expected_from_oracle(g[f"{tag}_W"], beta, g[f"{tag}_theta"], g[f"{tag}_bmin"], g[f"{tag}_bmax"],
                                g[f"{tag}_bias"], g[f"{tag}_x"], g[f"{tag}_t"], i // 8)
    got = {"y": y.detach().cpu().numpy(), "dW": layer.weight.grad.cpu().numpy(), "dx": x.grad.cpu().numpy(),
           "dbias": layer.bias.grad.cpu().numpy(), "dtheta": layer.theta_beta.grad.cpu().numpy()}
    # (1) against the oracle with the layer's own scales
    assert np.array_equal(bits(wq), bits(want["Wq"]))
    for k in ("y", "dW", "dx", "dbias"):
        assert rel(got[k], want[k]) < 1e-5, k
    assert np.abs(got["dtheta"] - want["dtheta"]).max() <= 2e-4 * np.abs(want["dtheta"]).max() + 1e-9
    # (2) against the reference layer's own outputs, row by row
    want_wq = g[f"{tag}_Wq"]
    same = (np.abs(wq - want_wq) <= 1e-6 * np.abs(want_wq)).all(axis=1)
    assert same.mean() >= 0.95, same.mean()
    assert (beta == g[f"{tag}_beta"]).mean() >= 0.5  # most scales are bit-identical to the CPU value
    assert rel(got["y"][:, same], g[f"{tag}_y"][:, same]) < 1e-5
    assert rel(got["dW"][same], g[f"{tag}_dW"][same]) < 1e-5
    assert rel(got["dbias"][same], g[f"{tag}_dbias"][same]) < 1e-5
    wt = g[f"{tag}_dtheta"]
    assert np.abs(got["dtheta"][same] - wt[same]).max() <= 2e-4 * np.abs(wt).max() + 1e-9
    if same.all():
        assert rel(got["dx"], g[f"{tag}_dx"]) < 1e-5


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


def test_graphed_train_step_keeps_the_statistics_schedule():
    """GraphedTrainStep replays forward + loss + backward as one CUDA graph and does the layer's host-side
    bookkeeping itself: after 520 steps (two statistics updates, weights changed in between) the EMA
    buffers, the step counter, the loss and the gradients are those of 520 eager steps."""
    from coset_b200.core.e8 import create_e8_hnlq_linear
    from coset_b200.core.layers import GraphedTrainStep
    torch.manual_seed(0)
    a = create_e8_hnlq_linear(64, 48, q=4, M=2, init_kwargs={"std": 20.0}, device="cuda")
    b = create_e8_hnlq_linear(64, 48, q=4, M=2, device="cuda")
    b.load_state_dict(a.state_dict())
    x = torch.randn(32, 64, device="cuda")
    t = torch.randn(32, 48, device="cuda")
    loss_fn = lambda y, tt: ((y - tt) ** 2).mean()
    step = GraphedTrainStep(b, loss_fn, (x, t))
    assert int(b.step_count) == int(a.step_count) == 0
    delta = torch.randn_like(a.weight) * 3.0
    for i in range(1, 521):
        a.zero_grad(set_to_none=True)
        la = loss_fn(a(x), t)
        la.backward()
        lb = step(x, t)
        if i == 300:
            with torch.no_grad():
                a.weight.add_(delta)
                b.weight.add_(delta)
    torch.cuda.synchronize()
    assert int(a.step_count) == int(b.step_count) == 520
    assert torch.equal(a.sigma_ema, b.sigma_ema) and torch.equal(a.xmax_ema, b.xmax_ema)
    assert not torch.equal(a.sigma_ema, torch.ones_like(a.sigma_ema))
    assert torch.equal(la, lb)
    assert torch.equal(a.weight.grad, b.weight.grad)
    assert torch.allclose(a.theta_beta.grad, b.theta_beta.grad, rtol=1e-6, atol=0)
