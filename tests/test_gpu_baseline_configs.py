"""Parity on the benchmark configurations themselves, at their stated shapes and data.

Each test runs the CUDA library through its C ABI on the data a measurement is quoted on and
compares with the CPU oracle (C restatement of coset.core.e8, pinned on reference-generated
fixtures by tests/test_oracle_golden.py):

  * bulk codec    : bench.make_values data (N(0, 0.02) with +-10 sigma outliers, which become exact
                    integers +-5.0 after scaling: the tie-heavy case), per-block scale 25, a
                    2^22-block chunk with a ragged tail; packed codes and reconstructions bit for bit,
                    float32 and bf16 input                     (coset/core/e8/codecs.py:63-89, 159-180)
  * QAT layer     : weight [3072, 768], 4096 tokens, std 0.02 and 20, row and block tiling
                                                               (coset/core/layers.py:398-484)
  * code-domain   : weight [4096, 4096] as codes, T in {1, 16, 256, 4096}, scale 25 and the literal
    product         scale, every kernel that can serve the product (coset/legacy/quant/vlut.py:72-117)
  * gradient      : 13 685 280 blocks x 8 ranks, decode-and-average kernel against the CPU recipe
    exchange        (prompts/design_instructions.md:104-110)
"""
import os

import numpy as np
import pytest
import torch

from conftest import bits
from oracle import oracle as O

pytestmark = pytest.mark.gpu

THREADS = os.cpu_count() or 1
BETA_MID = 0.021440971642732620


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


# ------------------------------------------------------------------------------- bulk codec
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bulk_codec_on_bench_data_matches_oracle(dtype):
    import bench
    from coset_b200 import _lib
    from coset_b200.core.e8 import e8_decode_packed, e8_encode_packed
    n = (1 << 22) + 77  # one 2^22-block chunk of the benchmark's stream plus a ragged tail
    x = bench.make_values(n * 8, 0).view(n, 8)
    if dtype == torch.bfloat16:
        x = x.to(torch.bfloat16)
    beta = torch.full((n,), bench.BETA_HEADLINE)
    x32 = x.float().numpy()
    # the +-10 sigma outliers scale to exactly +-5.0: rounding ties of the half-integer coset
    assert (np.abs(x32 * np.float32(25.0)) == 5.0).mean() > 5e-4 or dtype == torch.bfloat16
    digits = O.encode(x32, beta=beta.numpy(), scale_mode=2, blocks_per_tile=1, threads=THREADS)
    want_codes = O.pack_q4(digits)
    want_xhat = O.decode(digits, beta=beta.numpy(), scale_mode=2, blocks_per_tile=1, threads=THREADS)
    MT = _lib.SCALE_MUL_TILE
    xd, bd = x.cuda(), beta.cuda()
    codes = e8_encode_packed(xd, 4, 2, scale=bd, scale_mode=MT, blocks_per_tile=1)
    got_codes = codes.view(torch.int32).view(-1).cpu().numpy().view(np.uint32)
    assert np.array_equal(got_codes, want_codes), int((got_codes != want_codes).sum())
    assert (want_codes != 0).mean() > 0.5
    xhat = e8_decode_packed(codes, 4, 2, scale=bd, scale_mode=MT, blocks_per_tile=1)
    assert np.array_equal(bits(xhat.cpu().numpy()), bits(want_xhat))
    # fused round trip on the same data
    fused = torch.empty((n, 8), dtype=torch.float32, device="cuda")
    rc = _lib.lib().coset_e8_quantize(_lib.ptr(xd), _lib.dtype_code(xd, "x"), _lib.ptr(bd), MT, n, 1, 4, 2, 0.0,
                                      _lib.ptr(fused), 0, None, _lib.stream())
    assert rc == 0
    assert np.array_equal(bits(fused.cpu().numpy()), bits(want_xhat))


def test_bulk_codec_literal_scale_on_bench_data():
    import bench
    from coset_b200 import _lib
    from coset_b200.core.e8 import e8_encode_packed
    n = 1 << 20
    x = bench.make_values(n * 8, 0).view(n, 8)
    beta = torch.full((n,), bench.BETA_LITERAL)
    want = O.pack_q4(O.encode(x.numpy(), beta=beta.numpy(), scale_mode=2, blocks_per_tile=1, threads=THREADS))
    got = e8_encode_packed(x.cuda(), 4, 2, scale=beta.cuda(), scale_mode=_lib.SCALE_MUL_TILE).view(torch.int32).view(-1)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want)
    assert not want.any()  # every block maps to the all-zero code at the literal scale


# ------------------------------------------------------------------------------- QAT layer
@pytest.mark.parametrize("tiling", ["row", "block"])
@pytest.mark.parametrize("std", [0.02, 20.0])
def test_qat_layer_at_config_shape(tiling, std):
    from coset_b200.core.e8 import create_e8_hnlq_linear
    from test_gpu_layer import expected_from_oracle
    torch.manual_seed(0)
    d_in, d_out, tokens = 768, 3072, 4096
    layer = create_e8_hnlq_linear(d_in, d_out, q=4, M=2, tiling=tiling, init_kwargs={"std": std}, device="cpu")
    if std < 1:  # the config clamps its N(0, 0.02) weights to +-2 (a no-op at that sigma)
        with torch.no_grad():
            layer.weight.clamp_(-2.0, 2.0)
    layer = layer.cuda()
    x_cpu = torch.randn(tokens, d_in)
    t_cpu = torch.randn(tokens, d_out)
    W = layer.weight.detach().cpu().numpy()
    bmin, bmax = (v.detach().cpu().numpy() for v in layer._bounds())
    beta = layer._beta().detach().cpu().numpy()
    assert rel(beta, np.full_like(beta, BETA_MID)) < 1e-6
    theta = layer.theta_beta.detach().cpu().numpy()
    bpt = d_in // 8 if tiling == "row" else 1
    want = expected_from_oracle(W, beta, theta, bmin, bmax, layer.bias.detach().cpu().numpy(), x_cpu.numpy(),
                                t_cpu.numpy(), bpt)
    # float32 activations: 1e-5
    x = x_cpu.cuda().requires_grad_(True)
    y = layer(x)
    ((y - t_cpu.cuda()) ** 2).mean().backward()
    wq = layer._quantize_weights().detach().cpu().numpy()
    assert np.array_equal(bits(wq), bits(want["Wq"]))
    nonzero = float((want["Wq"] != 0).mean())
    assert (nonzero == 0.0) if std < 1 else (0.3 < nonzero < 0.8), nonzero
    assert rel(y.detach().cpu().numpy(), want["y"]) < 1e-5
    assert rel(layer.weight.grad.cpu().numpy(), want["dW"]) < 1e-5
    assert rel(x.grad.cpu().numpy(), want["dx"]) < 1e-5
    if std < 1:
        assert not x.grad.any()  # dx is identically zero when every weight quantises to 0
    assert rel(layer.bias.grad.cpu().numpy(), want["dbias"]) < 1e-5
    dth = layer.theta_beta.grad.cpu().numpy()
    assert np.abs(dth - want["dtheta"]).max() <= 2e-4 * np.abs(want["dtheta"]).max() + 1e-9
    # bf16 activations: 1e-2
    layer.zero_grad(set_to_none=True)
    xb = x_cpu.cuda().to(torch.bfloat16).requires_grad_(True)
    yb = layer(xb)
    assert yb.dtype == torch.bfloat16
    ((yb.float() - t_cpu.cuda()) ** 2).mean().backward()
    assert rel(yb.detach().float().cpu().numpy(), want["y"]) < 1e-2
    assert rel(layer.weight.grad.cpu().numpy(), want["dW"]) < 1e-2
    if std > 1:
        assert rel(xb.grad.float().cpu().numpy(), want["dx"]) < 1e-2


# ------------------------------------------------------------------------------- code-domain product
@pytest.fixture(scope="module")
def cfg4():
    """Weight [4096, 4096] N(0, 0.02), seed 0, encoded by the oracle with per-block scale 25."""
    torch.manual_seed(0)
    n = 4096
    W = torch.randn(n, n) * 0.02
    beta = np.full(n * n // 8, 25.0, np.float32)
    digits = O.encode(W.numpy().reshape(-1, 8), beta=beta, scale_mode=2, blocks_per_tile=1, threads=THREADS)
    w_hat = O.decode(digits, beta=beta, scale_mode=2, blocks_per_tile=1, threads=THREADS).reshape(n, n)
    return {"W": W, "beta": torch.from_numpy(beta), "codes": O.pack_q4(digits), "w_hat": w_hat}


@pytest.mark.parametrize("T", [1, 16, 256, 4096])
def test_code_domain_product_at_config_shape(cfg4, T):
    from coset_b200.vlut import E8CodeLinear, e8_decode_gemm, e8_dequant_gemm, e8_vlut_matmul
    lin = E8CodeLinear.from_weight(cfg4["W"].cuda(), cfg4["beta"].cuda(), 1)
    assert np.array_equal(lin.codes.cpu().numpy().view(np.uint32).reshape(-1), cfg4["codes"])
    torch.manual_seed(100 + T)
    x = torch.randn(T, 4096).to(torch.bfloat16)
    want = (x.float() @ torch.from_numpy(cfg4["w_hat"]).t()).numpy()  # decode, then float32 matmul
    xd = x.cuda()
    got_layer = lin(xd)
    assert got_layer.dtype == torch.bfloat16
    assert rel(got_layer.float().cpu().numpy(), want) < 1e-2
    got_gemm = e8_dequant_gemm(lin.codes, lin.beta, 1, xd, None, check=True)
    assert rel(got_gemm.cpu().numpy(), want) < 1e-2
    got_pair = e8_decode_gemm(lin.codes, lin.beta, 1, xd, None, check=True)
    assert rel(got_pair.cpu().numpy(), want) < 1e-2
    # same bf16 weights, same K order inside a K step: the two tensor-core forms differ by accumulation order at most
    assert rel(got_pair.cpu().numpy(), got_gemm.cpu().numpy()) < 1e-5
    if T <= 16:
        got_gemv = e8_vlut_matmul(lin.codes, lin.beta, 1, xd)
        assert rel(got_gemv.cpu().numpy(), want) < 1e-2
        # float32 activations through the few-token kernel: 1e-5 against a float64 product
        x32 = torch.randn(T, 4096)
        want32 = x32.double().numpy() @ cfg4["w_hat"].astype(np.float64).T
        assert rel(e8_vlut_matmul(lin.codes, lin.beta, 1, x32.cuda()).cpu().numpy(), want32) < 1e-5


def test_code_domain_product_literal_scale_is_zero(cfg4):
    from coset_b200.vlut import E8CodeLinear
    beta = torch.full((4096 * 4096 // 8,), BETA_MID)
    lin = E8CodeLinear.from_weight(cfg4["W"].cuda(), beta.cuda(), 1)
    want = O.pack_q4(O.encode(cfg4["W"].numpy().reshape(-1, 8), beta=beta.numpy(), scale_mode=2, blocks_per_tile=1,
                              threads=THREADS))
    assert np.array_equal(lin.codes.cpu().numpy().view(np.uint32).reshape(-1), want) and not want.any()
    for T in (1, 16, 256, 4096):
        assert not lin(torch.randn(T, 4096, device="cuda").to(torch.bfloat16)).any()


# ------------------------------------------------------------------------------- gradient exchange
def test_decode_mean_at_config_size():
    """W = 8 code streams of the BERT-base-shaped gradient (13 685 280 blocks each) built on one GPU;
    the decode-and-average kernel against the CPU recipe on every 64th block, and the encoder against
    the oracle on the same blocks."""
    from coset_b200 import _lib
    from coset_b200.gradcomm import CudaCodec, bert_base_gradient_numel
    from gradcomm_util import cpu_decode_mean
    n_values = bert_base_gradient_numel()
    assert n_values == 109_482_240
    n_blocks, world, scale = n_values // 8, 8, 500.0
    codec = CudaCodec()
    gathered = torch.empty((world, n_blocks), dtype=torch.int32, device="cuda")
    digits = []
    for r in range(world):
        g = torch.Generator().manual_seed(1000 + r)
        grad = torch.randn(n_values, generator=g) * 1e-3
        blocks = grad.view(n_blocks, 8)
        codec.encode(blocks.cuda(), scale, gathered[r])
        d = O.encode(blocks[::64].contiguous().numpy(), beta=np.array([scale], np.float32), scale_mode=2,
                     blocks_per_tile=n_blocks, threads=THREADS)
        assert np.array_equal(gathered[r][::64].cpu().numpy().view(np.uint32), O.pack_q4(d)), r
        digits.append(d)
    out = torch.empty((n_blocks, 8), dtype=torch.float32, device="cuda")
    codec.decode_mean(gathered, world, n_blocks, scale, out)
    want = cpu_decode_mean(digits, scale)
    assert np.array_equal(bits(out[::64].cpu().numpy()), bits(want))
    assert np.abs(want).max() > 0
