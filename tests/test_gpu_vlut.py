"""Code-domain matmul (E8CodeLinear) against decode-then-float32-matmul of the CPU restatement
of the reference (BASELINE config: weight stored as E8 codes, activations bf16 / float32)."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def make(n_out, n_in, tiling, beta_value=25.0, seed=0):
    torch.manual_seed(seed)
    W = torch.randn(n_out, n_in) * 0.02
    kb = n_in // 8
    if tiling == "block":
        beta = torch.full((n_out * kb,), beta_value) * (0.75 + 0.5 * torch.rand(n_out * kb))
        bpt = 1
    else:
        beta = torch.full((n_out,), beta_value) * (0.75 + 0.5 * torch.rand(n_out))
        bpt = kb
    digits = O.encode(W.numpy().reshape(-1, 8), beta=beta.numpy(), scale_mode=2, blocks_per_tile=bpt, threads=8)
    w_hat = O.decode(digits, beta=beta.numpy(), scale_mode=2, blocks_per_tile=bpt, threads=8).reshape(n_out, n_in)
    return W, beta, bpt, digits, w_hat


@pytest.mark.parametrize("tiling", ["block", "row"])
@pytest.mark.parametrize("T", [1, 3, 16, 40])
def test_small_t_fp32_activations(tiling, T):
    from coset_b200.vlut import E8CodeLinear
    W, beta, bpt, digits, w_hat = make(256, 512, tiling)
    bias = torch.randn(256)
    lin = E8CodeLinear.from_weight(W.cuda(), beta.cuda(), bpt, bias.cuda(), small_t_max=64)  # every T below: code-domain kernels
    assert np.array_equal(lin.codes.cpu().numpy().view(np.uint32).reshape(-1), O.pack_q4(digits))
    assert np.array_equal(lin.dense_weight().cpu().numpy(), w_hat)  # bit-exact dequantised weight
    x = torch.randn(T, 512)
    want = x.double().numpy() @ w_hat.astype(np.float64).T + bias.double().numpy()
    got = lin(x.cuda()).cpu().numpy()
    assert rel(got, want) < 1e-5


@pytest.mark.parametrize("T", [1, 16, 256])
def test_bf16_activations_config_shape(T):
    """BASELINE vLUT config at reduced width for the CPU oracle: beta = 25 (scaled sigma 0.5)."""
    from coset_b200.vlut import E8CodeLinear
    W, beta, bpt, digits, w_hat = make(512, 1024, "block")
    lin = E8CodeLinear.from_weight(W.cuda(), beta.cuda(), bpt)
    x = torch.randn(T, 1024).to(torch.bfloat16)
    want = x.float().numpy() @ w_hat.T
    got = lin(x.cuda()).float().cpu().numpy()
    assert rel(got, want) < 1e-2


def test_literal_scale_gives_zero_output():
    from coset_b200.vlut import E8CodeLinear
    W = torch.randn(64, 128) * 0.02
    beta = torch.full((64 * 16,), 0.021440971642732620)
    lin = E8CodeLinear.from_weight(W.cuda(), beta.cuda(), 1)
    assert not lin.codes.any()
    assert not lin(torch.randn(4, 128, device="cuda")).any()


def test_export_from_trained_layer():
    """Default weight_clip_value (2.0) with N(0, 20) weights: the clamp is active on most weights and the
    exported layer must still compute what the trained layer computes."""
    from coset_b200.core.e8 import create_e8_hnlq_linear
    from coset_b200.vlut import E8CodeLinear
    layer = create_e8_hnlq_linear(128, 64, device="cuda", init_kwargs={"std": 20.0})
    lin = E8CodeLinear.from_qat_layer(layer)
    assert lin.weight_clip_value == 2.0
    x = torch.randn(5, 128, device="cuda")
    with torch.no_grad():
        assert rel(lin(x).cpu().numpy(), layer(x).cpu().numpy()) < 1e-5
    with pytest.raises(ValueError):
        E8CodeLinear.from_weight(torch.zeros(4, 12, device="cuda"), torch.ones(4, device="cuda"), 1)


@pytest.mark.parametrize("tiling", ["block", "row"])
def test_weight_clip_in_every_kernel(tiling):
    """clamp(decode / beta, +-clip) with a clip that cuts about a third of the weights, against the CPU
    restatement: few-token kernel (float32 and bf16 activations), library path and both tcgen05 forms."""
    from coset_b200.vlut import E8CodeLinear, e8_decode_gemm, e8_dequant_gemm
    W, beta, bpt, digits, w_hat = make(256, 512, tiling)
    clip = 0.03
    w_clip = np.clip(w_hat, -clip, clip)
    assert 0.1 < (np.abs(w_hat) > clip).mean() < 0.6
    bias = torch.randn(256)
    lin = E8CodeLinear.from_weight(W.cuda(), beta.cuda(), bpt, bias.cuda(), weight_clip_value=clip, small_t_max=64)
    assert np.array_equal(lin.dense_weight().cpu().numpy(), w_clip)
    for T in (1, 3, 16, 40):
        x = torch.randn(T, 512)
        want = x.double().numpy() @ w_clip.astype(np.float64).T + bias.double().numpy()
        assert rel(lin(x.cuda()).cpu().numpy(), want) < 1e-5, T
    xb = torch.randn(300, 512).to(torch.bfloat16)
    want = xb.float().numpy().astype(np.float64) @ w_clip.astype(np.float64).T + bias.double().numpy()
    assert rel(lin(xb.cuda()).float().cpu().numpy(), want) < 1e-2
    got = e8_dequant_gemm(lin.codes, lin.beta, bpt, xb.cuda(), lin.bias, check=True, clip=clip)
    assert rel(got.cpu().numpy(), want) < 1e-2
    got2 = e8_decode_gemm(lin.codes, lin.beta, bpt, xb.cuda(), lin.bias, check=True, clip=clip)
    assert rel(got2.cpu().numpy(), want) < 1e-2


@pytest.mark.parametrize("form", ["fused", "decode_then_pair_gemm"])
@pytest.mark.parametrize("T,n_out,n_in,tiling", [(128, 128, 64, "block"), (256, 256, 512, "block"), (300, 200, 1024, "row"), (1100, 384, 256, "block"),
                                                  (1, 128, 128, "block"), (513, 640, 512, "row")])
def test_tcgen05_dequant_gemm(T, n_out, n_in, tiling, form):
    """Both tensor-core forms (decode fused into the K loop; decode to a transient bf16 buffer followed by the
    cta_group::2 GEMM) against decode-then-float32-matmul of the CPU restatement.  Shapes: ragged token counts,
    feature counts that are not multiples of a tile (200, 384, 640), one K step and sixteen."""
    from coset_b200.vlut import E8CodeLinear, e8_decode_gemm, e8_dequant_gemm
    gemm = e8_dequant_gemm if form == "fused" else e8_decode_gemm
    W, beta, bpt, digits, w_hat = make(n_out, n_in, tiling, seed=T)
    bias = torch.randn(n_out)
    lin = E8CodeLinear.from_weight(W.cuda(), beta.cuda(), bpt, bias.cuda())
    x = torch.randn(T, n_in).to(torch.bfloat16)
    got = gemm(lin.codes, lin.beta, bpt, x.cuda(), lin.bias, check=True).cpu().numpy()
    want = x.float().numpy().astype(np.float64) @ w_hat.astype(np.float64).T + bias.double().numpy()
    assert rel(got, want) < 1e-2
    # against the same product with bf16-rounded weights the kernel should agree to fp32 accumulation error
    w_bf = torch.from_numpy(w_hat).to(torch.bfloat16).double().numpy()
    want_bf = x.double().numpy() @ w_bf.T + bias.double().numpy()
    assert rel(got, want_bf) < 2e-3  # weights may differ from the exactly divided ones by one bf16 ulp
    if form != "fused":  # bf16 result: the same float32 accumulator plus bias, rounded once by the kernel
        got16 = gemm(lin.codes, lin.beta, bpt, x.cuda(), lin.bias, check=True, out_dtype=torch.bfloat16)
        assert got16.dtype == torch.bfloat16
        assert torch.equal(got16.cpu(), torch.from_numpy(got).to(torch.bfloat16))


@pytest.mark.parametrize("path", ["auto", "tcgen05", "cublas"])
def test_layer_dispatch_for_many_tokens(path):
    """Every large_t_path of E8CodeLinear at token counts on both sides of its thresholds (64 / 1024 / 2048):
    same product within the bf16 tolerance, result in the activations' type; 'tcgen05' keeps no dense copy."""
    from coset_b200.vlut import E8CodeLinear
    W, beta, bpt, digits, w_hat = make(256, 512, "row", seed=5)
    bias = torch.randn(256)
    lin = E8CodeLinear.from_weight(W.cuda(), beta.cuda(), bpt, bias.cuda(), large_t_path=path)
    assert lin.small_t_max == (48 if path == "tcgen05" else 16)
    for T in (16, 17, 48, 49, 65, 300, 1024, 1100, 2048, 2100):
        x = torch.randn(T, 512).to(torch.bfloat16)
        got = lin(x.cuda())
        assert got.dtype == torch.bfloat16 and tuple(got.shape) == (T, 256)
        want = x.float().numpy().astype(np.float64) @ w_hat.astype(np.float64).T + bias.double().numpy()
        assert rel(got.float().cpu().numpy(), want) < 1e-2, (path, T)
    assert (lin._dense is None) == (path == "tcgen05")
    lin.check()  # no bounded wait gave up in any of the tensor-core kernels above
    if path != "cublas":
        lin._status.fill_(1)  # what a kernel whose wait expired leaves behind
        with pytest.raises(RuntimeError):
            lin.check()
        lin.check()  # reported once, then clear
    with pytest.raises(ValueError):
        E8CodeLinear.from_weight(W.cuda(), beta.cuda(), bpt, large_t_path="fastest")


def test_decode_gemm_through_the_c_abi_with_strides_and_without_scales():
    """coset_e8_decode_gemm called as a foreign runtime would: raw pointers, activation rows and result rows
    with padding between them (ldx > n_in, ldy > n_out), no scales (beta = NULL: weights are the plain
    reconstructions), no bias; and the empty shapes return at once."""
    from coset_b200 import _lib
    L = _lib.lib()
    torch.manual_seed(3)
    n_out, n_in, T = 200, 192, 333
    W = torch.randn(n_out, n_in) * 0.6
    digits = O.encode(W.numpy().reshape(-1, 8), threads=8)
    w_hat = O.decode(digits, threads=8).reshape(n_out, n_in)
    codes = torch.from_numpy(O.pack_q4(digits).view(np.int32).reshape(n_out, n_in // 8)).cuda()
    ldx, ldy = n_in + 16, n_out + 5
    xbuf = torch.zeros(T, ldx, dtype=torch.bfloat16, device="cuda")
    x = torch.randn(T, n_in).to(torch.bfloat16)
    xbuf[:, :n_in] = x.cuda()
    ybuf = torch.full((T, ldy), 7.0, dtype=torch.float32, device="cuda")
    scratch = torch.empty(n_out * n_in, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = L.coset_e8_decode_gemm(_lib.ptr(codes), None, 1, n_out, n_in, _lib.ptr(xbuf), ldx, T, None, _lib.ptr(ybuf), _lib.DTYPE_F32, ldy,
                                0.0, _lib.ptr(scratch), scratch.numel() * 2, _lib.ptr(status), _lib.stream())
    assert rc == 0, L.coset_last_error_string()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = x.float().numpy().astype(np.float64) @ w_hat.astype(np.float64).T
    assert rel(ybuf[:, :n_out].cpu().numpy(), want) < 1e-2
    assert bool((ybuf[:, n_out:] == 7.0).all())  # the padding between result rows is untouched
    assert torch.equal(scratch.view(n_out, n_in).float().cpu(), torch.from_numpy(w_hat).to(torch.bfloat16).float())  # exact: halves of small integers
    for shape in ((0, n_in, T), (n_out, n_in, 0)):
        assert L.coset_e8_decode_gemm(_lib.ptr(codes), None, 1, shape[0], shape[1], _lib.ptr(xbuf), ldx, shape[2], None, _lib.ptr(ybuf),
                                      _lib.DTYPE_F32, ldy, 0.0, _lib.ptr(scratch), scratch.numel() * 2, None, _lib.stream()) == 0
    # refused: scratch too small, n_in not a multiple of 64, unknown result type
    assert L.coset_e8_decode_gemm(_lib.ptr(codes), None, 1, n_out, n_in, _lib.ptr(xbuf), ldx, T, None, _lib.ptr(ybuf), _lib.DTYPE_F32, ldy,
                                  0.0, _lib.ptr(scratch), 16, None, _lib.stream()) < 0
    assert L.coset_e8_decode_gemm(_lib.ptr(codes), None, 1, n_out, 100, _lib.ptr(xbuf), ldx, T, None, _lib.ptr(ybuf), _lib.DTYPE_F32, ldy,
                                  0.0, _lib.ptr(scratch), scratch.numel() * 2, None, _lib.stream()) < 0
    assert L.coset_e8_decode_gemm(_lib.ptr(codes), None, 1, n_out, n_in, _lib.ptr(xbuf), ldx, T, None, _lib.ptr(ybuf), 9, ldy,
                                  0.0, _lib.ptr(scratch), scratch.numel() * 2, None, _lib.stream()) < 0


def test_decode_gemm_scratch_is_checked_and_reusable():
    """The transient weight buffer: refused when too small or of the wrong type; one buffer serves layers of
    different shapes one after the other (nothing in it survives a call)."""
    from coset_b200.vlut import E8CodeLinear, e8_decode_gemm
    scratch = torch.empty(512 * 256, dtype=torch.bfloat16, device="cuda")
    for n_out, n_in in ((512, 256), (128, 192), (256, 512)):
        W, beta, bpt, digits, w_hat = make(n_out, n_in, "block", seed=n_out)
        lin = E8CodeLinear.from_weight(W.cuda(), beta.cuda(), bpt)
        x = torch.randn(70, n_in).to(torch.bfloat16)
        got = e8_decode_gemm(lin.codes, lin.beta, bpt, x.cuda(), None, check=True, scratch=scratch).cpu().numpy()
        assert rel(got, x.float().numpy().astype(np.float64) @ w_hat.astype(np.float64).T) < 1e-2
    with pytest.raises(ValueError):
        e8_decode_gemm(lin.codes, lin.beta, bpt, x.cuda(), None, scratch=scratch[:100])
    with pytest.raises(ValueError):
        e8_decode_gemm(lin.codes, lin.beta, bpt, x.cuda(), None, scratch=scratch.float())
    from coset_b200 import _lib
    assert _lib.lib().coset_e8_decode_gemm_scratch_bytes(256, 512) == 256 * 512 * 2


SHARD_WORKER = r'''
import os, sys
import torch
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from coset_b200.vlut import ColumnParallelE8CodeLinear, E8CodeLinear
rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
torch.manual_seed(3)
n_out, n_in = 256, 512
W = (torch.randn(n_out, n_in) * 0.02).cuda()
for bpt, nbeta in ((1, n_out * n_in // 8), (n_in // 8, n_out)):
    beta = (20.0 + 10.0 * torch.rand(nbeta)).cuda()
    bias = torch.randn(n_out).cuda()
    full = E8CodeLinear.from_weight(W, beta, bpt, bias)
    shard = ColumnParallelE8CodeLinear.from_weight(W, beta, bpt, bias)
    peer = ColumnParallelE8CodeLinear.from_weight(W, beta, bpt, bias, transport="peer")
    for T in (1, 5, 200):
        x = torch.randn(T, n_in).cuda()
        assert torch.equal(shard(x), full(x)), (bpt, T)
        for _ in range(3):  # several calls: both halves of the result buffer are reused
            assert torch.equal(peer(x), full(x)), ("peer", bpt, T)
torch.cuda.synchronize()
if rank == 0:
    print("SHARD_OK")
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_column_parallel_equals_unsharded(tmp_path):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "shard_worker.py"
    script.write_text(SHARD_WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29621", str(script), root]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "SHARD_OK" in res.stdout
