"""E8 gradient exchange on the GPU: the decode-and-average kernel against the CPU recipe, and
the NCCL exchange on 2 GPUs (skipped when only one is visible)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import bits
from gradcomm_util import cpu_decode_mean, oracle_encode_saturating
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_decode_mean_matches_cpu_recipe(world):
    from coset_b200.gradcomm import CudaCodec
    n, scale = 5000, 500.0
    codec = CudaCodec()
    gathered = torch.empty((world, n), dtype=torch.int32, device="cuda")
    digits = []
    for r in range(world):
        g = torch.Generator().manual_seed(1000 + r)
        grad = (torch.randn(n, 8, generator=g) * 1e-3)
        codec.encode(grad.cuda(), scale, gathered[r])
        d = oracle_encode_saturating(grad.numpy(), scale)
        assert np.array_equal(gathered[r].cpu().numpy().view(np.uint32), O.pack_q4(d))
        digits.append(d)
    out = torch.empty((n, 8), device="cuda")
    codec.decode_mean(gathered, world, n, scale, out)
    assert np.array_equal(bits(out.cpu().numpy()), bits(cpu_decode_mean(digits, scale)))


def test_outlier_block_is_clipped_not_wrapped():
    """One gradient value far outside the two-level code's range: the saturating encode clips it to
    3.9 / scale (bit for bit the CPU recipe with the clamp); the plain codec wraps it to an unrelated
    small value, which is what the exchange must never do silently."""
    from coset_b200.gradcomm import CudaCodec, E8GradientExchange, SATURATION
    from gradcomm_util import oracle_encode_saturating
    n, scale = 4096, 500.0
    g = torch.Generator().manual_seed(7)
    grad = torch.randn(n, 8, generator=g) * 1e-3
    grad[17, 3] = 0.25        # 125 lattice units: far beyond the range of the code
    grad[900] = -0.05         # a whole block at -25 units
    grad[901, 0] = float("inf")
    codes = torch.empty(n, dtype=torch.int32, device="cuda")
    CudaCodec().encode(grad.cuda(), scale, codes)
    want = oracle_encode_saturating(grad.numpy(), scale)
    assert np.array_equal(codes.cpu().numpy().view(np.uint32), O.pack_q4(want))
    out = torch.empty((n, 8), device="cuda")
    CudaCodec().decode_mean(codes.view(1, n), 1, n, scale, out)
    out = out.cpu()
    assert abs(float(out[17, 3]) - SATURATION / scale) <= 1.0 / scale      # clipped, within a lattice unit
    assert float((out[900] + SATURATION / scale).abs().max()) <= 1.5 / scale
    assert bool(torch.isfinite(out).all())
    # the plain codec wraps the same value around
    plain = torch.empty(n, dtype=torch.int32, device="cuda")
    CudaCodec(saturate=False).encode(grad.nan_to_num(posinf=0.0).cuda(), scale, plain)
    out2 = torch.empty((n, 8), device="cuda")
    CudaCodec().decode_mean(plain.view(1, n), 1, n, scale, out2)
    assert abs(float(out2[17, 3].cpu()) - 0.25) > 0.2
    frac = E8GradientExchange(scale=scale).overloaded_fraction(grad.nan_to_num(posinf=0.0).reshape(-1).cuda())
    assert 2 / n <= frac <= 8 / n


def test_single_gpu_exchange_roundtrip():
    from coset_b200.gradcomm import E8GradientExchange
    g = torch.randn(8 * 4096 + 3, device="cuda") * 1e-3
    avg = E8GradientExchange(scale=500.0).all_reduce_mean(g)
    assert avg.shape == g.shape
    # typical per-value error is a fraction of a lattice unit (1/scale); rare blocks land on a
    # farther coset (reference semantics), so the check is on the median and on the total
    assert float((avg - g).abs().median()) < 0.5 / 500.0
    assert float((avg - g).norm() / g.norm()) < 1.0


def test_bounded_arrival_gives_up_and_guards_the_decode():
    """The cross-rank wait is bounded.  One GPU plays rank 0 of a two-rank world whose "peer" is a
    plain device array that nothing ever writes: the wait must run out, report the missing rank in
    the status word and leave the context usable; the decode that follows must then touch nothing.
    Once the peer's word is set the same calls pass and decode as the all-gather form does."""
    import ctypes
    from coset_b200 import _lib
    from coset_b200.gradcomm import CudaCodec
    L = _lib.lib()
    n, scale = 3000, 500.0
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(2)]
    fptr = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flags])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    codec = CudaCodec()
    gathered = torch.empty((2, n), dtype=torch.int32, device="cuda")
    for r in range(2):
        g = torch.Generator().manual_seed(50 + r)
        codec.encode((torch.randn(n, 8, generator=g) * 1e-3).cuda(), scale, gathered[r])
    cptr = (ctypes.c_void_p * 2)(*[gathered[r].data_ptr() for r in range(2)])
    out = torch.full((n, 8), -7.0, device="cuda")

    def arrive(epoch):
        rc = L.coset_peer_signal_wait(ctypes.cast(fptr, ctypes.c_void_p), 2, 0, epoch, 50, _lib.ptr(status), _lib.stream())
        assert rc == 0, L.coset_last_error_string()

    def decode():
        rc = L.coset_e8_decode_mean_peers(ctypes.cast(cptr, ctypes.c_void_p), 2, 0, n, scale, _lib.ptr(out), 0,
                                          _lib.ptr(status), _lib.stream())
        assert rc == 0, L.coset_last_error_string()

    arrive(1)
    decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 2                      # 1 + the rank that never arrived
    assert int(flags[0][0]) == 1 and int(flags[1][0]) == 1  # this rank did signal itself and its peer
    assert bool((out == -7.0).all())                    # the guarded decode wrote nothing
    status.zero_()
    flags[0][1] = 2                                     # "rank 1 has reached epoch 2"
    arrive(2)
    decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = torch.empty((n, 8), device="cuda")
    codec.decode_mean(gathered, 2, n, scale, want)
    assert torch.equal(out, want)
    assert L.coset_peer_signal_wait(ctypes.cast(fptr, ctypes.c_void_p), 17, 0, 1, 50, None, None) < 0


WORKER = r'''
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
from coset_b200.gradcomm import E8GradientExchange
from gradcomm_util import cpu_decode_mean
from oracle import oracle as O
n_values = 8 * 20000 + 6
g = torch.Generator().manual_seed(1000 + rank)
grad = torch.randn(n_values, generator=g) * 1e-3
avg = E8GradientExchange(scale=500.0).all_reduce_mean(grad.cuda())
torch.cuda.synchronize()
if rank == 0:
    digits = []
    for r in range(world):
        gg = torch.Generator().manual_seed(1000 + r)
        x = torch.randn(n_values, generator=gg) * 1e-3
        p = np.zeros(((n_values + 7) // 8) * 8, np.float32); p[:n_values] = x.numpy()
        digits.append(O.encode(p.reshape(-1, 8), beta=np.array([500.0], np.float32), scale_mode=2, blocks_per_tile=p.size // 8))
    want = cpu_decode_mean(digits, 500.0).reshape(-1)[:n_values]
    assert np.array_equal(avg.cpu().numpy(), want), "exchange differs from the CPU recipe"
    print("EXCHANGE_OK")
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_nccl_exchange(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29617", str(script), ROOT]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "EXCHANGE_OK" in res.stdout


DDP_WORKER = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn
sys.path.insert(0, sys.argv[1])
from coset_b200.gradcomm import E8GradientExchange, e8_allreduce_hook
rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
torch.manual_seed(0)
model = nn.Sequential(nn.Linear(64, 48), nn.Tanh(), nn.Linear(48, 10)).cuda()
ddp = nn.parallel.DistributedDataParallel(model, device_ids=[local])
ex = E8GradientExchange(scale=500.0)
ddp.register_comm_hook(ex, e8_allreduce_hook)
g = torch.Generator().manual_seed(100 + rank)
x = torch.randn(32, 64, generator=g).cuda()
loss = ddp(x).square().mean() * 0.01  # keeps every gradient inside the two-level code range at scale 500
loss.backward()
torch.cuda.synchronize()
flat = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
# every rank must hold the same bits
gathered = [torch.empty_like(flat) for _ in range(world)]
dist.all_gather(gathered, flat)
assert all(torch.equal(gathered[0], t) for t in gathered), "ranks disagree after the hook"
# and they must be close to the exact mean of the local gradients (quantisation step 0.5 / 500 per value)
plain = nn.Sequential(nn.Linear(64, 48), nn.Tanh(), nn.Linear(48, 10)).cuda()
plain.load_state_dict(model.state_dict())
(plain(x).square().mean() * 0.01).backward()
exact = torch.cat([p.grad.reshape(-1) for p in plain.parameters()])
dist.all_reduce(exact)
exact /= world
err = (flat - exact).abs()
assert float(exact.abs().max()) < 4.0 / 500.0, float(exact.abs().max())
assert float(err.max()) <= 1.5 / 500.0 + 1e-7, float(err.max())
if rank == 0:
    print("DDP_HOOK_OK")
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_ddp_comm_hook(tmp_path):
    script = tmp_path / "ddp_worker.py"
    script.write_text(DDP_WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29619", str(script), ROOT]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "DDP_HOOK_OK" in res.stdout


PEER_WORKER = r'''
import os, sys
import torch
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from coset_b200.gradcomm import E8GradientExchange
rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
via_nccl = E8GradientExchange(scale=500.0)
via_peer = E8GradientExchange(scale=500.0, transport="peer")
chunked = E8GradientExchange(scale=500.0, transport="peer", chunks=4)
chunked.CHUNK_MIN_BLOCKS = 4096  # cut these small gradients into pieces too: decode of piece k beside the encode of piece k+1
n_values = 8 * 50000 + 3
for it in range(6):  # several calls in a row: both halves of the double buffer are reused; two sizes alternate
    g = torch.Generator().manual_seed(1000 * it + rank)
    size = 8 * 777 if it % 2 == 0 else (n_values if it % 4 == 1 else 8 * 50000)  # the second call grows the symmetric allocation
    grad = (torch.randn(size, generator=g) * 1e-3).cuda()
    a = via_nccl.all_reduce_mean(grad)
    b = via_peer.all_reduce_mean(grad)
    torch.cuda.synchronize()
    assert torch.equal(a, b), f"transports differ at call {it}"
    c = chunked.all_reduce_mean(grad)
    torch.cuda.synchronize()
    assert torch.equal(a, c), f"chunked peer transport differs at call {it}"
    if grad.numel() % 8 == 0:  # in place: the decode of a piece overwrites values whose encode has finished
        inplace = grad.clone()
        chunked.all_reduce_mean(inplace, out=inplace)
        torch.cuda.synchronize()
        assert torch.equal(a, inplace), f"in-place chunked exchange differs at call {it}"
via_peer.check()
chunked.check()
dist.barrier()
if rank == 0:
    print("PEER_OK")
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_peer_memory_transport_equals_all_gather(tmp_path):
    """The exchange that decodes straight from the peers' buffers returns the bits of the all-gather form."""
    script = tmp_path / "peer_worker.py"
    script.write_text(PEER_WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29623", str(script), ROOT]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "PEER_OK" in res.stdout
