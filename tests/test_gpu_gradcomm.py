"""E8 gradient exchange on the GPU: the decode-and-average kernel against the CPU recipe, and
the NCCL exchange on 2 GPUs (skipped when only one is visible)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import bits
from gradcomm_util import cpu_decode_mean
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
        d = O.encode(grad.numpy(), beta=np.array([scale], np.float32), scale_mode=2, blocks_per_tile=n)
        assert np.array_equal(gathered[r].cpu().numpy().view(np.uint32), O.pack_q4(d))
        digits.append(d)
    out = torch.empty((n, 8), device="cuda")
    codec.decode_mean(gathered, world, n, scale, out)
    assert np.array_equal(bits(out.cpu().numpy()), bits(cpu_decode_mean(digits, scale)))


def test_single_gpu_exchange_roundtrip():
    from coset_b200.gradcomm import E8GradientExchange
    g = torch.randn(8 * 4096 + 3, device="cuda") * 1e-3
    avg = E8GradientExchange(scale=500.0).all_reduce_mean(g)
    assert avg.shape == g.shape
    # typical per-value error is a fraction of a lattice unit (1/scale); rare blocks land on a
    # farther coset (reference semantics), so the check is on the median and on the total
    assert float((avg - g).abs().median()) < 0.5 / 500.0
    assert float((avg - g).norm() / g.norm()) < 1.0


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
n_values = 8 * 50000 + 3
for it in range(6):  # several calls in a row: both halves of the double buffer are reused; two sizes alternate
    g = torch.Generator().manual_seed(1000 * it + rank)
    grad = (torch.randn(n_values if it % 2 == 0 else 8 * 777, generator=g) * 1e-3).cuda()
    a = via_nccl.all_reduce_mean(grad)
    b = via_peer.all_reduce_mean(grad)
    torch.cuda.synchronize()
    assert torch.equal(a, b), f"transports differ at call {it}"
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
