"""Host logic of the E8 gradient exchange on CPU ranks (gloo, world size 2): padding, gather
layout, averaging recipe.  The device codec is replaced by the oracle-backed stand-in; the CUDA
kernels themselves are covered by the gpu tests."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _worker(rank, world, port, n_values, out_dir):
    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, HERE)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coset_b200.gradcomm import E8GradientExchange
    from gradcomm_util import OracleCodec
    g = torch.Generator().manual_seed(1000 + rank)
    grad = torch.randn(n_values, generator=g) * 1e-3
    ex = E8GradientExchange(scale=500.0, codec=OracleCodec())
    avg = ex.all_reduce_mean(grad)
    np.save(os.path.join(out_dir, f"avg{rank}.npy"), avg.numpy())
    dist.destroy_process_group()


def test_two_rank_exchange_matches_single_process_recipe(tmp_path):
    from oracle import oracle as O
    from gradcomm_util import cpu_decode_mean
    world, n_values = 2, 8 * 1000 + 5  # ragged tail: padded with zeros and stripped
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, n_values, str(tmp_path)), nprocs=world, join=True)
    got = [np.load(tmp_path / f"avg{r}.npy") for r in range(world)]
    assert np.array_equal(got[0], got[1])  # every rank holds the same bits
    codes = []
    grads = []
    for r in range(world):
        g = torch.Generator().manual_seed(1000 + r)
        grad = torch.randn(n_values, generator=g) * 1e-3
        grads.append(grad.numpy())
        padded = np.zeros(((n_values + 7) // 8) * 8, np.float32)
        padded[:n_values] = grad.numpy()
        codes.append(O.encode(padded.reshape(-1, 8), beta=np.array([500.0], np.float32), scale_mode=2,
                              blocks_per_tile=padded.size // 8))
    want = cpu_decode_mean(codes, 500.0).reshape(-1)[:n_values]
    assert np.array_equal(got[0], want)
    true_mean = (grads[0] + grads[1]) / 2
    # per-value error: at most 1.5 lattice units (the reference flip rule can move a coordinate
    # away from the input), i.e. 1.5 / scale, averaged over the ranks
    assert np.median(np.abs(got[0] - true_mean)) < 0.5 / 500.0
    rel = np.linalg.norm(got[0] - true_mean) / np.linalg.norm(true_mean)
    assert rel < 1.0, rel


def test_single_process_without_process_group():
    sys.path.insert(0, HERE)
    from coset_b200.gradcomm import E8GradientExchange
    from gradcomm_util import OracleCodec
    grad = torch.randn(64) * 1e-3
    avg = E8GradientExchange(scale=500.0, codec=OracleCodec()).all_reduce_mean(grad)
    assert avg.shape == grad.shape
    assert float((avg - grad).abs().median()) < 0.5 / 500.0


def _ddp_worker(rank, world, port, out_dir):
    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, HERE)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torch.nn as nn
    from coset_b200.gradcomm import E8GradientExchange, e8_allreduce_hook
    from gradcomm_util import OracleCodec
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 12), nn.Tanh(), nn.Linear(12, 3))
    ddp = nn.parallel.DistributedDataParallel(model)
    ddp.register_comm_hook(E8GradientExchange(scale=500.0, codec=OracleCodec()), e8_allreduce_hook)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(8, 16, generator=g)
    (ddp(x).square().mean() * 0.01).backward()
    flat = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
    plain = nn.Sequential(nn.Linear(16, 12), nn.Tanh(), nn.Linear(12, 3))
    plain.load_state_dict(model.state_dict())
    (plain(x).square().mean() * 0.01).backward()
    exact = torch.cat([p.grad.reshape(-1) for p in plain.parameters()])
    dist.all_reduce(exact)
    exact /= world
    np.save(os.path.join(out_dir, f"ddp{rank}.npy"), np.stack([flat.numpy(), exact.numpy()]))
    dist.destroy_process_group()


def test_ddp_comm_hook_on_cpu_ranks(tmp_path):
    """The hook registered on a real DistributedDataParallel module (gloo): DDP accepts its
    signature, every rank ends with the same gradient, close to the exact mean."""
    port = 33500 + (os.getpid() % 2000)
    mp.spawn(_ddp_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got = [np.load(tmp_path / f"ddp{r}.npy") for r in range(2)]
    assert np.array_equal(got[0][0], got[1][0])
    err = np.abs(got[0][0] - got[0][1])
    assert err.max() <= 1.5 / 500.0 + 1e-7, err.max()
    assert np.abs(got[0][1]).max() < 4.0 / 500.0  # the gradients stay inside the code range
