"""Host logic of the column-parallel code-domain linear layer on CPU ranks (gloo, world size 2):
the output-feature partition, the scale slice each rank takes and the all-gather layout.  The
device product is replaced by a dense CPU product of the oracle's reconstruction; the CUDA
kernels themselves are covered by the gpu tests."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
N_OUT, N_IN, T = 16, 64, 3


def _full_problem():
    g = torch.Generator().manual_seed(5)
    W = torch.randn(N_OUT, N_IN, generator=g) * 0.02
    beta = 20.0 + 10.0 * torch.rand(N_OUT * N_IN // 8, generator=g)
    x = torch.randn(T, N_IN, generator=g)
    return W, beta, x


def _oracle_dense(W, beta):
    from oracle import oracle as O
    b = beta.numpy().astype(np.float32)
    return torch.from_numpy(O.fake_quant(W.numpy().reshape(-1, 8), b, 1, 4, 1e30)[1].reshape(W.shape))


class _CpuLocal(torch.nn.Module):
    """Stand-in for E8CodeLinear: same attributes, dense product on the CPU."""

    def __init__(self, dense):
        super().__init__()
        self.dense = dense
        self.out_features, self.in_features = dense.shape

    def forward(self, x):
        return x @ self.dense.T


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, HERE)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coset_b200.vlut import ColumnParallelE8CodeLinear, out_feature_shard
    W, beta, x = _full_problem()
    lo, hi = out_feature_shard(N_OUT, world, rank)
    tiles_per_row = N_IN // 8
    local = _CpuLocal(_oracle_dense(W[lo:hi], beta[lo * tiles_per_row:hi * tiles_per_row]))
    lin = ColumnParallelE8CodeLinear(local, N_OUT)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), lin(x).numpy())
    dist.destroy_process_group()


def test_two_rank_column_parallel_matches_unsharded(tmp_path):
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got = [np.load(tmp_path / f"y{r}.npy") for r in range(2)]
    assert np.array_equal(got[0], got[1])
    W, beta, x = _full_problem()
    want = (x @ _oracle_dense(W, beta).T).numpy()
    assert got[0].shape == (T, N_OUT)
    assert np.allclose(got[0], want, rtol=0, atol=1e-6)


def test_partition_helpers():
    sys.path.insert(0, os.path.dirname(HERE))
    from coset_b200.vlut import assemble_gathered, out_feature_shard
    assert [out_feature_shard(12, 3, r) for r in range(3)] == [(0, 4), (4, 8), (8, 12)]
    with pytest.raises(ValueError):
        out_feature_shard(10, 4, 0)
    with pytest.raises(ValueError):
        out_feature_shard(8, 2, 2)
    g = torch.arange(2 * 3 * 4).reshape(2, 3, 4)
    full = assemble_gathered(g)
    assert full.shape == (3, 8)
    assert torch.equal(full[:, :4], g[0]) and torch.equal(full[:, 4:], g[1])
