"""Babai projection: rounding in the lattice basis (pub/main.tex, algorithm "Babai projection onto
E8"; weight path of ref/qat_auto.py:120-124).

    z = Ginv x,  z_hat = round(z / step) * step,  y = G z_hat

A cheaper, slightly less accurate stand-in for the closest-point search; `babai_quantize_ste` is the
straight-through form the reference's QAT-lite layer trains with (ste_round, ref/qat_auto.py:7).
"""
import ctypes

import torch

from .. import _lib


def babai_project(x: torch.Tensor, lattice, step: float = 1.0) -> torch.Tensor:
    """Rows of x ([d] or [N, d], float32, CUDA; d = lattice.d in {4, 8}) -> Babai point in `lattice`."""
    _lib.require_cuda(x, "x")
    if x.dtype != torch.float32:
        raise TypeError(f"babai_project expects float32, got {x.dtype}")
    d = int(lattice.d)
    if x.shape[-1] != d:
        raise ValueError(f"Input dimension {tuple(x.shape)} doesn't match {lattice.name} dimension {d}")
    x2 = x.reshape(-1, d).contiguous()
    y = torch.empty_like(x2)
    G = lattice.G.detach().to("cpu", torch.float32).contiguous()
    Gi = lattice.G_inv.detach().to("cpu", torch.float32).contiguous()
    with torch.cuda.device(x2.device):
        rc = _lib.lib().coset_lattice_babai(_lib.ptr(x2), x2.shape[0], d, ctypes.c_void_p(G.data_ptr()),
                                            ctypes.c_void_p(Gi.data_ptr()), float(step), _lib.ptr(y), _lib.stream())
    _lib.check(rc, "coset_lattice_babai")
    return y.view(x.shape)


class _BabaiSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, lattice, step):
        return babai_project(x, lattice, step)

    @staticmethod
    def backward(ctx, grad_out):
        # G ste_round(Ginv x / step) step has the gradient of G Ginv x = x
        return grad_out, None, None


def babai_quantize_ste(x: torch.Tensor, lattice, step: float = 1.0) -> torch.Tensor:
    """babai_project with the identity gradient of the reference's ste_round graph."""
    return _BabaiSTE.apply(x, lattice, float(step))
