"""create_d4_hnlq_linear (mirror of coset/core/d4/layers.py:15-68) and the fused D4 weight path."""
import torch

from ... import _lib
from .lattice import D4Lattice


def d4_quantize(x: torch.Tensor, q=None) -> torch.Tensor:
    """The layer's quantize_fn for D4: the lattice projection (coset/core/d4/layers.py:44-46; q is
    accepted and unused, as in the reference).  x: [..., 4] float32 on a CUDA device."""
    _lib.require_float32(x, "x")
    _lib.require_cuda(x, "x")
    if x.shape[-1] != 4:
        raise ValueError(f"Input dimension {tuple(x.shape)} doesn't match D4 dimension 4")
    x2 = x.reshape(-1, 4).contiguous()
    y = torch.empty_like(x2)
    with torch.cuda.device(x2.device):
        rc = _lib.lib().coset_d4_projection(_lib.ptr(x2), x2.shape[0], _lib.ptr(y), _lib.stream())
    _lib.check(rc, "coset_d4_projection")
    return y.view(x.shape)


class _D4FakeQuant(torch.autograd.Function):
    """clamp(projection(W * beta) / beta, +-clip) with the reference graph's gradients.

    forward : coset_d4_quantize (COSET_SCALE_MUL_TILE)
    backward: coset_d4_fake_quant_bwd -> dL/dW and dL/dbeta per tile
    """

    @staticmethod
    def forward(ctx, weight, beta, blocks_per_tile, clip, out_dtype):
        _lib.require_float32(weight, "weight")
        _lib.require_cuda(weight, "weight")
        w = weight.contiguous()
        b = beta.detach().to(torch.float32).contiguous().view(-1)
        n_blocks = w.numel() // 4
        out = torch.empty(w.shape, dtype=out_dtype, device=w.device)
        with torch.cuda.device(w.device):
            rc = _lib.lib().coset_d4_quantize(_lib.ptr(w), _lib.DTYPE_F32, _lib.ptr(b), _lib.SCALE_MUL_TILE, n_blocks,
                                              blocks_per_tile, float(clip), _lib.ptr(out), _lib.dtype_code(out, "out"),
                                              _lib.stream())
        _lib.check(rc, "coset_d4_quantize")
        ctx.save_for_backward(w, b)
        ctx.meta = (blocks_per_tile, float(clip), beta.shape)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        w, b = ctx.saved_tensors
        blocks_per_tile, clip, beta_shape = ctx.meta
        g = grad_out.contiguous()
        if g.dtype not in (torch.float32, torch.bfloat16):
            g = g.float()
        grad_w = torch.empty_like(w)
        need_beta = ctx.needs_input_grad[1]
        grad_beta = torch.empty_like(b) if need_beta else None
        with torch.cuda.device(w.device):
            rc = _lib.lib().coset_d4_fake_quant_bwd(_lib.ptr(g), _lib.dtype_code(g, "grad"), _lib.ptr(w), _lib.ptr(b),
                                                    w.numel() // 4, blocks_per_tile, clip, _lib.ptr(grad_w),
                                                    _lib.ptr(grad_beta), _lib.stream())
        _lib.check(rc, "coset_d4_fake_quant_bwd")
        return grad_w, (grad_beta.view(beta_shape) if need_beta else None), None, None, None


def d4_fake_quantize(weight, beta, blocks_per_tile, clip=2.0, out_dtype=torch.float32):
    """Differentiable fused D4 weight quantiser used by HNLQLinearQAT (see _D4FakeQuant)."""
    return _D4FakeQuant.apply(weight, beta, int(blocks_per_tile), float(clip), out_dtype)


def create_d4_hnlq_linear(in_dim, out_dim, device=None, **kwargs):
    """HNLQLinearQAT configured for the D4 lattice, with the reference's defaults."""
    from ..layers import HNLQLinearQAT

    if in_dim % 4 != 0:
        raise ValueError(f"Input dimension {in_dim} must be divisible by 4 for D4 lattice")
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    lattice = D4Lattice(device=device)
    defaults = {
        "lattice": lattice,
        "quantize_fn": d4_quantize,
        "block_size": 4,
        "q": 4,
        "M": 2,
        "Delta0": None,
        "warmup_epochs": 0,
        "enable_diagnostics": False,
        "weight_clip_value": 2.0,
        "theta_trainable": True,
        "theta_init_value": 0.0,
        "rho": 0.95,
    }
    defaults.update(kwargs)
    layer = HNLQLinearQAT(in_dim, out_dim, **defaults)
    return layer.to(device)
