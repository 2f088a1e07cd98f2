"""HNLQLinearQAT: quantisation-aware linear layer with hierarchical nested-lattice weights
(mirror of coset/core/layers.py; constructor arguments, buffers, state_dict keys and public
methods are the reference's).

What differs underneath: the weight path W -> clamp(e8_quantize(W * beta) / beta) is ONE fused
CUDA kernel (plus one for the straight-through backward) instead of ~250 small torch ops, the
step counter is mirrored on the host so a forward pass never synchronises the device, and
tiling='block' works (the reference raises at coset/core/layers.py:459).
"""
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib


def ste_round(x):
    """round() forward, identity backward (coset/core/layers.py:20-22)."""
    return (x - x.detach()) + torch.round(x).detach()


def ste_clip(x, min_val, max_val):
    """clamp() forward, identity backward (coset/core/layers.py:24-26)."""
    return (x - x.detach()) + torch.clamp(x, min_val, max_val).detach()


def get_generators(lattice):
    """(G, G_inv) of a lattice object (coset/core/layers.py:29-51)."""
    return lattice.get_generators()


class StraightThroughQuantize(torch.autograd.Function):
    """quantize_fn(x, q=q) forward, identity backward (coset/core/layers.py:62-95)."""

    @staticmethod
    def forward(ctx, x, quantize_fn, q):
        return quantize_fn(x, q=q)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None, None


def ste_quantize(x, quantize_fn, q):
    return StraightThroughQuantize.apply(x, quantize_fn, q)


class _E8FakeQuant(torch.autograd.Function):
    """clamp(e8_quantize(W * beta) / beta, +-clip) with the reference graph's gradients.

    forward : coset_e8_quantize (COSET_SCALE_MUL_TILE), also keeps the packed codes (4 B/block)
    backward: coset_e8_fake_quant_bwd -> dL/dW and dL/dbeta per tile
    """

    @staticmethod
    def forward(ctx, weight, beta, blocks_per_tile, q, clip, out_dtype):
        _lib.require_float32(weight, "weight")
        _lib.require_cuda(weight, "weight")
        w = weight.contiguous()
        b = beta.detach().to(torch.float32).contiguous().view(-1)
        n_blocks = w.numel() // 8
        lib = _lib.lib()
        code_bytes = lib.coset_e8_code_bytes(q, 2)
        if code_bytes == 0:
            raise ValueError(f"unsupported q={q} for the fused E8 weight quantiser (2 <= q <= 16)")
        codes = torch.empty((n_blocks, code_bytes), dtype=torch.uint8, device=w.device)
        out = torch.empty(w.shape, dtype=out_dtype, device=w.device)
        with torch.cuda.device(w.device):
            rc = lib.coset_e8_quantize(_lib.ptr(w), _lib.DTYPE_F32, _lib.ptr(b), _lib.SCALE_MUL_TILE, n_blocks,
                                       blocks_per_tile, q, 2, float(clip), _lib.ptr(out),
                                       _lib.dtype_code(out, "out"), _lib.ptr(codes), _lib.stream())
        _lib.check(rc, "coset_e8_quantize")
        ctx.save_for_backward(w, b, codes)
        ctx.meta = (blocks_per_tile, q, float(clip), beta.shape)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        w, b, codes = ctx.saved_tensors
        blocks_per_tile, q, clip, beta_shape = ctx.meta
        g = grad_out.contiguous()
        if g.dtype not in (torch.float32, torch.bfloat16):
            g = g.float()
        n_blocks = w.numel() // 8
        grad_w = torch.empty_like(w)
        need_beta = ctx.needs_input_grad[1]
        grad_beta = torch.empty_like(b) if need_beta else None
        with torch.cuda.device(w.device):
            rc = _lib.lib().coset_e8_fake_quant_bwd(_lib.ptr(g), _lib.dtype_code(g, "grad"), _lib.ptr(w),
                                                    _lib.ptr(codes), _lib.ptr(b), n_blocks, blocks_per_tile, q, clip,
                                                    _lib.ptr(grad_w), _lib.ptr(grad_beta), _lib.stream())
        _lib.check(rc, "coset_e8_fake_quant_bwd")
        return grad_w, (grad_beta.view(beta_shape) if need_beta else None), None, None, None, None


class _E8LayerFakeQuant(torch.autograd.Function):
    """The layer's whole weight path in one call each way: the per-tile scale
    beta = beta_min + sigmoid(theta) * (beta_max - beta_min) is computed on the device
    (coset_e8_layer_fake_quant_fwd), and the backward call returns dL/dW and dL/dtheta directly
    (coset_e8_layer_fake_quant_bwd), so no small torch kernels sit around the two CUDA kernels."""

    @staticmethod
    def forward(ctx, weight, theta, beta_min, beta_range, blocks_per_tile, q, clip, out_dtype):
        _lib.require_float32(weight, "weight")
        _lib.require_cuda(weight, "weight")
        w = weight.contiguous()
        th = theta.detach().to(torch.float32).contiguous().view(-1)
        n_blocks = w.numel() // 8
        lib = _lib.lib()
        code_bytes = lib.coset_e8_code_bytes(q, 2)
        if code_bytes == 0:
            raise ValueError(f"unsupported q={q} for the fused E8 weight quantiser (2 <= q <= 16)")
        codes = torch.empty((n_blocks, code_bytes), dtype=torch.uint8, device=w.device)
        out = torch.empty(w.shape, dtype=out_dtype, device=w.device)
        beta = torch.empty_like(th)
        with torch.cuda.device(w.device):
            rc = lib.coset_e8_layer_fake_quant_fwd(_lib.ptr(w), _lib.ptr(th), _lib.ptr(beta_min), _lib.ptr(beta_range), n_blocks,
                                                   blocks_per_tile, q, float(clip), _lib.ptr(out), _lib.dtype_code(out, "out"),
                                                   _lib.ptr(codes), _lib.ptr(beta), _lib.stream())
        _lib.check(rc, "coset_e8_layer_fake_quant_fwd")
        ctx.save_for_backward(w, th, beta, codes)
        # the bounds tensors are refreshed in place once every stat_update_interval steps (so that a captured
        # graph keeps reading them); kept outside save_for_backward, whose version check would turn a refresh
        # between this forward and its backward into an error
        ctx.beta_range = beta_range
        ctx.meta = (blocks_per_tile, q, float(clip), theta.shape)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        w, th, beta, codes = ctx.saved_tensors
        beta_range = ctx.beta_range
        blocks_per_tile, q, clip, theta_shape = ctx.meta
        g = grad_out.contiguous()
        if g.dtype not in (torch.float32, torch.bfloat16):
            g = g.float()
        grad_w = torch.empty_like(w)
        need_theta = ctx.needs_input_grad[1]
        grad_theta = torch.empty_like(th) if need_theta else None
        with torch.cuda.device(w.device):
            rc = _lib.lib().coset_e8_layer_fake_quant_bwd(_lib.ptr(g), _lib.dtype_code(g, "grad"), _lib.ptr(w), _lib.ptr(codes),
                                                          _lib.ptr(beta), _lib.ptr(th), _lib.ptr(beta_range), w.numel() // 8,
                                                          blocks_per_tile, q, clip, _lib.ptr(grad_w), _lib.ptr(grad_theta),
                                                          _lib.stream())
        _lib.check(rc, "coset_e8_layer_fake_quant_bwd")
        return grad_w, (grad_theta.view(theta_shape) if need_theta else None), None, None, None, None, None, None


def e8_fake_quantize(weight, beta, blocks_per_tile, q=4, clip=2.0, out_dtype=torch.float32):
    """Differentiable fused weight quantiser used by HNLQLinearQAT (see _E8FakeQuant)."""
    return _E8FakeQuant.apply(weight, beta, int(blocks_per_tile), int(q), float(clip), out_dtype)


class LSQActivation(nn.Module):
    """Learnable symmetric per-tensor activation quantiser (coset/core/layers.py:117-137)."""

    def __init__(self, bit_width: int = 8, init_alpha: float = 1.0):
        super().__init__()
        self.bit_width = bit_width
        self.qmax = 2 ** (bit_width - 1) - 1
        self.alpha = nn.Parameter(torch.tensor(init_alpha))

    def forward(self, x):
        alpha = torch.relu(self.alpha) + 1e-8
        scale = alpha / self.qmax
        return ste_round(ste_clip(x, -alpha, alpha) / scale) * scale


@dataclass
class HNLQConfig:
    """Plain parameter bundle kept for API compatibility (coset/core/layers.py:141-163)."""

    q: int = 4
    M: int = 2
    Delta0: float = 1.5
    eta: float = 0.1
    k: int = 1
    tiling: str = "row"
    block_size: int = 8
    quantize_activations: bool = False
    act_bit_width: int = 8
    act_init_alpha: float = 1.0
    init_method: str = "normal"
    init_kwargs: Dict[str, Any] = None

    def __post_init__(self):
        if self.init_kwargs is None:
            self.init_kwargs = {}
        if self.tiling not in ["row", "block"]:
            raise ValueError(f"tiling must be 'row' or 'block', got {self.tiling}")
        if self.block_size <= 0:
            raise ValueError(f"block_size must be positive, got {self.block_size}")


class HNLQLinearQAT(nn.Module):
    """Linear layer whose weights are fake-quantised to the E8 nested lattice during training.

    Arguments are those of the reference constructor (coset/core/layers.py:207-231).
    """

    def __init__(self, in_features: int, out_features: int, lattice, quantize_fn, q: int = 4, M: int = 2,
                 Delta0: Optional[float] = None, eta: float = 0.1, tiling: str = "row", block_size: int = 8,
                 quantize_activations: bool = False, act_bit_width: int = 8, act_init_alpha: float = 1.0,
                 init_method: str = "normal", init_kwargs: Optional[Dict[str, Any]] = None, bias: bool = True,
                 warmup_epochs: int = 0, enable_diagnostics: bool = False, weight_clip_value: float = 2.0,
                 theta_trainable: bool = True, theta_init_value: float = 0.0, rho: float = 0.95):
        super().__init__()
        if tiling not in ("row", "block"):
            raise ValueError(f"tiling must be 'row' or 'block', got {tiling}")
        if in_features % block_size != 0:
            raise ValueError(f"Input dimension {in_features} must be divisible by block_size {block_size}")
        self.in_features = in_features
        self.out_features = out_features
        self.quantize_fn = quantize_fn
        self.lattice = lattice
        self.lattice_type = lattice.name
        self.q = q
        self.M = M
        self.eta = eta
        self.tiling = tiling
        self.block_size = block_size
        self.quantize_activations = quantize_activations
        self.init_method = init_method
        self.init_kwargs = init_kwargs or {}
        self.theta_trainable = theta_trainable
        self.theta_init_value = theta_init_value
        self.rho = rho
        self.Delta0 = lattice.compute_delta0(q, M, rho) if Delta0 is None else Delta0

        G, Ginv = lattice.get_generators()
        self.register_buffer("G", G)
        self.register_buffer("Ginv", Ginv)
        self.blocks_per_row = in_features // block_size

        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self._initialize_weights()
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features))
        else:
            self.register_parameter("bias", None)

        tiles = out_features if tiling == "row" else out_features * self.blocks_per_row
        theta = torch.full((tiles,), float(theta_init_value))
        if theta_trainable:
            self.theta_beta = nn.Parameter(theta)
        else:
            self.register_buffer("theta_beta", theta)
        self.register_buffer("sigma_ema", torch.ones(tiles))
        self.register_buffer("xmax_ema", torch.ones(tiles))
        self.ema_momentum = 0.99
        self.stat_update_interval = 256
        self.register_buffer("step_count", torch.tensor(0, dtype=torch.long))
        self._step_host = 0  # host mirror of step_count: no device sync in forward
        self.register_buffer("gamma_inv", Ginv.abs().sum(dim=1).max())
        self._gamma_inv_host = float(Ginv.abs().sum(dim=1).max())

        self.actq = LSQActivation(act_bit_width, act_init_alpha) if quantize_activations else None

        self.warmup_epochs = warmup_epochs
        self.current_epoch = 0
        self.quantization_enabled = warmup_epochs == 0
        self.enable_diagnostics = enable_diagnostics
        self.weight_clip_value = weight_clip_value
        self._weight_history = [] if enable_diagnostics else None
        self._quantization_errors = [] if enable_diagnostics else None

        # The fused kernels implement the E8 and the D4 quantiser; any other quantize_fn runs op by op.
        from .d4.layers import d4_quantize as _fused_d4_fn
        from .e8.codecs import e8_quantize as _fused_fn
        self._fused = (quantize_fn is _fused_fn) and block_size == 8
        self._fused_d4 = (quantize_fn is _fused_d4_fn) and block_size == 4

    # ------------------------------------------------------------------ weights
    def _initialize_weights(self):
        m = self.init_method
        if m == "normal":
            nn.init.normal_(self.weight, **self.init_kwargs)
        elif m == "xavier":
            nn.init.xavier_normal_(self.weight, **self.init_kwargs)
        elif m == "kaiming":
            nn.init.kaiming_normal_(self.weight, **self.init_kwargs)
        elif m == "zeros":
            nn.init.zeros_(self.weight)
        elif m == "ones":
            nn.init.ones_(self.weight)
        elif m == "load":
            pass
        else:
            raise ValueError(f"Unknown init_method: {m}")

    def load_weights(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if weight.shape != (self.out_features, self.in_features):
            raise ValueError(f"Weight shape {weight.shape} doesn't match expected {(self.out_features, self.in_features)}")
        self.weight.data = weight.clone().to(self.weight.device)
        if bias is not None:
            if self.bias is None:
                raise ValueError("Cannot load bias: layer was initialized with bias=False")
            if bias.shape != (self.out_features,):
                raise ValueError(f"Bias shape {bias.shape} doesn't match expected {(self.out_features,)}")
            self.bias.data = bias.clone().to(self.bias.device)

    def load_from_linear(self, linear_layer: nn.Linear):
        if linear_layer.in_features != self.in_features:
            raise ValueError(f"Input features mismatch: {linear_layer.in_features} vs {self.in_features}")
        if linear_layer.out_features != self.out_features:
            raise ValueError(f"Output features mismatch: {linear_layer.out_features} vs {self.out_features}")
        self.load_weights(linear_layer.weight.data, linear_layer.bias.data if linear_layer.bias is not None else None)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        self._step_host = int(self._buffers["step_count"].item())

    def _sync_step_count(self):
        self._buffers["step_count"].fill_(self._step_host)

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        self._sync_step_count()
        super()._save_to_state_dict(destination, prefix, keep_vars)

    def __getattr__(self, name):
        if name == "step_count" and "step_count" in self.__dict__.get("_buffers", {}):
            # reading the buffer brings it up to date with the host-side counter
            buf = self.__dict__["_buffers"]["step_count"]
            buf.fill_(self.__dict__.get("_step_host", 0))
            return buf
        return super().__getattr__(name)

    # ------------------------------------------------------------------ scale bounds
    def _gather_stats(self, W_blocks):
        """EMA of per-tile std and abs-max (coset/core/layers.py:366-379)."""
        with torch.no_grad():
            m = self.ema_momentum
            if self.tiling == "row":
                sigma = W_blocks.std(dim=(1, 2)) + 1e-8
                xmax = W_blocks.abs().amax(dim=(1, 2)) + 1e-8
            else:
                sigma = W_blocks.std(dim=2).reshape(-1) + 1e-8
                xmax = W_blocks.abs().amax(dim=2).reshape(-1) + 1e-8
            self.sigma_ema.mul_(m).add_((1 - m) * sigma)
            self.xmax_ema.mul_(m).add_((1 - m) * xmax)

    def _bounds(self):
        """Adaptive (beta_min, beta_max) per tile (coset/core/layers.py:381-396).

        The bounds depend only on the two statistics buffers, which change once every 256 quantised
        forwards, so they are kept until one of the buffers is written (in place or replaced) or a
        hyper-parameter changes; the arithmetic and its order are the reference's."""
        key = (self.sigma_ema._version, self.xmax_ema._version, self.sigma_ema.data_ptr(), self.xmax_ema.data_ptr(),
               self.Delta0, self.eta, self.q, self.M)
        if getattr(self, "_bounds_key", None) != key:
            with torch.no_grad():
                qM = float(self.q ** self.M)
                ginv = self._gamma_inv_host
                beta_min = (self.Delta0 / qM) / (self.eta * ginv * self.sigma_ema)
                beta_max_det = (self.Delta0 * (qM - 1)) / (2 * ginv * self.xmax_ema)
                beta_max_prob = (self.Delta0 * (qM - 1)) / (2 * self.eta * ginv * self.sigma_ema)
                beta_max = torch.minimum(beta_max_det, beta_max_prob)
                beta_min = torch.minimum(beta_min, beta_max * 0.9)
                fresh = (beta_min, beta_max, beta_max - beta_min)
                old = getattr(self, "_bounds_cache", None)
                if old is not None and old[0].shape == beta_min.shape and old[0].device == beta_min.device:
                    # refreshed in place: a captured CUDA graph of the step keeps reading the same memory
                    for dst, src in zip(old, fresh):
                        dst.copy_(src)
                else:
                    self._bounds_cache = fresh
            self._bounds_key = key
        return self._bounds_cache[0], self._bounds_cache[1]

    def _beta(self):
        """beta = beta_min + sigmoid(theta) * (beta_max - beta_min) per tile (coset/core/layers.py:415-417),
        differentiable w.r.t. theta.  For CUDA parameters the forward value comes from the library's own
        kernel (coset_layer_beta), the same arithmetic the fused weight path uses, so that the scales a
        caller reads here are bit for bit the ones the weights were quantised with."""
        beta_min, _ = self._bounds()
        rng = self._bounds_cache[2]
        th = self.theta_beta
        soft = beta_min + torch.sigmoid(th) * rng
        if not th.is_cuda or th.dtype != torch.float32:
            return soft
        exact = torch.empty_like(beta_min)
        with torch.cuda.device(th.device):
            rc = _lib.lib().coset_layer_beta(_lib.ptr(th.detach().contiguous()), _lib.ptr(beta_min), _lib.ptr(rng), th.numel(),
                                             _lib.ptr(exact), _lib.stream())
        _lib.check(rc, "coset_layer_beta")
        return exact + (soft - soft.detach())  # value of the kernel, gradient of the torch expression

    # ------------------------------------------------------------------ quantised weights
    def _quantize_weights(self, out_dtype=torch.float32):
        W = self.weight
        if not self.quantization_enabled:
            if self.enable_diagnostics:
                self._weight_history.append(W.detach().clone())
            return W
        # the step counter lives on the host; the `step_count` buffer is brought up to date when it is
        # read (state_dict, int(layer.step_count) through the property below) -- one launch less per step
        self._step_host += 1
        if self._step_host % self.stat_update_interval == 0:
            self._sync_step_count()
            self._gather_stats(W.detach().view(self.out_features, self.blocks_per_row, self.block_size))
        bpt = self.blocks_per_row if self.tiling == "row" else 1
        if self._fused and W.is_cuda:
            beta_min, _ = self._bounds()
            W_q = _E8LayerFakeQuant.apply(W, self.theta_beta, beta_min, self._bounds_cache[2], bpt, int(self.q),
                                          float(self.weight_clip_value), out_dtype)
        elif self._fused_d4 and W.is_cuda:
            from .d4.layers import d4_fake_quantize
            W_q = d4_fake_quantize(W, self._beta(), bpt, self.weight_clip_value, out_dtype)
        elif self._fused or self._fused_d4:
            raise ValueError("HNLQLinearQAT with the E8 / D4 quantiser needs its parameters on a CUDA device "
                             "(coset_b200 has no CPU path); call .to('cuda')")
        else:
            W_q = self._quantize_weights_opwise(W, self._beta())
        if self.enable_diagnostics:
            self._weight_history.append(W.detach().clone())
            self._quantization_errors.append(torch.norm(W - W_q.float()).item())
        return W_q

    def _quantize_weights_opwise(self, W, beta):
        """Same graph as the reference for a user-supplied quantize_fn."""
        b3 = beta.view(self.out_features, -1, 1)
        Wb = W.view(self.out_features, self.blocks_per_row, self.block_size) * b3
        Wq = ste_quantize(Wb.reshape(-1, self.block_size), self.quantize_fn, self.q)
        Wq = Wq.view(self.out_features, self.blocks_per_row, self.block_size) / b3
        return torch.clamp(Wq.reshape(self.out_features, self.in_features), -self.weight_clip_value, self.weight_clip_value)

    def forward(self, x):
        low = x.dtype == torch.bfloat16
        W_q = self._quantize_weights(torch.bfloat16 if low else torch.float32)
        bias = self.bias
        if low:
            if W_q.dtype != torch.bfloat16:  # warm-up (dense weights) or a user-supplied quantiser
                W_q = W_q.to(torch.bfloat16)
            bias = bias.to(torch.bfloat16) if bias is not None else None
        x = F.linear(x, W_q, bias)
        if self.quantize_activations and self.actq is not None:
            x = self.actq(x)
        return x

    # ------------------------------------------------------------------ cold start control
    def update_epoch(self, epoch: int):
        self.current_epoch = epoch
        if epoch >= self.warmup_epochs and not self.quantization_enabled:
            self.quantization_enabled = True
            print(f"Epoch {epoch}: Enabling quantization (warmup complete)")

    def enable_quantization(self):
        self.quantization_enabled = True
        print("Quantization manually enabled")

    def disable_quantization(self):
        self.quantization_enabled = False
        print("Quantization manually disabled")

    def is_quantization_enabled(self) -> bool:
        return self.quantization_enabled

    # ------------------------------------------------------------------ diagnostics
    def get_weight_quantiles(self, quantiles: List[float] = None) -> torch.Tensor:
        if quantiles is None:
            quantiles = [0.0, 0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9, 1.0]
        W = self.weight.detach().flatten()
        return torch.quantile(W, torch.tensor(quantiles, device=W.device))

    def get_weight_statistics(self) -> Dict[str, float]:
        W = self.weight.detach()
        return {"mean": W.mean().item(), "std": W.std().item(), "min": W.min().item(), "max": W.max().item(),
                "median": W.median().item(), "l2_norm": torch.norm(W).item(), "l1_norm": torch.norm(W, p=1).item()}

    def _quantized_detached(self):
        with torch.no_grad():
            return self._quantize_weights().detach().float()

    def get_quantization_error(self) -> float:
        if not self.quantization_enabled:
            return 0.0
        return torch.norm(self.weight.detach() - self._quantized_detached()).item()

    def get_scaling_factors(self) -> torch.Tensor:
        return self.theta_beta.detach()

    def get_quantization_histogram(self, bins: int = 50) -> Tuple[torch.Tensor, torch.Tensor]:
        W = self.weight.detach() if not self.quantization_enabled else self._quantized_detached()
        return torch.histogram(W.flatten().cpu(), bins=bins)

    def get_sparsity_ratio(self, threshold: float = 1e-6) -> float:
        return (self.weight.detach().abs() < threshold).float().mean().item()

    def get_effective_bits(self) -> float:
        if not self.quantization_enabled:
            return 32.0
        n = torch.unique(self._quantized_detached()).numel()
        return torch.log2(torch.tensor(n, dtype=torch.float32)).item()

    def compare_weights(self) -> Dict[str, float]:
        if not self.quantization_enabled:
            return {"error": 0.0, "relative_error": 0.0, "cosine_similarity": 1.0}
        W, Wq = self.weight.detach(), self._quantized_detached()
        err = torch.norm(W - Wq).item()
        return {"error": err, "relative_error": err / torch.norm(W).item(),
                "cosine_similarity": F.cosine_similarity(W.flatten(), Wq.flatten(), dim=0).item()}

    def get_weight_clipping_stats(self) -> Dict[str, float]:
        W = self.weight.detach()
        clipped = torch.sum((W.abs() > self.weight_clip_value).float()).item()
        return {"clipping_ratio": clipped / W.numel(), "clipped_count": clipped, "total_count": W.numel(),
                "clip_value": self.weight_clip_value, "max_weight": W.abs().max().item()}

    def get_diagnostic_summary(self) -> Dict[str, Any]:
        summary = {
            "epoch": self.current_epoch,
            "quantization_enabled": self.quantization_enabled,
            "warmup_epochs": self.warmup_epochs,
            "weight_stats": self.get_weight_statistics(),
            "quantization_error": self.get_quantization_error(),
            "effective_bits": self.get_effective_bits(),
            "sparsity_ratio": self.get_sparsity_ratio(),
            "weight_clipping": self.get_weight_clipping_stats(),
        }
        if self.quantization_enabled:
            summary["weight_comparison"] = self.compare_weights()
        return summary

    def export_quantized(self, packed: bool = False):
        """Dense fake-quantised weights + metadata, as the reference returns them
        (coset/core/layers.py:620-650).

        packed=True (q = 4 with the E8 quantiser only): instead of the dense float weights, the packed
        two-level E8 codes (int32 [out_features, in_features / 8], 4 bytes per 8 weights), the scales
        beta, blocks_per_tile, the bias and metadata including weight_clip_value -- everything
        coset_b200.vlut.E8CodeLinear.from_exported needs to compute clamp(decode(codes) / beta) @ x."""
        with torch.no_grad():
            metadata = {"lattice_type": self.lattice_type, "q": self.q, "M": self.M, "Delta0": self.Delta0,
                        "tiling": self.tiling, "block_size": self.block_size,
                        "quantize_activations": self.quantize_activations}
            if self.quantize_activations and self.actq is not None:
                metadata.update({"act_bit_width": self.actq.bit_width, "act_alpha": self.actq.alpha.item()})
            if not packed:
                return {"weight": self._quantize_weights(), "bias": self.bias, "metadata": metadata}
            if not (self._fused and self.q == 4):
                raise ValueError("packed export stores q=4 two-level E8 codes; this layer uses "
                                 f"lattice {self.lattice_type}, q={self.q}")
            from .e8.codecs import e8_encode_packed
            _lib.require_float32(self.weight, "weight")
            beta = self._beta().detach().to(torch.float32).contiguous()
            bpt = self.blocks_per_row if self.tiling == "row" else 1
            codes = e8_encode_packed(self.weight.detach().contiguous().view(-1, 8), 4, 2, scale=beta.view(-1),
                                     scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=bpt)
            metadata.update({"packed_M": 2, "weight_clip_value": float(self.weight_clip_value),
                             "code_layout": "uint32 per block: level m digit j at bit 16 m + 2 j"})
            return {"codes": codes.view(torch.int32).view(self.out_features, self.blocks_per_row), "beta": beta,
                    "blocks_per_tile": bpt, "bias": self.bias.detach().clone() if self.bias is not None else None,
                    "metadata": metadata}

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"lattice_type={self.lattice_type}, q={self.q}, M={self.M}, "
                f"Delta0={self.Delta0:.4f}, tiling={self.tiling}, block_size={self.block_size}, "
                f"quantize_activations={self.quantize_activations}, bias={self.bias is not None}, "
                f"theta_trainable={self.theta_trainable}, theta_init_value={self.theta_init_value}, "
                f"rho={self.rho}")


HNLQLinear = HNLQLinearQAT


class GraphedTrainStep:
    """Forward + loss + backward of a module with HNLQLinearQAT layers as ONE CUDA graph.

    An eager step of a small layer is bound by the Python and launch path (about 0.5 ms for the
    [3072, 768] layer with 4096 tokens, against 0.24 ms of device work); the layers' kernels only enqueue
    work on the current stream, so the whole step can be captured once and replayed.  What a replay skips
    is the layers' host-side bookkeeping, which this wrapper performs itself before every replay: the
    quantised-forward counter and, every `stat_update_interval` steps, the EMA statistics update
    (coset/core/layers.py:409-413), whose new scale bounds are written in place into the tensors the
    captured kernels read.

        step = GraphedTrainStep(model, loss_fn, example_inputs)   # loss_fn(model_output, *extra) -> scalar
        loss = step(x, target)                                     # gradients are in p.grad afterwards

    The inputs of every call must have the shapes and dtypes of the examples.  Gradients are rewritten
    (not accumulated) by every replay; read or apply them before the next call."""

    def __init__(self, module: nn.Module, loss_fn, example_inputs, warmup: int = 3):
        self.module, self.loss_fn = module, loss_fn
        self.layers = [m for m in module.modules() if isinstance(m, HNLQLinearQAT)]
        self.static = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # warm-up outside the capture: lazy initialisation, allocator, autotuning
            for _ in range(warmup):
                module.zero_grad(set_to_none=True)
                self._run().backward()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        steps = [l._step_host for l in self.layers]
        module.zero_grad(set_to_none=True)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = self._run()
            self.loss.backward()
        for l, n in zip(self.layers, steps):  # neither the warm-up nor the capture is a training step
            l._step_host = n - warmup if n >= warmup else 0

    def _run(self):
        return self.loss_fn(self.module(self.static[0]), *self.static[1:])

    def __call__(self, *inputs):
        for dst, src in zip(self.static, inputs):
            dst.copy_(src)
        for l in self.layers:
            if l.quantization_enabled:
                l._step_host += 1
                if l._step_host % l.stat_update_interval == 0:
                    l._sync_step_count()
                    l._gather_stats(l.weight.detach().view(l.out_features, l.blocks_per_row, l.block_size))
                    l._bounds()  # refreshes the bounds in place for the captured kernels
        self.graph.replay()
        return self.loss

