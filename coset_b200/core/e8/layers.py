"""create_e8_hnlq_linear (mirror of coset/core/e8/layers.py:15-66)."""
import torch

from .lattice import E8Lattice
from .codecs import e8_quantize


def create_e8_hnlq_linear(in_dim, out_dim, device=None, **kwargs):
    """HNLQLinearQAT configured for the E8 lattice, with the reference's defaults."""
    from ..layers import HNLQLinearQAT

    if in_dim % 8 != 0:
        raise ValueError(f"Input dimension {in_dim} must be divisible by 8 for E8 lattice")
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    lattice = E8Lattice(device=device)
    defaults = {
        "lattice": lattice,
        "quantize_fn": e8_quantize,
        "block_size": 8,
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
