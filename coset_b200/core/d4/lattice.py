"""D4Lattice: integer points with an even coordinate sum (mirror of coset/core/d4/lattice.py and of
the Lattice base class, coset/core/base.py:63-292).

`projection` runs the CUDA kernel; the small helpers are elementwise torch ops whose float32
results do not depend on the device.
"""
import math
from typing import Optional

import torch

from ... import _lib
from ..e8.lattice import E8Lattice, _default_device

_G_ROWS = [[-1, -1, 0, 0], [1, -1, 0, 0], [0, 1, -1, 0], [0, 0, 1, -1]]
# torch.linalg.inv of the reference's G in float32 (exact)
_GINV = [[-0.5, -0.5, -0.5, -0.5], [0.5, -0.5, -0.5, -0.5], [0.0, 0.0, -1.0, -1.0], [0.0, 0.0, 0.0, -1.0]]


class D4Lattice(E8Lattice):
    """`G` has the basis vectors as columns (coset/core/d4/lattice.py:31-37).  Inherits the
    dimension-independent helpers (custom_round, g_x, encode_coords, decode_coords, compute_delta0);
    g_x has the same +1 / -1 rule in both reference lattices (d4/lattice.py:97-104)."""

    def __init__(self, device: Optional[torch.device] = None, config=None):
        self.device = _default_device(device)
        self.G = torch.tensor(_G_ROWS, dtype=torch.float32, device=self.device).T.contiguous()
        self.G_inv = torch.tensor(_GINV, dtype=torch.float32, device=self.device)
        self.name = "D4"
        self.d = 4
        self.config = config
        self.r_pack = 1.0 / math.sqrt(2)  # d4/lattice.py:39-49
        self.r_cov = 1.0  # d4/lattice.py:51-60

    def projection(self, x: torch.Tensor) -> torch.Tensor:
        """Reference-exact D4 point of every row of x ([4] or [N, 4], float32, CUDA)."""
        _lib.require_cuda(x, "x")
        if x.dtype != torch.float32:
            raise TypeError(f"projection expects float32, got {x.dtype}")
        squeeze = x.dim() == 1
        x2 = x.unsqueeze(0) if squeeze else x
        if x2.dim() != 2 or x2.shape[1] != 4:
            raise ValueError(f"Input dimension {tuple(x.shape)} doesn't match D4 dimension 4")
        x2 = x2.contiguous()
        y = torch.empty_like(x2)
        with torch.cuda.device(x2.device):
            rc = _lib.lib().coset_d4_projection(_lib.ptr(x2), x2.shape[0], _lib.ptr(y), _lib.stream())
        _lib.check(rc, "coset_d4_projection")
        return y.squeeze(0) if squeeze else y
