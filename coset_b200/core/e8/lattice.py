"""E8Lattice: generator matrix, geometric constants and the closest-point search
(mirror of coset/core/e8/lattice.py and of the Lattice base class, coset/core/base.py:63-292).

`projection` runs the CUDA kernel; the small helpers (custom_round, g_x, encode_coords,
decode_coords) are written with elementwise torch ops whose float32 results do not depend on
the device.
"""
import math
from typing import Optional

import torch

from ... import _lib

_G_ROWS = [
    [2, 0, 0, 0, 0, 0, 0, 0],
    [-1, 1, 0, 0, 0, 0, 0, 0],
    [0, -1, 1, 0, 0, 0, 0, 0],
    [0, 0, -1, 1, 0, 0, 0, 0],
    [0, 0, 0, -1, 1, 0, 0, 0],
    [0, 0, 0, 0, -1, 1, 0, 0],
    [0, 0, 0, 0, 0, -1, 1, 0],
    [0.5, 0.5, 0.5, 0.5, 0.5, 0.5, 0.5, 0.5],
]
# Exact inverse of G (the float32 result of torch.linalg.inv on the reference's G).
_GINV = [
    [0.5, 0.5, 0.5, 0.5, 0.5, 0.5, 0.5, -3.5],
    [0, 1, 1, 1, 1, 1, 1, -6],
    [0, 0, 1, 1, 1, 1, 1, -5],
    [0, 0, 0, 1, 1, 1, 1, -4],
    [0, 0, 0, 0, 1, 1, 1, -3],
    [0, 0, 0, 0, 0, 1, 1, -2],
    [0, 0, 0, 0, 0, 0, 1, -1],
    [0, 0, 0, 0, 0, 0, 0, 2],
]


def _default_device(device):
    if device is None:
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return torch.device(device)


class E8Lattice:
    """E8 = D8 u (D8 + 1/2).  `G` has the basis vectors as columns (lattice.py:32-41)."""

    def __init__(self, device: Optional[torch.device] = None, config=None):
        self.device = _default_device(device)
        self.G = torch.tensor(_G_ROWS, dtype=torch.float32, device=self.device).T.contiguous()
        self.G_inv = torch.tensor(_GINV, dtype=torch.float32, device=self.device)
        self.name = "E8"
        self.d = 8
        self.config = config
        self.r_pack = 0.5  # lattice.py:44-54
        self.r_cov = math.sqrt(2) / 2  # lattice.py:56-65

    def get_generators(self):
        return self.G.clone().detach(), self.G_inv.clone().detach()

    def compute_delta0(self, q: int, M: int, rho: float = 0.95) -> float:
        """Delta0 = 2 rho r_pack / (q^M - 1)   (base.py:270-284)."""
        return (2.0 * rho * self.r_pack) / (q ** M - 1)

    # ---- elementwise helpers (base.py:179-202, lattice.py:67-112, base.py:134-176)
    def custom_round(self, x: torch.Tensor, tiny: Optional[float] = None) -> torch.Tensor:
        if tiny is None:
            tiny = torch.finfo(x.dtype if x.dtype.is_floating_point else torch.float32).eps
        y = x - torch.sign(x) * tiny
        return torch.floor(y + 0.5)

    def g_x(self, x: torch.Tensor) -> torch.Tensor:
        squeeze = x.dim() == 1
        if squeeze:
            x = x.unsqueeze(0)
        f = self.custom_round(x)
        k = torch.argmax(torch.abs(x - f), dim=-1, keepdim=True)
        xk = torch.gather(x, -1, k)
        fk = torch.gather(f, -1, k)
        up = (xk >= 0) & (fk < xk)
        step = torch.where(up, torch.ones_like(fk), -torch.ones_like(fk))
        out = f.scatter(-1, k, fk + step)
        return out.squeeze(0) if squeeze else out

    def encode_coords(self, x: torch.Tensor, q: int) -> torch.Tensor:
        G_inv = self.G_inv.to(x.device)
        if x.dim() == 1:
            return torch.round(torch.matmul(G_inv, x)) % q
        return torch.round(torch.matmul(G_inv, x.T)).T % q

    def decode_coords(self, b: torch.Tensor, q: int) -> torch.Tensor:
        G = self.G.to(b.device)
        if b.dim() == 1:
            return torch.matmul(G, b.float())
        return torch.matmul(G, b.float().T).T

    # ---- the search itself
    def projection(self, x: torch.Tensor) -> torch.Tensor:
        """Reference-exact E8 'closest' point of every row of x ([8] or [N, 8], float32, CUDA)."""
        _lib.require_cuda(x, "x")
        if x.dtype != torch.float32:
            raise TypeError(f"projection expects float32, got {x.dtype}")
        squeeze = x.dim() == 1
        x2 = x.unsqueeze(0) if squeeze else x
        if x2.dim() != 2 or x2.shape[1] != 8:
            raise ValueError(f"Input dimension {tuple(x.shape)} doesn't match E8 dimension 8")
        x2 = x2.contiguous()
        y = torch.empty_like(x2)
        with torch.cuda.device(x2.device):
            rc = _lib.lib().coset_e8_projection(_lib.ptr(x2), x2.shape[0], _lib.ptr(y), _lib.stream())
        _lib.check(rc, "coset_e8_projection")
        return y.squeeze(0) if squeeze else y

    def __repr__(self) -> str:
        return f"{self.name}Lattice(d={self.d})"

    __str__ = __repr__
