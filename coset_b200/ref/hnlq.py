"""HNLQ: the E8 quantiser of ref/hnlq.py on the GPU (float64), batched.

`encode` / `decode` / `quantize` accept one vector `[8]` (returning what the reference returns:
a tuple of M integer vectors and T) or a batch `[N, 8]` (returning digits `[N, M, 8]` int32 and
T `[N]` int32).  Results are bit-identical to ref.hnlq.HNLQ run vector by vector.
"""
import ctypes
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from .. import _lib

# generate_tie_dither(8) of ref/utils.py:309-324 (float64 values as the reference computes them)
TIE_DITHER_E8 = tuple(float.fromhex(h) for h in (
    "-0x1.254ab98a68347p-44", "0x1.8cacb9e24bcfep-43", "-0x1.c32c65ece7921p-43", "0x1.f24daf0aef791p-44",
    "-0x1.3977980135725p-43", "0x1.68dd78c4ef9e4p-44", "-0x1.422329c1bb29ap-42", "-0x1.e267a62230fccp-44"))


@dataclass
class HNLQConfig:
    """Parameters of ref/hnlq.py:11-76 (same names, defaults and validation)."""

    lattice_type: str
    q: int
    M: int
    beta: float = 1.0
    alpha: float = 1.0
    eps: float = 1e-8
    overload: bool = True
    decoding: str = "full"
    max_scaling_iterations: int = 10
    with_tie_dither: bool = True
    with_dither: bool = False

    def __post_init__(self):
        if self.lattice_type != "E8":
            raise ValueError(f"Unsupported lattice type: {self.lattice_type} (this build implements E8)")
        if self.q <= 0:
            raise ValueError("Quantization parameter q must be positive")
        if self.beta <= 0:
            raise ValueError("Scaling parameter beta must be positive")
        if self.alpha <= 0:
            raise ValueError("Scaling parameter alpha must be positive")
        if self.M <= 0:
            raise ValueError("Number of hierarchical levels M must be positive")
        if self.max_scaling_iterations <= 0:
            raise ValueError("max_scaling_iterations must be positive")
        if self.decoding not in ["full", "coarse_to_fine", "progressive"]:
            raise ValueError(f"Unknown decoding method: {self.decoding}")


class HNLQ:
    def __init__(self, config: HNLQConfig, device=None):
        if isinstance(config, dict):
            config = HNLQConfig(**config)
        self.config = config
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        dither = TIE_DITHER_E8 if config.with_tie_dither else (config.eps,) * 8  # ref/hnlq.py:172-179
        self._dither = (ctypes.c_double * 8)(*dither)

    @classmethod
    def create_e8_quantizer(cls, q: int, M: int, beta: float = 1.0, alpha: float = 1.0, eps: float = 1e-8,
                            overload: bool = True, decoding: str = "full", with_tie_dither: bool = True,
                            with_dither: bool = False, device=None) -> "HNLQ":
        return cls(HNLQConfig("E8", q, M, beta, alpha, eps, overload, decoding, 10, with_tie_dither, with_dither), device)

    def _blocks(self, x):
        x = torch.as_tensor(x, dtype=torch.float64)
        single = x.dim() == 1
        x2 = x.reshape(1, -1) if single else x
        if x2.dim() != 2 or x2.shape[1] != 8:
            raise ValueError(f"expected [8] or [N, 8], got {tuple(x.shape)}")
        return x2.to(self.device).contiguous(), single

    def encode(self, x, with_dither: bool = False):
        """HNLQ.encode (ref/hnlq.py:344-383)."""
        if with_dither:
            raise NotImplementedError("subtractive dither is all-zero in the reference unless set by hand")
        x2, single = self._blocks(x)
        c = self.config
        n = x2.shape[0]
        digits = torch.empty((n, c.M, 8), dtype=torch.int32, device=self.device)
        T = torch.empty(n, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            rc = _lib.lib().coset_e8_ref_encode(_lib.ptr(x2), n, c.beta, c.alpha, c.q, c.M, int(c.overload),
                                                c.max_scaling_iterations, ctypes.cast(self._dither, ctypes.c_void_p),
                                                _lib.ptr(digits), _lib.ptr(T), _lib.stream())
        _lib.check(rc, "coset_e8_ref_encode")
        if single:
            return tuple(digits[0, m].cpu().numpy().astype(int) for m in range(c.M)), int(T[0])
        return digits, T

    def _decode_levels(self, b_list, T, depth):
        c = self.config
        single = not isinstance(b_list, torch.Tensor)
        if single:
            import numpy as np
            digits = torch.from_numpy(np.stack([np.asarray(b) for b in b_list]).astype("int32")).reshape(1, c.M, 8)
            Tt = torch.tensor([int(T)], dtype=torch.int32)
        else:
            digits, Tt = b_list, T
        digits = digits.to(self.device, torch.int32).contiguous()
        Tt = Tt.to(self.device, torch.int32).contiguous()
        n = digits.shape[0]
        out = torch.empty((n, 8), dtype=torch.float64, device=self.device)
        with torch.cuda.device(self.device):
            rc = _lib.lib().coset_e8_ref_decode_coarse(_lib.ptr(digits), _lib.ptr(Tt), n, c.beta, c.alpha, c.q, c.M,
                                                       int(depth), ctypes.cast(self._dither, ctypes.c_void_p),
                                                       _lib.ptr(out), _lib.stream())
        _lib.check(rc, "coset_e8_ref_decode_coarse")
        return out[0].cpu().numpy() if single else out

    def decode(self, b_list, T, with_dither: bool = False):
        """HNLQ.decode (ref/hnlq.py:422-445)."""
        if with_dither:
            raise NotImplementedError("subtractive dither is all-zero in the reference unless set by hand")
        return self._decode_levels(b_list, T, self.config.M)

    def decode_coarse_to_fine(self, b_list, T, with_dither: bool = False, depth: Optional[int] = None):
        """HNLQ.decode_coarse_to_fine (ref/hnlq.py:447-507): the `depth` coarsest levels only."""
        if with_dither:
            raise NotImplementedError("subtractive dither is all-zero in the reference unless set by hand")
        if depth is None:
            return self.decode(b_list, T, with_dither)
        if not (1 <= depth <= self.config.M):
            raise ValueError(f"depth must be between 1 and {self.config.M}, got {depth}")
        return self._decode_levels(b_list, T, depth)

    def decode_progressive(self, b_list, T, with_dither: bool = False) -> List:
        """HNLQ.decode_progressive (ref/hnlq.py:509-536): reconstructions for depth 1 .. M."""
        return [self.decode_coarse_to_fine(b_list, T, with_dither, level) for level in range(1, self.config.M + 1)]

    def get_default_decoding(self, b_list, T, with_dither: bool = False, depth: Optional[int] = None):
        """HNLQ.get_default_decoding (ref/hnlq.py:538-571): dispatch on config.decoding."""
        d = self.config.decoding
        if d == "full":
            return self.decode(b_list, T, with_dither)
        if d == "coarse_to_fine":
            return self.decode_coarse_to_fine(b_list, T, with_dither, depth=depth)
        if d == "progressive":
            return self.decode_progressive(b_list, T, with_dither)
        raise ValueError(f"Unknown decoding method: {d}")

    def decode_with_depth(self, b_list, T, depth: int, with_dither: bool = False):
        """HNLQ.decode_with_depth (ref/hnlq.py:573-601)."""
        if depth < 1 or depth > self.config.M:
            raise ValueError(f"Depth must be between 1 and {self.config.M}, got {depth}")
        return self.decode_coarse_to_fine(b_list, T, with_dither, depth)

    def quantize(self, x, with_dither: bool = False):
        """encode followed by decode (ref/hnlq.py:608-628)."""
        b, T = self.encode(x, with_dither)
        return self.decode(b, T, with_dither)
