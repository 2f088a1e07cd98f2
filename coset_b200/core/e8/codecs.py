"""E8 HNLQ codec functions with the reference's signatures (coset/core/e8/codecs.py).

e8_encode / e8_decode / e8_quantize keep the reference's calling convention (float32 digits of
shape [N, M, 8]); e8_encode_packed / e8_decode_packed expose the library's packed format
(4 bytes per block for q=4, M=2), which is what the bandwidth figures are quoted on.
"""
from enum import Enum
from typing import Optional, Tuple

import torch

from ... import _lib
from .lattice import E8Lattice


def _as_blocks(x: torch.Tensor, name="x"):
    _lib.require_cuda(x, name)
    squeeze = x.dim() == 1
    x2 = x.unsqueeze(0) if squeeze else x
    if x2.dim() != 2:
        raise ValueError(f"{name} must be 1-D or 2-D, got {x.dim()} dimensions")  # reference: unpack error
    if x2.shape[1] != 8:
        raise ValueError(f"Input dimension {x2.shape[1]} doesn't match E8 dimension 8")
    return x2.contiguous(), squeeze


def _code_dtype(q: int, M: int):
    nbytes = _lib.lib().coset_e8_code_bytes(q, M)
    if nbytes == 0:
        raise ValueError(f"unsupported (q={q}, M={M}); the CUDA library handles 2 <= q <= 16, 1 <= M <= 8")
    return nbytes


def _scale_args(scale, scale_mode, n_blocks, blocks_per_tile, device):
    if scale_mode == _lib.SCALE_NONE or scale is None:
        return None, _lib.SCALE_NONE, 1
    if not isinstance(scale, torch.Tensor):
        scale = torch.tensor([float(scale)], dtype=torch.float32, device=device)
    _lib.require_cuda(scale, "scale")
    scale = scale.to(torch.float32).contiguous().view(-1)
    if scale_mode == _lib.SCALE_DIV_SCALAR:
        if scale.numel() != 1:
            raise ValueError("the codec (divide) convention takes one scalar beta")
    else:
        tiles = (n_blocks + blocks_per_tile - 1) // blocks_per_tile
        if scale.numel() != tiles:
            raise ValueError(f"expected {tiles} per-tile scales, got {scale.numel()}")
    return scale, scale_mode, blocks_per_tile


def e8_encode_packed(x: torch.Tensor, q: int = 4, M: int = 2, scale=None, scale_mode: int = _lib.SCALE_NONE,
                     blocks_per_tile: int = 1, out: Optional[torch.Tensor] = None,
                     literal: bool = False) -> torch.Tensor:
    """x [N, 8] float32/bfloat16 -> packed codes, uint8 tensor [N, code_bytes(q, M)].

    For q=4, M=2 the result can be viewed as int32 [N] (`codes.view(torch.int32)`).
    scale_mode: SCALE_DIV_SCALAR divides by one beta (codec convention); SCALE_MUL_TILE
    multiplies block b by scale[b // blocks_per_tile] (layer convention).
    literal=True forces the op-by-op search for every block (validation of the fast path).
    """
    x2, _ = _as_blocks(x)
    n = x2.shape[0]
    nbytes = _code_dtype(q, M)
    scale_t, mode, bpt = _scale_args(scale, scale_mode, n, blocks_per_tile, x2.device)
    if out is None:
        out = torch.empty((n, nbytes), dtype=torch.uint8, device=x2.device)
    elif out.numel() * out.element_size() != n * nbytes or not out.is_contiguous() or out.device != x2.device:
        raise ValueError("out has the wrong size, layout or device")
    with torch.cuda.device(x2.device):
        rc = _lib.lib().coset_e8_encode(_lib.ptr(x2), _lib.dtype_code(x2, "x"), _lib.ptr(scale_t), mode, n, bpt,
                                        q, M, _lib.SEM_CORE_LITERAL if literal else _lib.SEM_CORE, _lib.ptr(out),
                                        _lib.stream())
    _lib.check(rc, "coset_e8_encode")
    return out


def e8_decode_packed(codes: torch.Tensor, q: int = 4, M: int = 2, scale=None, scale_mode: int = _lib.SCALE_NONE,
                     blocks_per_tile: int = 1, dtype: torch.dtype = torch.float32,
                     out: Optional[torch.Tensor] = None, depth: Optional[int] = None) -> torch.Tensor:
    """packed codes (as produced by e8_encode_packed) -> reconstruction [N, 8].

    depth (1 .. M): coarse-to-fine reconstruction from the `depth` coarsest levels only, the
    float32 counterpart of ref/hnlq.py:447-507.  The residual of an all-zero level word is the
    zero vector, so the finer level words are cleared and the full decoder runs."""
    _lib.require_cuda(codes, "codes")
    nbytes = _code_dtype(q, M)
    total = codes.numel() * codes.element_size()
    if total % nbytes or not codes.is_contiguous():
        raise ValueError("codes is not a contiguous array of packed block codes")
    n = total // nbytes
    if depth is not None:
        if not (1 <= depth <= M):
            raise ValueError(f"depth must be between 1 and {M}, got {depth}")
        if depth < M:
            levels = codes.view(torch.uint8).reshape(n, M, nbytes // M).clone()
            levels[:, :M - depth] = 0
            codes = levels.view(-1)
    scale_t, mode, bpt = _scale_args(scale, scale_mode, n, blocks_per_tile, codes.device)
    if out is None:
        out = torch.empty((n, 8), dtype=dtype, device=codes.device)
    elif out.shape != (n, 8) or not out.is_contiguous() or out.device != codes.device:
        raise ValueError("out has the wrong shape, layout or device")
    with torch.cuda.device(codes.device):
        rc = _lib.lib().coset_e8_decode(_lib.ptr(codes), _lib.ptr(scale_t), mode, n, bpt, q, M, _lib.SEM_CORE,
                                        _lib.ptr(out), _lib.dtype_code(out, "out"), _lib.stream())
    _lib.check(rc, "coset_e8_decode")
    return out


def e8_encode(x: torch.Tensor, config, lattice=None, dither: Optional[torch.Tensor] = None,
              device: Optional[torch.device] = None) -> Tuple[torch.Tensor, int]:
    """Hierarchical E8 encoding (coset/core/e8/codecs.py:17-89).

    Returns (digits, 0): float32 digits in {0..q-1} of shape [N, M, 8] ([M, 8] for a 1-D input)
    and the reference's always-zero scaling count.  x must be float32 on a CUDA device.
    """
    if device is not None:
        x = x.to(device)
    x2, squeeze = _as_blocks(x)
    if x2.dtype != torch.float32:
        raise TypeError(f"e8_encode expects float32 like the reference; got {x2.dtype} "
                        "(use e8_encode_packed for bfloat16 input)")
    q, M, beta = int(config.q), int(config.M), float(config.beta)
    if getattr(config, "with_dither", False) and dither is not None:
        # codecs.py:64-69: x / beta + dither, then quantise without further scaling.  The
        # division uses a device tensor so that it is an IEEE division, as on the CPU.
        d = dither.to(x2.device)
        if d.dim() == 1:
            d = d.unsqueeze(0)
        xs = x2 / torch.tensor(beta, dtype=torch.float32, device=x2.device) + d
        packed = e8_encode_packed(xs.contiguous(), q, M)
    else:
        packed = e8_encode_packed(x2, q, M, scale=beta, scale_mode=_lib.SCALE_DIV_SCALAR)
    digits = torch.empty((x2.shape[0], M, 8), dtype=torch.float32, device=x2.device)
    with torch.cuda.device(x2.device):
        rc = _lib.lib().coset_e8_unpack_codes_f32(_lib.ptr(packed), x2.shape[0], q, M, _lib.ptr(digits), _lib.stream())
    _lib.check(rc, "coset_e8_unpack_codes_f32")
    if squeeze:
        digits = digits.squeeze(0)
    return digits, 0


class DecodingMethod(Enum):
    """Available decoding methods (coset/core/e8/codecs.py:92-96)."""

    FULL = "full"


def _decode_digits(b: torch.Tensor, config) -> torch.Tensor:
    _lib.require_cuda(b, "b")
    squeeze = b.dim() == 2
    b3 = b.unsqueeze(0) if squeeze else b
    if b3.dim() != 3 or b3.shape[2] != 8:
        raise ValueError(f"encoding vectors must have shape [N, M, 8] or [M, 8], got {tuple(b.shape)}")
    n, M, _ = b3.shape
    q, beta = int(config.q), float(config.beta)
    nbytes = _code_dtype(q, M)
    digits = b3.to(torch.float32).contiguous()
    packed = torch.empty((n, nbytes), dtype=torch.uint8, device=b3.device)
    with torch.cuda.device(b3.device):
        rc = _lib.lib().coset_e8_pack_codes_f32(_lib.ptr(digits), n, q, M, _lib.ptr(packed), _lib.stream())
    _lib.check(rc, "coset_e8_pack_codes_f32")
    out = e8_decode_packed(packed, q, M, scale=beta, scale_mode=_lib.SCALE_DIV_SCALAR)
    return out.squeeze(0) if squeeze else out


class E8Decoder:
    """Decoder object of the reference API (coset/core/e8/codecs.py:99-180)."""

    def __init__(self, device: Optional[torch.device] = None):
        self.device = device
        self.lattice = E8Lattice(device=device)

    def decode(self, b: torch.Tensor, config, method: DecodingMethod = DecodingMethod.FULL) -> torch.Tensor:
        if method == DecodingMethod.FULL:
            return _decode_digits(b, config)
        raise ValueError(f"Unknown decoding method: {method}. Only 'full' is currently supported.")


def e8_decode(b: torch.Tensor, config, method: str = "full", device: Optional[torch.device] = None) -> torch.Tensor:
    """Hierarchical E8 decoding (coset/core/e8/codecs.py:185-218); b holds digits [N, M, 8] or [M, 8]."""
    method_map = {"full": DecodingMethod.FULL}
    if method not in method_map:
        raise ValueError(f"Unknown decoding method: {method}. Available: {list(method_map.keys())}")
    if device is not None:
        b = b.to(device)
    return _decode_digits(b, config)


def e8_quantize(x: torch.Tensor, q: int, lattice: Optional[E8Lattice] = None) -> torch.Tensor:
    """decode(encode(x)) with M = 2 and beta = 1, as the reference hard-wires
    (coset/core/e8/codecs.py:221-286), in one fused kernel."""
    x2, squeeze = _as_blocks(x)
    _code_dtype(q, 2)
    out = torch.empty((x2.shape[0], 8), dtype=torch.float32, device=x2.device)
    with torch.cuda.device(x2.device):
        rc = _lib.lib().coset_e8_quantize(_lib.ptr(x2), _lib.dtype_code(x2, "x"), None, _lib.SCALE_NONE, x2.shape[0],
                                          1, q, 2, 0.0, _lib.ptr(out), _lib.DTYPE_F32, None, _lib.stream())
    _lib.check(rc, "coset_e8_quantize")
    return out.squeeze(0) if squeeze else out


def e8_quant_stats(x: torch.Tensor, scale=None, scale_mode: int = _lib.SCALE_NONE, blocks_per_tile: int = 1) -> dict:
    """Quantisation statistics of the q=4, M=2 codec over x [N, 8] in one pass: squared error and
    signal energy (scaled domain), overloaded blocks (the overload test of ref/hnlq.py:341 with
    the core search) and blocks with a non-zero code."""
    x2, _ = _as_blocks(x)
    n = x2.shape[0]
    scale_t, mode, bpt = _scale_args(scale, scale_mode, n, blocks_per_tile, x2.device)
    lib = _lib.lib()
    nbytes = lib.coset_e8_quant_stats_scratch_bytes(n)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x2.device)
    out = torch.empty(4, dtype=torch.float64, device=x2.device)
    with torch.cuda.device(x2.device):
        rc = lib.coset_e8_quant_stats(_lib.ptr(x2), _lib.dtype_code(x2, "x"), _lib.ptr(scale_t), mode, n, bpt,
                                      _lib.ptr(scratch), nbytes, _lib.ptr(out), _lib.stream())
    _lib.check(rc, "coset_e8_quant_stats")
    err2, overload, nonzero, sig2 = out.tolist()
    return {"squared_error": err2, "signal_energy": sig2, "overloaded_blocks": int(overload),
            "nonzero_blocks": int(nonzero), "n_blocks": n,
            "sqnr_db": float("inf") if err2 == 0 else 10.0 * __import__("math").log10(max(sig2, 1e-300) / err2)}
