"""ctypes/numpy front-end of the CPU oracle (oracle/e8_oracle.c, oracle/d4_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's
CPU-baseline legs.  Nothing under coset_b200/ may import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libe8_oracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_u32p = ctypes.POINTER(ctypes.c_uint32)


def build(force=False):
    """Compile the C oracle with gcc (oracle/Makefile)."""
    srcs = [os.path.join(_HERE, f) for f in ("e8_oracle.c", "d4_oracle.c")]
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < max(os.path.getmtime(f) for f in srcs):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.e8o_custom_round.restype = ctypes.c_float
        _lib.e8o_custom_round.argtypes = [ctypes.c_float]
    return _lib


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def generators():
    g = np.empty((8, 8), np.float32)
    gi = np.empty((8, 8), np.float32)
    lib().e8o_generators(g.ctypes.data_as(_f32p), gi.ctypes.data_as(_f32p))
    return g, gi


def custom_round(x):
    x = np.asarray(x, np.float32)
    out = np.empty_like(x)
    L = lib()
    flat_in, flat_out = x.reshape(-1), out.reshape(-1)
    for i in range(flat_in.size):
        flat_out[i] = L.e8o_custom_round(float(flat_in[i]))
    return out


def _rows(fn, x, *extra):
    x, xp = _f32(x)
    assert x.shape[-1] == 8
    out = np.empty_like(x)
    flat = x.reshape(-1, 8)
    o = out.reshape(-1, 8)
    L = lib()
    f = getattr(L, fn)
    for i in range(flat.shape[0]):
        f(flat[i].ctypes.data_as(_f32p), *extra, o[i].ctypes.data_as(_f32p))
    return out


def g_x(x):
    return _rows("e8o_g_x", x)


def projection(x):
    return _rows("e8o_projection", x)


def encode_coords(p, q):
    return _rows("e8o_encode_coords", p, ctypes.c_int(q))


def decode_coords(b):
    return _rows("e8o_decode_coords", b)


def _beta_arg(beta, scale_mode):
    if scale_mode == 0 or beta is None:
        b = np.ones(1, np.float32)
    else:
        b = np.ascontiguousarray(np.atleast_1d(beta), dtype=np.float32).reshape(-1)
    return b, b.ctypes.data_as(_f32p)


def encode(x, beta=None, scale_mode=0, blocks_per_tile=1, q=4, M=2, threads=1):
    """-> float32 digits [n, M, 8], exactly what the reference's e8_encode returns."""
    x, xp = _f32(x)
    n = x.shape[0]
    b, bp = _beta_arg(beta, scale_mode)
    codes = np.empty((n, M, 8), np.float32)
    lib().e8o_encode_mt(xp, ctypes.c_int64(n), bp, scale_mode, ctypes.c_int64(blocks_per_tile), q, M,
                        codes.ctypes.data_as(_f32p), threads)
    return codes


def decode(codes, beta=None, scale_mode=0, blocks_per_tile=1, q=4, threads=1):
    codes, cp = _f32(codes)
    n, M, _ = codes.shape
    b, bp = _beta_arg(beta, scale_mode)
    out = np.empty((n, 8), np.float32)
    lib().e8o_decode_mt(cp, ctypes.c_int64(n), bp, scale_mode, ctypes.c_int64(blocks_per_tile), q, M,
                        out.ctypes.data_as(_f32p), threads)
    return out


def quantize(x, q=4):
    x, xp = _f32(x)
    out = np.empty_like(x)
    lib().e8o_quantize(xp, ctypes.c_int64(x.shape[0]), q, out.ctypes.data_as(_f32p))
    return out


def fake_quant(w_blocks, beta, blocks_per_tile, q=4, clip=2.0):
    """-> (clamped, unclipped) float32 [n, 8]."""
    w, wp = _f32(w_blocks)
    b, bp = _beta_arg(beta, 2)
    wq = np.empty_like(w)
    un = np.empty_like(w)
    lib().e8o_fake_quant(wp, ctypes.c_int64(w.shape[0]), bp, ctypes.c_int64(blocks_per_tile), q,
                         ctypes.c_float(clip), wq.ctypes.data_as(_f32p), un.ctypes.data_as(_f32p))
    return wq, un


def pack_q4(codes):
    """float digits [n, M<=2, 8] -> uint32 [n] in the CUDA library's packed layout."""
    codes, cp = _f32(codes)
    n, M, _ = codes.shape
    out = np.empty(n, np.uint32)
    lib().e8o_pack_q4(cp, ctypes.c_int64(n), M, out.ctypes.data_as(_u32p))
    return out


def codes_to_int(codes):
    """Reference digits are float32 and may be -0.0; compare them as integers."""
    return np.asarray(codes).astype(np.int64)


# ---- "ref" semantics (ref/hnlq.py, float64) ------------------------------------------------
# Tie-dither vector of ref/utils.py:309-324 for d = 8 (values produced by the reference itself).
TIE_DITHER = np.array([float.fromhex(h) for h in (
    "-0x1.254ab98a68347p-44", "0x1.8cacb9e24bcfep-43", "-0x1.c32c65ece7921p-43", "0x1.f24daf0aef791p-44",
    "-0x1.3977980135725p-43", "0x1.68dd78c4ef9e4p-44", "-0x1.422329c1bb29ap-42", "-0x1.e267a62230fccp-44")])

_f64p = ctypes.POINTER(ctypes.c_double)
_i32p = ctypes.POINTER(ctypes.c_int32)


def ref_encode(x, beta=1.0, alpha=1.0, q=4, M=2, overload=True, max_iter=10, dither=None):
    """-> (digits int32 [n, M, 8], T int32 [n]) as ref.hnlq.HNLQ.encode yields per vector."""
    x = np.ascontiguousarray(x, dtype=np.float64)
    n = x.shape[0]
    d = np.ascontiguousarray(TIE_DITHER if dither is None else dither, dtype=np.float64)
    digits = np.empty((n, M, 8), np.int32)
    T = np.empty(n, np.int32)
    lib().e8o_ref_encode(x.ctypes.data_as(_f64p), ctypes.c_int64(n), ctypes.c_double(beta), ctypes.c_double(alpha), q, M,
                         int(bool(overload)), max_iter, d.ctypes.data_as(_f64p), digits.ctypes.data_as(_i32p),
                         T.ctypes.data_as(_i32p))
    return digits, T


def ref_decode(digits, T, beta=1.0, alpha=1.0, q=4, dither=None, depth=None):
    """ref.hnlq.HNLQ.decode, or decode_coarse_to_fine(depth) when depth is given."""
    digits = np.ascontiguousarray(digits, dtype=np.int32)
    T = np.ascontiguousarray(T, dtype=np.int32)
    n, M, _ = digits.shape
    d = np.ascontiguousarray(TIE_DITHER if dither is None else dither, dtype=np.float64)
    out = np.empty((n, 8), np.float64)
    lib().e8o_ref_decode_depth(digits.ctypes.data_as(_i32p), T.ctypes.data_as(_i32p), ctypes.c_int64(n),
                               ctypes.c_double(beta), ctypes.c_double(alpha), q, M, M if depth is None else int(depth),
                               d.ctypes.data_as(_f64p), out.ctypes.data_as(_f64p))
    return out


# ---- D4 lattice path and Babai projection (oracle/d4_oracle.c)
def d4_projection(x):
    x, xp = _f32(x)
    out = np.empty_like(x)
    lib().d4o_projection_rows(xp, ctypes.c_int64(x.shape[0]), out.ctypes.data_as(_f32p))
    return out


def d4_g_x(x):
    x, xp = _f32(x)
    out = np.empty_like(x)
    lib().d4o_g_x_rows(xp, ctypes.c_int64(x.shape[0]), out.ctypes.data_as(_f32p))
    return out


def d4_fake_quant(w_blocks, beta, blocks_per_tile, clip=2.0):
    """-> (clamped, unclipped) float32 [n, 4]."""
    w, wp = _f32(w_blocks)
    b, bp = _beta_arg(beta, 2)
    wq = np.empty_like(w)
    un = np.empty_like(w)
    lib().d4o_fake_quant(wp, ctypes.c_int64(w.shape[0]), bp, ctypes.c_int64(blocks_per_tile), ctypes.c_float(clip),
                         wq.ctypes.data_as(_f32p), un.ctypes.data_as(_f32p))
    return wq, un


def babai(x, G, Ginv, step=1.0):
    """Babai rounding of the rows of x in the basis G (d x d, basis vectors as columns)."""
    x, xp = _f32(x)
    G, Gp = _f32(G)
    Gi, Gip = _f32(Ginv)
    out = np.empty_like(x)
    lib().lato_babai(xp, ctypes.c_int64(x.shape[0]), int(x.shape[1]), Gp, Gip, ctypes.c_float(step),
                     out.ctypes.data_as(_f32p))
    return out
