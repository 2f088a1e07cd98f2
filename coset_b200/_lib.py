"""ctypes binding of libcoset_b200.so, the C-ABI CUDA library.

There is no CPU fallback: if the library is missing or a tensor is not on a CUDA device the
call fails loudly.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libcoset_b200.so")

DTYPE_F32, DTYPE_BF16 = 0, 1
SCALE_NONE, SCALE_DIV_SCALAR, SCALE_MUL_TILE = 0, 1, 2
SEM_CORE, SEM_REF, SEM_CORE_LITERAL, SEM_CORE_SATURATE = 0, 1, 2, 3

_lib = None

_vp, _i64, _i32, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float

# name -> argtypes; every symbol declared in include/coset_b200.h
SIGNATURES = {
    "coset_version": [],
    "coset_last_error_string": [],
    "coset_e8_code_bytes": [_i32, _i32],
    "coset_e8_projection": [_vp, _i64, _vp, _vp],
    "coset_e8_encode": [_vp, _i32, _vp, _i32, _i64, _i64, _i32, _i32, _i32, _vp, _vp],
    "coset_e8_decode": [_vp, _vp, _i32, _i64, _i64, _i32, _i32, _i32, _vp, _i32, _vp],
    "coset_e8_quantize": [_vp, _i32, _vp, _i32, _i64, _i64, _i32, _i32, _f32, _vp, _i32, _vp, _vp],
    "coset_e8_unpack_codes_f32": [_vp, _i64, _i32, _i32, _vp, _vp],
    "coset_e8_pack_codes_f32": [_vp, _i64, _i32, _i32, _vp, _vp],
    "coset_host_ctx_create": [_i64, _i32, ctypes.POINTER(ctypes.c_void_p)],
    "coset_host_ctx_destroy": [_vp],
    "coset_e8_encode_host": [_vp, _vp, _i32, _vp, _i32, _i64, _i64, _i32, _i32, _vp],
    "coset_e8_decode_host": [_vp, _vp, _vp, _i32, _i64, _i64, _i32, _i32, _vp, _i32],
    "coset_e8_quantize_host": [_vp, _vp, _i32, _vp, _i32, _i64, _i64, _i32, _i32, _f32, _vp, _i32, _vp],
    "coset_e8_decode_mean": [_vp, _i32, _i64, _i64, _f32, _vp, _i32, _vp],
    "coset_e8_decode_mean_peers": [_vp, _i32, _i32, _i64, _f32, _vp, _i32, _vp, _vp],
    "coset_peer_signal_wait": [_vp, _i32, _i32, ctypes.c_uint32, _i32, _vp, _vp],
    "coset_e8_vlut_gemv": [_vp, _vp, _i64, _i32, _i32, _vp, _i32, _i64, _i32, _vp, _vp, _i32, _i64, _f32, _vp],
    "coset_e8_vlut_gemv_scatter": [_vp, _vp, _i64, _i32, _i32, _vp, _i32, _i64, _i32, _vp, _vp, _i32, _i64, _f32, _vp],
    "coset_e8_quant_stats_scratch_bytes": [_i64],
    "coset_e8_quant_stats": [_vp, _i32, _vp, _i32, _i64, _i64, _vp, _i64, _vp, _vp],
    "coset_e8_quant_stats_static_max_blocks": [],
    "coset_e8_quant_stats_static": [_vp, _i32, _vp, _i32, _i64, _i64, _vp, _vp],
    "coset_e8_ref_encode": [_vp, _i64, ctypes.c_double, ctypes.c_double, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp],
    "coset_e8_ref_decode": [_vp, _vp, _i64, ctypes.c_double, ctypes.c_double, _i32, _i32, _vp, _vp, _vp],
    "coset_e8_ref_decode_coarse": [_vp, _vp, _i64, ctypes.c_double, ctypes.c_double, _i32, _i32, _i32, _vp, _vp, _vp],
    "coset_d4_projection": [_vp, _i64, _vp, _vp],
    "coset_d4_quantize": [_vp, _i32, _vp, _i32, _i64, _i64, _f32, _vp, _i32, _vp],
    "coset_d4_fake_quant_bwd": [_vp, _i32, _vp, _vp, _i64, _i64, _f32, _vp, _vp, _vp],
    "coset_lattice_babai": [_vp, _i64, _i32, _vp, _vp, _f32, _vp, _vp],
    "coset_e8_dequant_gemm": [_vp, _vp, _i64, _i32, _i32, _vp, _i64, _i32, _vp, _vp, _i64, _f32, _vp, _vp],
    "coset_e8_decode_gemm_scratch_bytes": [_i32, _i32],
    "coset_e8_decode_gemm": [_vp, _vp, _i64, _i32, _i32, _vp, _i64, _i32, _vp, _vp, _i32, _i64, _f32, _vp, _i64, _vp, _vp],
    "coset_layer_beta": [_vp, _vp, _vp, _i64, _vp, _vp],
    "coset_e8_layer_fake_quant_fwd": [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _f32, _vp, _i32, _vp, _vp, _vp],
    "coset_e8_layer_fake_quant_bwd": [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _f32, _vp, _vp, _vp],
    "coset_e8_fake_quant_bwd": [_vp, _i32, _vp, _vp, _vp, _i64, _i64, _i32, _f32, _vp, _vp, _vp],
}


def lib():
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m coset_b200.build` "
                "(coset_b200 has no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = (ctypes.c_char_p if name == "coset_last_error_string"
                          else ctypes.c_int64 if name.endswith(("_scratch_bytes", "_max_blocks")) else ctypes.c_int)
        _lib = L
    return _lib


def check(rc, what):
    if rc != 0:
        msg = lib().coset_last_error_string().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed with status {rc}: {msg}")


def require_cuda(t, name):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise ValueError(f"{name} must live on a CUDA device (coset_b200 has no CPU path); got {t.device}")
    return t


def require_float32(t, name):
    """The weight-path kernels read their parameter as float32 rows; any other dtype would be
    misread (and over-read), so it is refused before a launch."""
    if t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32 (the fused weight kernels read float32 rows), got {t.dtype}; "
                        "keep the layer's parameters in float32 and pass low-precision activations instead")
    return t


def dtype_code(t, name):
    if t.dtype == torch.float32:
        return DTYPE_F32
    if t.dtype == torch.bfloat16:
        return DTYPE_BF16
    raise TypeError(f"{name} must be float32 or bfloat16, got {t.dtype}")


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() > 0 else ctypes.c_void_p(0)


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
