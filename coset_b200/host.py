"""Codec over HOST arrays: the drop-in for CPU-side callers of e8_encode / e8_decode.

HostCodec stages pinned host tensors through the GPU in chunks (copy in, kernel, copy out, all
overlapped) and returns host tensors.  This is the end-to-end path the benchmark's `e2e`
figure is measured on.
"""
import ctypes

import torch

from . import _lib


class HostCodec:
    def __init__(self, chunk_blocks: int = 1 << 21, n_slots: int = 4, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._ctx = ctypes.c_void_p(0)
        with torch.cuda.device(self.device):
            rc = _lib.lib().coset_host_ctx_create(int(chunk_blocks), int(n_slots), ctypes.byref(self._ctx))
        _lib.check(rc, "coset_host_ctx_create")

    def close(self):
        if self._ctx:
            _lib.lib().coset_host_ctx_destroy(self._ctx)
            self._ctx = ctypes.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _host(t, name):
        if not isinstance(t, torch.Tensor) or t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CPU tensor")
        return ctypes.c_void_p(t.data_ptr())

    def encode(self, x, scale=None, scale_mode=_lib.SCALE_NONE, blocks_per_tile=1, q=4, M=2, out=None):
        """x: CPU [N, 8] float32/bfloat16 (pinned for overlap) -> CPU uint8 [N, code_bytes]."""
        n = x.shape[0]
        cb = _lib.lib().coset_e8_code_bytes(q, M)
        if out is None:
            out = torch.empty((n, cb), dtype=torch.uint8, pin_memory=True)
        sp = self._host(scale, "scale") if scale is not None else None
        with torch.cuda.device(self.device):
            rc = _lib.lib().coset_e8_encode_host(self._ctx, self._host(x, "x"), _lib.dtype_code(x, "x"), sp, scale_mode,
                                                 n, blocks_per_tile, q, M, self._host(out, "out"))
        _lib.check(rc, "coset_e8_encode_host")
        return out

    def decode(self, codes, scale=None, scale_mode=_lib.SCALE_NONE, blocks_per_tile=1, q=4, M=2,
               dtype=torch.float32, out=None):
        """codes: CPU packed codes -> CPU [N, 8] reconstruction."""
        cb = _lib.lib().coset_e8_code_bytes(q, M)
        n = codes.numel() * codes.element_size() // cb
        if out is None:
            out = torch.empty((n, 8), dtype=dtype, pin_memory=True)
        sp = self._host(scale, "scale") if scale is not None else None
        with torch.cuda.device(self.device):
            rc = _lib.lib().coset_e8_decode_host(self._ctx, self._host(codes, "codes"), sp, scale_mode, n,
                                                 blocks_per_tile, q, M, self._host(out, "out"), _lib.dtype_code(out, "out"))
        _lib.check(rc, "coset_e8_decode_host")
        return out

    def quantize(self, x, scale=None, scale_mode=_lib.SCALE_NONE, blocks_per_tile=1, q=4, M=2, clip=0.0,
                 dtype=torch.float32, out=None, codes_out=None, return_codes=False):
        """Round trip decode(encode(x)) in one pass over the host array: the input goes to the device while
        the reconstructions (and the packed codes, if asked for) of earlier chunks come back.
        -> CPU [N, 8] reconstruction, or (reconstruction, codes) with return_codes / codes_out."""
        n = x.shape[0]
        cb = _lib.lib().coset_e8_code_bytes(q, M)
        if out is None:
            out = torch.empty((n, 8), dtype=dtype, pin_memory=True)
        if return_codes and codes_out is None:
            codes_out = torch.empty((n, cb), dtype=torch.uint8, pin_memory=True)
        sp = self._host(scale, "scale") if scale is not None else None
        cp = self._host(codes_out, "codes_out") if codes_out is not None else None
        with torch.cuda.device(self.device):
            rc = _lib.lib().coset_e8_quantize_host(self._ctx, self._host(x, "x"), _lib.dtype_code(x, "x"), sp, scale_mode, n,
                                                   blocks_per_tile, q, M, float(clip), self._host(out, "out"),
                                                   _lib.dtype_code(out, "out"), cp)
        _lib.check(rc, "coset_e8_quantize_host")
        return (out, codes_out) if codes_out is not None else out
