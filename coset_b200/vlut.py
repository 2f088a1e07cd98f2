"""Inference with weights kept as E8 codes: E8CodeLinear.

The weight of a trained HNLQLinearQAT layer is exported as packed q=4, M=2 codes (4 bytes per 8
weights) plus the scales beta, and applied from the codes:

  * few tokens  (T <= small_t_max): the code-domain kernels of coset_e8_vlut_gemv, which read the code
    stream (8.4 - 16.8 MB for a 4096 x 4096 weight instead of 64 MB of float32);
  * many tokens (from 2048 by default): the weight is decoded into a transient bf16 buffer and multiplied by
    this library's tcgen05 GEMM (coset_e8_decode_gemm); nothing dense survives the call;
  * in between, by default, the library GEMM on a cached dense bf16 copy (`large_t_path` chooses).

The math is the reference's one-sided vLUT inner product (coset/legacy/quant/vlut.py:72-117) in
the layer's scale convention W_q = decode(codes) / beta (coset/core/layers.py:453-460).
"""
from typing import Optional

import torch
import torch.nn as nn

from . import _lib
from .core.e8.codecs import e8_decode_packed, e8_encode_packed


def e8_vlut_matmul(codes: torch.Tensor, beta: Optional[torch.Tensor], blocks_per_tile: int, x: torch.Tensor,
                   bias: Optional[torch.Tensor] = None, clip: float = 0.0, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """y = x @ Wq.T + bias with Wq = decode(codes) / beta (clamped to +-clip when clip > 0);
    codes int32 [n_out, n_in / 8]; x [T, n_in]; y float32, or bf16 rounded once from the float32 sums."""
    _lib.require_cuda(codes, "codes")
    _lib.require_cuda(x, "x")
    if codes.dtype != torch.int32 or codes.dim() != 2 or not codes.is_contiguous():
        raise ValueError("codes must be a contiguous int32 tensor [n_out, n_in / 8]")
    n_out, kb = codes.shape
    if x.dim() != 2 or x.shape[1] != kb * 8:
        raise ValueError(f"x must be [T, {kb * 8}], got {tuple(x.shape)}")
    x = x.contiguous()
    T = x.shape[0]
    y = torch.empty((T, n_out), dtype=out_dtype, device=x.device)
    b = beta.to(torch.float32).contiguous().view(-1) if beta is not None else None
    bias32 = bias.to(torch.float32).contiguous() if bias is not None else None
    with torch.cuda.device(x.device):
        rc = _lib.lib().coset_e8_vlut_gemv(_lib.ptr(codes), _lib.ptr(b) if b is not None else None, int(blocks_per_tile),
                                           n_out, kb * 8, _lib.ptr(x), _lib.dtype_code(x, "x"), x.stride(0), T,
                                           _lib.ptr(bias32) if bias32 is not None else None, _lib.ptr(y),
                                           _lib.dtype_code(y, "y"), y.stride(0), float(clip), _lib.stream())
    _lib.check(rc, "coset_e8_vlut_gemv")
    return y


def e8_dequant_gemm(codes: torch.Tensor, beta: Optional[torch.Tensor], blocks_per_tile: int, x: torch.Tensor,
                    bias: Optional[torch.Tensor] = None, check: bool = False, clip: float = 0.0,
                    status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same product as e8_vlut_matmul for many tokens, on the tcgen05 tensor cores: weight tiles are
    decoded to bf16 in shared memory and never written to HBM.  x: bf16 [T, n_in], n_in % 64 == 0.
    check=True synchronises and raises if a bounded barrier wait expired inside the kernel."""
    _lib.require_cuda(codes, "codes")
    _lib.require_cuda(x, "x")
    if x.dtype != torch.bfloat16:
        raise TypeError("e8_dequant_gemm takes bfloat16 activations")
    if codes.dtype != torch.int32 or codes.dim() != 2 or not codes.is_contiguous():
        raise ValueError("codes must be a contiguous int32 tensor [n_out, n_in / 8]")
    n_out, kb = codes.shape
    if x.dim() != 2 or x.shape[1] != kb * 8 or (kb * 8) % 64:
        raise ValueError(f"x must be [T, {kb * 8}] with n_in a multiple of 64, got {tuple(x.shape)}")
    x = x.contiguous()
    T = x.shape[0]
    y = torch.empty((T, n_out), dtype=torch.float32, device=x.device)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=x.device)
    b = beta.to(torch.float32).contiguous().view(-1) if beta is not None else None
    bias32 = bias.to(torch.float32).contiguous() if bias is not None else None
    with torch.cuda.device(x.device):
        rc = _lib.lib().coset_e8_dequant_gemm(_lib.ptr(codes), _lib.ptr(b) if b is not None else None,
                                              int(blocks_per_tile), n_out, kb * 8, _lib.ptr(x), x.stride(0), T,
                                              _lib.ptr(bias32) if bias32 is not None else None, _lib.ptr(y),
                                              y.stride(0), float(clip), _lib.ptr(status), _lib.stream())
    _lib.check(rc, "coset_e8_dequant_gemm")
    if check and int(status.item()) != 0:
        raise RuntimeError("coset_e8_dequant_gemm: a barrier wait expired inside the kernel; the result is invalid")
    return y


def e8_decode_gemm(codes: torch.Tensor, beta: Optional[torch.Tensor], blocks_per_tile: int, x: torch.Tensor,
                   bias: Optional[torch.Tensor] = None, check: bool = False, clip: float = 0.0,
                   scratch: Optional[torch.Tensor] = None, out_dtype=torch.float32,
                   status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The product of e8_dequant_gemm in two launches: the weight is decoded to bf16 into `scratch` (transient,
    n_out * n_in bf16 values, allocated here when not given) and multiplied by a TMA-fed tcgen05 GEMM on pairs
    of CTAs (cta_group::2).  Same bits as e8_dequant_gemm and, measured, the same speed up to 8192 tokens, a few
    percent more beyond; nothing dense survives the call.  out_dtype: float32 or bfloat16 (rounded once from the
    float32 accumulator)."""
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("out_dtype must be float32 or bfloat16")
    _lib.require_cuda(codes, "codes")
    _lib.require_cuda(x, "x")
    if x.dtype != torch.bfloat16:
        raise TypeError("e8_decode_gemm takes bfloat16 activations")
    if codes.dtype != torch.int32 or codes.dim() != 2 or not codes.is_contiguous():
        raise ValueError("codes must be a contiguous int32 tensor [n_out, n_in / 8]")
    n_out, kb = codes.shape
    if x.dim() != 2 or x.shape[1] != kb * 8 or (kb * 8) % 64:
        raise ValueError(f"x must be [T, {kb * 8}] with n_in a multiple of 64, got {tuple(x.shape)}")
    x = x.contiguous()
    T = x.shape[0]
    need = n_out * kb * 8
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.bfloat16, device=x.device)
    elif scratch.dtype != torch.bfloat16 or scratch.numel() < need or not scratch.is_contiguous() or scratch.device != x.device:
        raise ValueError(f"scratch must be a contiguous bfloat16 tensor of at least {need} values on {x.device}")
    y = torch.empty((T, n_out), dtype=out_dtype, device=x.device)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=x.device)
    b = beta.to(torch.float32).contiguous().view(-1) if beta is not None else None
    bias32 = bias.to(torch.float32).contiguous() if bias is not None else None
    with torch.cuda.device(x.device):
        rc = _lib.lib().coset_e8_decode_gemm(_lib.ptr(codes), _lib.ptr(b) if b is not None else None,
                                             int(blocks_per_tile), n_out, kb * 8, _lib.ptr(x), x.stride(0), T,
                                             _lib.ptr(bias32) if bias32 is not None else None, _lib.ptr(y),
                                             _lib.dtype_code(y, "y"), y.stride(0), float(clip), _lib.ptr(scratch), scratch.numel() * 2,
                                             _lib.ptr(status), _lib.stream())
    _lib.check(rc, "coset_e8_decode_gemm")
    if check and int(status.item()) != 0:
        raise RuntimeError("coset_e8_decode_gemm: a barrier wait expired inside the kernel; the result is invalid")
    return y


class E8CodeLinear(nn.Module):
    """Linear layer that owns E8 codes + scales instead of a dense weight (inference only).

    Its state_dict is self-describing (codes, beta, bias, blocks_per_tile, weight_clip_value), so a
    layer can be rebuilt from a checkpoint alone with `E8CodeLinear.from_state_dict`.
    Up to small_t_max tokens go to the code-domain kernels; more bf16 tokens go to (large_t_path): "tcgen05" --
    this library's tensor-core kernels, which keep no dense weight: decode to a transient bf16 buffer + TMA-fed
    cta_group::2 GEMM from 1024 tokens, the single-launch fused kernel below; "cublas" -- a cached dense bf16 copy
    and the library GEMM; "auto" (default) -- the own kernels from PAIR_GEMM_MIN_T tokens, the library path for
    the tokens in between, where decoding the whole weight per call costs more than the product itself.
    small_t_max defaults to 16 ("auto", "cublas") or 48 ("tcgen05"): measured on a 4096 x 4096 layer the
    code-domain kernels take 9.7 / 23 / 44 / 86 us for 1 / 16 / 32 / 64 tokens (they re-read and re-decode the
    codes for every 16 tokens), the library on the cached copy 7-13 us, the fused kernel 64 us.
    weight_clip_value > 0: the weights are clamp(decode(codes) / beta, +-clip), the clamp the training
    layer applies after de-scaling (coset/core/layers.py:463); 0 disables it."""

    PAIR_GEMM_MIN_T = 2048  # from here on the decode + cta_group::2 GEMM is within 10-25 % of the library on a dense copy

    def __init__(self, codes: torch.Tensor, beta: torch.Tensor, blocks_per_tile: int,
                 bias: Optional[torch.Tensor] = None, small_t_max: Optional[int] = None, large_t_path: str = "auto",
                 weight_clip_value: float = 0.0):
        super().__init__()
        self.out_features, kb = codes.shape
        self.in_features = kb * 8
        if large_t_path not in ("auto", "cublas", "tcgen05"):
            raise ValueError("large_t_path must be 'auto', 'cublas' (dequantise once, keep the dense copy, library GEMM) "
                             "or 'tcgen05' (this library's tensor-core kernels only, no dense copy kept)")
        self.large_t_path = large_t_path
        self.small_t_max = int(small_t_max) if small_t_max is not None else (48 if large_t_path == "tcgen05" else 16)
        self.register_buffer("codes", codes.contiguous())
        self.register_buffer("beta", beta.to(torch.float32).contiguous().view(-1))
        self.register_buffer("bias", bias.detach().clone() if bias is not None else None)
        self.register_buffer("blocks_per_tile_t", torch.tensor(int(blocks_per_tile), dtype=torch.int64))
        self.register_buffer("weight_clip_value_t", torch.tensor(float(weight_clip_value), dtype=torch.float32))
        self.blocks_per_tile = int(blocks_per_tile)
        self.weight_clip_value = float(weight_clip_value)
        self._dense, self._dense_key = None, None  # bf16 copy for the library GEMM, rebuilt when codes / scales change
        self._status = None                         # device word the tensor-core kernels set when a bounded wait gave up

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        self.blocks_per_tile = int(self.blocks_per_tile_t.item())
        self.weight_clip_value = float(self.weight_clip_value_t.item())
        self._dense, self._dense_key = None, None

    @classmethod
    def from_weight(cls, weight: torch.Tensor, beta: torch.Tensor, blocks_per_tile: int, bias=None, **kw):
        """Quantise a dense float32 weight [n_out, n_in] with scales beta (layer convention)."""
        _lib.require_cuda(weight, "weight")
        n_out, n_in = weight.shape
        if n_in % 8:
            raise ValueError(f"Input dimension {n_in} must be divisible by 8 for E8 lattice")
        packed = e8_encode_packed(weight.contiguous().view(-1, 8), 4, 2, scale=beta.contiguous().view(-1),
                                  scale_mode=_lib.SCALE_MUL_TILE, blocks_per_tile=blocks_per_tile)
        codes = packed.view(torch.int32).view(n_out, n_in // 8)
        return cls(codes, beta, blocks_per_tile, bias, **kw)

    @classmethod
    def from_qat_layer(cls, layer, **kw):
        """Export of a trained HNLQLinearQAT (q must be 4): codes, scales, bias and the layer's
        weight_clip_value, so that this layer computes what the trained one computes."""
        return cls.from_exported(layer.export_quantized(packed=True), **kw)

    @classmethod
    def from_exported(cls, exported: dict, **kw):
        """Rebuild from HNLQLinearQAT.export_quantized(packed=True)."""
        meta = exported["metadata"]
        if meta.get("q") != 4 or meta.get("packed_M", 2) != 2:
            raise ValueError("E8CodeLinear stores q=4, M=2 codes")
        kw.setdefault("weight_clip_value", meta.get("weight_clip_value", 0.0))
        return cls(exported["codes"], exported["beta"], int(exported["blocks_per_tile"]), exported.get("bias"), **kw)

    @classmethod
    def from_state_dict(cls, state_dict: dict, prefix: str = "", **kw):
        """Rebuild from a checkpoint of this class alone (no codes in hand)."""
        g = lambda k: state_dict[prefix + k]
        bias = state_dict.get(prefix + "bias")
        kw.setdefault("weight_clip_value", float(g("weight_clip_value_t")))
        return cls(g("codes"), g("beta"), int(g("blocks_per_tile_t")), bias, **kw)

    def dense_weight(self, dtype=torch.float32) -> torch.Tensor:
        """Wq = clamp(decode(codes) / beta) as a dense [n_out, n_in] tensor."""
        w = e8_decode_packed(self.codes.view(-1), 4, 2, scale=self.beta, scale_mode=_lib.SCALE_MUL_TILE,
                             blocks_per_tile=self.blocks_per_tile, dtype=torch.float32 if self.weight_clip_value > 0 else dtype)
        if self.weight_clip_value > 0:
            w = w.clamp_(-self.weight_clip_value, self.weight_clip_value).to(dtype)
        return w.view(self.out_features, self.in_features)

    def _dense_bf16(self):
        key = (self.codes._version, self.beta._version, self.codes.data_ptr(), self.beta.data_ptr(), self.codes.device,
               self.weight_clip_value, self.blocks_per_tile)
        if self._dense is None or self._dense_key != key:
            self._dense, self._dense_key = self.dense_weight(torch.bfloat16), key
        return self._dense

    def check(self):
        """Synchronises and raises if a bounded barrier wait expired inside one of the tensor-core kernels since
        the last check (their results are then invalid).  The kernels never hang: they give up after 0.2 s."""
        if self._status is not None and int(self._status.item()) != 0:
            self._status.zero_()
            raise RuntimeError("E8CodeLinear: a barrier wait expired inside a tensor-core kernel; results since the last check are invalid")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        clip = self.weight_clip_value
        if x2.shape[0] <= self.small_t_max:
            out_dtype = torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float32
            y = e8_vlut_matmul(self.codes, self.beta, self.blocks_per_tile, x2, self.bias, clip, out_dtype)
            y = y.to(x.dtype) if x.dtype != out_dtype else y
        else:
            if x2.dtype == torch.float32:
                y = torch.nn.functional.linear(x2, self.dense_weight(torch.float32), self.bias)
            elif x2.dtype == torch.bfloat16 and self.in_features % 64 == 0 and (
                    self.large_t_path == "tcgen05" or (self.large_t_path == "auto" and x2.shape[0] >= self.PAIR_GEMM_MIN_T)):
                if self._status is None or self._status.device != x2.device:
                    self._status = torch.zeros(1, dtype=torch.int32, device=x2.device)
                if x2.shape[0] >= 1024:
                    y = e8_decode_gemm(self.codes, self.beta, self.blocks_per_tile, x2, self.bias, clip=clip, out_dtype=torch.bfloat16,
                                       status=self._status)
                else:
                    y = e8_dequant_gemm(self.codes, self.beta, self.blocks_per_tile, x2, self.bias, clip=clip,
                                        status=self._status).to(x2.dtype)
            else:
                b = self.bias.to(x2.dtype) if self.bias is not None else None
                y = torch.nn.functional.linear(x2, self._dense_bf16().to(x2.dtype), b)
        return y.reshape(*lead, self.out_features)


def out_feature_shard(n_out: int, world: int, rank: int):
    """[start, stop) of the output features rank `rank` owns: contiguous, equal sizes (n_out must
    divide by world so that the gathered result needs no padding)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if n_out % world:
        raise ValueError(f"out_features {n_out} must be divisible by the world size {world}")
    per = n_out // world
    return rank * per, (rank + 1) * per


def assemble_gathered(gathered: torch.Tensor) -> torch.Tensor:
    """[world, T, n_out / world] (the layout an all-gather of the local products yields) -> [T, n_out]."""
    world, T, per = gathered.shape
    return gathered.permute(1, 0, 2).reshape(T, world * per)


class ColumnParallelE8CodeLinear(nn.Module):
    """E8CodeLinear sharded along the output features over a process group: every rank owns the
    codes and scales of out_features / world rows, multiplies the (replicated) activations with
    them and the slices are exchanged with one all-gather of [T, out_features / world] floats.

    The codes never cross the link; at T = 1 the all-gather is latency-bound.

    transport="peer" (few tokens, T <= local.small_t_max): the product kernel writes every result row
    straight into the result buffer of EVERY rank (symmetric memory, plain stores over NVLink), the
    library's bounded cross-rank arrival follows (coset_b200.peer), and no all-gather is issued."""

    def __init__(self, local: E8CodeLinear, out_features: int, group=None, transport: str = "nccl", timeout_ms: int = 2000):
        super().__init__()
        import torch.distributed as dist
        if transport not in ("nccl", "peer"):
            raise ValueError("transport must be 'nccl' or 'peer'")
        self.transport = transport
        self.timeout_ms = int(timeout_ms)
        self._region, self._cap_tokens, self._parity = None, 0, 0  # symmetric result buffer [2, tokens, out_features]
        self.local = local
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.out_features = out_features
        self.in_features = local.in_features
        lo, hi = out_feature_shard(out_features, self.world, self.rank)
        if local.out_features != hi - lo:
            raise ValueError(f"local shard has {local.out_features} rows, expected {hi - lo}")

    @classmethod
    def from_weight(cls, weight: torch.Tensor, beta: torch.Tensor, blocks_per_tile: int, bias=None, group=None,
                    transport: str = "nccl", **kw):
        """Quantise this rank's rows of a full [n_out, n_in] weight; beta holds the scales of the
        full weight (one per block for blocks_per_tile = 1, one per row for n_in / 8)."""
        import torch.distributed as dist
        n_out, n_in = weight.shape
        lo, hi = out_feature_shard(n_out, dist.get_world_size(group), dist.get_rank(group))
        tiles_per_row = (n_in // 8) // int(blocks_per_tile)
        if tiles_per_row * int(blocks_per_tile) * 8 != n_in:
            raise ValueError("a scale tile must not straddle two rows")
        b = beta.contiguous().view(-1)[lo * tiles_per_row:hi * tiles_per_row]
        local = E8CodeLinear.from_weight(weight[lo:hi].contiguous(), b, blocks_per_tile,
                                         bias[lo:hi] if bias is not None else None, **kw)
        return cls(local, n_out, group, transport)

    def _forward_peer(self, x2: torch.Tensor) -> torch.Tensor:
        import ctypes
        import torch.distributed as dist
        from .peer import SymmetricRegion
        T = x2.shape[0]
        if T > self._cap_tokens:  # collective: every rank sees the same sequence of token counts
            if self._region is not None:  # peers may still be writing into the old allocation
                torch.cuda.synchronize(x2.device)
                dist.barrier(group=self.group)
            self._cap_tokens = T
            self._region = SymmetricRegion(2 * T * self.out_features * 4, x2.device, self.group, self.timeout_ms)
            self._parity = 0
        region, parity = self._region, self._parity
        self._parity ^= 1
        half_elems = self._cap_tokens * self.out_features
        lo, _ = out_feature_shard(self.out_features, self.world, self.rank)
        offset = (parity * half_elems + lo) * 4  # this rank's columns inside half `parity`
        targets = region.pointers(offset)
        loc = self.local
        x2 = x2.contiguous()
        bias32 = loc.bias.to(torch.float32).contiguous() if loc.bias is not None else None
        with torch.cuda.device(x2.device):
            rc = _lib.lib().coset_e8_vlut_gemv_scatter(
                _lib.ptr(loc.codes), _lib.ptr(loc.beta), loc.blocks_per_tile, loc.out_features, loc.in_features,
                _lib.ptr(x2), _lib.dtype_code(x2, "x"), x2.stride(0), T, _lib.ptr(bias32) if bias32 is not None else None,
                ctypes.cast(targets, ctypes.c_void_p), self.world, self.out_features, float(loc.weight_clip_value),
                _lib.stream())
        _lib.check(rc, "coset_e8_vlut_gemv_scatter")
        region.arrive()  # bounded: all ranks have written their columns into this rank's buffer
        # the half is written again two calls from now, after the arrival of the call in between
        mine = region.data(torch.float32)[parity * half_elems: parity * half_elems + T * self.out_features]
        return mine.view(T, self.out_features).clone()

    def check(self):
        """Raises if a bounded cross-rank wait of the peer-store path, or a bounded barrier wait inside a
        tensor-core kernel of the local product, gave up (synchronises)."""
        self.local.check()
        if self._region is not None:
            self._region.check()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if self.transport == "peer" and self.world > 1 and x2.shape[0] <= self.local.small_t_max:
            y = self._forward_peer(x2)
            y = y.to(x.dtype) if x.dtype != torch.float32 else y
            return y.reshape(*lead, self.out_features)
        y_loc = self.local(x2).contiguous()
        gathered = torch.empty(self.world * y_loc.numel(), dtype=y_loc.dtype, device=y_loc.device)
        dist.all_gather_into_tensor(gathered, y_loc.view(-1), group=self.group)
        return assemble_gathered(gathered.view(self.world, *y_loc.shape)).reshape(*lead, self.out_features)
