"""E8-quantised gradient averaging across data-parallel ranks.

The reference plans this ("quantize gradient buckets along the last dim, pad to d, decode",
prompts/design_instructions.md:104-110) but ships no code.  The exchange here is:

    1. pad the flat gradient to a multiple of 8 values, view it as blocks [n, 8]
    2. encode x * scale with the q=4, M=2 E8 codec -> 4 bytes per block
    3. all-gather the packed codes (NCCL over NVLink; 1/8 of the float32 payload)
    4. one kernel decodes the W code streams and writes (sum_r x_hat_r) / (scale * W)

With transport="nccl" (default) each rank only reads its own memory; the collective is a plain
all_gather_into_tensor.  With transport="peer" steps 3 and 4 are ONE kernel: every rank encodes into a
buffer in symmetric memory, the library's own bounded arrival (coset_peer_signal_wait) orders "all
encoded", and the decode kernel reads the W code streams straight from the peers' memory over NVLink
(plain loads, no multicast) while it decodes -- no gathered copy is written or re-read.  The
arithmetic is fixed (exact sum of reconstructions, one float32 division), so every rank obtains
bit-identical averages with either transport and a CPU run of the same recipe reproduces them.
"""
import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib


SATURATION = 3.9  # bound of a scaled coordinate under the saturating encode (COSET_SEM_CORE_SATURATE)


class CudaCodec:
    """The two device operations of the exchange, through the C ABI.

    saturate=True (default): every scaled value is clamped to +-SATURATION before it is quantised.
    The q=4, M=2 code is periodic (it wraps modulo 16 E8), so without the clamp one gradient value
    beyond the code's range would decode to an unrelated small number on every rank; with it the value
    is clipped to SATURATION / scale, a bounded and visible error.  Blocks inside the range are coded
    exactly as without the clamp."""

    def __init__(self, saturate: bool = True):
        self.saturate = bool(saturate)
        self._scales = {}  # (device, scale) -> 1-element tensor: no allocation or host-to-device copy per call

    def encode(self, blocks: torch.Tensor, scale: float, out: torch.Tensor) -> torch.Tensor:
        n = blocks.shape[0]
        key = (blocks.device, float(scale))
        s = self._scales.get(key)
        if s is None:
            s = self._scales[key] = torch.full((1,), float(scale), dtype=torch.float32, device=blocks.device)
        sem = _lib.SEM_CORE_SATURATE if self.saturate else _lib.SEM_CORE
        with torch.cuda.device(blocks.device):
            rc = _lib.lib().coset_e8_encode(_lib.ptr(blocks), _lib.dtype_code(blocks, "grad"), _lib.ptr(s),
                                            _lib.SCALE_MUL_TILE, n, max(n, 1), 4, 2, sem, _lib.ptr(out),
                                            _lib.stream())
        _lib.check(rc, "coset_e8_encode")
        return out

    def decode_mean(self, codes: torch.Tensor, world: int, n_blocks: int, scale: float, out: torch.Tensor):
        with torch.cuda.device(codes.device):
            rc = _lib.lib().coset_e8_decode_mean(_lib.ptr(codes), world, n_blocks, codes.shape[1], float(scale),
                                                 _lib.ptr(out), _lib.dtype_code(out, "out"), _lib.stream())
        _lib.check(rc, "coset_e8_decode_mean")
        return out


class E8GradientExchange:
    """Averages a flat gradient over the ranks of `group` through E8 codes.

    scale: shared multiplier applied before quantisation (the quantiser's step is 1/scale); it
    must be the same on every rank.  With gradients of standard deviation sigma, scale = 0.5/sigma
    keeps the two-level code away from overload; values beyond SATURATION / scale are clipped there
    (see CudaCodec), and `overloaded_fraction` reports how many blocks that concerns.
    timeout_ms: bound of the cross-rank wait of the peer-memory transport (see coset_b200.peer).
    chunks: the peer-memory transport can cut a large gradient into this many pieces and decode piece k (NVLink
    reads, on a high-priority side stream) while piece k+1 is being encoded.  Default 1 = one piece: on 4 B200s
    the 109.5 M-value gradient takes 0.460 / 0.491 / 0.544 / 0.665 ms with 1 / 2 / 4 / 8 pieces (on 8: 0.767 / 0.797 /
    0.856 / 0.963 ms) -- encoder and
    decoder both want every SM, so running them side by side moves no work off the critical path, while each
    extra piece adds an arrival (a cross-GPU round trip) and three launches.
    """

    CHUNK_MIN_BLOCKS = 1 << 18  # below this a piece is too small for the overlap to pay for its extra arrival

    def __init__(self, group: Optional[dist.ProcessGroup] = None, scale: float = 500.0, codec=None,
                 transport: str = "nccl", timeout_ms: int = 2000, chunks: int = 1):
        if transport not in ("nccl", "peer"):
            raise ValueError("transport must be 'nccl' (all-gather, then decode) or 'peer' (decode from peer memory)")
        self.group = group
        self.scale = float(scale)
        self.codec = codec if codec is not None else CudaCodec()
        self.transport = transport
        self.timeout_ms = int(timeout_ms)
        self.chunks = max(1, int(chunks))
        self._decode_stream = None  # high-priority stream of the chunked peer transport
        self._codes = None
        self._gathered = None
        self._region = None      # one symmetric allocation [2, capacity] int32, grown (collectively) when a larger bucket arrives
        self._capacity = 0
        self._parity = 0
        self._side = None        # stream of the asynchronous DDP hook
        self.phase_events = None  # set to a list: a CUDA event is appended after encode, transfer and decode

    def _mark(self):
        if self.phase_events is not None and torch.cuda.is_available():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.phase_events.append(ev)

    def _world(self):
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def _buffers(self, n_blocks, world, device):
        if self._codes is None or self._codes.numel() != n_blocks or self._codes.device != device:
            self._codes = torch.empty(n_blocks, dtype=torch.int32, device=device)
        if self._gathered is None or self._gathered.shape != (world, n_blocks) or self._gathered.device != device:
            self._gathered = torch.empty((world, n_blocks), dtype=torch.int32, device=device)
        return self._codes, self._gathered

    def all_reduce_mean(self, flat: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """flat: 1-D float32 (or bfloat16) gradient on this rank -> 1-D float32 average, same length.
        out (float32, contiguous, same length) receives the result; it may be `flat` itself."""
        if flat.dim() != 1:
            raise ValueError("expected a flat 1-D gradient")
        if isinstance(self.codec, CudaCodec):
            _lib.require_cuda(flat, "flat")
        n_values = flat.numel()
        n_blocks = (n_values + 7) // 8
        if n_blocks * 8 != n_values:  # pad the tail with zeros, stripped again below
            padded = torch.zeros(n_blocks * 8, dtype=flat.dtype, device=flat.device)
            padded[:n_values] = flat
        else:
            padded = flat.contiguous()
        world = self._world()
        # the decode kernel writes straight into `out` when its layout allows (no padding, float32)
        direct = (out is not None and n_blocks * 8 == n_values and out.dtype == torch.float32 and out.is_contiguous()
                  and out.numel() == n_values and out.device == flat.device)
        res = out.view(n_blocks, 8) if direct else torch.empty((n_blocks, 8), dtype=torch.float32, device=flat.device)
        if self.transport == "peer" and world > 1:
            self._all_reduce_mean_peer(padded, n_blocks, world, res)
        else:
            self._all_reduce_mean_gathered(padded, n_blocks, world, res)
        if direct:
            return out
        res = res.view(-1)[:n_values]
        if out is not None:
            out.copy_(res)
            return out
        return res

    def _all_reduce_mean_gathered(self, padded, n_blocks, world, res):
        """Encode, all-gather the packed codes, decode-and-average, one after the other on the caller's stream.
        (Pipelining the three over pieces of the gradient -- all-gather of piece k on a second stream beside the
        encode of piece k+1 and the decode of piece k-1 -- was measured on 8 B200s at 1.126 / 1.196 / 1.106 /
        1.177 / 1.437 ms for 1 / 2 / 3 / 4 / 8 pieces: the collective's own kernels and ours compete for the
        same SMs, so nothing is gained and the form stays sequential.)"""
        codes, gathered = self._buffers(n_blocks, world, padded.device)
        self._mark()
        self.codec.encode(padded.view(n_blocks, 8), self.scale, codes)
        self._mark()
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), codes, group=self.group)
        else:
            gathered.view(-1).copy_(codes)
        self._mark()
        self.codec.decode_mean(gathered, world, n_blocks, self.scale, res)
        self._mark()
        return res

    def overloaded_fraction(self, flat: torch.Tensor) -> float:
        """Fraction of this rank's 8-value blocks whose scaled values leave the two-level code's range
        (the overload test of ref/hnlq.py:341 through coset_e8_quant_stats).  Diagnostic: it reads the
        tensor once more and synchronises; use it to pick `scale`, not on every step."""
        from .core.e8.codecs import e8_quant_stats
        n_values = flat.numel()
        n_blocks = n_values // 8
        if n_blocks == 0:
            return 0.0
        s = torch.full((1,), self.scale, dtype=torch.float32, device=flat.device)
        stats = e8_quant_stats(flat[:n_blocks * 8].contiguous().view(n_blocks, 8), scale=s, scale_mode=_lib.SCALE_MUL_TILE,
                               blocks_per_tile=n_blocks)
        return float(stats["overloaded_blocks"]) / n_blocks

    def check(self):
        """Raises if a bounded cross-rank wait of the peer-memory transport gave up (synchronises)."""
        if self._region is not None:
            self._region.check()

    def _all_reduce_mean_peer(self, padded, n_blocks, world, res):
        """Encode into one half of the symmetric allocation, bounded arrival, decode from every rank's
        half -- piece by piece, so that the NVLink reads of one piece run beside the encode of the next.
        One arrival per piece is enough: a rank overwrites half p only two calls later, after the arrivals
        of the call in between, which no rank passes before its own decodes of half p have finished (they
        are joined into the caller's stream ahead of those arrivals)."""
        from .peer import SymmetricRegion
        dev = padded.device
        if n_blocks > self._capacity:  # collective: every rank sees the same sequence of sizes
            if self._region is not None:  # peers may still be reading the old allocation
                torch.cuda.synchronize(dev)
                dist.barrier(group=self.group)
            self._capacity = n_blocks
            self._region = SymmetricRegion(2 * n_blocks * 4, dev, self.group, self.timeout_ms)
            self._parity = 0
        region, parity = self._region, self._parity
        self._parity ^= 1
        half = region.data(torch.int32)[parity * self._capacity: parity * self._capacity + n_blocks]
        blocks = padded.view(n_blocks, 8)
        pieces = min(self.chunks, max(1, n_blocks // self.CHUNK_MIN_BLOCKS))
        step = (n_blocks + pieces - 1) // pieces
        step = (step + 1023) // 1024 * 1024  # whole 4 KiB of codes per piece
        main = torch.cuda.current_stream(dev)
        if pieces > 1 and self._decode_stream is None:
            self._decode_stream = torch.cuda.Stream(device=dev, priority=-1)
        lib = _lib.lib()
        for lo in range(0, n_blocks, step):
            hi = min(lo + step, n_blocks)
            self.codec.encode(blocks[lo:hi], self.scale, half[lo:hi])
            region.arrive()  # every rank's piece is in its buffer (or the wait gave up and set the status word)
            ptrs = region.pointers((parity * self._capacity + lo) * 4)
            stream = main
            if pieces > 1:  # decode this piece beside the encode of the next one
                stream = self._decode_stream
                stream.wait_stream(main)
            with torch.cuda.device(dev), torch.cuda.stream(stream):
                rc = lib.coset_e8_decode_mean_peers(ctypes.cast(ptrs, ctypes.c_void_p), world, region.rank, hi - lo,
                                                    float(self.scale), _lib.ptr(res[lo:hi]), _lib.dtype_code(res, "out"),
                                                    _lib.ptr(region.status), _lib.stream())
            _lib.check(rc, "coset_e8_decode_mean_peers")
        if pieces > 1:
            # the caller's stream continues after the last decode; this join is also what keeps the reuse of
            # the buffer halves safe (see above: the next arrival is enqueued behind it)
            main.wait_stream(self._decode_stream)
        return res


def e8_allreduce_hook(state: E8GradientExchange, bucket) -> torch.futures.Future[torch.Tensor]:
    """torch DDP communication hook: `ddp.register_comm_hook(E8GradientExchange(group), e8_allreduce_hook)`.

    The bucket's flat gradient is replaced by its E8-quantised average.  On a CUDA device the exchange
    runs on a side stream of `state` and the returned future completes with it, so the exchange of one
    bucket overlaps the backward pass that fills the next; buckets are exchanged in order on that one
    stream, which is also what makes the reuse of `state`'s buffers safe."""
    buf = bucket.buffer()
    if not buf.is_cuda:
        avg = state.all_reduce_mean(buf.float() if buf.dtype not in (torch.float32, torch.bfloat16) else buf)
        fut = torch.futures.Future()
        fut.set_result(avg.to(buf.dtype))
        return fut
    if state._side is None:
        state._side = torch.cuda.Stream(device=buf.device)
    side = state._side
    side.wait_stream(torch.cuda.current_stream(buf.device))
    fut = torch.futures.Future(devices=[buf.device])
    with torch.cuda.stream(side):
        src = buf.float() if buf.dtype not in (torch.float32, torch.bfloat16) else buf
        if buf.dtype == torch.float32:
            state.all_reduce_mean(src, out=buf)  # decoded straight into the bucket
            result = buf
        else:
            result = state.all_reduce_mean(src).to(buf.dtype)
        buf.record_stream(side)
        fut.set_result(result)  # records the side stream's work; consumers wait for it on their own stream
    return fut


def bert_base_gradient_numel() -> int:
    """Parameter count of the BERT-base-shaped set used by the gradient-exchange benchmark:
    embeddings 30522/512/2 x 768 + LayerNorm, 12 x (4 attention projections, 2 FFN matrices,
    2 LayerNorms), pooler."""
    h, f, v = 768, 3072, 30522
    emb = v * h + 512 * h + 2 * h + 2 * h
    layer = 4 * (h * h + h) + 2 * h + (h * f + f) + (f * h + h) + 2 * h
    return emb + 12 * layer + h * h + h
