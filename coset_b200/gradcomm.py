"""E8-quantised gradient averaging across data-parallel ranks.

The reference plans this ("quantize gradient buckets along the last dim, pad to d, decode",
prompts/design_instructions.md:104-110) but ships no code.  The exchange here is:

    1. pad the flat gradient to a multiple of 8 values, view it as blocks [n, 8]
    2. encode x * scale with the q=4, M=2 E8 codec -> 4 bytes per block
    3. all-gather the packed codes (NCCL over NVLink; 1/8 of the float32 payload)
    4. one kernel decodes the W code streams and writes (sum_r x_hat_r) / (scale * W)

With transport="nccl" (default) each rank only reads its own memory; the collective is a plain
all_gather_into_tensor.  With transport="peer" steps 3 and 4 are ONE kernel: every rank encodes into a
buffer in symmetric memory, a device-side barrier of torch's symmetric-memory handle orders "all
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


class CudaCodec:
    """The two device operations of the exchange, through the C ABI."""

    def encode(self, blocks: torch.Tensor, scale: float, out: torch.Tensor) -> torch.Tensor:
        n = blocks.shape[0]
        s = torch.full((1,), float(scale), dtype=torch.float32, device=blocks.device)
        with torch.cuda.device(blocks.device):
            rc = _lib.lib().coset_e8_encode(_lib.ptr(blocks), _lib.dtype_code(blocks, "grad"), _lib.ptr(s),
                                            _lib.SCALE_MUL_TILE, n, max(n, 1), 4, 2, _lib.SEM_CORE, _lib.ptr(out),
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
    keeps the two-level code away from overload.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, scale: float = 500.0, codec=None,
                 transport: str = "nccl"):
        if transport not in ("nccl", "peer"):
            raise ValueError("transport must be 'nccl' (all-gather, then decode) or 'peer' (decode from peer memory)")
        self.group = group
        self.scale = float(scale)
        self.codec = codec if codec is not None else CudaCodec()
        self.transport = transport
        self._codes = None
        self._gathered = None
        self._symm = {}  # n_blocks -> [buffer [2, n_blocks] int32, handle, parity]; one entry per bucket size

    def _world(self):
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def _buffers(self, n_blocks, world, device):
        if self._codes is None or self._codes.numel() != n_blocks or self._codes.device != device:
            self._codes = torch.empty(n_blocks, dtype=torch.int32, device=device)
        if self._gathered is None or self._gathered.shape != (world, n_blocks) or self._gathered.device != device:
            self._gathered = torch.empty((world, n_blocks), dtype=torch.int32, device=device)
        return self._codes, self._gathered

    def all_reduce_mean(self, flat: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """flat: 1-D float32 (or bfloat16) gradient on this rank -> 1-D average, same length."""
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
        if self.transport == "peer" and world > 1:
            res = self._all_reduce_mean_peer(padded, n_blocks, world)
            res = res.view(-1)[:n_values]
            if out is not None:
                out.copy_(res)
                return out
            return res
        codes, gathered = self._buffers(n_blocks, world, flat.device)
        self.codec.encode(padded.view(n_blocks, 8), self.scale, codes)
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), codes, group=self.group)
        else:
            gathered.view(-1).copy_(codes)
        res = torch.empty((n_blocks, 8), dtype=torch.float32, device=flat.device)
        self.codec.decode_mean(gathered, world, n_blocks, self.scale, res)
        res = res.view(-1)[:n_values]
        if out is not None:
            out.copy_(res)
            return out
        return res


def _peer_exchange(self, padded, n_blocks, world):
    """Encode into this rank's half of a double-buffered symmetric allocation, barrier, decode from
    every rank's buffer.  One barrier per call is enough: a rank overwrites half p only two calls
    later, after the barrier of the call in between, which no rank passes before its own decode of
    half p has been enqueued ahead of it on the same stream."""
    import torch.distributed._symmetric_memory as symm
    dev = padded.device
    if n_blocks not in self._symm:  # collective: every rank sees the same sequence of sizes
        buf = symm.empty(2, n_blocks, dtype=torch.int32, device=dev)
        group = self.group if self.group is not None else dist.group.WORLD
        hdl = symm.rendezvous(buf, group.group_name)
        self._symm[n_blocks] = [buf, hdl, 0]
    entry = self._symm[n_blocks]
    buf, hdl, parity = entry
    entry[2] = parity ^ 1
    self.codec.encode(padded.view(n_blocks, 8), self.scale, buf[parity])
    hdl.barrier(channel=parity)
    res = torch.empty((n_blocks, 8), dtype=torch.float32, device=dev)
    offset = parity * n_blocks * 4
    ptrs = (ctypes.c_void_p * world)(*[int(p) + offset for p in hdl.buffer_ptrs])
    with torch.cuda.device(dev):
        rc = _lib.lib().coset_e8_decode_mean_peers(ctypes.cast(ptrs, ctypes.c_void_p), world, hdl.rank, n_blocks,
                                                   float(self.scale), _lib.ptr(res), _lib.dtype_code(res, "out"),
                                                   _lib.stream())
    _lib.check(rc, "coset_e8_decode_mean_peers")
    return res


E8GradientExchange._all_reduce_mean_peer = _peer_exchange


def e8_allreduce_hook(state: E8GradientExchange, bucket) -> torch.futures.Future[torch.Tensor]:
    """torch DDP communication hook: `ddp.register_comm_hook(E8GradientExchange(group), e8_allreduce_hook)`.

    The bucket's flat gradient is replaced by its E8-quantised average."""
    buf = bucket.buffer()
    avg = state.all_reduce_mean(buf.float() if buf.dtype not in (torch.float32, torch.bfloat16) else buf)
    fut = torch.futures.Future()
    fut.set_result(avg.to(buf.dtype))
    return fut


def bert_base_gradient_numel() -> int:
    """Parameter count of the BERT-base-shaped set used by the gradient-exchange benchmark:
    embeddings 30522/512/2 x 768 + LayerNorm, 12 x (4 attention projections, 2 FFN matrices,
    2 LayerNorms), pooler."""
    h, f, v = 768, 3072, 30522
    emb = v * h + 512 * h + 2 * h + 2 * h
    layer = 4 * (h * h + h) + 2 * h + (h * f + f) + (f * h + h) + 2 * h
    return emb + 12 * layer + h * h + h
