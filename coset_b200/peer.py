"""Symmetric (peer-mapped) device memory with the library's own bounded cross-rank arrival.

Every rank allocates the same number of bytes through torch.distributed._symmetric_memory, which
maps all ranks' buffers into every process; the last 64 bytes of each buffer are that rank's arrival
words.  `arrive()` enqueues coset_peer_signal_wait on the current stream: "everything I wrote before
this point is visible to my peers, and every peer has reached the same point".  The wait inside that
kernel is bounded (default 2 s): when a peer never arrives the kernel records it in `status` and
returns, the kernels that follow check `status` before touching a peer's data, and `check()` raises
on the host -- no GPU is left spinning on a rank that died.
"""
import ctypes

import torch
import torch.distributed as dist

from . import _lib

_FLAG_BYTES = 64  # 16 arrival words: coset_peer_signal_wait handles up to 16 ranks


class SymmetricRegion:
    """`nbytes` of symmetric memory per rank plus the arrival words.  Construction is collective."""

    def __init__(self, nbytes: int, device, group=None, timeout_ms: int = 2000):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 16:
            raise ValueError("the peer-memory transport handles at most 16 ranks")
        self.nbytes = (int(nbytes) + 15) // 16 * 16
        self.timeout_ms = int(timeout_ms)
        self.buffer = symm.empty(self.nbytes + _FLAG_BYTES, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buffer, self.group.group_name)
        self.base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[p + self.nbytes for p in self.base_ptrs])
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        # arrival words start at zero on every rank before anyone signals
        self.buffer[self.nbytes:].zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def data(self, dtype=torch.uint8):
        return self.buffer[:self.nbytes].view(dtype)

    def pointers(self, byte_offset: int = 0):
        """ctypes array of every rank's buffer address (+ offset), for the kernels that take peer pointers."""
        return (ctypes.c_void_p * self.world)(*[p + int(byte_offset) for p in self.base_ptrs])

    def arrive(self):
        """Enqueue the bounded arrival on the current stream (collective: every rank calls it once per step)."""
        self.epoch = (self.epoch + 1) & 0xFFFFFFFF
        with torch.cuda.device(self.buffer.device):
            rc = _lib.lib().coset_peer_signal_wait(ctypes.cast(self._flag_ptrs, ctypes.c_void_p), self.world, self.rank,
                                                   self.epoch, self.timeout_ms, _lib.ptr(self.status), _lib.stream())
        _lib.check(rc, "coset_peer_signal_wait")

    def check(self):
        """Synchronises and raises if a bounded wait gave up since the last check."""
        s = int(self.status.item())
        if s != 0:
            self.status.zero_()
            raise RuntimeError(f"peer-memory arrival timed out after {self.timeout_ms} ms: rank {s - 1} did not arrive; "
                               "results produced since the last check are invalid")
