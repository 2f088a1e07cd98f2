"""Helpers shared by the gradient-exchange tests: the CPU recipe (oracle-based) of the exchange."""
import numpy as np
import torch

from oracle import oracle as O


def cpu_decode_mean(codes_per_rank, scale):
    """codes_per_rank: list of float digit arrays [n, 2, 8] -> (sum_r x_hat_r) / RN(scale * W)."""
    total = None
    for c in codes_per_rank:
        xh = O.decode(c)  # exact half-integers
        total = xh if total is None else (total + xh).astype(np.float32)
    div = np.float32(np.float32(scale) * np.float32(len(codes_per_rank)))
    return (total / div).astype(np.float32)


SATURATION = np.float32(3.9)  # coset_b200.gradcomm.SATURATION / COSET_SEM_CORE_SATURATE


def oracle_encode_saturating(blocks, scale):
    """The exchange's encode step on the CPU: x * scale in float32, every value clamped to
    +-SATURATION, then the reference codec without further scaling -> float digits [n, 2, 8]."""
    xs = (np.asarray(blocks, np.float32) * np.float32(scale)).astype(np.float32)
    xs = np.minimum(np.maximum(xs, -SATURATION), SATURATION)
    return O.encode(xs)


class OracleCodec:
    """Drop-in for coset_b200.gradcomm.CudaCodec on CPU tensors (tests of the host logic only)."""

    def encode(self, blocks, scale, out):
        digits = oracle_encode_saturating(blocks.numpy(), scale)
        out.copy_(torch.from_numpy(O.pack_q4(digits).view(np.int32)))
        return out

    def decode_mean(self, codes, world, n_blocks, scale, out):
        per_rank = []
        for r in range(world):
            w = codes[r].numpy().view(np.uint32)
            digits = np.stack([np.stack([(w >> (16 * m + 2 * j)) & 3 for j in range(8)], axis=1) for m in range(2)], axis=1)
            per_rank.append(digits.astype(np.float32))
        out.copy_(torch.from_numpy(cpu_decode_mean(per_rank, scale)))
        return out
