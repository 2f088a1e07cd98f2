"""Small fixed case of the fused tcgen05 dequant-GEMM for profiling:
    python -m coset_b200.benchmarks_profile_gemm          (T = 2048, W 4096 x 4096, per-block scales)
Runs the kernel three times and checks its status word."""
import torch

from .vlut import E8CodeLinear, e8_dequant_gemm


def main():
    torch.manual_seed(0)
    n = 4096
    W = (torch.randn(n, n) * 0.02).cuda()
    beta = torch.full((n * n // 8,), 25.0, device="cuda")
    lin = E8CodeLinear.from_weight(W, beta, 1)
    x = torch.randn(2048, n, device="cuda").to(torch.bfloat16)
    for _ in range(3):
        e8_dequant_gemm(lin.codes, lin.beta, 1, x, None, check=True)
    torch.cuda.synchronize()
    print("ok")


if __name__ == "__main__":
    main()
