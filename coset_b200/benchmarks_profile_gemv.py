"""Small fixed case of the few-token code-domain product for profiling:
    python -m coset_b200.benchmarks_profile_gemv          (T = 1, W 4096 x 4096, per-block scales)
Runs the layer five times."""
import torch

from .vlut import E8CodeLinear


def main():
    torch.manual_seed(0)
    n = 4096
    W = (torch.randn(n, n) * 0.02).cuda()
    beta = torch.full((n * n // 8,), 25.0, device="cuda")
    lin = E8CodeLinear.from_weight(W, beta, 1)
    x = torch.randn(1, n, device="cuda").to(torch.bfloat16)
    for _ in range(5):
        lin(x)
    torch.cuda.synchronize()
    print("ok")


if __name__ == "__main__":
    main()
