"""Golden vectors of the D4 lattice path (coset/core/d4) and of the Babai projection, produced by
the unmodified reference:  python tests/golden/make_golden_d4.py /path/to/reference"""
import os
import sys
import warnings

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden_d4.py /path/to/reference")
ref_root = sys.argv[1]
sys.path.insert(0, ref_root)
sys.dont_write_bytecode = True
warnings.filterwarnings("ignore")
from coset.core.d4 import D4Lattice, create_d4_hnlq_linear  # noqa: E402
from coset.core.e8 import E8Lattice  # noqa: E402
from coset.core.layers import ste_quantize  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
torch.set_num_threads(1)
out = {}
lat = D4Lattice()
out["G"] = lat.G.numpy()
out["G_inv"] = lat.G_inv.numpy()
out["r_pack"] = np.float64(lat.r_pack)
out["r_cov"] = np.float64(lat.r_cov)
out["delta0_q4_M2"] = np.float64(lat.compute_delta0(4, 2))

# --- projection / g_x: random inputs at several scales plus rows on the decision boundaries
g = torch.Generator().manual_seed(0)
rows = [torch.randn(2500, 4, generator=g) * s for s in (0.3, 1.0, 4.0, 50.0)]
grid = torch.tensor([-2.5, -1.5, -1.0, -0.5, 0.0, 0.25, 0.5, 1.0, 1.5])
adv = torch.cartesian_prod(grid, grid, grid, grid)  # every tie pattern of halves and integers
eps = torch.tensor([1.1920929e-07, -1.1920929e-07, 5.9604645e-08, 0.0])
rows += [adv, adv + eps, adv - eps, adv * 0.5, torch.zeros(3, 4), -torch.zeros(3, 4)]
x = torch.cat(rows).contiguous()
out["x"] = x.numpy()
out["projection"] = lat.projection(x).numpy()
out["g_x"] = lat.g_x(x).numpy()
out["custom_round"] = lat.custom_round(x).numpy()

# --- layer: row tiling through the reference layer, block tiling through reference functions
for tag, std, (o, i) in [("small", 0.02, (24, 64)), ("big", 20.0, (24, 64)), ("mid", 1.0, (16, 128))]:
    torch.manual_seed(0)
    layer = create_d4_hnlq_linear(i, o, q=4, M=2, init_kwargs={"std": std})
    torch.manual_seed(1)
    with torch.no_grad():
        layer.theta_beta.copy_(torch.randn(o) * 0.5)
        layer.sigma_ema.copy_(torch.rand(o) * (0.01 if tag == "mid" else 1.0) + 0.005)
        layer.xmax_ema.copy_(layer.sigma_ema * 3.0)
    xin = torch.randn(16, i)
    tgt = torch.randn(16, o)
    bmin, bmax = layer._bounds()
    beta = bmin + torch.sigmoid(layer.theta_beta) * (bmax - bmin)
    xin2 = xin.clone().requires_grad_(True)
    y = layer(xin2)
    ((y - tgt) ** 2).mean().backward()
    out[f"{tag}_W"] = layer.weight.detach().numpy()
    out[f"{tag}_bias"] = layer.bias.detach().numpy()
    out[f"{tag}_theta"] = layer.theta_beta.detach().numpy()
    out[f"{tag}_sigma"] = layer.sigma_ema.numpy()
    out[f"{tag}_xmax"] = layer.xmax_ema.numpy()
    out[f"{tag}_beta"] = beta.detach().numpy()
    out[f"{tag}_x"] = xin.numpy()
    out[f"{tag}_t"] = tgt.numpy()
    out[f"{tag}_y"] = y.detach().numpy()
    out[f"{tag}_dW"] = layer.weight.grad.numpy().copy()
    out[f"{tag}_dtheta"] = layer.theta_beta.grad.numpy().copy()
    out[f"{tag}_dbias"] = layer.bias.grad.numpy().copy()
    out[f"{tag}_dx"] = xin2.grad.numpy()
    layer.step_count.zero_()
    out[f"{tag}_Wq"] = layer._quantize_weights().detach().numpy()
    out[f"{tag}_Delta0"] = np.float64(layer.Delta0)
    out[f"{tag}_gamma_inv"] = layer.gamma_inv.numpy()
    # block tiling: the reference layer raises at its rescale step, so the expectation is
    # assembled from reference functions (projection on W*beta, then /beta, clamp)
    torch.manual_seed(2)
    W = layer.weight.detach().clone().requires_grad_(True)
    beta_b = (beta.detach().view(o, 1).expand(o, i // 4) * (0.5 + torch.rand(o, i // 4))).contiguous()
    beta_b.requires_grad_(True)
    Wb = W.view(o, i // 4, 4) * beta_b.view(o, i // 4, 1)
    Wq = ste_quantize(Wb.reshape(-1, 4), lambda v, q: lat.projection(v), 4).view(o, i // 4, 4) / beta_b.view(o, i // 4, 1)
    Wq = torch.clamp(Wq.reshape(o, i), -2.0, 2.0)
    yb = torch.nn.functional.linear(xin, Wq, layer.bias.detach())
    ((yb - tgt) ** 2).mean().backward()
    out[f"{tag}_blk_beta"] = beta_b.detach().numpy()
    out[f"{tag}_blk_Wq"] = Wq.detach().numpy()
    out[f"{tag}_blk_dW"] = W.grad.numpy()
    out[f"{tag}_blk_dbeta"] = beta_b.grad.numpy()

# --- Babai projection (pub/main.tex "Babai projection onto E8"; ref/qat_auto.py:120-124):
# z = x Ginv^T, z_hat = round(z / step) * step, y = z_hat G^T, evaluated in float64 so that the
# fixture does not depend on a BLAS summation order; rows whose z/step comes within 1e-4 of a
# rounding boundary are flagged for the tests to skip in float32.
for name, L in (("e8", E8Lattice()), ("d4", lat)):
    d = L.d
    g = torch.Generator().manual_seed(7)
    xb = (torch.randn(2000, d, generator=g) * 1.5).double()
    G, Ginv = L.G.double(), L.G_inv.double()
    for step in (1.0, 0.25):
        z = xb @ Ginv.T / step
        frac = (z - torch.floor(z) - 0.5).abs().min(dim=1).values
        y = (torch.round(z) * step) @ G.T
        out[f"babai_{name}_step{step}_y"] = y.numpy()
        out[f"babai_{name}_step{step}_safe"] = (frac > 1e-4).numpy()
    out[f"babai_{name}_x"] = xb.float().numpy()

np.savez_compressed(os.path.join(OUT, "d4.npz"), **out)
print(len(x), os.path.getsize(os.path.join(OUT, "d4.npz")))
