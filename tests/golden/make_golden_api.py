"""Generates tests/golden/api.npz by running the UNMODIFIED reference layer (CPU, float32):

    python tests/golden/make_golden_api.py /path/to/reference

  * ema_*   : the statistics update of HNLQLinearQAT (coset/core/layers.py:366-379, 409-413): 512
              quantised forwards of a 24 x 32 layer with a weight change after forward 300, the two
              EMA buffers and the bounds after forward 256 and after forward 512
  * lsq_*   : LSQActivation forward / backward (coset/core/layers.py:117-137)
  * qa_*    : a layer with quantize_activations=True (coset/core/layers.py:481-482)
  * diag_*  : the get_* diagnostics and export_quantized of a layer (coset/core/layers.py:509-650)
  * dec_*   : E8Decoder.decode / DecodingMethod (coset/core/e8/codecs.py:99-180)
Nothing at test time reads the reference tree.
"""
import os
import sys
import warnings

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden_api.py /path/to/reference")
sys.path.insert(0, sys.argv[1])
sys.dont_write_bytecode = True
warnings.filterwarnings("ignore")

from coset.core.base import LatticeConfig  # noqa: E402
from coset.core.e8 import e8_encode  # noqa: E402
from coset.core.e8.codecs import DecodingMethod, E8Decoder  # noqa: E402
from coset.core.e8.layers import create_e8_hnlq_linear  # noqa: E402
from coset.core.layers import LSQActivation  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
torch.set_num_threads(4)
out = {}

# ---- EMA statistics
torch.manual_seed(0)
layer = create_e8_hnlq_linear(32, 24, q=4, M=2, init_kwargs={"std": 0.7})
torch.manual_seed(1)
x = torch.randn(4, 32)
delta = torch.randn(24, 32) * 0.5
out["ema_W0"] = layer.weight.detach().numpy().copy()
out["ema_delta"] = delta.numpy()
out["ema_x"] = x.numpy()
with torch.no_grad():
    for step in range(1, 513):
        y = layer(x)
        if step == 300:
            layer.weight.add_(delta)
        if step in (256, 512):
            bmin, bmax = layer._bounds()
            out[f"ema_sigma_{step}"] = layer.sigma_ema.numpy().copy()
            out[f"ema_xmax_{step}"] = layer.xmax_ema.numpy().copy()
            out[f"ema_bmin_{step}"] = bmin.numpy().copy()
            out[f"ema_bmax_{step}"] = bmax.numpy().copy()
            out[f"ema_y_{step}"] = y.numpy().copy()
out["ema_step_count"] = np.int64(int(layer.step_count))

# ---- LSQ activation quantiser
for tag, bits, alpha in (("a", 8, 1.3), ("b", 4, 0.7)):
    torch.manual_seed(2)
    act = LSQActivation(bits, alpha)
    xa = (torch.randn(64, 16) * 2).requires_grad_(True)
    t = torch.randn(64, 16)
    ya = act(xa)
    (ya * t).sum().backward()
    out[f"lsq_{tag}_x"] = xa.detach().numpy()
    out[f"lsq_{tag}_t"] = t.numpy()
    out[f"lsq_{tag}_y"] = ya.detach().numpy()
    out[f"lsq_{tag}_dx"] = xa.grad.numpy()
    out[f"lsq_{tag}_dalpha"] = act.alpha.grad.numpy()

# ---- layer with activation quantisation
torch.manual_seed(3)
qa = create_e8_hnlq_linear(32, 16, q=4, M=2, init_kwargs={"std": 20.0}, quantize_activations=True, act_bit_width=6, act_init_alpha=2.5)
xq = torch.randn(8, 32)
tq = torch.randn(8, 16)
yq = qa(xq)
((yq - tq) ** 2).mean().backward()
out["qa_W"] = qa.weight.detach().numpy()
out["qa_x"], out["qa_t"], out["qa_y"] = xq.numpy(), tq.numpy(), yq.detach().numpy()
out["qa_dW"] = qa.weight.grad.numpy()
out["qa_dalpha"] = qa.actq.alpha.grad.numpy()
out["qa_dtheta"] = qa.theta_beta.grad.numpy()

# ---- diagnostics and the dense export
torch.manual_seed(4)
dg = create_e8_hnlq_linear(64, 24, q=4, M=2, init_kwargs={"std": 20.0}, enable_diagnostics=True)
out["diag_W"] = dg.weight.detach().numpy()
stats = dg.get_weight_statistics()
for k, v in stats.items():
    out[f"diag_stat_{k}"] = np.float64(v)
out["diag_quantiles"] = dg.get_weight_quantiles().numpy()
out["diag_qerr"] = np.float64(dg.get_quantization_error())
out["diag_bits"] = np.float64(dg.get_effective_bits())
out["diag_sparsity"] = np.float64(dg.get_sparsity_ratio())
cmp = dg.compare_weights()
for k, v in cmp.items():
    out[f"diag_cmp_{k}"] = np.float64(v)
clipst = dg.get_weight_clipping_stats()
for k, v in clipst.items():
    out[f"diag_clip_{k}"] = np.float64(v)
hist, edges = dg.get_quantization_histogram(bins=20)
out["diag_hist"], out["diag_edges"] = hist.numpy(), edges.numpy()
ex = dg.export_quantized()
out["diag_export_weight"] = ex["weight"].detach().numpy()
out["diag_export_meta_q"] = np.int64(ex["metadata"]["q"])
lin = torch.nn.Linear(64, 24)
dg.load_from_linear(lin)
out["diag_lin_W"], out["diag_lin_b"] = lin.weight.detach().numpy(), lin.bias.detach().numpy()
out["diag_after_load_Wq"] = dg._quantize_weights().detach().numpy()

# ---- decoder class
torch.manual_seed(5)
c = LatticeConfig(lattice_type="E8", q=4, M=2, beta=0.5)
xd = torch.randn(300, 8)
b, _ = e8_encode(xd, c)
out["dec_x"], out["dec_codes"] = xd.numpy(), b.numpy()
out["dec_xhat"] = E8Decoder(torch.device("cpu")).decode(b, c, method=DecodingMethod.FULL).numpy()

np.savez_compressed(os.path.join(OUT, "api.npz"), **out)
print("api.npz", len(out), "arrays", os.path.getsize(os.path.join(OUT, "api.npz")), "bytes")
