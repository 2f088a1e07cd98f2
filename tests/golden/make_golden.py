"""Generates tests/golden/*.npz by running the UNMODIFIED reference (imported from its source
tree, CPU, float32).  Run once where the reference is mounted:

    python tests/golden/make_golden.py /path/to/reference

The fixtures are small, committed, and are what pins both the CPU oracle and the CUDA library;
nothing at test time reads the reference tree.
"""
import os
import sys
import warnings

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
ref_root = sys.argv[1]
sys.path.insert(0, ref_root)
sys.dont_write_bytecode = True
warnings.filterwarnings("ignore")

from coset.core.base import LatticeConfig  # noqa: E402
from coset.core.e8 import E8Lattice, e8_decode, e8_encode, e8_quantize  # noqa: E402
from coset.core.e8.layers import create_e8_hnlq_linear  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
torch.set_num_threads(4)
L = E8Lattice()

BETA_MID = 0.021440971642732620  # beta(theta=0) of the layer at sigma_ema = xmax_ema = 1, q=4, M=2


def cfg(q=4, M=2, beta=1.0):
    return LatticeConfig(lattice_type="E8", q=q, M=M, beta=beta)


def adversarial_rows():
    rows = []
    e = np.float32(2.0 ** -23)
    base = [0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 3.5, -3.5, 0.0, -0.0, 100.5, -100.5,
            0.5 + 2.0 ** -24, 0.5 + 2.0 ** -23, 0.5 - 2.0 ** -25, 1.5 + 2.0 ** -23, 1.5 - 2.0 ** -23,
            -0.5 - 2.0 ** -24, -0.5 - 2.0 ** -23, -0.5 - 3 * 2.0 ** -24, -1.5 - 2.0 ** -23,
            0.25, -0.25, 0.75, -0.75, 1.0, -1.0, 2.0, -2.0, 1e-8, -1e-8, 1e-30, -1e-30,
            8388608.5, 4194304.5, -4194304.5, 1048576.5, 0.49999997, -0.49999997]
    base = np.array(base, np.float32)
    rng = np.random.default_rng(7)
    # every special value in every position against random companions, plus constant rows
    for v in base:
        rows.append(np.full(8, v, np.float32))
        for pos in range(8):
            r = rng.standard_normal(8).astype(np.float32)
            r[pos] = v
            rows.append(r)
    # all-equal deltas (argmax must take the first index), exact ties between the two cosets
    for v in [0.25, 0.75, -0.25, -0.75, 0.5, 1.25]:
        for k in range(9):
            r = np.full(8, v, np.float32)
            r[:k] += 1.0
            rows.append(r)
    # multiples of 1/8 (what the decoder feeds the search) and small integers / half-integers
    for _ in range(1500):
        rows.append((rng.integers(-16, 17, 8) / 8.0).astype(np.float32))
    for _ in range(500):
        rows.append((rng.integers(-6, 7, 8) / 2.0).astype(np.float32))
    # near-tie between the two cosets: points near deep holes / midpoints
    for _ in range(1500):
        a = rng.integers(-3, 4, 8).astype(np.float32)
        if a.sum() % 2:
            a[0] += 1
        b = a + 0.5
        mid = (a + b) / 2 + rng.standard_normal(8).astype(np.float32) * np.float32(1e-6)
        rows.append(mid.astype(np.float32))
    for _ in range(500):
        r = rng.standard_normal(8).astype(np.float32)
        r[rng.integers(0, 8)] = np.float32(rng.integers(-3, 4) + 0.5) + np.float32(rng.integers(-3, 4)) * e
        rows.append(r)
    return np.stack(rows).astype(np.float32)


def main():
    out = {}
    G, Ginv = L.get_generators()
    out["G"] = G.numpy()
    out["Ginv"] = Ginv.numpy()

    # --- custom_round known answers (reference's own test pins +-0.5 -> 0) ---
    cr_in = adversarial_rows().reshape(-1)
    cr_in = np.unique(cr_in.view(np.uint32)).view(np.float32)
    out["cr_in"] = cr_in
    out["cr_out"] = L.custom_round(torch.from_numpy(cr_in)).numpy()

    # --- projection / g_x ---
    torch.manual_seed(123)
    pj = [adversarial_rows()]
    for s in [0.05, 0.3, 1.0, 3.0, 20.0, 1000.0]:
        pj.append((torch.randn(3000, 8) * s).numpy())
    pj = np.concatenate(pj).astype(np.float32)
    out["proj_in"] = pj
    out["proj_out"] = L.projection(torch.from_numpy(pj)).numpy()
    out["gx_out"] = L.g_x(torch.from_numpy(pj)).numpy()

    # --- encode/decode: config-1 input (seed 0, N(0,1), clip +-2), first 8192 rows ---
    torch.manual_seed(0)
    x = torch.randn(65536, 8).clamp_(-2, 2)
    xs = x[:8192].contiguous()
    out["cfg1_x"] = xs.numpy()
    bm = torch.tensor(BETA_MID, dtype=torch.float32)
    for name, s in [("s0p25", 0.25), ("s0p5", 0.5), ("s1", 1.0), ("s2", 2.0), ("s4", 4.0), ("s8", 8.0)]:
        codes, _ = e8_encode(xs * s, cfg())
        out[f"cfg1_codesA_{name}"] = codes.numpy().astype(np.int8)
        out[f"cfg1_xhatA_{name}"] = e8_decode(codes, cfg()).numpy()
    # convention A literal (layer): x*beta_mid, all-zero codes
    codes, _ = e8_encode(xs * bm, cfg())
    out["cfg1_codesA_lit"] = codes.numpy().astype(np.int8)
    out["cfg1_xhatA_lit"] = (e8_decode(codes, cfg()) / bm).numpy()
    # convention B (codec): x / beta
    for name, b in [("mid", BETA_MID), ("0p3", 0.3), ("1p7", 1.7)]:
        codes, _ = e8_encode(xs, cfg(beta=b))
        out[f"cfg1_codesB_{name}"] = codes.numpy().astype(np.int8)
        out[f"cfg1_xhatB_{name}"] = e8_decode(codes, cfg(beta=b)).numpy()
    # other (q, M)
    for q, M in [(2, 1), (3, 2), (4, 1), (4, 3), (5, 2), (8, 2), (16, 2)]:
        codes, _ = e8_encode(xs[:2048] * 3.0, cfg(q=q, M=M, beta=0.7))
        out[f"qm_codes_{q}_{M}"] = codes.numpy().astype(np.int8)
        out[f"qm_xhat_{q}_{M}"] = e8_decode(codes, cfg(q=q, M=M, beta=0.7)).numpy()
    # adversarial rows through the whole codec
    adv = torch.from_numpy(adversarial_rows())
    adv = adv[(adv.abs().amax(dim=1) < 1e6)]
    out["adv_x"] = adv.numpy()
    codes, _ = e8_encode(adv, cfg())
    out["adv_codes"] = codes.numpy().astype(np.int8)
    out["adv_xhat"] = e8_decode(codes, cfg()).numpy()
    out["adv_quant"] = e8_quantize(adv, 4).numpy()

    # e8_quantize
    out["cfg1_quant_s1"] = e8_quantize(xs, 4).numpy()
    out["cfg1_quant_s4"] = e8_quantize(xs * 4.0, 4).numpy()
    np.savez_compressed(os.path.join(OUT, "codec.npz"), **out)

    # --- exhaustive single-level decode: all 4^8 codes -> residual G b - 4 Q(G b / 4) ---
    idx = np.arange(65536, dtype=np.int64)
    digits = np.stack([(idx >> (2 * j)) & 3 for j in range(8)], axis=1).astype(np.float32)
    res = e8_decode(torch.from_numpy(digits).unsqueeze(1), cfg(M=1)).numpy()
    assert (res * 2 == np.round(res * 2)).all()
    np.savez_compressed(os.path.join(OUT, "decode_q4_exhaustive.npz"), twice_residual=(res * 2).astype(np.int8))

    # --- layer: row tiling through the reference layer, block tiling through reference functions ---
    lay = {}
    for tag, std, (o, i) in [("small", 0.02, (48, 64)), ("big", 20.0, (48, 64)), ("mid", 1.0, (32, 128))]:
        torch.manual_seed(0)
        layer = create_e8_hnlq_linear(i, o, q=4, M=2, init_kwargs={"std": std})
        torch.manual_seed(1)
        with torch.no_grad():
            layer.theta_beta.copy_(torch.randn(o) * 0.5)
            layer.sigma_ema.copy_(torch.rand(o) * (0.01 if tag == "mid" else 1.0) + 0.005)
            layer.xmax_ema.copy_(layer.sigma_ema * 3.0)
        xin = torch.randn(16, i)
        tgt = torch.randn(16, o)
        bmin, bmax = layer._bounds()
        beta = bmin + torch.sigmoid(layer.theta_beta) * (bmax - bmin)
        y = layer(xin)
        loss = ((y - tgt) ** 2).mean()
        loss.backward()
        xin2 = xin.clone().requires_grad_(True)
        layer.zero_grad()
        layer.step_count.zero_()
        y2 = layer(xin2)
        ((y2 - tgt) ** 2).mean().backward()
        lay[f"{tag}_W"] = layer.weight.detach().numpy()
        lay[f"{tag}_bias"] = layer.bias.detach().numpy()
        lay[f"{tag}_theta"] = layer.theta_beta.detach().numpy()
        lay[f"{tag}_sigma"] = layer.sigma_ema.numpy()
        lay[f"{tag}_xmax"] = layer.xmax_ema.numpy()
        lay[f"{tag}_beta"] = beta.detach().numpy()
        lay[f"{tag}_bmin"] = bmin.numpy()
        lay[f"{tag}_bmax"] = bmax.numpy()
        lay[f"{tag}_x"] = xin.numpy()
        lay[f"{tag}_t"] = tgt.numpy()
        lay[f"{tag}_y"] = y2.detach().numpy()
        layer.step_count.zero_()
        lay[f"{tag}_Wq"] = layer._quantize_weights().detach().numpy()
        lay[f"{tag}_dW"] = layer.weight.grad.numpy()
        lay[f"{tag}_dtheta"] = layer.theta_beta.grad.numpy()
        lay[f"{tag}_dbias"] = layer.bias.grad.numpy()
        lay[f"{tag}_dx"] = xin2.grad.numpy()
        lay[f"{tag}_Delta0"] = np.float64(layer.Delta0)
        lay[f"{tag}_gamma_inv"] = layer.gamma_inv.numpy()
        # block tiling: the reference layer raises at the rescale step, so the expected values
        # are assembled from reference functions (e8_quantize on W*beta, then /beta, clamp)
        torch.manual_seed(2)
        W = layer.weight.detach().clone().requires_grad_(True)
        beta_b = (beta.detach().view(o, 1).expand(o, i // 8) * (0.5 + torch.rand(o, i // 8))).contiguous()
        beta_b.requires_grad_(True)
        from coset.core.layers import ste_quantize
        Wb = W.view(o, i // 8, 8) * beta_b.view(o, i // 8, 1)
        Wq = ste_quantize(Wb.reshape(-1, 8), e8_quantize, 4).view(o, i // 8, 8) / beta_b.view(o, i // 8, 1)
        Wq = torch.clamp(Wq.reshape(o, i), -2.0, 2.0)
        yb = torch.nn.functional.linear(xin, Wq, layer.bias.detach())
        ((yb - tgt) ** 2).mean().backward()
        lay[f"{tag}_blk_beta"] = beta_b.detach().numpy()
        lay[f"{tag}_blk_Wq"] = Wq.detach().numpy()
        lay[f"{tag}_blk_dW"] = W.grad.numpy()
        lay[f"{tag}_blk_dbeta"] = beta_b.grad.numpy()
    np.savez_compressed(os.path.join(OUT, "layer.npz"), **lay)
    for f in ["codec.npz", "decode_q4_exhaustive.npz", "layer.npz"]:
        print(f, os.path.getsize(os.path.join(OUT, f)))


if __name__ == "__main__":
    main()
