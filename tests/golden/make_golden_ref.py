"""Golden vectors of the paper-faithful quantiser ref/hnlq.py (numpy, per vector), produced by the
unmodified reference:  python tests/golden/make_golden_ref.py /path/to/reference"""
import os
import sys
import warnings

import numpy as np

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden_ref.py /path/to/reference")
ref_root = sys.argv[1]
sys.path.insert(0, ref_root)
sys.dont_write_bytecode = True
warnings.filterwarnings("ignore")
from ref.hnlq import HNLQ  # noqa: E402
from ref.utils import generate_tie_dither  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
rng = np.random.default_rng(0)
x = np.clip(rng.standard_normal((1500, 8)), -2, 2)
out = {"x": x, "tie_dither": generate_tie_dither(8)}
cases = [("b1", 1.0, True, 4, 2, 1.0), ("b025", 0.25, True, 4, 2, 1.0), ("b025_noover", 0.25, False, 4, 2, 1.0),
         ("b01", 0.1, True, 4, 2, 1.0), ("q3m3", 0.5, True, 3, 3, 1.0), ("b4", 4.0, True, 4, 2, 1.0)]
for tag, beta, over, q, M, alpha in cases:
    h = HNLQ.create_e8_quantizer(q=q, M=M, beta=beta, alpha=alpha, overload=over)
    digits = np.empty((len(x), M, 8), np.int32)
    T = np.empty(len(x), np.int32)
    xh = np.empty((len(x), 8))
    for i, v in enumerate(x):
        b_list, t = h.encode(v)
        digits[i] = np.stack(b_list)
        T[i] = t
        xh[i] = h.decode(b_list, t)
    out[f"{tag}_digits"], out[f"{tag}_T"], out[f"{tag}_xhat"] = digits, T, xh
    out[f"{tag}_params"] = np.array([beta, alpha, q, M, float(over)])
    print(tag, "T>0:", (T > 0).mean(), "max digit", digits.max())
np.savez_compressed(os.path.join(OUT, "ref_mode.npz"), **out)
print(os.path.getsize(os.path.join(OUT, "ref_mode.npz")))

# decode_coarse_to_fine / decode_progressive (ref/hnlq.py:447-536) on the codes above
coarse = {}
n_c = 400
for tag, beta, over, q, M, alpha in cases:
    if tag not in ("b025", "q3m3", "b01"):
        continue
    h = HNLQ.create_e8_quantizer(q=q, M=M, beta=beta, alpha=alpha, overload=over)
    digits, T = out[f"{tag}_digits"], out[f"{tag}_T"]
    res = np.empty((M, n_c, 8))
    for i in range(n_c):
        b_list = tuple(digits[i, m] for m in range(M))
        prog = h.decode_progressive(b_list, int(T[i]))
        for depth in range(1, M + 1):
            one = h.decode_coarse_to_fine(b_list, int(T[i]), depth=depth)
            assert np.array_equal(one, prog[depth - 1])
            res[depth - 1, i] = one
        assert np.array_equal(res[M - 1, i], out[f"{tag}_xhat"][i])
    coarse[f"{tag}_by_depth"] = res
np.savez_compressed(os.path.join(OUT, "ref_coarse.npz"), **coarse)
print(os.path.getsize(os.path.join(OUT, "ref_coarse.npz")))
