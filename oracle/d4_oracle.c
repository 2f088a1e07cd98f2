/*
 * CPU restatement of the reference's D4 lattice path and of the Babai projection.
 *
 * TEST INFRASTRUCTURE ONLY: checked against fixtures produced by the reference
 * (tests/golden/d4.npz) and used by the tests as the expectation for the CUDA kernels.  Nothing
 * in the shipped library links or calls it.
 *
 * Each function performs the same IEEE binary32 operations, in the same order, as the torch CPU
 * op chain it restates (file:line per function).  Built with -ffp-contract=off.
 */
#include <math.h>
#include <stdint.h>

#define D4_D 4

float e8o_custom_round(float x); /* coset/core/base.py:179-202, shared with the E8 oracle */

static int d4_argmax_first(const float* v) {
    int k = 0;
    float best = v[0];
    if (best != best) return 0;
    for (int i = 1; i < D4_D; ++i) {
        if (v[i] != v[i]) return i;
        if (v[i] > best) { best = v[i]; k = i; }
    }
    return k;
}

/* D4Lattice.g_x (coset/core/d4/lattice.py:62-109): the coordinate with the largest |x - f| moves by
 * +1 only under `flip_positive` (x_k >= 0 and f_k < x_k); every other row gets -1, the
 * `flip_negative` mask being computed and not used (lattice.py:97-104). */
void d4o_g_x(const float* x, float* out) {
    float f[D4_D], delta[D4_D];
    for (int i = 0; i < D4_D; ++i) {
        f[i] = e8o_custom_round(x[i]);
        delta[i] = fabsf(x[i] - f[i]);
        out[i] = f[i];
    }
    int k = d4_argmax_first(delta);
    int flip_positive = (x[k] >= 0.0f) && (f[k] < x[k]);
    out[k] = flip_positive ? out[k] + 1.0f : out[k] - 1.0f;
}

/* D4Lattice.projection (coset/core/d4/lattice.py:111-146): f = custom_round(x) if its coordinate
 * sum is even (python float `% 2 == 0`), else g_x(x). */
void d4o_projection(const float* x, float* out) {
    float f[D4_D], s = 0.0f;
    for (int i = 0; i < D4_D; ++i) {
        f[i] = e8o_custom_round(x[i]);
        s = s + f[i];
    }
    float r = fmodf(s, 2.0f);
    if (r != 0.0f && ((r < 0.0f) != (2.0f < 0.0f))) r += 2.0f;
    if (r == 0.0f) {
        for (int i = 0; i < D4_D; ++i) out[i] = f[i];
    } else {
        d4o_g_x(x, out);
    }
}

void d4o_projection_rows(const float* x, int64_t n, float* out) {
    for (int64_t b = 0; b < n; ++b) d4o_projection(x + b * D4_D, out + b * D4_D);
}

void d4o_g_x_rows(const float* x, int64_t n, float* out) {
    for (int64_t b = 0; b < n; ++b) d4o_g_x(x + b * D4_D, out + b * D4_D);
}

/* Weight path of HNLQLinearQAT built by create_d4_hnlq_linear (coset/core/d4/layers.py:15-68;
 * coset/core/layers.py:429-463): clamp(projection(W * beta) / beta, +-clip), one beta per
 * `blocks_per_tile` blocks of 4.  `unclipped` (optional) receives the value before the clamp. */
void d4o_fake_quant(const float* w, int64_t n, const float* beta, int64_t blocks_per_tile, float clip, float* wq,
                    float* unclipped) {
    for (int64_t b = 0; b < n; ++b) {
        float xs[D4_D], p[D4_D];
        float bt = beta[b / blocks_per_tile];
        for (int i = 0; i < D4_D; ++i) xs[i] = w[b * D4_D + i] * bt;
        d4o_projection(xs, p);
        for (int i = 0; i < D4_D; ++i) {
            float v = p[i] / bt;
            if (unclipped) unclipped[b * D4_D + i] = v;
            float c = v < -clip ? -clip : (v > clip ? clip : v);
            if (v != v) c = v;
            wq[b * D4_D + i] = c;
        }
    }
}

/* Babai projection (pub/main.tex, algorithm "Babai projection onto E8"; ref/qat_auto.py:120-124):
 * z = Ginv x, z_hat = round_half_even(z / step) * step, y = G z_hat, for a d x d generator given
 * row-major (basis vectors as columns, like Lattice.G).  Products and sums are rounded separately
 * and accumulated left to right. */
void lato_babai(const float* x, int64_t n, int d, const float* G, const float* Ginv, float step, float* out) {
    for (int64_t b = 0; b < n; ++b) {
        float z[8];
        for (int a = 0; a < d; ++a) {
            float acc = 0.0f;
            for (int i = 0; i < d; ++i) acc = acc + Ginv[a * d + i] * x[b * d + i];
            z[a] = rintf(acc / step) * step;
        }
        for (int a = 0; a < d; ++a) {
            float acc = 0.0f;
            for (int i = 0; i < d; ++i) acc = acc + G[a * d + i] * z[i];
            out[b * d + a] = acc;
        }
    }
}
