// Literal device restatement of the reference's float32 E8 search, one rounding per operation.
//
// Every function performs the same IEEE binary32 operations, in the same order, as the torch
// CPU op chain it replaces (file:line given per function), so results are bit-identical on the
// exactness domain (finite inputs, |x| <= 2^20).  No FMA contraction: all arithmetic that has to
// round like the reference uses the __f*_rn intrinsics, which the compiler never fuses.
//
// These are the "always correct" paths: the generic (q, M) kernels use them directly and the
// tuned q=4 kernels fall back to them whenever their cheaper evaluation cannot prove its result.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace e8 {

// Lattice.custom_round (coset/core/base.py:179-202):
// y = x - sign(x) * eps32 ; floor(y + 0.5), two separately rounded adds.
__device__ __forceinline__ float custom_round(float x) {
    const float eps = 1.1920928955078125e-07f;
    float s = (x > 0.0f) ? eps : ((x < 0.0f) ? -eps : __fmul_rn(x, 0.0f));
    float y = __fsub_rn(x, s);
    float t = __fadd_rn(y, 0.5f);
    return floorf(t);
}

// First index of the maximum of v[0..7]; NaN counts as the maximum (torch.argmax).
__device__ __forceinline__ int argmax_first(const float (&v)[8]) {
    int k = 0;
    float best = v[0];
    bool done = (best != best);
#pragma unroll
    for (int i = 1; i < 8; ++i) {
        bool isn = (v[i] != v[i]);
        bool take = !done && (isn || v[i] > best);
        if (take) { best = v[i]; k = i; }
        done = done || isn;
    }
    return k;
}

// E8Lattice.g_x (coset/core/e8/lattice.py:67-112) applied on top of f = custom_round(x):
// the coordinate with the largest |x - f| (first index on ties) moves by +1 only when
// x_k >= 0 and f_k < x_k, and by -1 in every other case (the reference ignores its
// flip_negative mask, lattice.py:102-107).
__device__ __forceinline__ void g_x_inplace(const float (&x)[8], float (&f)[8]) {
    float delta[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) delta[i] = fabsf(__fsub_rn(x[i], f[i]));
    int k = argmax_first(delta);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (i == k) {
            bool up = (x[i] >= 0.0f) && (f[i] < x[i]);
            f[i] = up ? __fadd_rn(f[i], 1.0f) : __fsub_rn(f[i], 1.0f);
        }
    }
}

// torch.norm(v, dim=-1) over 8 contiguous float32 on the CPU: sqrt of the left-to-right
// float32 sum of separately rounded squares.
__device__ __forceinline__ float norm8(const float (&v)[8]) {
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = __fadd_rn(acc, __fmul_rn(v[i], v[i]));
    return __fsqrt_rn(acc);
}

__device__ __forceinline__ bool even_sum(const float (&f)[8]) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s = __fadd_rn(s, f[i]);
    return fmodf(s, 2.0f) == 0.0f;  // python float `% 2 == 0`; NaN/inf -> false
}

// E8Lattice.projection (coset/core/e8/lattice.py:114-169).
// Returns true when the half-integer coset D8 + 1/2 was chosen (dist0 < dist1 is false).
__device__ __forceinline__ bool projection(const float (&x)[8], float (&y)[8]) {
    float y0[8], xs[8], y1[8], e0[8], e1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y0[i] = custom_round(x[i]);
    if (!even_sum(y0)) g_x_inplace(x, y0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        xs[i] = __fsub_rn(x[i], 0.5f);
        y1[i] = custom_round(xs[i]);
    }
    if (!even_sum(y1)) g_x_inplace(xs, y1);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        y1[i] = __fadd_rn(y1[i], 0.5f);
        e0[i] = __fsub_rn(x[i], y0[i]);
        e1[i] = __fsub_rn(x[i], y1[i]);
    }
    bool closer0 = norm8(e0) < norm8(e1);
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = closer0 ? y0[i] : y1[i];
    return !closer0;
}

__device__ __forceinline__ int floored_mod(int a, int q) {
    int r = a % q;
    return r < 0 ? r + q : r;
}

// Lattice.encode_coords (coset/core/base.py:134-154) for a lattice point y = h + c/2:
// round(G^-1 y) mod q.  G^-1 has the suffix-sum structure
//   z7 = 2 y7,  zj = sum_{i=j..6} yi - (7-j) y7  (j = 1..6),  z0 = (sum_{i<7} yi - 7 y7) / 2,
// and every z is an integer for y in E8, so the float matmul + round of the reference equals
// this integer evaluation.  digits[j] in [0, q).
__device__ __forceinline__ void encode_coords(const float (&y)[8], bool half, int q, int (&digits)[8]) {
    int h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = __float2int_rd(y[i]);
    int c = half ? 1 : 0;
    int s = 0;
    digits[7] = floored_mod(2 * h[7] + c, q);
#pragma unroll
    for (int j = 6; j >= 1; --j) {
        s += h[j];
        digits[j] = floored_mod(s - (7 - j) * h[7], q);
    }
    s += h[0];
    digits[0] = floored_mod((s - 7 * h[7]) >> 1, q);
}

// Lattice.decode_coords (coset/core/base.py:156-176): p = G b (exact in float32).
__device__ __forceinline__ void decode_coords(const int (&b)[8], float (&p)[8]) {
    float hb = __fmul_rn(0.5f, (float)b[7]);
    p[0] = __fadd_rn((float)(2 * b[0] - b[1]), hb);
#pragma unroll
    for (int i = 1; i <= 5; ++i) p[i] = __fadd_rn((float)(b[i] - b[i + 1]), hb);
    p[6] = __fadd_rn((float)b[6], hb);
    p[7] = hb;
}

// One level of E8Decoder._full_decode (coset/core/e8/codecs.py:161-167):
// r = G b - q * projection(G b / q).
__device__ __forceinline__ void level_residual(const int (&b)[8], float qf, float (&r)[8]) {
    float p[8], s[8], pr[8];
    decode_coords(b, p);
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = __fdiv_rn(p[i], qf);
    projection(s, pr);
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = __fsub_rn(p[i], __fmul_rn(qf, pr[i]));
}

}  // namespace e8
