// Cheapest tier of the q = 4 encode level: digits of encode_coords(projection(x), 4)
// (coset/core/e8/lattice.py:114-169 followed by coset/core/base.py:134-154) for blocks whose
// every decision is clear of a rounding tie, in about half the instructions of level_fast_q4.
//
// What it uses, all of it valid only under the guards below (a block that fails one is reported and
// finished by the exact tiers of e8_fast.cuh):
//   * ONE rounding pass.  With f = rint(x), d = x - f and g_i = [d_i < 0], the half-integer coset's
//     rounded values are f' = f - g, its residuals have |d'_i| = 1/2 - |d_i| (up to 2^-23), so its flip
//     coordinate is the arg-MIN of |d| -- taken from the same integer keys as the arg-max -- as long as
//     that minimum is separated from the runner-up by more than the rounding noise (checked), and the
//     parity of sum f' is the parity of sum f xor the parity of the number of negative d_i.
//   * The two squared distances share sum d_i^2: dist1 - dist0 = 2 - sum|d_i| (+- the flip costs).
//   * The reference's flip rule only needs two signs at the flip coordinate k: coset 0 moves up iff
//     d_k > 0 and x_k >= 0 (away from x iff d_k > 0 and x_k < 0); coset 1 moves up iff d_k < 0 and
//     x_k > 0 (away iff d_k < 0 and x_k < 0).
//   * The digits are a linear map of the rounded integers.  Four float accumulators hold two 7-bit
//     lanes each (digit i of the level word in the lane at bit 2i+1, so that the low two bits of every
//     lane are already in place), built on the FP32 pipe with exact small-integer arithmetic; the flip
//     adds one table row; three bit-selects and a shift leave the 16-bit level word.
// Guards: max|x| <= 1.96 and sum|x| <= 7.96 (which also makes the NEXT level the origin and keeps every
// lane in range), max|d| < 1/2 - 2.96 * 2^-21 and min|d| > 2.96 * 2^-21 (rint equals the reference's
// custom_round for x and x - 1/2), minimum of |d| unique by 2^-21, |dist1 - dist0| > 2^-14.
#pragma once
#include "e8_fast.cuh"

namespace e8 {

constexpr float kMagic0 = 8388608.0f + 64.0f * (1.0f + 512.0f);     // coordinate 0 starts digit word A
constexpr float kMagicB = 8388608.0f + 64.0f * (8.0f + 2048.0f);
constexpr float kMagicC = 8388608.0f + 64.0f * (32.0f + 8192.0f);
constexpr float kMagicD = 8388608.0f + 64.0f * (128.0f + 32768.0f);

// Row k: what one unit step of rounded integer k adds to the digit words A, B, C, D.
__device__ __constant__ uint4 kFlipRows[8] = {
    {1u, 0u, 0u, 0u},     {1u, 8u, 0u, 0u},       {1u, 8u, 32u, 0u},       {1u, 8u, 32u, 128u},
    {513u, 8u, 32u, 128u}, {513u, 2056u, 32u, 128u}, {513u, 2056u, 8224u, 128u}, {513u, 4112u, 24672u, 66048u}};

__device__ __forceinline__ uint32_t xor3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x96;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
// prmt.b32 with the full 4-bit selectors (bit 3 of a selector replicates the sign of the chosen byte)
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t s) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(s));
    return r;
}
// (a & m) | (b & ~m)
__device__ __forceinline__ uint32_t bitselect(uint32_t a, uint32_t b, uint32_t m) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(r) : "r"(m), "r"(a), "r"(b));
    return r;
}

// x: scaled block with max|x| <= 1.96 and sum|x| <= 7.96 (the caller's pre-test).  Returns true and the
// 16-bit level word, or false when a guard refuses.
// rows: the eight kFlipRows entries, in shared memory when the caller has a copy there (lanes index it
// with different values; constant memory would serialise those reads), else kFlipRows itself.
__device__ __forceinline__ bool level_fast2_q4(const float (&x)[8], uint32_t& digits, const uint4* rows = kFlipRows) {
    const float kTie = 2.96f * 4.76837158203125e-07f;
    float w[8], f[8], d[8], g[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float M = i == 0 ? kMagic0 : kMagic;
        w[i] = __fadd_rn(x[i], M);
        f[i] = __fsub_rn(w[i], M);
        d[i] = __fsub_rn(x[i], f[i]);
        g[i] = __saturatef(__fmul_rn(d[i], -1.099511627776e12f));  // 1 where d < 0
    }
    float l1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) l1 = __fadd_rn(l1, fabsf(d[i]));
    // keys: |d| bits * 4 + byte lane; group B = coordinates 0..3 (lanes 3..0), group A = 4..7
    uint32_t k[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) k[i] = __float_as_uint(d[i]) * 4u + (uint32_t)(3 - (i & 3));
    const uint32_t maxB = max(umax3(k[0], k[1], k[2]), k[3]), maxA = max(umax3(k[4], k[5], k[6]), k[7]);
    const uint32_t minB = min(__vimin3_u32(k[0], k[1], k[2]), k[3]), minA = min(__vimin3_u32(k[4], k[5], k[6]), k[7]);
    const bool low0 = (maxB | 3u) >= maxA;  // equal |d|: the lower coordinate index wins (torch.argmax)
    const bool low1 = minB <= minA;
    const uint32_t key0 = low0 ? maxB : maxA, key1 = low1 ? minB : minA;
    const float m0 = __uint_as_float(key0 >> 2), mn = __uint_as_float(key1 >> 2);
    bool ok = (m0 < 0.5f - kTie) && (mn > kTie);
    // the minimum must be unique by ~2^-21: sum of sat(1 - (|d_i| - mn) 2^20) is 1 from the minimum itself
    const float cu = __fmaf_rn(mn, 1048576.0f, 1.0f);
    float u = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) u = __fadd_rn(u, __saturatef(__fmaf_rn(fabsf(d[i]), -1048576.0f, cu)));
    ok = ok && (u < 1.5f);
    // sign bytes of d and of x, one byte per coordinate in key-lane order
    const uint32_t sA = gather_bytes<0x0073>(d[7], d[6], d[5], d[4]), sB = gather_bytes<0x0073>(d[3], d[2], d[1], d[0]);
    const uint32_t xA = gather_bytes<0x0073>(x[7], x[6], x[5], x[4]), xB = gather_bytes<0x0073>(x[3], x[2], x[1], x[0]);
    const uint32_t sel0 = (key0 & 3u) | (low0 ? 0u : 4u), sel1 = (key1 & 3u) | (low1 ? 0u : 4u);
    const uint32_t rep0 = (sel0 | 8u) * 0x1111u, rep1 = (sel1 | 8u) * 0x1111u;  // sign-replicating selectors
    const uint32_t dneg0 = prmt(sB, sA, rep0), xneg0 = prmt(xB, xA, rep0);  // 0 or ~0
    const uint32_t dneg1 = prmt(sB, sA, rep1), xneg1 = prmt(xB, xA, rep1);
    const uint32_t away0 = ~dneg0 & xneg0, up0 = ~(dneg0 | xneg0);
    const uint32_t away1 = dneg1 & xneg1, up1 = dneg1 & ~xneg1;
    // parities: sum f odd?  sum f' odd? (one more flip per negative d)
    const uint32_t pw = xor3(xor3(__float_as_uint(w[0]), __float_as_uint(w[1]), __float_as_uint(w[2])),
                             xor3(__float_as_uint(w[3]), __float_as_uint(w[4]), __float_as_uint(w[5])),
                             __float_as_uint(w[6]) ^ __float_as_uint(w[7]));
    const uint32_t pd = xor3(xor3(__float_as_uint(d[0]), __float_as_uint(d[1]), __float_as_uint(d[2])),
                             xor3(__float_as_uint(d[3]), __float_as_uint(d[4]), __float_as_uint(d[5])),
                             __float_as_uint(d[6]) ^ __float_as_uint(d[7]));
    const bool odd0 = (pw & 1u) != 0u;
    const bool odd1 = ((pw ^ (pd >> 31)) & 1u) != 0u;
    // flip costs: 1 -+ 2 m0 for the integer coset, 1 -+ 2 (1/2 - mn) for the half-integer coset
    const float m0s = __uint_as_float(__float_as_uint(m0) ^ (away0 & 0x80000000u));
    const float c0 = __fmaf_rn(-2.0f, m0s, 1.0f);
    const float c1 = away1 ? __fmaf_rn(-2.0f, mn, 2.0f) : __fmul_rn(2.0f, mn);
    float delta = __fsub_rn(2.0f, l1);  // dist1 - dist0 (the shared sum d^2 cancels)
    if (odd1) delta = __fadd_rn(delta, c1);
    if (odd0) delta = __fsub_rn(delta, c0);
    ok = ok && (fabsf(delta) > 6.103515625e-05f);
    const bool half = delta < 0.0f;
    const float hf = half ? 1.0f : 0.0f, nhf = half ? -1.0f : 0.0f;
    const bool odd = half ? odd1 : odd0;
    const uint32_t up = half ? up1 : up0;
    const uint32_t row = (half ? sel1 : sel0) ^ 3u;  // coordinate index of the flip
    const uint32_t stp = odd ? (up ? 1u : 0xffffffffu) : 0u;  // +1 when the rule moves up, -1 otherwise
    // digit words from the chosen coset's rounded integers fs = f - half * g (coordinate 0 keeps its magic)
    float fs[8];
    fs[0] = __fmaf_rn(nhf, g[0], w[0]);
#pragma unroll
    for (int i = 1; i < 8; ++i) fs[i] = __fmaf_rn(nhf, g[i], f[i]);
    const float t56 = __fadd_rn(fs[5], fs[6]), t46 = __fadd_rn(fs[4], t56), t36 = __fadd_rn(fs[3], t46);
    const float t26 = __fadd_rn(fs[2], t36), t16 = __fadd_rn(fs[1], t26), t06 = __fadd_rn(fs[0], t16);
    const float A = __fmaf_rn(fs[7], 513.0f, __fmaf_rn(t46, 512.0f, t06));
    const float B = __fmaf_rn(fs[7], 4112.0f, __fmaf_rn(t56, 2048.0f, __fmaf_rn(t16, 8.0f, kMagicB)));
    const float C = __fmaf_rn(fs[7], 24672.0f, __fmaf_rn(fs[6], 8192.0f, __fmaf_rn(t26, 32.0f, kMagicC)));
    const float D = __fmaf_rn(hf, 32768.0f, __fmaf_rn(fs[7], 66048.0f, __fmaf_rn(t36, 128.0f, kMagicD)));
    const uint4 r = rows[row];
    const uint32_t a = __float_as_uint(A) + stp * r.x, b = __float_as_uint(B) + stp * r.y;
    const uint32_t c = __float_as_uint(C) + stp * r.z, e = __float_as_uint(D) + stp * r.w;
    const uint32_t t = bitselect(bitselect(a, b, 0x606u), bitselect(c, e, 0x6060u), 0x1E1Eu);
    digits = (t >> 1) & 0xffffu;
    return ok;
}

}  // namespace e8
