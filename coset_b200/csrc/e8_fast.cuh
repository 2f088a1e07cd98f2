// q = 4, M = 2 codec primitives: one uint32 per block, level m digit j at bit 16*m + 2*j.
#pragma once
#include "e8_io.cuh"
#include "e8_literal.cuh"

namespace e8 {

// ---------------------------------------------------------------------------------------------
// Fast evaluation of one encode level: digits of encode_coords(projection(x), 4)
// (coset/core/e8/lattice.py:114-169 followed by coset/core/base.py:134-154).
//
// The literal search costs ~600 instructions per level; this path reaches the same digits in
// ~200 by (1) rounding with the 1.5*2^23 magic constant, (2) finding the flip coordinate of
// both cosets with exact integer keys (|delta| bits * 4 + lane: first index wins ties, as
// torch.argmax does), (3) deciding between the cosets from squared distances with a guard band
// and (4) forming the base-4 digits with byte-lane arithmetic.  It only answers when every
// shortcut is provably equivalent to the reference arithmetic:
//   * no coordinate of x or x - 1/2 lies within (amax + 1) * 2^-21 of a rounding tie, so
//     rint() equals the reference's custom_round();
//   * the two squared distances differ by more than 2^-14, far above the rounding noise of the
//     reference's sequential float32 norm, so `dist0 < dist1` is decided identically.
// Otherwise it reports failure and the caller runs the literal code for that block.  The model
// was checked against the CPU restatement of the reference on > 2*10^8 random, structured and
// near-tie vectors; the GPU tests compare it with the literal kernels on 2^25 blocks.
constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: x + kMagic rounds x to an integer (ties to even)

__device__ __forceinline__ uint32_t umax3(uint32_t a, uint32_t b, uint32_t c) { return __vimax3_u32(a, b, c); }

// low bytes (SEL = 0x0040 pairs) or top bytes (0x0073) of four floats, coordinate order hi..lo
template <uint32_t PAIR_SEL>
__device__ __forceinline__ uint32_t gather_bytes(float c3, float c2, float c1, float c0) {
    uint32_t a = __byte_perm(__float_as_uint(c3), __float_as_uint(c2), PAIR_SEL);
    uint32_t b = __byte_perm(__float_as_uint(c1), __float_as_uint(c0), PAIR_SEL);
    return __byte_perm(a, b, 0x5410);
}

struct CosetScan {
    uint32_t key;     // winning key: (|delta| bits << 2) | lane
    bool low_group;   // flip coordinate is one of 0..3
    uint32_t hA, hB;  // low bytes of the rounded integers: A = (c7,c6,c5,c4), B = (c3,c2,c1,c0), lanes 0..3
    bool odd, up, away;
    float m, sumsq;
};

// Scan of one D8 coset: x is the (shifted) input, w = x + kMagic, d = x - rint(x).
// sA / sB: top bytes (sign bits) of d, coordinates (7..4) and (3..0).  GIVEN = false: gathered here and
// returned; GIVEN = true: supplied by the caller.
template <bool GIVEN>
__device__ __forceinline__ void scan_coset(const float (&w)[8], const float (&d)[8], CosetScan& s, uint32_t& sA, uint32_t& sB) {
    uint32_t kb = max(umax3(__float_as_uint(d[0]) * 4u + 3u, __float_as_uint(d[1]) * 4u + 2u, __float_as_uint(d[2]) * 4u + 1u),
                      __float_as_uint(d[3]) * 4u);
    uint32_t ka = max(umax3(__float_as_uint(d[4]) * 4u + 3u, __float_as_uint(d[5]) * 4u + 2u, __float_as_uint(d[6]) * 4u + 1u),
                      __float_as_uint(d[7]) * 4u);
    s.low_group = (kb | 3u) >= ka;  // equal |delta|: the lower coordinate index wins
    s.key = s.low_group ? kb : ka;
    s.m = __uint_as_float(s.key >> 2);
    s.hA = gather_bytes<0x0040>(w[7], w[6], w[5], w[4]);
    s.hB = gather_bytes<0x0040>(w[3], w[2], w[1], w[0]);
    if (!GIVEN) {
        sA = gather_bytes<0x0073>(d[7], d[6], d[5], d[4]);
        sB = gather_bytes<0x0073>(d[3], d[2], d[1], d[0]);
    }
    uint32_t par = __float_as_uint(w[0]) ^ __float_as_uint(w[1]) ^ __float_as_uint(w[2]) ^ __float_as_uint(w[3]) ^
                   __float_as_uint(w[4]) ^ __float_as_uint(w[5]) ^ __float_as_uint(w[6]) ^ __float_as_uint(w[7]);
    s.odd = (par & 1u) != 0u;
    uint32_t sh = 8u * (s.key & 3u);
    uint32_t hb = (s.low_group ? s.hB : s.hA) >> sh;  // rounded integer at the flip coordinate (low byte)
    uint32_t sb = (s.low_group ? sB : sA) >> sh;      // top byte of delta there
    bool dpos = ((sb & 0x80u) == 0u) && ((s.key >> 2) != 0u);
    bool rneg = (hb & 0x80u) != 0u;
    s.up = dpos && !rneg;    // reference rule: +1 only when x_k >= 0 and f_k < x_k
    s.away = dpos && rneg;   // ... so a negative x_k that was rounded down moves AWAY from x
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) a = __fmaf_rn(d[i], d[i], a);
    float c = s.away ? __fmaf_rn(2.0f, s.m, 1.0f) : __fmaf_rn(-2.0f, s.m, 1.0f);
    s.sumsq = s.odd ? a + c : a;
}

// kMagic + custom_round(x), evaluated exactly as the reference does (coset/core/base.py:194-202:
// nudge by eps toward zero, add 0.5, floor); the floor is a round-down add of the magic constant.
__device__ __forceinline__ float magic_custom_round(float x) {
    float nudge = __uint_as_float((__float_as_uint(x) & 0x80000000u) | 0x34000000u);  // copysign(2^-23, x)
    float t = __fadd_rn(__fsub_rn(x, nudge), 0.5f);
    return __fadd_rd(t, kMagic);
}

// Returns true and the 16-bit level word when the fast path can answer; amax >= max |x_i|.
// EXACT_ROUND = false: rint() by one magic add, valid only away from rounding ties (guarded).
// EXACT_ROUND = true : the reference's custom_round op by op (3 more instructions per
//   coordinate and coset), valid everywhere, so exact ties -- zeros, integers, half-integers in
//   the data -- stay on this path; only the distance guard can still refuse.
template <bool EXACT_ROUND>
__device__ __forceinline__ bool level_fast_q4(const float (&x)[8], float amax, uint32_t& digits) {
    if (!(amax < 60.0f)) return false;
    float thr = __fmaf_rn(amax + 1.0f, -4.76837158203125e-07f, 0.5f);
    float w[8], d[8], ws[8], ds[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float xs = __fsub_rn(x[i], 0.5f);
        w[i] = EXACT_ROUND ? magic_custom_round(x[i]) : __fadd_rn(x[i], kMagic);
        ws[i] = EXACT_ROUND ? magic_custom_round(xs) : __fadd_rn(xs, kMagic);
        d[i] = __fsub_rn(x[i], __fsub_rn(w[i], kMagic));
        ds[i] = __fsub_rn(xs, __fsub_rn(ws[i], kMagic));
    }
    CosetScan s0, s1;
    uint32_t sA, sB;
    scan_coset<false>(w, d, s0, sA, sB);
    if (EXACT_ROUND) {
        scan_coset<false>(ws, ds, s1, sA, sB);
    } else {
        // Away from rounding ties (enforced below for this tier) x - 1/2 lies on the other side of its
        // nearest integer than x does of its own: sign(ds_i) = !sign(d_i).  Blocks for which that
        // fails have some |d_i| or |ds_i| at the tie threshold and are rejected by the guard.
        sA = ~sA;
        sB = ~sB;
        scan_coset<true>(ws, ds, s1, sA, sB);
    }
    if (!EXACT_ROUND && (!(s0.m < thr) || !(s1.m < thr))) return false;
    float delta = s1.sumsq - s0.sumsq;
    if (!(fabsf(delta) > 6.103515625e-05f)) return false;
    bool half = delta < 0.0f;  // the D8 + 1/2 candidate is strictly closer
    uint32_t hA = half ? s1.hA : s0.hA, hB = half ? s1.hB : s0.hB;
    uint32_t key = half ? s1.key : s0.key;
    bool low_group = half ? s1.low_group : s0.low_group;
    bool odd = half ? s1.odd : s0.odd, up = half ? s1.up : s0.up;
    // flip: +-1 (mod 16) in the byte lane of the flip coordinate
    uint32_t step = odd ? ((up ? 1u : 15u) << (8u * (key & 3u))) : 0u;
    uint32_t A = (hA & 0x0f0f0f0fu) + (low_group ? 0u : step);
    uint32_t B = (hB & 0x0f0f0f0fu) + (low_group ? step : 0u);
    A &= 0x0f0f0f0fu;
    B &= 0x0f0f0f0fu;
    // encode_coords: with S'_i = sum_{k>=i} h_k (mod 16 per lane, no carries: lanes stay < 256)
    //   b_7 = 2 h_7 + c,  b_i = S'_i + i h_7 (i = 1..6),  b_0 = S'_0 / 2      (all mod 4)
    uint32_t PA = A * 0x01010101u;                  // lanes S'_7, S'_6, S'_5, S'_4
    uint32_t PB = (B + (PA >> 24)) * 0x01010101u;   // lanes S'_3, S'_2, S'_1, S'_0
    uint32_t h7 = A & 0xfu;
    uint32_t VA = PA + h7 * 0x04050601u + (half ? 1u : 0u);
    uint32_t VB = PB + h7 * 0x00010203u;
    uint32_t dA = (((VA & 0x03030303u) * 0x40100401u) >> 16) & 0xff00u;  // digits 7..4 -> bits 14..8
    uint32_t dB = (((VB & 0x00030303u) * 0x40100401u) >> 24) & 0xfcu;    // digits 3..1 -> bits 6..2
    digits = dA | dB | ((VB >> 25) & 3u);
    return true;
}

// Second and third attempt, out of line (rare): exact-rounding fast path, then the literal search.
static __device__ __noinline__ uint32_t level_slow_q4(const float (&x)[8], float amax) {
    uint32_t digits;
    if (level_fast_q4<true>(x, amax, digits)) return digits;
    float y[8];
    int dg[8];
    bool half = projection(x, y);
    encode_coords(y, half, 4, dg);
    return pack_level<2>(dg);
}

// One level, always exact: the cheapest path that can prove its answer.
__device__ __forceinline__ uint32_t level_q4(const float (&x)[8], float amax) {
    uint32_t digits;
    if (level_fast_q4<false>(x, amax, digits)) return digits;
    return level_slow_q4(x, amax);
}

// Completes a block whose levels `start`..1 are still open, using the tiers that accept every
// input (exact-rounding fast path, then the literal search).  x holds the level-0 (scaled) input.
// Used for the deferred, warp-compacted work of the queued encoder.
__device__ __forceinline__ uint32_t finish_block_q4(float (&x)[8], uint32_t code, int start) {
    float amax = 0.0f, s1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        amax = fmaxf(amax, fabsf(x[i]));
        s1 += fabsf(x[i]);
    }
    bool finite = (s1 - s1) == 0.0f;
#pragma unroll 1
    for (int m = 0; m < 2; ++m) {
        bool origin = finite && amax <= 0.49f && s1 <= 1.99f;
        if (m >= start && !origin) {
            uint32_t digits;
            if (!level_fast_q4<true>(x, finite ? amax : __int_as_float(0x7fc00000), digits)) {
                float y[8];
                int dg[8];
                bool half = projection(x, y);
                encode_coords(y, half, 4, dg);
                digits = pack_level<2>(dg);
            }
            code |= digits << (16 * m);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], 0.25f);
        amax *= 0.25f;
        s1 *= 0.25f;
    }
    return code;
}

// Both levels of e8_encode for q = 4 (coset/core/e8/codecs.py:75-81).  x / 4 is exact in
// float32, so level 1 sees x * 0.25.
//
// Shortcut per level: if every |x_i| <= 0.49 and sum |x_i| <= 1.99 the projection is the origin
// (the integer candidate is 0 at squared distance sum x_i^2, every half-integer candidate is at
// least 2 - sum |x_i| farther), so the level word is 0.  In a quantiser that is not overloaded
// the top level is almost always in this regime.
template <bool LITERAL>
__device__ __forceinline__ uint32_t encode_q4m2(float (&x)[8]) {
    uint32_t code = 0;
    if (LITERAL) {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float y[8];
            int d[8];
            bool half = projection(x, y);
            encode_coords(y, half, 4, d);
            code |= pack_level<2>(d) << (16 * m);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], 0.25f);
        }
        return code;
    }
    float amax = 0.0f, s1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        amax = fmaxf(amax, fabsf(x[i]));
        s1 += fabsf(x[i]);
    }
    bool finite = (s1 - s1) == 0.0f;  // false for NaN / inf anywhere in the block
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        bool origin = finite && amax <= 0.49f && s1 <= 1.99f;
        if (!origin) code |= level_q4(x, finite ? amax : __int_as_float(0x7fc00000)) << (16 * m);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], 0.25f);
        amax *= 0.25f;
        s1 *= 0.25f;
    }
    return code;
}

// ---------------------------------------------------------------------------------------------
// Table-driven decode.
//
// Residual table entry for a 16-bit level word b: eight biased bytes t_i = 2 r_i(b) + 7 in
// [0, 18], where r(b) = G b - 4 Q(G b / 4) (E8Decoder._full_decode, coset/core/e8/codecs.py:161-167).
// With two levels, 2 x_hat_i = (t0_i - 7) + 4 (t1_i - 7) = (t0_i + 4 t1_i) - 35; the packed sum
// t0 + 4 t1 stays below 256 per byte lane, so one 32-bit multiply-add handles four coordinates.
constexpr int kTableBias = 7;

// byte `lane` of v -> float(byte) without the conversion pipe: build 0x4B4000bb (= 1.5*2^23 + bb).
template <int LANE>
__device__ __forceinline__ float biased_byte_to_float(uint32_t v) {
    return __uint_as_float(__byte_perm(v, 0x4B400000u, 0x7640u + LANE));
}

// Twice the reconstruction (an integer in [-35, 55]) of every coordinate, as exact floats.
// twice_from_entries: the same from the two table entries, already loaded.
__device__ __forceinline__ void twice_from_entries(uint2 t0, uint2 t1, float (&v2)[8]) {
    uint32_t lo = t0.x + 4u * t1.x, hi = t0.y + 4u * t1.y;
    const float kOff = 12582912.0f + 5.0f * kTableBias;
    v2[0] = __fsub_rn(biased_byte_to_float<0>(lo), kOff);
    v2[1] = __fsub_rn(biased_byte_to_float<1>(lo), kOff);
    v2[2] = __fsub_rn(biased_byte_to_float<2>(lo), kOff);
    v2[3] = __fsub_rn(biased_byte_to_float<3>(lo), kOff);
    v2[4] = __fsub_rn(biased_byte_to_float<0>(hi), kOff);
    v2[5] = __fsub_rn(biased_byte_to_float<1>(hi), kOff);
    v2[6] = __fsub_rn(biased_byte_to_float<2>(hi), kOff);
    v2[7] = __fsub_rn(biased_byte_to_float<3>(hi), kOff);
}

__device__ __forceinline__ void decode_q4m2_twice(uint32_t code, const uint2* __restrict__ table, float (&v2)[8]) {
    twice_from_entries(__ldg(table + (code & 0xffffu)), __ldg(table + (code >> 16)), v2);
}

// Packed form of the same table: 4 bytes per level word.  With t_i = 2 r_i(b) (an integer in
// [-7, 11]; |t_7| <= 5), all t_i of one entry have the same parity p (integer or half-integer
// coset), so
//     nibble i (bits 4i..4i+3) = (t_i - p + 8) / 2  in [0, 9]   for i < 7,
//     nibble 7 low 3 bits      = (t_7 - p + 6) / 2  in [0, 5],  bit 31 = p.
// With two levels, 2 x_hat_i = t0_i + 4 t1_i = 2 (n0_i + 4 n1_i) + (p0 + 4 p1) - 5 bias_i; even and
// odd nibbles are widened to byte lanes, so four coordinates share each 32-bit multiply-add and the
// byte B_i = 2 (n0_i + 4 n1_i) + p0 + 4 p1 stays below 96.
constexpr int kNibbleBias = 8, kNibbleBias7 = 6;
constexpr uint32_t kPackedZeroEntry = 0x34444444u;  // residual 0: nibbles 8/2 (6/2 for coordinate 7), parity 0

// Byte lanes B of the two packed entries of one code: `even` holds coordinates 0, 2, 4, 6 and `odd`
// coordinates 1, 3, 5, 7; coordinate i is B_i - 40 (B_7 - 30) = twice the reconstruction.
__device__ __forceinline__ void biased_bytes_q4m2(uint32_t e0, uint32_t e1, uint32_t& even, uint32_t& odd) {
    const uint32_t s_even = (e0 & 0x0f0f0f0fu) + 4u * (e1 & 0x0f0f0f0fu);
    const uint32_t s_odd = ((e0 >> 4) & 0x070f0f0fu) + 4u * ((e1 >> 4) & 0x070f0f0fu);
    const uint32_t rep = ((e0 >> 31) + 4u * (e1 >> 31)) * 0x01010101u;  // p0 + 4 p1 in every byte lane
    even = 2u * s_even + rep;
    odd = 2u * s_odd + rep;
}

// Twice the reconstruction from the two packed entries of a code, already loaded.
__device__ __forceinline__ void twice_from_packed(uint32_t e0, uint32_t e1, float (&v2)[8]);

__device__ __forceinline__ void decode_q4m2_twice(uint32_t code, const uint32_t* __restrict__ packed, float (&v2)[8]) {
    const uint32_t w0 = code & 0xffffu, w1 = code >> 16;
    // The residual of an all-zero level word is the zero vector, and the top level of a quantiser that is
    // not overloaded is almost always that word: its lookup is skipped (measured +2 % on the decoder).
    uint32_t e0 = kPackedZeroEntry, e1 = kPackedZeroEntry;
    if (w0) e0 = __ldg(packed + w0);
    if (w1) e1 = __ldg(packed + w1);
    twice_from_packed(e0, e1, v2);
}

__device__ __forceinline__ void twice_from_packed(uint32_t e0, uint32_t e1, float (&v2)[8]) {
    uint32_t even, odd;
    biased_bytes_q4m2(e0, e1, even, odd);
    const float kOff = 12582912.0f + 5.0f * kNibbleBias, kOff7 = 12582912.0f + 5.0f * kNibbleBias7;
    v2[0] = __fsub_rn(biased_byte_to_float<0>(even), kOff);
    v2[1] = __fsub_rn(biased_byte_to_float<0>(odd), kOff);
    v2[2] = __fsub_rn(biased_byte_to_float<1>(even), kOff);
    v2[3] = __fsub_rn(biased_byte_to_float<1>(odd), kOff);
    v2[4] = __fsub_rn(biased_byte_to_float<2>(even), kOff);
    v2[5] = __fsub_rn(biased_byte_to_float<2>(odd), kOff);
    v2[6] = __fsub_rn(biased_byte_to_float<3>(even), kOff);
    v2[7] = __fsub_rn(biased_byte_to_float<3>(odd), kOff7);
}

// x_hat = v2 / 2 with the reference's output scaling applied as the same IEEE operation:
//   MODE 0: x_hat                      (exact halving)
//   MODE 1: x_hat * s                  (coset/core/e8/codecs.py:175)   = RN(v2 * (s/2))
//   MODE 2: x_hat / s                  (coset/core/layers.py:455-460)  = RN(v2 / (2 s))
// For MODE 2 the quotient is formed as q0 = v2*r, q = fma(fma(-q0, 2s, v2), r, q0) with
// r = RN(1/(2s)); for the integer numerators that occur (|v2| <= 55) this equals the correctly
// rounded IEEE quotient for every float32 significand of s (checked exhaustively on the CPU),
// as long as s is far from the exponent limits -- outside that range the IEEE division is used.
template <int MODE>
__device__ __forceinline__ void scale_twice(const float (&v2)[8], float s, float (&out)[8]) {
    if (MODE == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = __fmul_rn(v2[i], 0.5f);
    } else if (MODE == 1) {
        float a = fabsf(s);
        if (a > 1e-30f && a < 1e30f) {
            float hs = __fmul_rn(s, 0.5f);
#pragma unroll
            for (int i = 0; i < 8; ++i) out[i] = __fmul_rn(v2[i], hs);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) out[i] = __fmul_rn(__fmul_rn(v2[i], 0.5f), s);
        }
    } else {
        float a = fabsf(s);
        if (a > 1e-18f && a < 1e18f) {
            float s2 = __fmul_rn(s, 2.0f);
            float r = __frcp_rn(s2);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float q0 = __fmul_rn(v2[i], r);
                float e = __fmaf_rn(-q0, s2, v2[i]);
                out[i] = __fmaf_rn(e, r, q0);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) out[i] = __fdiv_rn(__fmul_rn(v2[i], 0.5f), s);
        }
    }
}

// E8Decoder._full_decode for q = 4, M = 2 without output scaling.
__device__ __forceinline__ void decode_q4m2(uint32_t code, const uint2* __restrict__ table, float (&xh)[8]) {
    float v2[8];
    decode_q4m2_twice(code, table, v2);
    scale_twice<0>(v2, 1.0f, xh);
}

}  // namespace e8
