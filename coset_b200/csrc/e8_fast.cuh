// q = 4, M = 2 codec primitives: one uint32 per block, level m digit j at bit 16*m + 2*j.
#pragma once
#include "e8_io.cuh"
#include "e8_literal.cuh"

namespace e8 {

// Both levels of e8_encode for q = 4 (coset/core/e8/codecs.py:75-81).  x / 4 is exact in
// float32 (barring underflow to subnormals, which the reference shares), so level 1 simply
// sees x * 0.25.
__device__ __forceinline__ uint32_t encode_q4m2(float (&x)[8]) {
    uint32_t code = 0;
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

// Small signed integer -> float without the conversion pipe: 1.5*2^23 + v has v in its low
// mantissa bits for |v| < 2^22.
__device__ __forceinline__ float small_int_to_float(int v) {
    return __fsub_rn(__int_as_float(0x4B400000 + v), 12582912.0f);
}

// E8Decoder._full_decode for q = 4, M = 2 (coset/core/e8/codecs.py:159-172) through the
// residual table: x_hat = r(b0) + 4 r(b1), every term an exact half-integer, so the integer
// evaluation 2 x_hat = t0 + 4 t1 followed by an exact halving reproduces the float32 chain.
__device__ __forceinline__ void decode_q4m2(uint32_t code, const uint2* __restrict__ table, float (&xh)[8]) {
    uint2 t0 = __ldg(table + (code & 0xffffu));
    uint2 t1 = __ldg(table + (code >> 16));
    uint32_t a[2] = {t0.x, t0.y}, b[2] = {t1.x, t1.y};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int va = (int)(int8_t)(a[i >> 2] >> (8 * (i & 3)));
        int vb = (int)(int8_t)(b[i >> 2] >> (8 * (i & 3)));
        xh[i] = __fmul_rn(small_int_to_float(va + 4 * vb), 0.5f);
    }
}

}  // namespace e8
