// Global-memory access helpers shared by the codec kernels: 128-bit block loads/stores for
// float32 and bf16 rows of 8, per-tile scale lookup and the packed-code layout.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace e8 {

// Exact unsigned division of a block index (< 2^31) by blocks_per_tile, precomputed on the host.
struct TileDiv {
    uint32_t mul;
    uint32_t shr;
    int64_t divisor;  // blocks_per_tile; 1 = one scale per block
    int wide;         // 1: indices may reach 2^31, use the 64-bit division
};

inline TileDiv make_tile_div(int64_t divisor, int64_t n_blocks) {
    TileDiv t;
    t.divisor = divisor < 1 ? 1 : divisor;
    t.wide = (n_blocks >= (int64_t(1) << 31)) || (t.divisor >= (int64_t(1) << 31)) ? 1 : 0;
    t.mul = 0;
    t.shr = 0;
    if (!t.wide && t.divisor > 1) {
        uint32_t d = (uint32_t)t.divisor;
        int lg = 0;
        while ((uint64_t(1) << lg) < d) ++lg;  // ceil(log2 d)
        int p = 31 + lg;
        t.mul = (uint32_t)(((uint64_t(1) << p) + d - 1) / d);
        t.shr = (uint32_t)(p - 32);
    }
    return t;
}

__device__ __forceinline__ int64_t tile_of(const TileDiv& t, int64_t block) {
    if (t.divisor == 1) return block;
    if (t.wide) return block / t.divisor;
    return (int64_t)(__umulhi((uint32_t)block, t.mul) >> t.shr);
}

template <int DTYPE>
struct Row8;

template <>
struct Row8<0> {  // float32
    static __device__ __forceinline__ void load(const void* base, int64_t block, float (&v)[8]) {
        const float4* p = reinterpret_cast<const float4*>(base) + block * 2;
        float4 a = __ldcs(p), b = __ldcs(p + 1);  // streamed once: do not displace the residual table in L1
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(void* base, int64_t block, const float (&v)[8]) {
        float4* p = reinterpret_cast<float4*>(base) + block * 2;
        __stcs(p, make_float4(v[0], v[1], v[2], v[3]));
        __stcs(p + 1, make_float4(v[4], v[5], v[6], v[7]));
    }
};

template <>
struct Row8<1> {  // bf16: widened exactly on load, rounded to nearest-even on store
    static __device__ __forceinline__ void load(const void* base, int64_t block, float (&v)[8]) {
        uint4 a = __ldcs(reinterpret_cast<const uint4*>(base) + block);
        uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store(void* base, int64_t block, const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        __stcs(reinterpret_cast<uint4*>(base) + block, make_uint4(w[0], w[1], w[2], w[3]));
    }
};

// Level word of 8 digits, BPD bits each, digit j at bit BPD*j.
template <int BPD>
__device__ __forceinline__ uint32_t pack_level(const int (&d)[8]) {
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) w |= (uint32_t)d[j] << (BPD * j);
    return w;
}
template <int BPD>
__device__ __forceinline__ void unpack_level(uint32_t w, int (&d)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) d[j] = (int)((w >> (BPD * j)) & ((1u << BPD) - 1u));
}

}  // namespace e8
