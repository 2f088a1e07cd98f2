// D4 lattice path: the reference's second lattice (coset/core/d4/lattice.py) behind the same layer.
//
//   projection   D4Lattice.projection, coset/core/d4/lattice.py:111-146
//   quantize     weight path of the layer built by create_d4_hnlq_linear
//                (coset/core/d4/layers.py:15-68; coset/core/layers.py:429-463):
//                clamp(projection(W * beta) / beta, +-clip)
//   backward     straight-through gradients of that graph (coset/core/layers.py:62-95)
//
// A D4 block is 4 values.  The search is short (4 roundings, a parity test, one flip), so these
// kernels are bound by HBM: 16 B in + 16 B out per block.  Each thread owns two consecutive
// blocks (one 32-byte row) so that accesses stay 128-bit and fully coalesced; an odd last block is
// handled by the last thread alone.  Every value that reaches the output is produced by the reference's
// float32 operations in the reference's order (__f*_rn intrinsics are never contracted) or by a
// sequence shown to round identically, so results are bit-identical.
#include <cuda_bf16.h>
#include <math.h>

#include "common.cuh"
#include "e8_io.cuh"
#include "e8_literal.cuh"

using namespace coset;

namespace {

constexpr int kThreads = 256;

template <int DTYPE>
struct Row4;

template <>
struct Row4<0> {
    static __device__ __forceinline__ void load(const void* base, int64_t block, float (&v)[4]) {
        float4 a = __ldcs(reinterpret_cast<const float4*>(base) + block);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
    static __device__ __forceinline__ void store(void* base, int64_t block, const float (&v)[4]) {
        __stcs(reinterpret_cast<float4*>(base) + block, make_float4(v[0], v[1], v[2], v[3]));
    }
};

template <>
struct Row4<1> {
    static __device__ __forceinline__ void load(const void* base, int64_t block, float (&v)[4]) {
        uint2 a = __ldcs(reinterpret_cast<const uint2*>(base) + block);
        v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xffff0000u);
        v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xffff0000u);
    }
    static __device__ __forceinline__ void store(void* base, int64_t block, const float (&v)[4]) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        __stcs(reinterpret_cast<uint2*>(base) + block,
               make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi)));
    }
};

// custom_round with the nudge taken as copysign(2^-23, x): for x = +-0 the reference's nudge is 0,
// here it is +-2^-23, and both give floor(0.5 -+ tiny) = 0, so the results agree for every input.
__device__ __forceinline__ float d4_round(float x) {
    float nudge = __uint_as_float((__float_as_uint(x) & 0x80000000u) | 0x34000000u);
    return floorf(__fadd_rn(__fsub_rn(x, nudge), 0.5f));
}

// D4Lattice.projection on one block: f = custom_round(x); if sum(f) is odd (python float `% 2`),
// the coordinate with the largest |x - f| (first index on ties; NaN counts as largest) moves by
// +1 when x_k >= 0 and f_k < x_k and by -1 in every other case -- the reference computes a
// `flip_negative` mask and does not use it (coset/core/d4/lattice.py:97-104).
__device__ __forceinline__ void d4_projection(const float (&x)[4], float (&y)[4]) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        y[i] = d4_round(x[i]);
        s = __fadd_rn(s, y[i]);
    }
    // python float `s % 2 == 0`: integer parity below 2^24, every finite float from 2^24 up is an
    // even integer, and NaN / inf compare false (those rows take the g_x branch like the reference)
    float as = fabsf(s);
    bool even = as < 16777216.0f ? ((__float2int_rn(s) & 1) == 0) : (as < __int_as_float(0x7f800000));
    if (even) return;
    int k = 0;
    float best = fabsf(__fsub_rn(x[0], y[0]));
    bool done = best != best;
#pragma unroll
    for (int i = 1; i < 4; ++i) {
        float d = fabsf(__fsub_rn(x[i], y[i]));
        bool isn = d != d;
        if (!done && (isn || d > best)) { best = d; k = i; }
        done = done || isn;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (i == k) {
            bool up = (x[i] >= 0.0f) && (y[i] < x[i]);
            y[i] = up ? __fadd_rn(y[i], 1.0f) : __fsub_rn(y[i], 1.0f);
        }
    }
}

// One block of the layer's weight path; u = value before the clamp.
template <bool SCALED>
__device__ __forceinline__ void d4_fake_quant_block(const float (&w)[4], float beta, float clip, float (&u)[4], float (&c)[4]) {
    float xs[4], p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) xs[i] = SCALED ? __fmul_rn(w[i], beta) : w[i];
    d4_projection(xs, p);
    if (SCALED) {
        // p / beta: for integer numerators up to 64 the sequence q0 = p r, q = fma(fma(-q0, beta, p), r, q0)
        // with r = RN(1 / beta) is the correctly rounded quotient for every float32 significand of
        // beta (checked exhaustively on the CPU) while beta stays far from the exponent limits;
        // anything else takes the IEEE division.
        float amax = fmaxf(fmaxf(fabsf(p[0]), fabsf(p[1])), fmaxf(fabsf(p[2]), fabsf(p[3])));
        float ab = fabsf(beta);
        if (amax <= 64.0f && ab > 1e-18f && ab < 1e18f) {
            float r = __frcp_rn(beta);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float q0 = __fmul_rn(p[i], r);
                u[i] = __fmaf_rn(__fmaf_rn(-q0, beta, p[i]), r, q0);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) u[i] = __fdiv_rn(p[i], beta);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) u[i] = p[i];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float v = u[i];
        c[i] = (clip > 0.0f && v == v) ? fminf(fmaxf(v, -clip), clip) : v;  // torch.clamp keeps NaN
    }
}

__global__ void __launch_bounds__(kThreads) k_d4_projection(const float* __restrict__ x, int64_t n, float* __restrict__ out) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    float v[4], y[4];
    Row4<0>::load(x, b, v);
    d4_projection(v, y);
    Row4<0>::store(out, b, y);
}

template <int DTI, bool SCALED, int DTO>
__global__ void __launch_bounds__(kThreads)
k_d4_quantize(const void* __restrict__ x, const float* __restrict__ beta, e8::TileDiv td, int64_t n, float clip,
              void* __restrict__ out) {
    int64_t pair = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    int64_t b0 = pair * 2;
    if (b0 >= n) return;
    if (b0 + 1 < n) {
        float v[8], o[8];
        e8::Row8<DTI>::load(x, pair, v);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float w[4] = {v[4 * h], v[4 * h + 1], v[4 * h + 2], v[4 * h + 3]}, u[4], c[4];
            float bt = SCALED ? __ldg(beta + e8::tile_of(td, b0 + h)) : 1.0f;
            d4_fake_quant_block<SCALED>(w, bt, clip, u, c);
#pragma unroll
            for (int i = 0; i < 4; ++i) o[4 * h + i] = c[i];
        }
        e8::Row8<DTO>::store(out, pair, o);
    } else {
        float w[4], u[4], c[4];
        Row4<DTI>::load(x, b0, w);
        float bt = SCALED ? __ldg(beta + e8::tile_of(td, b0)) : 1.0f;
        d4_fake_quant_block<SCALED>(w, bt, clip, u, c);
        Row4<DTO>::store(out, b0, c);
    }
}

// Backward of clamp(projection(W beta) / beta, +-clip) as torch autograd evaluates the reference
// graph (clamp -> div -> straight-through -> mul):
//   g_c = g * 1[-clip <= U <= clip],  t = g_c / beta,  dW = t * beta,  dbeta = sum_tile t * (W - U)
// U is recomputed from W (16 B/block) instead of being saved by the forward pass.
template <int DTG>
__device__ __forceinline__ float d4_bwd_block(const void* __restrict__ g, const float* __restrict__ w, float beta,
                                              float clip, int64_t b, float* __restrict__ dw) {
    float gv[4], wv[4], u[4], c[4], o[4];
    Row4<DTG>::load(g, b, gv);
    Row4<0>::load(w, b, wv);
    d4_fake_quant_block<true>(wv, beta, clip, u, c);
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        bool pass = (clip > 0.0f) ? (u[i] >= -clip && u[i] <= clip) : (u[i] == u[i]);
        float gc = pass ? gv[i] : 0.0f;
        float t = __fdiv_rn(gc, beta);
        o[i] = __fmul_rn(t, beta);
        acc += t * (wv[i] - u[i]);
    }
    Row4<0>::store(dw, b, o);
    return acc;
}

template <int DTG>
__global__ void __launch_bounds__(kThreads)
k_d4_bwd_block_tiles(const void* __restrict__ g, const float* __restrict__ w, const float* __restrict__ beta, float clip,
                     int64_t n, float* __restrict__ dw, float* __restrict__ dbeta) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    float acc = d4_bwd_block<DTG>(g, w, __ldg(beta + b), clip, b, dw);
    if (dbeta) dbeta[b] = acc;
}

// One warp per scale tile (a weight row): lanes stride over the tile's blocks, shuffle reduction.
template <int DTG>
__global__ void __launch_bounds__(kThreads)
k_d4_bwd_row_tiles(const void* __restrict__ g, const float* __restrict__ w, const float* __restrict__ beta, float clip,
                   int64_t n, int64_t bpt, int64_t tiles, float* __restrict__ dw, float* __restrict__ dbeta) {
    int64_t tile = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (tile >= tiles) return;
    float bt = __ldg(beta + tile);
    int64_t lo = tile * bpt, hi = lo + bpt;
    if (hi > n) hi = n;
    float acc = 0.0f;
    for (int64_t b = lo + lane; b < hi; b += 32) acc += d4_bwd_block<DTG>(g, w, bt, clip, b, dw);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0 && dbeta) dbeta[tile] = acc;
}

// Babai rounding in a d x d basis (d = 4 or 8): z = Ginv x, z_hat = rint(z / step) * step, y = G z_hat,
// products and sums rounded separately, accumulated left to right.
struct Basis {
    float G[64];
    float Ginv[64];
};

template <int D>
__global__ void __launch_bounds__(kThreads)
k_babai(const float* __restrict__ x, int64_t n, Basis basis, float step, float inv_step, float* __restrict__ out) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    float v[D], z[D], y[D];
    const float4* p = reinterpret_cast<const float4*>(x) + b * (D / 4);
#pragma unroll
    for (int h = 0; h < D / 4; ++h) {
        float4 a = __ldcs(p + h);
        v[4 * h] = a.x; v[4 * h + 1] = a.y; v[4 * h + 2] = a.z; v[4 * h + 3] = a.w;
    }
#pragma unroll
    for (int a = 0; a < D; ++a) {
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < D; ++i) acc = __fadd_rn(acc, __fmul_rn(basis.Ginv[a * D + i], v[i]));
        // inv_step != 0: step is a power of two, so the product equals the IEEE quotient
        float t = inv_step != 0.0f ? __fmul_rn(acc, inv_step) : __fdiv_rn(acc, step);
        z[a] = __fmul_rn(rintf(t), step);
    }
#pragma unroll
    for (int a = 0; a < D; ++a) {
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < D; ++i) acc = __fadd_rn(acc, __fmul_rn(basis.G[a * D + i], z[i]));
        y[a] = acc;
    }
    float4* q = reinterpret_cast<float4*>(out) + b * (D / 4);
#pragma unroll
    for (int h = 0; h < D / 4; ++h) __stcs(q + h, make_float4(y[4 * h], y[4 * h + 1], y[4 * h + 2], y[4 * h + 3]));
}

}  // namespace

extern "C" {

int coset_d4_projection(const float* x, int64_t n_blocks, float* out, void* stream) {
    if (n_blocks < 0) return fail(COSET_E_BADARG, "n_blocks is negative");
    if (n_blocks == 0) return 0;
    if (!x || !out) return fail(COSET_E_BADARG, "null pointer");
    if (!aligned(x, 16) || !aligned(out, 16)) return fail(COSET_E_ALIGN, "x and out must be 16-byte aligned");
    if (n_blocks > ((int64_t)1 << 38)) return fail(COSET_E_BADARG, "n_blocks too large");
    k_d4_projection<<<(unsigned)((n_blocks + kThreads - 1) / kThreads), kThreads, 0, (cudaStream_t)stream>>>(x, n_blocks, out);
    return check_launch("d4_projection");
}

int coset_d4_quantize(const void* x, int x_dtype, const float* scale, int scale_mode, int64_t n_blocks,
                      int64_t blocks_per_tile, float clip, void* out, int out_dtype, void* stream) {
    if (n_blocks < 0) return fail(COSET_E_BADARG, "n_blocks is negative");
    if (n_blocks == 0) return 0;
    if (!x || !out) return fail(COSET_E_BADARG, "null pointer");
    if ((x_dtype != COSET_DTYPE_F32 && x_dtype != COSET_DTYPE_BF16) || (out_dtype != COSET_DTYPE_F32 && out_dtype != COSET_DTYPE_BF16))
        return fail(COSET_E_BADARG, "unknown dtype");
    if (scale_mode != COSET_SCALE_NONE && scale_mode != COSET_SCALE_MUL_TILE)
        return fail(COSET_E_UNSUPPORTED, "the D4 path takes COSET_SCALE_NONE or COSET_SCALE_MUL_TILE");
    const bool scaled = scale_mode == COSET_SCALE_MUL_TILE;
    if (scaled && (!scale || blocks_per_tile < 1)) return fail(COSET_E_BADARG, "scale is null or blocks_per_tile < 1");
    if (!aligned(x, 16) || !aligned(out, 16)) return fail(COSET_E_ALIGN, "x and out must be 16-byte aligned");
    if (n_blocks > ((int64_t)1 << 38)) return fail(COSET_E_BADARG, "n_blocks too large");
    e8::TileDiv td = e8::make_tile_div(scaled ? blocks_per_tile : 1, n_blocks);
    cudaStream_t st = (cudaStream_t)stream;
    int64_t pairs = (n_blocks + 1) / 2;
    unsigned grid = (unsigned)((pairs + kThreads - 1) / kThreads);
#define D4Q(DTI, DTO)                                                                                          \
    do {                                                                                                       \
        if (scaled) k_d4_quantize<DTI, true, DTO><<<grid, kThreads, 0, st>>>(x, scale, td, n_blocks, clip, out); \
        else k_d4_quantize<DTI, false, DTO><<<grid, kThreads, 0, st>>>(x, scale, td, n_blocks, clip, out);       \
    } while (0)
    if (x_dtype == COSET_DTYPE_F32) {
        if (out_dtype == COSET_DTYPE_F32) D4Q(0, 0); else D4Q(0, 1);
    } else {
        if (out_dtype == COSET_DTYPE_F32) D4Q(1, 0); else D4Q(1, 1);
    }
#undef D4Q
    return check_launch("d4_quantize");
}

int coset_d4_fake_quant_bwd(const void* grad_out, int grad_dtype, const float* w, const float* beta, int64_t n_blocks,
                            int64_t blocks_per_tile, float clip, float* grad_w, float* grad_beta, void* stream) {
    if (n_blocks < 0 || blocks_per_tile < 1) return fail(COSET_E_BADARG, "bad n_blocks / blocks_per_tile");
    if (n_blocks == 0) return 0;
    if (!grad_out || !w || !beta || !grad_w) return fail(COSET_E_BADARG, "null pointer");
    if (grad_dtype != COSET_DTYPE_F32 && grad_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown grad_dtype");
    if (!aligned(grad_out, 16) || !aligned(w, 16) || !aligned(grad_w, 16))
        return fail(COSET_E_ALIGN, "grad_out, w and grad_w must be 16-byte aligned");
    if (n_blocks > ((int64_t)1 << 36)) return fail(COSET_E_BADARG, "n_blocks too large");
    cudaStream_t st = (cudaStream_t)stream;
    if (blocks_per_tile == 1) {
        unsigned grid = (unsigned)((n_blocks + kThreads - 1) / kThreads);
        if (grad_dtype == COSET_DTYPE_F32) k_d4_bwd_block_tiles<0><<<grid, kThreads, 0, st>>>(grad_out, w, beta, clip, n_blocks, grad_w, grad_beta);
        else k_d4_bwd_block_tiles<1><<<grid, kThreads, 0, st>>>(grad_out, w, beta, clip, n_blocks, grad_w, grad_beta);
    } else {
        int64_t tiles = (n_blocks + blocks_per_tile - 1) / blocks_per_tile;
        unsigned grid = (unsigned)((tiles * 32 + kThreads - 1) / kThreads);
        if (grad_dtype == COSET_DTYPE_F32) k_d4_bwd_row_tiles<0><<<grid, kThreads, 0, st>>>(grad_out, w, beta, clip, n_blocks, blocks_per_tile, tiles, grad_w, grad_beta);
        else k_d4_bwd_row_tiles<1><<<grid, kThreads, 0, st>>>(grad_out, w, beta, clip, n_blocks, blocks_per_tile, tiles, grad_w, grad_beta);
    }
    return check_launch("d4_fake_quant_bwd");
}

int coset_lattice_babai(const float* x, int64_t n_blocks, int dim, const float* G_host, const float* Ginv_host, float step,
                        float* out, void* stream) {
    if (n_blocks < 0) return fail(COSET_E_BADARG, "n_blocks is negative");
    if (dim != 4 && dim != 8) return fail(COSET_E_UNSUPPORTED, "Babai rounding is built for dimension 4 and 8");
    if (!(step > 0.0f)) return fail(COSET_E_BADARG, "step must be positive");
    if (n_blocks == 0) return 0;
    if (!x || !out || !G_host || !Ginv_host) return fail(COSET_E_BADARG, "null pointer");
    if (!aligned(x, 16) || !aligned(out, 16)) return fail(COSET_E_ALIGN, "x and out must be 16-byte aligned");
    if (n_blocks > ((int64_t)1 << 38)) return fail(COSET_E_BADARG, "n_blocks too large");
    Basis basis;
    for (int i = 0; i < dim * dim; ++i) {
        basis.G[i] = G_host[i];
        basis.Ginv[i] = Ginv_host[i];
    }
    for (int i = dim * dim; i < 64; ++i) basis.G[i] = basis.Ginv[i] = 0.0f;
    int exp2 = 0;
    const bool pow2 = frexpf(step, &exp2) == 0.5f && exp2 > -100 && exp2 < 100;
    const float inv_step = pow2 ? 1.0f / step : 0.0f;
    unsigned grid = (unsigned)((n_blocks + kThreads - 1) / kThreads);
    if (dim == 4) k_babai<4><<<grid, kThreads, 0, (cudaStream_t)stream>>>(x, n_blocks, basis, step, inv_step, out);
    else k_babai<8><<<grid, kThreads, 0, (cudaStream_t)stream>>>(x, n_blocks, basis, step, inv_step, out);
    return check_launch("lattice_babai");
}

}  // extern "C"
