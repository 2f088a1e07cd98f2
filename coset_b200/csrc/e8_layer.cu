// Backward pass of the HNLQLinearQAT weight path (straight-through estimator).
//
// Forward (coset/core/layers.py:429-463):  U = e8_quantize(W * beta) / beta,  Wq = clamp(U, +-clip)
// is coset_e8_quantize with COSET_SCALE_MUL_TILE; it also emits the packed codes, so the backward
// pass re-creates U from 4 B/block instead of re-reading a saved 32 B/block tensor.
//
// Backward, as torch autograd evaluates the reference graph (clamp -> div -> STE -> mul,
// coset/core/layers.py:62-95 for the STE):
//   g_c      = g * 1[-clip <= U <= clip]
//   t        = g_c / beta                       (div backward w.r.t. the numerator)
//   dW       = t * beta                         (mul backward)
//   dbeta    = sum_tile  t * W - g_c * Q / beta^2  =  sum_tile t * (W - U),   Q = beta * U
#include "common.cuh"
#include "e8_fast.cuh"
#include "e8_io.cuh"
#include "e8_literal.cuh"

using namespace coset;

namespace {

constexpr int kThreads = 256;

// One block's contribution; returns the block's dbeta partial.
template <int DTG, bool Q4>
__device__ __forceinline__ float bwd_block(const void* __restrict__ g, const float* __restrict__ w,
                                           const void* __restrict__ codes, const uint2* __restrict__ table, float beta,
                                           float clip, int q, int64_t b, float* __restrict__ dw) {
    float gv[8], wv[8], qv[8], uv[8], out[8];
    e8::Row8<DTG>::load(g, b, gv);
    e8::Row8<0>::load(w, b, wv);
    if (Q4) {
        float v2[8];
        e8::decode_q4m2_twice(__ldg(reinterpret_cast<const uint32_t*>(codes) + b), table, v2);
        e8::scale_twice<2>(v2, beta, uv);
    } else {
        uint32_t words[2];
        if (q <= 4) {
            const uint16_t* c = reinterpret_cast<const uint16_t*>(codes) + b * 2;
            words[0] = c[0]; words[1] = c[1];
        } else {
            const uint32_t* c = reinterpret_cast<const uint32_t*>(codes) + b * 2;
            words[0] = c[0]; words[1] = c[1];
        }
        float qf = (float)q, wgt = 1.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) qv[i] = 0.0f;
        for (int m = 0; m < 2; ++m) {
            int d[8];
            float r[8];
            if (q <= 4) e8::unpack_level<2>(words[m], d); else e8::unpack_level<4>(words[m], d);
            e8::level_residual(d, qf, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) qv[i] = __fadd_rn(qv[i], __fmul_rn(wgt, r[i]));
            wgt = __fmul_rn(wgt, qf);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) uv[i] = __fdiv_rn(qv[i], beta);
    }
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float u = uv[i];
        bool pass = (clip > 0.0f) ? (u >= -clip && u <= clip) : (u == u);
        float gc = pass ? gv[i] : 0.0f;
        float t = __fdiv_rn(gc, beta);
        out[i] = __fmul_rn(t, beta);
        acc += t * (wv[i] - u);
    }
    e8::Row8<0>::store(dw, b, out);
    return acc;
}

// blocks_per_tile == 1: one thread per block, dbeta written directly.
template <int DTG, bool Q4>
__global__ void __launch_bounds__(kThreads)
k_bwd_block_tiles(const void* __restrict__ g, const float* __restrict__ w, const void* __restrict__ codes,
                  const uint2* __restrict__ table, const float* __restrict__ beta, float clip, int q, int64_t n,
                  float* __restrict__ dw, float* __restrict__ dbeta) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    float bt = __ldg(beta + b);
    float acc = bwd_block<DTG, Q4>(g, w, codes, table, bt, clip, q, b, dw);
    if (dbeta) dbeta[b] = acc;
}

// blocks_per_tile > 1 (one scale per weight row): one warp per tile, lanes stride over the
// tile's blocks (coalesced 1 KiB per step), shuffle reduction, no scratch memory.
template <int DTG, bool Q4>
__global__ void __launch_bounds__(kThreads)
k_bwd_row_tiles(const void* __restrict__ g, const float* __restrict__ w, const void* __restrict__ codes,
                const uint2* __restrict__ table, const float* __restrict__ beta, float clip, int q, int64_t n,
                int64_t bpt, int64_t tiles, float* __restrict__ dw, float* __restrict__ dbeta) {
    int64_t tile = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (tile >= tiles) return;
    float bt = __ldg(beta + tile);
    int64_t lo = tile * bpt, hi = lo + bpt;
    if (hi > n) hi = n;
    float acc = 0.0f;
    for (int64_t b = lo + lane; b < hi; b += 32) acc += bwd_block<DTG, Q4>(g, w, codes, table, bt, clip, q, b, dw);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0 && dbeta) dbeta[tile] = acc;
}

// Per-tile scale of the layer (coset/core/layers.py:415-417):
//   beta = beta_min + sigmoid(theta) * (beta_max - beta_min),   sigmoid(t) = 1 / (1 + exp(-t))
// and its backward: d theta = (d beta * range) * (1 - s) * s, the product torch autograd forms for
// mul followed by sigmoid.
__device__ __forceinline__ float sigmoidf_exact(float t) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-t))); }

__global__ void __launch_bounds__(kThreads)
k_layer_beta(const float* __restrict__ theta, const float* __restrict__ bmin, const float* __restrict__ brange, int64_t tiles,
             float* __restrict__ beta) {
    int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= tiles) return;
    beta[i] = __fadd_rn(__ldg(bmin + i), __fmul_rn(sigmoidf_exact(__ldg(theta + i)), __ldg(brange + i)));
}

__global__ void __launch_bounds__(kThreads)
k_layer_dtheta(const float* __restrict__ theta, const float* __restrict__ brange, int64_t tiles, float* __restrict__ grad) {
    int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= tiles) return;
    const float s = sigmoidf_exact(__ldg(theta + i));
    const float t = __fmul_rn(grad[i], __ldg(brange + i));
    grad[i] = __fmul_rn(__fmul_rn(t, __fsub_rn(1.0f, s)), s);
}

}  // namespace

extern "C" int coset_layer_beta(const float* theta, const float* beta_min, const float* beta_range, int64_t n_tiles,
                                float* beta, void* stream) {
    if (n_tiles < 0) return fail(COSET_E_BADARG, "n_tiles is negative");
    if (n_tiles == 0) return 0;
    if (!theta || !beta_min || !beta_range || !beta) return fail(COSET_E_BADARG, "null pointer");
    k_layer_beta<<<(unsigned)((n_tiles + kThreads - 1) / kThreads), kThreads, 0, (cudaStream_t)stream>>>(theta, beta_min, beta_range,
                                                                                                      n_tiles, beta);
    return check_launch("layer_beta");
}

extern "C" int coset_e8_layer_fake_quant_fwd(const float* w, const float* theta, const float* beta_min, const float* beta_range,
                                             int64_t n_blocks, int64_t blocks_per_tile, int q, float clip, void* out,
                                             int out_dtype, void* codes, float* beta, void* stream) {
    if (n_blocks < 0 || blocks_per_tile < 1) return fail(COSET_E_BADARG, "bad n_blocks / blocks_per_tile");
    const int64_t tiles = (n_blocks + blocks_per_tile - 1) / blocks_per_tile;
    if (int e = coset_layer_beta(theta, beta_min, beta_range, tiles, beta, stream)) return e;
    return coset_e8_quantize(w, COSET_DTYPE_F32, beta, COSET_SCALE_MUL_TILE, n_blocks, blocks_per_tile, q, 2, clip, out,
                             out_dtype, codes, stream);
}

extern "C" int coset_e8_fake_quant_bwd(const void* grad_out, int grad_dtype, const float* w, const void* codes,
                                       const float* beta, int64_t n_blocks, int64_t blocks_per_tile, int q, float clip,
                                       float* grad_w, float* grad_beta, void* stream);

extern "C" int coset_e8_layer_fake_quant_bwd(const void* grad_out, int grad_dtype, const float* w, const void* codes,
                                             const float* beta, const float* theta, const float* beta_range, int64_t n_blocks,
                                             int64_t blocks_per_tile, int q, float clip, float* grad_w, float* grad_theta,
                                             void* stream) {
    if (int e = coset_e8_fake_quant_bwd(grad_out, grad_dtype, w, codes, beta, n_blocks, blocks_per_tile, q, clip, grad_w,
                                        grad_theta, stream))
        return e;
    if (!grad_theta || n_blocks == 0) return 0;
    if (!theta || !beta_range) return fail(COSET_E_BADARG, "null pointer");
    const int64_t tiles = (n_blocks + blocks_per_tile - 1) / blocks_per_tile;
    k_layer_dtheta<<<(unsigned)((tiles + kThreads - 1) / kThreads), kThreads, 0, (cudaStream_t)stream>>>(theta, beta_range, tiles,
                                                                                                       grad_theta);
    return check_launch("layer_dtheta");
}

extern "C" int coset_e8_fake_quant_bwd(const void* grad_out, int grad_dtype, const float* w, const void* codes,
                                       const float* beta, int64_t n_blocks, int64_t blocks_per_tile, int q,
                                       float clip, float* grad_w, float* grad_beta, void* stream) {
    if (n_blocks < 0 || blocks_per_tile < 1) return fail(COSET_E_BADARG, "bad n_blocks / blocks_per_tile");
    if (n_blocks == 0) return 0;
    if (!grad_out || !w || !codes || !beta || !grad_w) return fail(COSET_E_BADARG, "null pointer");
    if (grad_dtype != COSET_DTYPE_F32 && grad_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown grad_dtype");
    if (q < 2 || q > 16) return fail(COSET_E_UNSUPPORTED, "unsupported q=%d", q);
    if (!aligned(grad_out, 16) || !aligned(w, 16) || !aligned(grad_w, 16) || !aligned(codes, 4))
        return fail(COSET_E_ALIGN, "grad_out, w, grad_w must be 16-byte and codes 4-byte aligned");
    if (n_blocks > ((int64_t)1 << 36)) return fail(COSET_E_BADARG, "n_blocks too large");
    cudaStream_t st = (cudaStream_t)stream;
    const uint2* table = nullptr;
    if (q == 4) {
        table = residual_table_q4(st);
        if (!table) return COSET_E_STATE;
    }
#define LAUNCH_BWD(DTG, Q4)                                                                                       \
    do {                                                                                                          \
        if (blocks_per_tile == 1) {                                                                               \
            unsigned grid = (unsigned)((n_blocks + kThreads - 1) / kThreads);                                     \
            k_bwd_block_tiles<DTG, Q4><<<grid, kThreads, 0, st>>>(grad_out, w, codes, table, beta, clip, q,       \
                                                                  n_blocks, grad_w, grad_beta);                   \
        } else {                                                                                                  \
            int64_t tiles = (n_blocks + blocks_per_tile - 1) / blocks_per_tile;                                   \
            unsigned grid = (unsigned)((tiles * 32 + kThreads - 1) / kThreads);                                   \
            k_bwd_row_tiles<DTG, Q4><<<grid, kThreads, 0, st>>>(grad_out, w, codes, table, beta, clip, q,         \
                                                                n_blocks, blocks_per_tile, tiles, grad_w,         \
                                                                grad_beta);                                       \
        }                                                                                                         \
    } while (0)
    if (grad_dtype == COSET_DTYPE_F32) {
        if (q == 4) LAUNCH_BWD(0, true); else LAUNCH_BWD(0, false);
    } else {
        if (q == 4) LAUNCH_BWD(1, true); else LAUNCH_BWD(1, false);
    }
#undef LAUNCH_BWD
    return check_launch("e8_fake_quant_bwd");
}
