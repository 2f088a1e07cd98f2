// Code-domain matrix product for inference: y[T, N] = x[T, K] * Wq^T (+ bias), with the weight
// held only as packed E8 codes (q=4, M=2: 4 B per 8 weights) plus its scales.
//
// The reference defines the math through per-query lookup tables of inner products with every
// codeword residual, <y, x_hat> = sum_m q^m <y, r(b_m)> (coset/legacy/quant/vlut.py:72-117,
// driver tests/legacy/test_one_sided_vlut_pytest.py:22-43); a table of 4^8 inner products per
// 8 activations is 128 MB per token at K = 4096, so the GPU form keeps ONE table (the 65536
// residuals r(b), 512 KB, L2/L1 resident), rebuilds the weight block in registers and multiplies:
//     y += <r(b_0) + 4 r(b_1), x_block> / beta      (one scaling per block, after the inner product)
// Small T ("GEMV" regime): memory-bound on the code stream, 4 B (+ scale) per 8 weights.
// One warp owns one output row; lanes stride over the row's blocks (coalesced 128 B of codes per
// step), keep TT token accumulators in registers and reduce with shuffles at the end.
#include <cuda_bf16.h>

#include "common.cuh"
#include "e8_fast.cuh"
#include "e8_io.cuh"

using namespace coset;

namespace {

constexpr int kWarps = 8;

template <int XDT>
__device__ __forceinline__ void load_x8(const void* x, int64_t elem_offset, float (&v)[8]);
template <>
__device__ __forceinline__ void load_x8<0>(const void* x, int64_t off, float (&v)[8]) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + off);
    float4 a = __ldg(p), b = __ldg(p + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load_x8<1>(const void* x, int64_t off, float (&v)[8]) {
    uint4 a = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + off));
    uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Where a result row goes: one buffer, or (output-feature sharding over several GPUs) the same place
// in the result buffer of every rank -- this rank's own and its peers' (peer memory, plain stores over
// NVLink), which replaces the all-gather that would otherwise follow the product.
constexpr int kMaxTargets = 16;
struct Targets {
    float* y[kMaxTargets];
    int n;
};

// CLIP: the weights are clamp(decode / beta, +-clip) as the training layer applies it
// (coset/core/layers.py:463); the clamp acts on single weights, so every weight is scaled first.
template <int TT, int XDT, int MODE, bool CLIP>
__global__ void __launch_bounds__(kWarps * 32)
k_vlut_gemv(const uint32_t* __restrict__ codes, const float* __restrict__ beta, e8::TileDiv td, int n_out, int kb,
            const void* __restrict__ x, int64_t ldx, int T, const float* __restrict__ bias,
            const uint2* __restrict__ table, Targets out, int64_t ldy, float clip) {
    int row = blockIdx.x * kWarps + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    int t0 = blockIdx.y * TT;
    if (row >= n_out) return;
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; ++t) acc[t] = 0.0f;
    const int64_t row_base = (int64_t)row * kb;
    // Lanes stride over the row's blocks in groups of kGroup.  The codes (and scales) of the NEXT group are
    // requested before the table entries of the current one, and all entries of a group before the
    // first multiply, so a group costs one memory round trip (the longer of code fetch and gather)
    // instead of one code fetch plus one gather per block.
    constexpr int kGroup = 4;
    uint32_t code_n[kGroup];
    float s_n[kGroup];
    auto fetch = [&](int blk0) {
#pragma unroll
        for (int j = 0; j < kGroup; ++j) {
            const int blk = blk0 + 32 * j;
            code_n[j] = blk < kb ? __ldcs(codes + row_base + blk) : 0u;
            s_n[j] = (MODE == COSET_SCALE_MUL_TILE && blk < kb) ? __ldg(beta + e8::tile_of(td, row_base + blk)) : 1.0f;
        }
    };
    fetch(lane);
    for (int blk0 = lane; blk0 < kb; blk0 += 32 * kGroup) {
        uint32_t code_c[kGroup];
        float s_c[kGroup];
#pragma unroll
        for (int j = 0; j < kGroup; ++j) { code_c[j] = code_n[j]; s_c[j] = s_n[j]; }
        fetch(blk0 + 32 * kGroup);  // guarded per block: past the row's end it loads nothing
        uint2 t_lo[kGroup], t_hi[kGroup];
#pragma unroll
        for (int j = 0; j < kGroup; ++j) {
            t_lo[j] = __ldg(table + (code_c[j] & 0xffffu));
            t_hi[j] = __ldg(table + (code_c[j] >> 16));
        }
#pragma unroll
        for (int j = 0; j < kGroup; ++j) {
            const int blk = blk0 + 32 * j;
            if (blk < kb) {
                // the block's inner product is formed on twice the (integer) reconstruction and scaled
                // once by 0.5 / beta -- the look-up-table form of the product, 1 multiply per block and
                // token instead of 8 exact divisions per block
                float v2[8];
                e8::twice_from_entries(t_lo[j], t_hi[j], v2);
                const float half_inv = MODE == COSET_SCALE_MUL_TILE ? __fdividef(0.5f, s_c[j]) : 0.5f;
                if (TT >= 4 || CLIP) {  // many tokens share the block: scale the 8 weights once instead
                    float w[8];
                    e8::scale_twice<MODE == COSET_SCALE_MUL_TILE ? 2 : 0>(v2, s_c[j], w);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v2[i] = CLIP ? fminf(fmaxf(w[i], -clip), clip) : w[i];
                }
#pragma unroll
                for (int t = 0; t < TT; ++t) {
                    if (t0 + t < T) {
                        float xv[8];
                        load_x8<XDT>(x, (int64_t)(t0 + t) * ldx + (int64_t)blk * 8, xv);
                        if (TT >= 4 || CLIP) {
                            float a = acc[t];
#pragma unroll
                            for (int i = 0; i < 8; ++i) a = __fmaf_rn(v2[i], xv[i], a);
                            acc[t] = a;
                        } else {
                            float d = 0.0f;
#pragma unroll
                            for (int i = 0; i < 8; ++i) d = __fmaf_rn(v2[i], xv[i], d);
                            acc[t] = __fmaf_rn(d, half_inv, acc[t]);
                        }
                    }
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        float a = acc[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0 && t0 + t < T) {
            const float r = a + (bias ? __ldg(bias + row) : 0.0f);
            for (int k = 0; k < out.n; ++k) out.y[k][(int64_t)(t0 + t) * ldy + row] = r;
        }
    }
}

template <int XDT, int MODE, bool CLIP>
void launch_gemv(int tt, dim3 grid, cudaStream_t st, const uint32_t* codes, const float* beta, e8::TileDiv td, int n_out,
                 int kb, const void* x, int64_t ldx, int T, const float* bias, const uint2* table, const Targets& y, int64_t ldy,
                 float clip) {
#define GEMV_CASE(TT) k_vlut_gemv<TT, XDT, MODE, CLIP><<<grid, kWarps * 32, 0, st>>>(codes, beta, td, n_out, kb, x, ldx, T, bias, table, y, ldy, clip)
    switch (tt) {
        case 1: GEMV_CASE(1); break;
        case 2: GEMV_CASE(2); break;
        case 4: GEMV_CASE(4); break;
        case 8: GEMV_CASE(8); break;
        default: GEMV_CASE(16); break;
    }
#undef GEMV_CASE
}

}  // namespace

static int vlut_gemv_impl(const void* codes, const float* beta, int64_t blocks_per_tile, int n_out, int n_in, const void* x,
                          int x_dtype, int64_t ldx, int T, const float* bias, const Targets& y, int64_t ldy, float clip,
                          void* stream) {
    if (n_out < 0 || n_in < 0 || T < 0 || (n_in % 8) != 0) return fail(COSET_E_BADARG, "bad shape (n_in must be a multiple of 8)");
    if (n_out == 0 || T == 0) return 0;
    if (!codes || !x) return fail(COSET_E_BADARG, "null pointer");
    if (x_dtype != COSET_DTYPE_F32 && x_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown x_dtype");
    if (ldx < n_in || ldy < n_out) return fail(COSET_E_BADARG, "leading dimension too small");
    const int elem = x_dtype == COSET_DTYPE_F32 ? 4 : 2;
    if (!aligned(x, 16) || ((ldx * elem) % 16) != 0 || !aligned(codes, 4))
        return fail(COSET_E_ALIGN, "x rows must be 16-byte aligned and codes 4-byte aligned");
    if (beta && blocks_per_tile < 1) return fail(COSET_E_BADARG, "blocks_per_tile must be >= 1");
    cudaStream_t st = (cudaStream_t)stream;
    const uint2* table = residual_table_q4(st);
    if (!table) return COSET_E_STATE;
    int kb = n_in / 8;
    e8::TileDiv td = e8::make_tile_div(beta ? blocks_per_tile : 1, (int64_t)n_out * kb);
    int tt = T >= 16 ? 16 : (T >= 8 ? 8 : (T >= 4 ? 4 : (T >= 2 ? 2 : 1)));
    dim3 grid((n_out + kWarps - 1) / kWarps, (T + tt - 1) / tt);
    if (grid.y > 65535) return fail(COSET_E_UNSUPPORTED, "T too large for the small-T kernel");
    const uint32_t* c = (const uint32_t*)codes;
    if (!(clip == clip)) return fail(COSET_E_BADARG, "clip is not a number");
#define GEMV_LAUNCH(XDT, MODE)                                                                                              \
    if (clip > 0.0f) launch_gemv<XDT, MODE, true>(tt, grid, st, c, beta, td, n_out, kb, x, ldx, T, bias, table, y, ldy, clip); \
    else launch_gemv<XDT, MODE, false>(tt, grid, st, c, beta, td, n_out, kb, x, ldx, T, bias, table, y, ldy, 0.0f)
    if (x_dtype == COSET_DTYPE_F32) {
        if (beta) { GEMV_LAUNCH(0, 2); } else { GEMV_LAUNCH(0, 0); }
    } else {
        if (beta) { GEMV_LAUNCH(1, 2); } else { GEMV_LAUNCH(1, 0); }
    }
#undef GEMV_LAUNCH
    return check_launch("e8_vlut_gemv");
}

extern "C" int coset_e8_vlut_gemv(const void* codes, const float* beta, int64_t blocks_per_tile, int n_out, int n_in,
                                  const void* x, int x_dtype, int64_t ldx, int T, const float* bias, float* y,
                                  int64_t ldy, float clip, void* stream) {
    if (!y && n_out > 0 && T > 0) return fail(COSET_E_BADARG, "null pointer");
    Targets t = {};
    t.y[0] = y;
    t.n = 1;
    return vlut_gemv_impl(codes, beta, blocks_per_tile, n_out, n_in, x, x_dtype, ldx, T, bias, t, ldy, clip, stream);
}

extern "C" int coset_e8_vlut_gemv_scatter(const void* codes, const float* beta, int64_t blocks_per_tile, int n_out, int n_in,
                                          const void* x, int x_dtype, int64_t ldx, int T, const float* bias,
                                          float* const* y_targets, int n_targets, int64_t ldy, float clip, void* stream) {
    if (n_targets < 1 || n_targets > kMaxTargets || !y_targets) return fail(COSET_E_BADARG, "need 1..16 result buffers");
    Targets t = {};
    for (int k = 0; k < n_targets; ++k) {
        if (!y_targets[k]) return fail(COSET_E_BADARG, "result buffer %d is null", k);
        t.y[k] = y_targets[k];
    }
    t.n = n_targets;
    return vlut_gemv_impl(codes, beta, blocks_per_tile, n_out, n_in, x, x_dtype, ldx, T, bias, t, ldy, clip, stream);
}
