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
// residual-table entry of the all-zero level word: every coordinate 2 * 0 + kTableBias
__device__ __forceinline__ uint2 zero_entry() { return make_uint2(0x07070707u, 0x07070707u); }

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
    int bf16;  // 1: the buffers hold bf16 values (results are rounded to nearest even on the store)
};
__device__ __forceinline__ void store_result(const Targets& out, int64_t idx, float r) {
    for (int k = 0; k < out.n; ++k) {
        if (out.bf16) reinterpret_cast<__nv_bfloat16*>(out.y[k])[idx] = __float2bfloat16_rn(r);
        else out.y[k][idx] = r;
    }
}

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
            t_hi[j] = zero_entry();  // all-zero top-level word: zero residual, no gather
            if (code_c[j] >> 16) t_hi[j] = __ldg(table + (code_c[j] >> 16));
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
            store_result(out, (int64_t)(t0 + t) * ldy + row, r);
        }
    }
}

// One or two tokens: the product is bound by the latency of ONE dependent chain (code -> table entry ->
// multiply), so a row is split over kSplit warps of the same CTA and every lane owns at most kOwn blocks
// whose codes, scales, table entries and activations are ALL requested before the first multiply.  The
// partial sums of a row are added in a fixed order through shared memory (deterministic, no atomics).
constexpr int kSplit = 4;              // warps per output row
constexpr int kRowsPerCta = kWarps / kSplit;
constexpr int kOwn = 4;                // blocks per lane and pass

template <int TT, int XDT, int MODE, bool CLIP>
__global__ void __launch_bounds__(kWarps * 32)
k_vlut_gemv_split(const uint32_t* __restrict__ codes, const float* __restrict__ beta, e8::TileDiv td, int n_out, int kb,
                  const void* __restrict__ x, int64_t ldx, int T, const float* __restrict__ bias,
                  const uint2* __restrict__ table, const uint32_t* __restrict__ packed, Targets out, int64_t ldy, float clip) {
    __shared__ float part[kRowsPerCta][kSplit][TT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r_in = warp / kSplit, part_id = warp % kSplit;
    const int row = blockIdx.x * kRowsPerCta + r_in;
    const int t0 = blockIdx.y * TT;
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; ++t) acc[t] = 0.0f;
    if (row < n_out) {
        const int64_t row_base = (int64_t)row * kb;
        // lane l of part p owns blocks p*32 + l + j * (32 * kSplit): a warp reads 128 contiguous bytes of codes
        for (int blk0 = part_id * 32 + lane; blk0 < kb; blk0 += 32 * kSplit * kOwn) {
            uint32_t code[kOwn];
            float sc[kOwn];
#pragma unroll
            for (int j = 0; j < kOwn; ++j) {
                const int blk = blk0 + j * 32 * kSplit;
                code[j] = blk < kb ? __ldcs(codes + row_base + blk) : 0u;
                sc[j] = (MODE == COSET_SCALE_MUL_TILE && blk < kb) ? __ldg(beta + e8::tile_of(td, row_base + blk)) : 1.0f;
            }
            float xv[kOwn][TT][8];
#pragma unroll
            for (int j = 0; j < kOwn; ++j) {
                const int blk = blk0 + j * 32 * kSplit;
#pragma unroll
                for (int t = 0; t < TT; ++t) {
                    if (blk < kb && t0 + t < T) {
                        load_x8<XDT>(x, (int64_t)(t0 + t) * ldx + (int64_t)blk * 8, xv[j][t]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) xv[j][t][i] = 0.0f;
                    }
                }
            }
            // The residual of an all-zero level word is the zero vector and the top level of a quantiser that is
            // not overloaded is almost always that word: its lookup is skipped.  One token reads the 8-byte table
            // entries (fewest instructions: 9.7 us against 10.4 for a 4096 x 4096 weight), two tokens the packed
            // 4-byte entries (256 KB for all level words, mostly L1 hits: 13.7 us against 15.7).
            constexpr bool PACKED = TT == 2;
            uint2 t_lo[kOwn], t_hi[kOwn];
#pragma unroll
            for (int j = 0; j < kOwn; ++j) {
                if (PACKED) {
                    t_lo[j].x = t_hi[j].x = e8::kPackedZeroEntry;
                    if (code[j] & 0xffffu) t_lo[j].x = __ldg(packed + (code[j] & 0xffffu));
                    if (code[j] >> 16) t_hi[j].x = __ldg(packed + (code[j] >> 16));
                } else {
                    t_lo[j] = __ldg(table + (code[j] & 0xffffu));
                    t_hi[j] = zero_entry();
                    if (code[j] >> 16) t_hi[j] = __ldg(table + (code[j] >> 16));
                }
            }
#pragma unroll
            for (int j = 0; j < kOwn; ++j) {
                float v2[8];
                if (PACKED) e8::twice_from_packed(t_lo[j].x, t_hi[j].x, v2);
                else e8::twice_from_entries(t_lo[j], t_hi[j], v2);
                if (CLIP) {
                    float w[8];
                    e8::scale_twice<MODE == COSET_SCALE_MUL_TILE ? 2 : 0>(v2, sc[j], w);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v2[i] = fminf(fmaxf(w[i], -clip), clip);
                }
                const float half_inv = CLIP ? 1.0f : (MODE == COSET_SCALE_MUL_TILE ? __fdividef(0.5f, sc[j]) : 0.5f);
#pragma unroll
                for (int t = 0; t < TT; ++t) {
                    float d = 0.0f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) d = __fmaf_rn(v2[i], xv[j][t][i], d);
                    acc[t] = __fmaf_rn(d, half_inv, acc[t]);
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        float a = acc[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0) part[r_in][part_id][t] = a;
    }
    __syncthreads();
    if (part_id == 0 && lane < TT && row < n_out && t0 + lane < T) {
        float r = part[r_in][0][lane];
#pragma unroll
        for (int p = 1; p < kSplit; ++p) r += part[r_in][p][lane];
        r += bias ? __ldg(bias + row) : 0.0f;
        store_result(out, (int64_t)(t0 + lane) * ldy + row, r);
    }
}

// ---------------------------------------------------------------------------------------------
// bf16 activations, up to 16 tokens: the multiply-adds go to the tensor cores (mma.sync m16n8k16, bf16 in,
// float32 accumulate), which removes them and the per-token handling of the activations from the
// instruction stream -- the scalar kernel above spends 8 FMA + 8 activation unpacks per block AND token.
//
// One CTA owns 16 output rows and the whole K; its warps take interleaved units of 8 blocks (64 values
// of K) and their partial tiles are added in a fixed order through shared memory (deterministic).
// Per unit a warp reads the 16 x 8 codes (and scales) as ONE 16-byte vector per lane -- lane l holds row
// l/2, blocks 4 (l%2) .. 4 (l%2) + 3 -- and hands every code to the four lanes whose A-fragment slots it
// fills with shuffles: thread (g = lane/4, c = lane%4) of a k16 step needs the weights k = 2c, 2c+1 of two
// blocks of rows g and g+8, i.e. ONE 32-bit word of each residual-table entry (gathered as such).
// The bytes become floats through the byte-permute trick, are scaled by 0.5 / beta (clamped when asked)
// and packed to bf16 pairs.  The activations are the B fragments, read as 32-bit words from x (L1-resident).
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// float(byte `sel` of v) + 1.5 * 2^23, sel = 0..3 at run time
__device__ __forceinline__ float byte_to_magic_float(uint32_t v, uint32_t sel) {
    return __uint_as_float(__byte_perm(v, 0x4B400000u, 0x7640u + sel));
}

constexpr int kMmaWarps = 8;  // K is split over the warps of a CTA (16 warps measured slower: one CTA per SM, two waves)

template <int MODE, bool CLIP, int NT>
__global__ void __launch_bounds__(kMmaWarps * 32)
k_vlut_mma(const uint32_t* __restrict__ codes, const float* __restrict__ beta, int64_t blocks_per_tile, int n_out, int kb,
           const __nv_bfloat16* __restrict__ x, int64_t ldx, int T, const float* __restrict__ bias,
           const uint2* __restrict__ table, Targets out, int64_t ldy, float clip) {
    __shared__ float part[kMmaWarps][16][8 * NT + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int row0 = blockIdx.x * 16;
    const int t0 = blockIdx.y * (8 * NT);
    const int units = kb >> 3;
    // loading role: row l/2, blocks 4 (l%2) .. +3 of the unit
    const int lrow = row0 + (lane >> 1);
    const bool lrow_ok = lrow < n_out;
    const int64_t lbase = (int64_t)lrow * kb + (lane & 1) * 4;
    const bool per_block = MODE == COSET_SCALE_MUL_TILE && blocks_per_tile == 1;
    float d[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) d[n][0] = d[n][1] = d[n][2] = d[n][3] = 0.0f;
    const uint32_t wsel = (uint32_t)(c >> 1);          // which 32-bit word of a table entry holds k = 2c, 2c+1
    const uint32_t bsel = (uint32_t)((c & 1) * 2);     // first of the two bytes inside that word
    const char* table_w = reinterpret_cast<const char*>(table) + wsel * 4;
    const float kOff = 12582912.0f + 5.0f * e8::kTableBias;
    // activations of this thread's B fragments: token t0 + 8 n + g, k = k0 + 2c (+8)
    const __nv_bfloat16* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const int t = t0 + 8 * n + g;
        xok[n] = t < T;
        xrow[n] = x + (int64_t)(xok[n] ? t : 0) * ldx + 2 * c;
    }
    auto load_unit = [&](int u, uint4& cv, float4& iv) {
        cv = make_uint4(0u, 0u, 0u, 0u);
        iv = make_float4(0.5f, 0.5f, 0.5f, 0.5f);
        if (lrow_ok && u < units) {
            cv = __ldcs(reinterpret_cast<const uint4*>(codes + lbase + (int64_t)u * 8));
            if (per_block) {
                const float4 b = __ldcs(reinterpret_cast<const float4*>(beta + lbase + (int64_t)u * 8));
                iv = make_float4(__fdividef(0.5f, b.x), __fdividef(0.5f, b.y), __fdividef(0.5f, b.z), __fdividef(0.5f, b.w));
            } else if (MODE == COSET_SCALE_MUL_TILE) {
                const float b = __ldg(beta + (lbase + (int64_t)u * 8) / blocks_per_tile);
                const float r = __fdividef(0.5f, b);
                iv = make_float4(r, r, r, r);
            }
        }
    };
    uint4 cv_n;
    float4 iv_n;
    load_unit(warp, cv_n, iv_n);
    for (int u = warp; u < units; u += kMmaWarps) {
        const uint4 cv = cv_n;
        const float4 iv = iv_n;
        load_unit(u + kMmaWarps, cv_n, iv_n);
        const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
        const float iw[4] = {iv.x, iv.y, iv.z, iv.w};
        // codes and inverse scales of this thread's slots: step s uses blocks 2s, 2s+1 of rows g, g+8
        uint32_t code[4][4];
        float inv[4][4];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // j: 0 = (g, 2s), 1 = (g+8, 2s), 2 = (g, 2s+1), 3 = (g+8, 2s+1)
                const int blk = 2 * s + (j >> 1);
                const int src = 2 * (g + 8 * (j & 1)) + (blk >> 2);
                code[s][j] = __shfl_sync(0xffffffffu, cw[blk & 3], src);
                inv[s][j] = __shfl_sync(0xffffffffu, iw[blk & 3], src);
            }
        }
        uint32_t wlo[4][4], whi[4][4];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                wlo[s][j] = __ldg(reinterpret_cast<const uint32_t*>(table_w + (size_t)(code[s][j] & 0xffffu) * 8));
                whi[s][j] = 0x07070707u;  // all-zero top-level word: zero residual, no gather
                if (code[s][j] >> 16) whi[s][j] = __ldg(reinterpret_cast<const uint32_t*>(table_w + (size_t)(code[s][j] >> 16) * 8));
            }
        }
        const int k0 = u * 64;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            uint32_t a[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t bytes = wlo[s][j] + 4u * whi[s][j];
                float w0 = __fmul_rn(__fsub_rn(byte_to_magic_float(bytes, bsel), kOff), inv[s][j]);
                float w1 = __fmul_rn(__fsub_rn(byte_to_magic_float(bytes, bsel + 1u), kOff), inv[s][j]);
                if (CLIP) {
                    w0 = fminf(fmaxf(w0, -clip), clip);
                    w1 = fminf(fmaxf(w1, -clip), clip);
                }
                __nv_bfloat162 h = __floats2bfloat162_rn(w0, w1);
                a[j] = *reinterpret_cast<uint32_t*>(&h);
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                uint32_t b0 = 0u, b1 = 0u;
                if (xok[n]) {
                    b0 = __ldg(reinterpret_cast<const uint32_t*>(xrow[n] + k0 + 16 * s));
                    b1 = __ldg(reinterpret_cast<const uint32_t*>(xrow[n] + k0 + 16 * s + 8));
                }
                mma_bf16_16816(d[n], a, b0, b1);
            }
        }
    }

    // accumulator layout: d[0], d[1] = (row g, tokens 2c, 2c+1); d[2], d[3] = (row g+8, same tokens)
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        part[warp][g][8 * n + 2 * c] = d[n][0];
        part[warp][g][8 * n + 2 * c + 1] = d[n][1];
        part[warp][g + 8][8 * n + 2 * c] = d[n][2];
        part[warp][g + 8][8 * n + 2 * c + 1] = d[n][3];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 16 * 8 * NT; e += kMmaWarps * 32) {
        const int r = e & 15, t = e >> 4;  // consecutive threads write consecutive rows of one token
        if (row0 + r < n_out && t0 + t < T) {
            float v = part[0][r][t];
#pragma unroll
            for (int w = 1; w < kMmaWarps; ++w) v += part[w][r][t];
            v += bias ? __ldg(bias + row0 + r) : 0.0f;
            store_result(out, (int64_t)(t0 + t) * ldy + row0 + r, v);
        }
    }
}

template <int XDT, int MODE, bool CLIP>
void launch_gemv(int tt, dim3 grid, cudaStream_t st, const uint32_t* codes, const float* beta, e8::TileDiv td, int n_out,
                 int kb, const void* x, int64_t ldx, int T, const float* bias, const uint2* table, const Targets& y, int64_t ldy,
                 float clip) {
#define GEMV_CASE(TT) k_vlut_gemv<TT, XDT, MODE, CLIP><<<grid, kWarps * 32, 0, st>>>(codes, beta, td, n_out, kb, x, ldx, T, bias, table, y, ldy, clip)
    if (tt <= 2) {  // one or two tokens: the split-row kernel
        dim3 sgrid((n_out + kRowsPerCta - 1) / kRowsPerCta, grid.y);
        const uint32_t* packed = residual_table_q4_packed(st);
        if (tt == 1) k_vlut_gemv_split<1, XDT, MODE, CLIP><<<sgrid, kWarps * 32, 0, st>>>(codes, beta, td, n_out, kb, x, ldx, T, bias, table, packed, y, ldy, clip);
        else k_vlut_gemv_split<2, XDT, MODE, CLIP><<<sgrid, kWarps * 32, 0, st>>>(codes, beta, td, n_out, kb, x, ldx, T, bias, table, packed, y, ldy, clip);
        return;
    }
    switch (tt) {
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
    // bf16 activations, three tokens or more: tensor-core kernel when the layout allows 16-byte code vectors and
    // whole units per scale tile (one or two tokens are faster in the split-row kernel: 11 us against 17 us)
    if (T >= 3 && x_dtype == COSET_DTYPE_BF16 && (kb % 8) == 0 && aligned(codes, 16) && (ldx % 2) == 0 &&
        (!beta || blocks_per_tile == 1 || (blocks_per_tile % 8) == 0) && (!beta || blocks_per_tile != 1 || aligned(beta, 16))) {
        const int nt = T > 8 ? 2 : 1;
        dim3 mgrid((n_out + 15) / 16, (T + 8 * nt - 1) / (8 * nt));
        if (mgrid.y > 65535) return fail(COSET_E_UNSUPPORTED, "T too large for the small-T kernel");
        const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
#define MMA_LAUNCH(MODE, CLIPB, NT) k_vlut_mma<MODE, CLIPB, NT><<<mgrid, kMmaWarps * 32, 0, st>>>(c, beta, beta ? blocks_per_tile : 1, n_out, kb, xb, ldx, T, bias, table, y, ldy, clip)
        if (beta) {
            if (clip > 0.0f) { if (nt == 2) MMA_LAUNCH(2, true, 2); else MMA_LAUNCH(2, true, 1); }
            else { if (nt == 2) MMA_LAUNCH(2, false, 2); else MMA_LAUNCH(2, false, 1); }
        } else {
            if (clip > 0.0f) { if (nt == 2) MMA_LAUNCH(0, true, 2); else MMA_LAUNCH(0, true, 1); }
            else { if (nt == 2) MMA_LAUNCH(0, false, 2); else MMA_LAUNCH(0, false, 1); }
        }
#undef MMA_LAUNCH
        return check_launch("e8_vlut_gemv (tensor-core form)");
    }
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
                                  const void* x, int x_dtype, int64_t ldx, int T, const float* bias, void* y,
                                  int y_dtype, int64_t ldy, float clip, void* stream) {
    if (!y && n_out > 0 && T > 0) return fail(COSET_E_BADARG, "null pointer");
    if (y_dtype != COSET_DTYPE_F32 && y_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown y_dtype");
    Targets t = {};
    t.y[0] = (float*)y;
    t.n = 1;
    t.bf16 = y_dtype == COSET_DTYPE_BF16 ? 1 : 0;
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
