// E8 HNLQ codec kernels and their C-ABI entry points: projection, encode, decode, fused
// round trip (quantise), packed <-> float32 digit views, and the q=4 residual table.
//
// One thread owns one 8-vector ("block"): 32 B in (two 128-bit loads, a warp reads 1 KiB
// contiguously), all state in registers, 4 B packed code out.  The kernels are HBM-bound by
// design; algorithmic bytes per block (q=4, M=2, float32): encode 32+4 (+4 per-block scale),
// decode 4+32 (+4), round trip 32+32 (+4).
#include <stdarg.h>

#include <mutex>

#include "common.cuh"
#include "e8_fast.cuh"
#include "e8_io.cuh"
#include "e8_literal.cuh"

namespace coset {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
}
int check_launch(const char* what) { return check_cuda(cudaGetLastError(), what); }

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace coset

using namespace coset;

namespace {

constexpr int kThreads = 256;

template <int MODE>
__device__ __forceinline__ float scale_in(float v, float s) {
    if (MODE == COSET_SCALE_DIV_SCALAR) return __fdiv_rn(v, s);
    if (MODE == COSET_SCALE_MUL_TILE) return __fmul_rn(v, s);
    return v;
}
template <int MODE>
__device__ __forceinline__ float scale_out(float v, float s) {
    if (MODE == COSET_SCALE_DIV_SCALAR) return __fmul_rn(v, s);
    if (MODE == COSET_SCALE_MUL_TILE) return __fdiv_rn(v, s);
    return v;
}
template <int MODE>
__device__ __forceinline__ float load_scale(const float* scale, const e8::TileDiv& td, int64_t block) {
    if (MODE == COSET_SCALE_DIV_SCALAR) return __ldg(scale);
    if (MODE == COSET_SCALE_MUL_TILE) {
        // per-block scales are streamed once; per-row scales are reused by the whole row
        return td.divisor == 1 ? __ldcs(scale + block) : __ldg(scale + e8::tile_of(td, block));
    }
    return 1.0f;
}

__device__ __forceinline__ float clampf(float v, float clip) {
    // torch.clamp: NaN stays NaN
    if (clip > 0.0f) v = (v < -clip) ? -clip : ((v > clip) ? clip : v);
    return v;
}

// ---------------------------------------------------------------- projection
__global__ void __launch_bounds__(kThreads) k_projection(const float* __restrict__ x, int64_t n, float* __restrict__ y) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    float v[8], o[8];
    e8::Row8<0>::load(x, b, v);
    e8::projection(v, o);
    e8::Row8<0>::store(y, b, o);
}

// ---------------------------------------------------------------- generic (any 2<=q<=16, M<=8)
// e8_encode, coset/core/e8/codecs.py:63-83: x_l starts as the scaled input and is divided by q
// after every level (cumulative IEEE divisions, no re-quantisation).
template <int BPD>
__device__ __forceinline__ void encode_levels_generic(float (&xl)[8], int q, int M, uint32_t* words) {
    float qf = (float)q;
    for (int m = 0; m < M; ++m) {
        float y[8];
        int d[8];
        bool half = e8::projection(xl, y);
        e8::encode_coords(y, half, q, d);
        words[m] = e8::pack_level<BPD>(d);
#pragma unroll
        for (int i = 0; i < 8; ++i) xl[i] = __fdiv_rn(xl[i], qf);
    }
}

// E8Decoder._full_decode, coset/core/e8/codecs.py:159-172 (before the final scale).
template <int BPD>
__device__ __forceinline__ void decode_levels_generic(const uint32_t* words, int q, int M, float (&xh)[8]) {
    float qf = (float)q, w = 1.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) xh[i] = 0.0f;
    for (int m = 0; m < M; ++m) {
        int d[8];
        float r[8];
        e8::unpack_level<BPD>(words[m], d);
        e8::level_residual(d, qf, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) xh[i] = __fadd_rn(xh[i], __fmul_rn(w, r[i]));
        w = __fmul_rn(w, qf);
    }
}

template <int BPD>
struct LevelWord;
template <>
struct LevelWord<2> { typedef uint16_t type; };
template <>
struct LevelWord<4> { typedef uint32_t type; };

template <int DT, int MODE, int BPD>
__global__ void __launch_bounds__(kThreads)
k_encode_generic(const void* __restrict__ x, const float* __restrict__ scale, e8::TileDiv td, int64_t n, int q,
                 int M, void* __restrict__ codes) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    float v[8];
    e8::Row8<DT>::load(x, b, v);
    float s = load_scale<MODE>(scale, td, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = scale_in<MODE>(v[i], s);
    uint32_t words[8];
    encode_levels_generic<BPD>(v, q, M, words);
    typename LevelWord<BPD>::type* out = reinterpret_cast<typename LevelWord<BPD>::type*>(codes) + b * M;
    for (int m = 0; m < M; ++m) out[m] = (typename LevelWord<BPD>::type)words[m];
}

template <int DT, int MODE, int BPD>
__global__ void __launch_bounds__(kThreads)
k_decode_generic(const void* __restrict__ codes, const float* __restrict__ scale, e8::TileDiv td, int64_t n, int q,
                 int M, void* __restrict__ out) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    const typename LevelWord<BPD>::type* in = reinterpret_cast<const typename LevelWord<BPD>::type*>(codes) + b * M;
    uint32_t words[8];
    for (int m = 0; m < M; ++m) words[m] = in[m];
    float xh[8];
    decode_levels_generic<BPD>(words, q, M, xh);
    float s = load_scale<MODE>(scale, td, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) xh[i] = scale_out<MODE>(xh[i], s);
    e8::Row8<DT>::store(out, b, xh);
}

template <int DTI, int DTO, int MODE, int BPD>
__global__ void __launch_bounds__(kThreads)
k_quantize_generic(const void* __restrict__ x, const float* __restrict__ scale, e8::TileDiv td, int64_t n, int q,
                   int M, float clip, void* __restrict__ out, void* __restrict__ codes) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    float v[8];
    e8::Row8<DTI>::load(x, b, v);
    float s = load_scale<MODE>(scale, td, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = scale_in<MODE>(v[i], s);
    uint32_t words[8];
    encode_levels_generic<BPD>(v, q, M, words);
    if (codes) {
        typename LevelWord<BPD>::type* co = reinterpret_cast<typename LevelWord<BPD>::type*>(codes) + b * M;
        for (int m = 0; m < M; ++m) co[m] = (typename LevelWord<BPD>::type)words[m];
    }
    float xh[8];
    decode_levels_generic<BPD>(words, q, M, xh);
#pragma unroll
    for (int i = 0; i < 8; ++i) xh[i] = clampf(scale_out<MODE>(xh[i], s), clip);
    e8::Row8<DTO>::store(out, b, xh);
}

// ---------------------------------------------------------------- q = 4, M = 2 (one uint32 per block)
template <int DT, int MODE, bool LITERAL>
__global__ void __launch_bounds__(kThreads, 6)
k_encode_q4m2(const void* __restrict__ x, const float* __restrict__ scale, e8::TileDiv td, int64_t n,
              uint32_t* __restrict__ codes) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    float v[8];
    e8::Row8<DT>::load(x, b, v);
    float s = load_scale<MODE>(scale, td, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = scale_in<MODE>(v[i], s);
    __stcs(codes + b, e8::encode_q4m2<LITERAL>(v));
}

// Queued encoder (the production path for q=4, M=2).
//
// Warps are persistent; one loop iteration of a warp covers kRowsPerIter * 32 consecutive blocks,
// one row per lane and sub-step.  Every lane runs the cheap rint-based level-0 path; whatever that
// path cannot finish -- a block on a rounding tie, a block whose top level is not the origin, a
// non-finite block -- is NOT handled in place (that would idle the other 31 lanes for hundreds of
// instructions): the lane appends the block's index, its code so far and its first open level to
// a per-warp queue in shared memory (a shared-memory atomic hands out the slot, so no warp-wide
// vote sits on the common path).  Once per iteration the warp looks at the queue length; with 32
// or more entries (and at the end) it drains 32 of them with all lanes busy: every lane reads the
// row of its entry again -- one memory round trip per 32 deferred blocks -- and completes it with
// the always-valid tiers.  This also serves an overloaded quantiser, where most blocks need the top
// level: the queue then fills every iteration and is drained by full warps (running that level in
// place for the lanes that need it was measured and is slower at every scale).
constexpr int kRowsPerIter = 3;   // rows per lane and loop iteration (measured on 2^25 blocks: 2 -> 0.395 ms, 3 -> 0.387, 4 -> 0.388)
constexpr int kQueueSlots = 32 * (kRowsPerIter + 1);  // < 32 left after a drain + at most 32 per sub-step
constexpr int kEncWarps = kThreads / 32;

// CTAs of the queued encoder: enough for every warp to get one iteration, at most kEncCtasPerSm per SM.
constexpr int kEncCtasPerSm = 12;
inline unsigned encoder_grid(int64_t n_blocks) {
    const int64_t per_cta = (int64_t)kThreads * kRowsPerIter;
    const int64_t need = (n_blocks + per_cta - 1) / per_cta;
    const int64_t cap = (int64_t)sm_count() * kEncCtasPerSm;
    return (unsigned)(need < cap ? (need < 1 ? 1 : need) : cap);
}

// RECON = false: codes only (e8_encode).  RECON = true: the fused round trip -- every finished code is
// decoded through the residual table, unscaled, clamped and written as [n, 8] of type DTO; the
// packed code is stored only if `codes` is not null (e8_quantize / the layer's weight path).
template <int DT, int MODE, bool RECON, int DTO>
__global__ void __launch_bounds__(kThreads, 4)
k_encode_q4m2_queued(const void* __restrict__ x, const float* __restrict__ scale, e8::TileDiv td, int64_t n,
                     uint32_t* __restrict__ codes, const uint2* __restrict__ table, void* __restrict__ out, float clip) {
    __shared__ uint32_t q_meta[kEncWarps][4][kQueueSlots];  // block index lo / hi, code so far, first open level
    __shared__ int q_count[kEncWarps];
    auto emit = [&](int64_t b, uint32_t code, float s) {
        if (!RECON) {
            __stcs(codes + b, code);
        } else {
            if (codes) __stcs(codes + b, code);
            float v2[8], xh[8];
            e8::decode_q4m2_twice(code, table, v2);
            e8::scale_twice<MODE>(v2, s, xh);
#pragma unroll
            for (int i = 0; i < 8; ++i) xh[i] = clampf(xh[i], clip);
            e8::Row8<DTO>::store(out, b, xh);
        }
    };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) q_count[warp] = 0;
    __syncwarp();
    int count = 0;  // warp-uniform copy of q_count[warp] as of the last look

    // Scaled row of block b (only called for b < n).
    auto load_row = [&](int64_t b, float (&v)[8], float& s) {
        e8::Row8<DT>::load(x, b, v);
        s = load_scale<MODE>(scale, td, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = scale_in<MODE>(v[i], s);
    };
    // Completes the last min(count, 32) queued blocks with all lanes busy.
    auto drain = [&]() {
        const int take = count < 32 ? count : 32;
        if (lane < take) {
            const int e = count - take + lane;
            const int64_t b = (int64_t)(((uint64_t)q_meta[warp][1][e] << 32) | q_meta[warp][0][e]);
            const uint32_t code = q_meta[warp][2][e];
            const int start = (int)q_meta[warp][3][e];
            float v[8], s;
            load_row(b, v, s);
            emit(b, e8::finish_block_q4(v, code, start), s);
        }
        count -= take;
        __syncwarp();
        if (lane == 0) q_count[warp] = count;
        __syncwarp();
    };

    const int64_t span = 32 * kRowsPerIter;
    const int64_t stride = (int64_t)gridDim.x * kEncWarps * span;
    for (int64_t base = ((int64_t)blockIdx.x * kEncWarps + warp) * span; base < n; base += stride) {
        uint32_t code[kRowsPerIter];
        int open_level[kRowsPerIter];  // first level still open; 2 = finished, 3 = no block (past the end)
        float sc[kRowsPerIter];
        bool any_open = false;
        {
            // All rows are requested first; the level-0 path then runs row after row in straight-line
            // code, so the loads of the later rows and the FP32-heavy head of one row overlap the
            // ALU-heavy tail of the previous one.  The rows are not kept beyond this scope.
            float v[kRowsPerIter][8];
#pragma unroll
            for (int j = 0; j < kRowsPerIter; ++j) {
                const int64_t b = base + j * 32 + lane;
                sc[j] = 1.0f;
                if (b < n) {
                    e8::Row8<DT>::load(x, b, v[j]);
                    sc[j] = load_scale<MODE>(scale, td, b);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[j][i] = 0.0f;
                }
            }
#pragma unroll
            for (int j = 0; j < kRowsPerIter; ++j) {
                const bool active = base + j * 32 + lane < n;
                float s1 = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[j][i] = scale_in<MODE>(v[j][i], sc[j]);
                    s1 += fabsf(v[j][i]);
                }
                // max |x_i| as a tree of three-input maxima (4 instructions instead of 8)
                const float m0 = fmaxf(fmaxf(fabsf(v[j][0]), fabsf(v[j][1])), fabsf(v[j][2]));
                const float m1 = fmaxf(fmaxf(fabsf(v[j][3]), fabsf(v[j][4])), fabsf(v[j][5]));
                const float amax = fmaxf(fmaxf(m0, m1), fmaxf(fabsf(v[j][6]), fabsf(v[j][7])));
                const bool finite = (s1 - s1) == 0.0f;
                // top level: origin unless max|x| > 1.96 or sum|x| > 7.96 (the level sees x / 4); decided
                // here so that only one predicate, not amax and s1, lives across the level-0 path
                const bool top_open = !(amax <= 1.96f && s1 <= 7.96f);
                code[j] = 0;
                open_level[j] = 2;
                if (!finite) {
                    open_level[j] = 0;
                } else if (!(amax <= 0.49f && s1 <= 1.99f)) {
                    if (!e8::level_fast_q4<false>(v[j], amax, code[j])) open_level[j] = 0;
                }
                if (open_level[j] == 2 && top_open) open_level[j] = 1;
                if (!active) open_level[j] = 3;  // past the end: neither stored nor queued
                if (open_level[j] == 2) emit(base + j * 32 + lane, code[j], sc[j]);
                any_open = any_open || open_level[j] < 2;
            }
        }
        if (any_open) {  // rare: one branch per iteration keeps the queue code off the common path
#pragma unroll
            for (int j = 0; j < kRowsPerIter; ++j) {
                if (open_level[j] < 2) {
                    const int64_t b = base + j * 32 + lane;
                    const int pos = atomicAdd(&q_count[warp], 1);
                    q_meta[warp][0][pos] = (uint32_t)b;
                    q_meta[warp][1][pos] = (uint32_t)((uint64_t)b >> 32);
                    q_meta[warp][2][pos] = code[j];
                    q_meta[warp][3][pos] = (uint32_t)open_level[j];
                }
            }
        }
        __syncwarp();
        count = *reinterpret_cast<volatile int*>(&q_count[warp]);
        while (count >= 32) drain();
    }
    while (count > 0) drain();
}

// Two blocks per thread (kThreads apart, so every access stays coalesced): both codes are
// loaded before the first table lookup, which doubles the gathers in flight per thread.
constexpr int kDecPerThread = 2;
// TABLE is `uint2` (8-byte entries) or `uint32_t` (packed 4-byte entries, used for float32 output,
// where the kernel is bound by the gathers and not by instruction issue).
template <int DT, int MODE, typename TABLE>
__global__ void __launch_bounds__(kThreads)
k_decode_q4m2(const uint32_t* __restrict__ codes, const float* __restrict__ scale, e8::TileDiv td, int64_t n,
              const TABLE* __restrict__ table, void* __restrict__ out) {
    int64_t base = (int64_t)blockIdx.x * (kThreads * kDecPerThread) + threadIdx.x;
    uint32_t code[kDecPerThread];
    float s[kDecPerThread];
#pragma unroll
    for (int j = 0; j < kDecPerThread; ++j) {
        int64_t b = base + j * kThreads;
        code[j] = b < n ? __ldcs(codes + b) : 0u;
        s[j] = b < n ? load_scale<MODE>(scale, td, b) : 1.0f;
    }
#pragma unroll
    for (int j = 0; j < kDecPerThread; ++j) {
        int64_t b = base + j * kThreads;
        if (b < n) {
            float v2[8], xh[8];
            e8::decode_q4m2_twice(code[j], table, v2);
            e8::scale_twice<MODE>(v2, s[j], xh);
            e8::Row8<DT>::store(out, b, xh);
        }
    }
}

// Residual table of the q=4 decoder, produced by the literal float32 decoder itself:
// entry[w] = 2 * (G b - 4 Q(G b / 4)) + 7 for the 16-bit level word w, as 8 unsigned bytes.
__global__ void k_build_table_q4(uint2* __restrict__ table, uint32_t* __restrict__ packed, int* __restrict__ bad) {
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= 65536) return;
    int d[8];
    float r[8];
    e8::unpack_level<2>((uint32_t)w, d);
    e8::level_residual(d, 4.0f, r);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        lo |= ((uint32_t)((__float2int_rn(__fmul_rn(r[i], 2.0f)) + e8::kTableBias) & 0xff)) << (8 * i);
        hi |= ((uint32_t)((__float2int_rn(__fmul_rn(r[i + 4], 2.0f)) + e8::kTableBias) & 0xff)) << (8 * i);
    }
    table[w] = make_uint2(lo, hi);
    // packed entry (layout at e8::biased_bytes_q4m2); `bad` counts residuals that do not fit it
    int t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = __float2int_rn(__fmul_rn(r[i], 2.0f));
    const int p = t[0] & 1;
    uint32_t e = (uint32_t)p << 31;
    bool ok = true;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int nib = (t[i] - p + (i < 7 ? e8::kNibbleBias : e8::kNibbleBias7)) >> 1;
        ok = ok && ((t[i] & 1) == p) && nib >= 0 && nib <= (i < 7 ? 15 : 7);
        e |= ((uint32_t)nib & 0xfu) << (4 * i);
    }
    if (!ok) atomicAdd(bad, 1);
    packed[w] = e;
}

// ---------------------------------------------------------------- digit views
template <int BPD>
__global__ void __launch_bounds__(kThreads)
k_unpack_f32(const void* __restrict__ codes, int64_t n_words, float* __restrict__ digits) {
    int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;  // one level word per thread
    if (i >= n_words) return;
    uint32_t w = reinterpret_cast<const typename LevelWord<BPD>::type*>(codes)[i];
    int d[8];
    float f[8];
    e8::unpack_level<BPD>(w, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = (float)d[j];
    e8::Row8<0>::store(digits, i, f);
}

template <int BPD>
__global__ void __launch_bounds__(kThreads)
k_pack_f32(const float* __restrict__ digits, int64_t n_words, int q, void* __restrict__ codes) {
    int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n_words) return;
    float f[8];
    int d[8];
    e8::Row8<0>::load(digits, i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) d[j] = e8::floored_mod(__float2int_rn(f[j]), q);
    reinterpret_cast<typename LevelWord<BPD>::type*>(codes)[i] = (typename LevelWord<BPD>::type)e8::pack_level<BPD>(d);
}

inline unsigned grid_for(int64_t n) { return (unsigned)((n + kThreads - 1) / kThreads); }

int check_common(const void* a, const void* b, int64_t n_blocks, int q, int M) {
    if (n_blocks < 0) return fail(COSET_E_BADARG, "n_blocks is negative");
    if (n_blocks > 0 && (!a || !b)) return fail(COSET_E_BADARG, "null data pointer");
    if (q < 2 || q > 16 || M < 1 || M > 8) return fail(COSET_E_UNSUPPORTED, "unsupported q=%d M=%d (need 2<=q<=16, 1<=M<=8)", q, M);
    if ((int64_t)grid_for(n_blocks) != (n_blocks + kThreads - 1) / kThreads || n_blocks > ((int64_t)1 << 38))
        return fail(COSET_E_BADARG, "n_blocks too large");
    return 0;
}
int check_scale(const float* scale, int mode, int64_t bpt) {
    if (mode < 0 || mode > 2) return fail(COSET_E_BADARG, "unknown scale_mode %d", mode);
    if (mode != COSET_SCALE_NONE && !scale) return fail(COSET_E_BADARG, "scale is null");
    if (mode == COSET_SCALE_MUL_TILE && bpt < 1) return fail(COSET_E_BADARG, "blocks_per_tile must be >= 1");
    return 0;
}

}  // namespace

namespace coset {

const uint2* residual_table_q4(cudaStream_t stream) {
    static std::mutex mu;
    static uint2* tables[64] = {nullptr};
    int dev = 0;
    if (check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return nullptr;
    if (dev < 0 || dev >= 64) { fail(COSET_E_STATE, "device index %d out of range", dev); return nullptr; }
    std::lock_guard<std::mutex> lock(mu);
    if (!tables[dev]) {
        uint2* t = nullptr;  // 65536 x 8 B, then 65536 x 4 B packed, then the builder's self-check word
        if (check_cuda(cudaMalloc(&t, 65536 * (sizeof(uint2) + sizeof(uint32_t)) + 16), "cudaMalloc(residual table)")) return nullptr;
        uint32_t* packed = reinterpret_cast<uint32_t*>(t + 65536);
        int* bad = reinterpret_cast<int*>(packed + 65536);
        int bad_host = -1;
        // Built on the caller's stream: every later use on any stream must see it complete, so
        // the one-time build synchronises that stream.
        bool failed = check_cuda(cudaMemsetAsync(bad, 0, sizeof(int), stream), "table build") != 0;
        if (!failed) {
            k_build_table_q4<<<65536 / 256, 256, 0, stream>>>(t, packed, bad);
            failed = check_launch("k_build_table_q4") ||
                     check_cuda(cudaMemcpyAsync(&bad_host, bad, sizeof(int), cudaMemcpyDeviceToHost, stream), "table build") ||
                     check_cuda(cudaStreamSynchronize(stream), "table build");
        }
        if (!failed && bad_host != 0) {
            fail(COSET_E_STATE, "residual table: %d entries do not fit the packed layout", bad_host);
            failed = true;
        }
        if (failed) {
            cudaFree(t);
            return nullptr;
        }
        tables[dev] = t;
    }
    return tables[dev];
}

const uint32_t* residual_table_q4_packed(cudaStream_t stream) {
    const uint2* t = residual_table_q4(stream);
    return t ? reinterpret_cast<const uint32_t*>(t + 65536) : nullptr;
}

}  // namespace coset

#define DISPATCH_MODE(MODE_VAR, ...)                                   \
    switch (MODE_VAR) {                                                \
        case 0: { constexpr int MODE = 0; __VA_ARGS__; } break;         \
        case 1: { constexpr int MODE = 1; __VA_ARGS__; } break;         \
        default: { constexpr int MODE = 2; __VA_ARGS__; } break;        \
    }
#define DISPATCH_DT(DT_VAR, NAME, ...)                                 \
    if ((DT_VAR) == COSET_DTYPE_F32) { constexpr int NAME = 0; __VA_ARGS__; } else { constexpr int NAME = 1; __VA_ARGS__; }

extern "C" {

int coset_version(void) { return 100; }
const char* coset_last_error_string(void) { return coset::g_err; }

int coset_e8_code_bytes(int q, int M) {
    if (q < 2 || q > 16 || M < 1 || M > 8) return 0;
    return M * (q <= 4 ? 2 : 4);
}

int coset_e8_projection(const float* x, int64_t n_blocks, float* y, void* stream) {
    if (int e = check_common(x, y, n_blocks, 4, 2)) return e;
    if (n_blocks == 0) return 0;
    if (!aligned(x, 16) || !aligned(y, 16)) return fail(COSET_E_ALIGN, "x and y must be 16-byte aligned");
    k_projection<<<grid_for(n_blocks), kThreads, 0, (cudaStream_t)stream>>>(x, n_blocks, y);
    return check_launch("k_projection");
}

int coset_e8_encode(const void* x, int x_dtype, const float* scale, int scale_mode, int64_t n_blocks,
                    int64_t blocks_per_tile, int q, int M, int sem, void* codes, void* stream) {
    if (int e = check_common(x, codes, n_blocks, q, M)) return e;
    if (int e = check_scale(scale, scale_mode, blocks_per_tile)) return e;
    if (x_dtype != COSET_DTYPE_F32 && x_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown x_dtype %d", x_dtype);
    if (sem != COSET_SEM_CORE && sem != COSET_SEM_CORE_LITERAL) return fail(COSET_E_UNSUPPORTED, "semantics %d not available in this entry point", sem);
    if (n_blocks == 0) return 0;
    if (!aligned(x, 16) || !aligned(codes, 4)) return fail(COSET_E_ALIGN, "x must be 16-byte and codes 4-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    e8::TileDiv td = e8::make_tile_div(scale_mode == COSET_SCALE_MUL_TILE ? blocks_per_tile : 1, n_blocks);
    unsigned grid = grid_for(n_blocks);
    if (q == 4 && M == 2 && sem == COSET_SEM_CORE) {
        // persistent warps: at most kEncCtasPerSm CTAs per SM of grid (4 resident at a time)
        unsigned qgrid = encoder_grid(n_blocks);
        DISPATCH_DT(x_dtype, DT, DISPATCH_MODE(scale_mode, (k_encode_q4m2_queued<DT, MODE, false, 0><<<qgrid, kThreads, 0, st>>>(x, scale, td, n_blocks, (uint32_t*)codes, nullptr, nullptr, 0.0f))))
    } else if (q == 4 && M == 2) {
        DISPATCH_DT(x_dtype, DT, DISPATCH_MODE(scale_mode, (k_encode_q4m2<DT, MODE, true><<<grid, kThreads, 0, st>>>(x, scale, td, n_blocks, (uint32_t*)codes))))
    } else if (q <= 4) {
        DISPATCH_DT(x_dtype, DT, DISPATCH_MODE(scale_mode, (k_encode_generic<DT, MODE, 2><<<grid, kThreads, 0, st>>>(x, scale, td, n_blocks, q, M, codes))))
    } else {
        DISPATCH_DT(x_dtype, DT, DISPATCH_MODE(scale_mode, (k_encode_generic<DT, MODE, 4><<<grid, kThreads, 0, st>>>(x, scale, td, n_blocks, q, M, codes))))
    }
    return check_launch("e8_encode");
}

int coset_e8_decode(const void* codes, const float* scale, int scale_mode, int64_t n_blocks, int64_t blocks_per_tile,
                    int q, int M, int sem, void* out, int out_dtype, void* stream) {
    if (int e = check_common(codes, out, n_blocks, q, M)) return e;
    if (int e = check_scale(scale, scale_mode, blocks_per_tile)) return e;
    if (out_dtype != COSET_DTYPE_F32 && out_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown out_dtype %d", out_dtype);
    if (sem != COSET_SEM_CORE) return fail(COSET_E_UNSUPPORTED, "semantics %d not available in this entry point", sem);
    if (n_blocks == 0) return 0;
    if (!aligned(out, 16) || !aligned(codes, 4)) return fail(COSET_E_ALIGN, "out must be 16-byte and codes 4-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    e8::TileDiv td = e8::make_tile_div(scale_mode == COSET_SCALE_MUL_TILE ? blocks_per_tile : 1, n_blocks);
    unsigned grid = grid_for(n_blocks);
    if (q == 4 && M == 2) {
        const uint2* table = residual_table_q4(st);
        const uint32_t* packed = residual_table_q4_packed(st);
        if (!table || !packed) return COSET_E_STATE;
        unsigned grid2 = (unsigned)((n_blocks + kThreads * kDecPerThread - 1) / (kThreads * kDecPerThread));
        if (out_dtype == COSET_DTYPE_F32) {
            DISPATCH_MODE(scale_mode, (k_decode_q4m2<0, MODE, uint32_t><<<grid2, kThreads, 0, st>>>((const uint32_t*)codes, scale, td, n_blocks, packed, out)))
        } else {
            DISPATCH_MODE(scale_mode, (k_decode_q4m2<1, MODE, uint2><<<grid2, kThreads, 0, st>>>((const uint32_t*)codes, scale, td, n_blocks, table, out)))
        }
    } else if (q <= 4) {
        DISPATCH_DT(out_dtype, DT, DISPATCH_MODE(scale_mode, (k_decode_generic<DT, MODE, 2><<<grid, kThreads, 0, st>>>(codes, scale, td, n_blocks, q, M, out))))
    } else {
        DISPATCH_DT(out_dtype, DT, DISPATCH_MODE(scale_mode, (k_decode_generic<DT, MODE, 4><<<grid, kThreads, 0, st>>>(codes, scale, td, n_blocks, q, M, out))))
    }
    return check_launch("e8_decode");
}

int coset_e8_quantize(const void* x, int x_dtype, const float* scale, int scale_mode, int64_t n_blocks,
                      int64_t blocks_per_tile, int q, int M, float clip, void* out, int out_dtype, void* codes_out,
                      void* stream) {
    if (int e = check_common(x, out, n_blocks, q, M)) return e;
    if (int e = check_scale(scale, scale_mode, blocks_per_tile)) return e;
    if ((x_dtype != 0 && x_dtype != 1) || (out_dtype != 0 && out_dtype != 1)) return fail(COSET_E_BADARG, "unknown dtype");
    if (n_blocks == 0) return 0;
    if (!aligned(x, 16) || !aligned(out, 16) || !aligned(codes_out, 4)) return fail(COSET_E_ALIGN, "x/out must be 16-byte and codes 4-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    e8::TileDiv td = e8::make_tile_div(scale_mode == COSET_SCALE_MUL_TILE ? blocks_per_tile : 1, n_blocks);
    unsigned grid = grid_for(n_blocks);
    if (q == 4 && M == 2) {
        const uint2* table = residual_table_q4(st);
        if (!table) return COSET_E_STATE;
        unsigned qgrid = encoder_grid(n_blocks);
        DISPATCH_DT(x_dtype, DTI, DISPATCH_DT(out_dtype, DTO, DISPATCH_MODE(scale_mode, (k_encode_q4m2_queued<DTI, MODE, true, DTO><<<qgrid, kThreads, 0, st>>>(x, scale, td, n_blocks, (uint32_t*)codes_out, table, out, clip)))))
    } else if (q <= 4) {
        DISPATCH_DT(x_dtype, DTI, DISPATCH_DT(out_dtype, DTO, DISPATCH_MODE(scale_mode, (k_quantize_generic<DTI, DTO, MODE, 2><<<grid, kThreads, 0, st>>>(x, scale, td, n_blocks, q, M, clip, out, codes_out)))))
    } else {
        DISPATCH_DT(x_dtype, DTI, DISPATCH_DT(out_dtype, DTO, DISPATCH_MODE(scale_mode, (k_quantize_generic<DTI, DTO, MODE, 4><<<grid, kThreads, 0, st>>>(x, scale, td, n_blocks, q, M, clip, out, codes_out)))))
    }
    return check_launch("e8_quantize");
}

int coset_e8_unpack_codes_f32(const void* codes, int64_t n_blocks, int q, int M, float* digits, void* stream) {
    if (int e = check_common(codes, digits, n_blocks, q, M)) return e;
    if (n_blocks == 0) return 0;
    if (!aligned(digits, 16)) return fail(COSET_E_ALIGN, "digits must be 16-byte aligned");
    int64_t nw = n_blocks * M;
    if (q <= 4) k_unpack_f32<2><<<grid_for(nw), kThreads, 0, (cudaStream_t)stream>>>(codes, nw, digits);
    else k_unpack_f32<4><<<grid_for(nw), kThreads, 0, (cudaStream_t)stream>>>(codes, nw, digits);
    return check_launch("e8_unpack_codes_f32");
}

int coset_e8_pack_codes_f32(const float* digits, int64_t n_blocks, int q, int M, void* codes, void* stream) {
    if (int e = check_common(digits, codes, n_blocks, q, M)) return e;
    if (n_blocks == 0) return 0;
    if (!aligned(digits, 16)) return fail(COSET_E_ALIGN, "digits must be 16-byte aligned");
    int64_t nw = n_blocks * M;
    if (q <= 4) k_pack_f32<2><<<grid_for(nw), kThreads, 0, (cudaStream_t)stream>>>(digits, nw, q, codes);
    else k_pack_f32<4><<<grid_for(nw), kThreads, 0, (cudaStream_t)stream>>>(digits, nw, q, codes);
    return check_launch("e8_pack_codes_f32");
}

}  // extern "C"
