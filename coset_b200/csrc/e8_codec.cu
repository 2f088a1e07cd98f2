// E8 HNLQ codec kernels and their C-ABI entry points: projection, encode, decode, fused
// round trip (quantise), packed <-> float32 digit views, and the q=4 residual table.
//
// One thread owns one 8-vector ("block"): 32 B in (two 128-bit loads, a warp reads 1 KiB
// contiguously), all state in registers, 4 B packed code out.  The kernels are HBM-bound by
// design; algorithmic bytes per block (q=4, M=2, float32): encode 32+4 (+4 per-block scale),
// decode 4+32 (+4), round trip 32+32 (+4).
#include <stdarg.h>

#include <mutex>
#include <vector>

#include "common.cuh"
#include "e8_fast.cuh"
#include "e8_fast2.cuh"
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
// one row per lane and sub-step.  Every lane runs the cheapest tier (level_fast2_q4: one rounding
// pass, both cosets from it, digits on the FP32 pipe) behind one pre-test, max|x| <= 1.96 and
// sum|x| <= 7.96, which makes the top level the origin and bounds every quantity of that tier.
// Whatever the tier cannot prove -- a block near a rounding tie, a block whose top level is not the
// origin, a non-finite block -- is NOT handled in place (that would idle the other 31 lanes for
// hundreds of instructions): the lane appends the block's index to a per-warp queue in shared memory
// (a shared-memory atomic hands out the slot, so no warp-wide vote sits on the common path).  Once
// per iteration the warp looks at the queue length; with 32 or more entries (and at the end) it
// drains 32 of them with all lanes busy: every lane reads the row of its entry again -- one memory
// round trip per 32 deferred blocks -- and encodes it from scratch with the always-valid tiers.
// This also serves an overloaded quantiser, where most blocks need the top level: the queue then
// fills every iteration and is drained by full warps.
// SAT: every scaled coordinate is first clamped to +-kSaturate, which keeps the two-level code from
// wrapping around (the top level stays the origin); only deferred blocks can exceed the bound, so the
// clamp costs nothing on the common path.
constexpr int kRowsPerIter = 3;   // rows per lane and loop iteration
constexpr int kQueueSlots = 32 * (kRowsPerIter + 1);  // < 32 left after a drain + at most 32 per sub-step
constexpr int kEncWarps = kThreads / 32;
constexpr float kSaturate = 3.9f;  // 8 * 3.9 / 4 < 7.96 and 3.9 / 4 < 1.96: level 1 of a clamped block is the origin

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
template <int DT, int MODE, bool RECON, int DTO, bool SAT>
__global__ void __launch_bounds__(kThreads, 4)
k_encode_q4m2_queued(const void* __restrict__ x, const float* __restrict__ scale, e8::TileDiv td, int64_t n,
                     uint32_t* __restrict__ codes, const uint2* __restrict__ table, void* __restrict__ out, float clip) {
    __shared__ uint32_t q_index[kEncWarps][2][kQueueSlots];  // block index lo / hi
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

    // Completes the last min(count, 32) queued blocks with all lanes busy.
    auto drain = [&]() {
        const int take = count < 32 ? count : 32;
        if (lane < take) {
            const int e = count - take + lane;
            const int64_t b = (int64_t)(((uint64_t)q_index[warp][1][e] << 32) | q_index[warp][0][e]);
            float v[8];
            e8::Row8<DT>::load(x, b, v);
            const float s = load_scale<MODE>(scale, td, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = scale_in<MODE>(v[i], s);
                if (SAT) v[i] = fminf(fmaxf(v[i], -kSaturate), kSaturate);  // NaN -> -kSaturate: finite, harmless
            }
            emit(b, e8::finish_block_q4(v, 0u, 0), s);
        }
        count -= take;
        __syncwarp();
        if (lane == 0) q_count[warp] = count;
        __syncwarp();
    };

    const int64_t span = 32 * kRowsPerIter;
    const int64_t stride = (int64_t)gridDim.x * kEncWarps * span;
    for (int64_t base = ((int64_t)blockIdx.x * kEncWarps + warp) * span; base < n; base += stride) {
        bool defer[kRowsPerIter];
        bool any_defer = false;
        {
            // All rows are requested first; the tier then runs row after row in straight-line code, so
            // the loads of the later rows overlap the arithmetic of the earlier ones.  The rows are not
            // kept beyond this scope.
            float v[kRowsPerIter][8];
            float sc[kRowsPerIter];
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
                const int64_t b = base + j * 32 + lane;
                float s1 = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[j][i] = scale_in<MODE>(v[j][i], sc[j]);
                    s1 += fabsf(v[j][i]);
                }
                // max |x_i| as a tree of three-input maxima; a NaN is dropped by fmaxf but poisons s1
                const float m0 = fmaxf(fmaxf(fabsf(v[j][0]), fabsf(v[j][1])), fabsf(v[j][2]));
                const float m1 = fmaxf(fmaxf(fabsf(v[j][3]), fabsf(v[j][4])), fabsf(v[j][5]));
                const float amax = fmaxf(fmaxf(m0, m1), fmaxf(fabsf(v[j][6]), fabsf(v[j][7])));
                const bool pre = amax <= 1.96f && s1 <= 7.96f;       // top level is the origin, tier applicable
                const bool origin = amax <= 0.49f && s1 <= 1.99f;    // this level is the origin too: code 0
                uint32_t code;
                const bool proven = e8::level_fast2_q4(v[j], code);
                const bool done = origin || (pre && proven);
                defer[j] = b < n && !done;
                if (b < n && done) emit(b, origin ? 0u : code, sc[j]);
                any_defer = any_defer || defer[j];
            }
        }
        if (any_defer) {  // rare: one branch per iteration keeps the queue code off the common path
#pragma unroll
            for (int j = 0; j < kRowsPerIter; ++j) {
                if (defer[j]) {
                    const int64_t b = base + j * 32 + lane;
                    const int pos = atomicAdd(&q_count[warp], 1);
                    q_index[warp][0][pos] = (uint32_t)b;
                    q_index[warp][1][pos] = (uint32_t)((uint64_t)b >> 32);
                }
            }
        }
        __syncwarp();
        count = *reinterpret_cast<volatile int*>(&q_count[warp]);
        while (count >= 32) drain();
    }
    while (count > 0) drain();
}

// ---------------------------------------------------------------- encode-only production path
// The codes-only encoder is two launches.  Measured on this part, ANY state carried across the loop of
// the persistent kernel above (a queue length, a vote per iteration, a second loop) costs 10-25 % of
// its time through register pressure at the 64-register budget, so the main kernel carries none: a
// lane whose block the cheapest tier cannot prove stores a marker code (top level word non-zero, which
// that tier never produces) and appends the block index to a list in scratch memory with one atomic
// in a rare branch.  The fix-up kernel then finishes the listed blocks densely with the always-valid
// tiers.  When more blocks are deferred than the list holds (an overloaded quantiser) the fix-up kernel
// instead sweeps all codes for the marker and compacts the marked blocks warp by warp.
constexpr uint32_t kDeferredMark = 0x80000000u;
// The list is split into kDeferLists sub-lists (CTA i of the main kernel appends to sub-list i mod
// kDeferLists), each with its own counter in its own 32-byte sector: appends do not contend for one
// address (a single counter serialises: 2.7e5 appends took 0.4 ms).
constexpr int kDeferLists = 256;
constexpr int kCounterStride = 8;  // uint32 words between counters

struct EncodeScratch {
    uint32_t* ctrl;   // [kDeferLists * kCounterStride] counters, then [0] overflow flag, [1] fix-up CTAs finished
    int64_t* list;    // kDeferLists sub-lists of `cap` entries
    uint32_t cap;     // entries per sub-list
};
__device__ __forceinline__ uint32_t* scratch_tail(const EncodeScratch& s) { return s.ctrl + kDeferLists * kCounterStride; }

// rows per lane and iteration of the main kernel (with its rare deferral branch, 4 rows at 85 registers and
// 3 CTAs per SM measured 5 % slower than 3 rows at 64 registers and 4 CTAs per SM)
constexpr int kMainRows = 3;
inline unsigned main_grid(int64_t n_blocks) {
    const int64_t per_cta = (int64_t)kThreads * kMainRows;
    const int64_t need = (n_blocks + per_cta - 1) / per_cta;
    const int64_t cap = (int64_t)sm_count() * kEncCtasPerSm;
    return (unsigned)(need < cap ? (need < 1 ? 1 : need) : cap);
}

template <int DT, int MODE>
__global__ void __launch_bounds__(kThreads, 4)
k_encode_q4m2_main(const void* __restrict__ x, const float* __restrict__ scale, e8::TileDiv td, int64_t n,
                   uint32_t* __restrict__ codes, EncodeScratch sc_) {
    __shared__ uint4 flip_rows[8];
    if (threadIdx.x < 8) flip_rows[threadIdx.x] = e8::kFlipRows[threadIdx.x];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t span = 32 * kMainRows;
    const int64_t stride = (int64_t)gridDim.x * kEncWarps * span;
    for (int64_t base = ((int64_t)blockIdx.x * kEncWarps + warp) * span; base < n; base += stride) {
        float v[kMainRows][8];
        float sc[kMainRows];
#pragma unroll
        for (int j = 0; j < kMainRows; ++j) {
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
        for (int j = 0; j < kMainRows; ++j) {
            const int64_t b = base + j * 32 + lane;
            float s1 = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[j][i] = scale_in<MODE>(v[j][i], sc[j]);
                s1 += fabsf(v[j][i]);
            }
            // max |x_i| as a tree of three-input maxima; a NaN is dropped by fmaxf but poisons s1
            const float m0 = fmaxf(fmaxf(fabsf(v[j][0]), fabsf(v[j][1])), fabsf(v[j][2]));
            const float m1 = fmaxf(fmaxf(fabsf(v[j][3]), fabsf(v[j][4])), fabsf(v[j][5]));
            const float amax = fmaxf(fmaxf(m0, m1), fmaxf(fabsf(v[j][6]), fabsf(v[j][7])));
            const bool pre = amax <= 1.96f && s1 <= 7.96f;     // top level is the origin, tier applicable
            const bool origin = amax <= 0.49f && s1 <= 1.99f;  // this level is the origin too: code 0
            uint32_t code;
            const bool proven = e8::level_fast2_q4(v[j], code, flip_rows);
            const bool done = origin || (pre && proven);
            if (b < n) {
                if (done) {
                    __stcs(codes + b, origin ? 0u : code);
                } else {  // rare: mark the block and append it to this CTA's sub-list
                    codes[b] = kDeferredMark;
                    const uint32_t l = blockIdx.x % kDeferLists;
                    const uint32_t pos = atomicAdd(sc_.ctrl + l * kCounterStride, 1u);
                    if (pos < sc_.cap) sc_.list[(int64_t)l * sc_.cap + pos] = b;
                    else *scratch_tail(sc_) = 1u;  // full: the fix-up kernel will sweep for the markers instead
                }
            }
        }
    }
}

// One level of a deferred block: the cheapest tier when it applies, then the exact-rounding tier, then the
// literal search.  amax, s1: max and sum of |x_i|.
__device__ __forceinline__ uint32_t level_any_q4(const float (&x)[8], float amax, float s1) {
    uint32_t digits;
    if (amax <= 1.96f && s1 <= 7.96f && e8::level_fast2_q4(x, digits)) return digits;
    return e8::level_slow_q4(x, s1 == s1 && s1 - s1 == 0.0f ? amax : __int_as_float(0x7fc00000));
}

template <int DT, int MODE, bool SAT>
__global__ void __launch_bounds__(kThreads)
k_encode_q4m2_fix(const void* __restrict__ x, const float* __restrict__ scale, e8::TileDiv td, int64_t n,
                  uint32_t* __restrict__ codes, EncodeScratch sc_) {
    __shared__ uint32_t q_index[kEncWarps][2][64];
    __shared__ uint32_t prefix[kDeferLists + 1];
    const bool overflow = *reinterpret_cast<volatile uint32_t*>(scratch_tail(sc_)) != 0u;
    auto finish = [&](int64_t b) {
        float v[8];
        e8::Row8<DT>::load(x, b, v);
        const float s = load_scale<MODE>(scale, td, b);
        float amax = 0.0f, s1 = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = scale_in<MODE>(v[i], s);
            if (SAT) v[i] = fminf(fmaxf(v[i], -kSaturate), kSaturate);  // a NaN becomes -kSaturate: finite, harmless
            amax = fmaxf(amax, fabsf(v[i]));
            s1 += fabsf(v[i]);
        }
        uint32_t code = 0u;
#pragma unroll 1
        for (int m = 0; m < 2; ++m) {
            const bool origin = amax <= 0.49f && s1 <= 1.99f;
            if (!origin) code |= level_any_q4(v, amax, s1) << (16 * m);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], 0.25f);
            amax *= 0.25f;
            s1 *= 0.25f;
        }
        __stcs(codes + b, code);
    };
    if (!overflow) {
        // every deferred block is in a sub-list.  Flatten them: exclusive prefix of the kDeferLists
        // counters (one per thread), then one thread per entry across the whole grid, all lanes busy.
        uint32_t cnt = *reinterpret_cast<volatile uint32_t*>(sc_.ctrl + threadIdx.x * kCounterStride);
        prefix[threadIdx.x + 1] = cnt < sc_.cap ? cnt : sc_.cap;
        if (threadIdx.x == 0) prefix[0] = 0u;
        __syncthreads();
        for (int o = 1; o < kDeferLists; o <<= 1) {  // Hillis-Steele inclusive scan over prefix[1..]
            const uint32_t add = threadIdx.x + 1 > (unsigned)o ? prefix[threadIdx.x + 1 - o] : 0u;
            __syncthreads();
            prefix[threadIdx.x + 1] += add;
            __syncthreads();
        }
        const uint32_t total = prefix[kDeferLists];
        for (uint32_t f = blockIdx.x * kThreads + threadIdx.x; f < total; f += gridDim.x * kThreads) {
            int lo = 0, hi = kDeferLists;  // largest l with prefix[l] <= f
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (prefix[mid] <= f) lo = mid; else hi = mid;
            }
            finish(sc_.list[(int64_t)lo * sc_.cap + (f - prefix[lo])]);
        }
    } else {
        // a sub-list overflowed: sweep all codes for the marker, 32 marked blocks at a time per warp
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        int count = 0;
        auto drain = [&](int take) {
            if (lane < take) {
                const int e = count - take + lane;
                finish((int64_t)(((uint64_t)q_index[warp][1][e] << 32) | q_index[warp][0][e]));
            }
            count -= take;
            __syncwarp();
        };
        const int64_t stride = (int64_t)gridDim.x * kEncWarps * 32;
        for (int64_t base = ((int64_t)blockIdx.x * kEncWarps + warp) * 32; base < n; base += stride) {
            const int64_t b = base + lane;
            const bool marked = b < n && codes[b] == kDeferredMark;
            const uint32_t bal = __ballot_sync(0xffffffffu, marked);
            if (bal) {
                if (marked) {
                    const int pos = count + __popc(bal & ((1u << lane) - 1u));
                    q_index[warp][0][pos] = (uint32_t)b;
                    q_index[warp][1][pos] = (uint32_t)((uint64_t)b >> 32);
                }
                count += __popc(bal);
                __syncwarp();
                if (count >= 32) drain(32);
            }
        }
        if (count > 0) drain(count);
    }
    // the last CTA to finish clears the counters and the flag for the next call on this scratch
    __syncthreads();
    __shared__ bool last;
    if (threadIdx.x == 0) {
        __threadfence();
        last = atomicAdd(scratch_tail(sc_) + 1, 1u) == gridDim.x - 1u;
    }
    __syncthreads();
    if (last) {
        sc_.ctrl[threadIdx.x * kCounterStride] = 0u;
        if (threadIdx.x == 0) { scratch_tail(sc_)[0] = 0u; scratch_tail(sc_)[1] = 0u; }
        __threadfence();
    }
}
static_assert(kDeferLists == kThreads, "the fix-up kernel scans one counter per thread");

// Four blocks per thread (kThreads apart, so every access stays coalesced): all codes are
// loaded before the first table lookup, which multiplies the gathers in flight per thread
// (measured per 2^25 blocks: 2 per thread 0.236 ms, 4 per thread 0.231 ms, 8 per thread 0.231 ms).
constexpr int kDecPerThread = 4;
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

namespace {

// Scratch of the two-launch encoder, one per (device, stream): calls on one stream are ordered, so they
// may share it; the mutex keeps the two launches of one call together when several host threads use the
// same stream.  Allocated on first use and when a larger tensor arrives (never inside a stream capture:
// make the first call of a given size before capturing).
struct ScratchSlot {
    int device;
    cudaStream_t stream;
    EncodeScratch s;
};
std::mutex g_scratch_mu;
std::vector<ScratchSlot> g_scratch;

constexpr size_t kCtrlBytes = (size_t)(kDeferLists * kCounterStride + 8) * sizeof(uint32_t);

int alloc_scratch(EncodeScratch* s, uint32_t cap, cudaStream_t st) {
    *s = EncodeScratch{nullptr, nullptr, 0};
    if (int e = check_cuda(cudaMalloc(&s->ctrl, kCtrlBytes), "cudaMalloc(encode scratch)")) return e;
    if (int e = check_cuda(cudaMalloc(&s->list, (size_t)kDeferLists * cap * sizeof(int64_t)), "cudaMalloc(encode scratch)")) return e;
    if (int e = check_cuda(cudaMemsetAsync(s->ctrl, 0, kCtrlBytes, st), "cudaMemsetAsync(encode scratch)")) return e;
    s->cap = cap;
    return 0;
}

int encode_scratch(cudaStream_t st, int64_t n_blocks, EncodeScratch* out) {
    int dev = 0;
    if (int e = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return e;
    // room for one block in 32 deferred (the benchmark data defers one in 125), at least 64 per sub-list
    const uint32_t want = (uint32_t)(n_blocks / 32 / kDeferLists) + 64u;
    if ((uint64_t)want * kDeferLists >= 0xffffffffull) return fail(COSET_E_BADARG, "n_blocks too large");
    for (auto& slot : g_scratch) {
        if (slot.device == dev && slot.stream == st) {
            if (slot.s.cap >= want) { *out = slot.s; return 0; }
            // grow: earlier launches on this stream may still use the old buffers
            if (int e = check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize(encode scratch)")) return e;
            cudaFree(slot.s.ctrl);
            cudaFree(slot.s.list);
            if (int e = alloc_scratch(&slot.s, want, st)) return e;
            *out = slot.s;
            return 0;
        }
    }
    ScratchSlot slot{dev, st, EncodeScratch{nullptr, nullptr, 0}};
    if (int e = alloc_scratch(&slot.s, want, st)) return e;
    g_scratch.push_back(slot);
    *out = slot.s;
    return 0;
}

template <int DT, int MODE>
int launch_encode_q4m2(const void* x, const float* scale, e8::TileDiv td, int64_t n, uint32_t* codes, bool saturate,
                       cudaStream_t st) {
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    EncodeScratch sc;
    if (int e = encode_scratch(st, n, &sc)) return e;
    const unsigned mgrid = main_grid(n);
    k_encode_q4m2_main<DT, MODE><<<mgrid, kThreads, 0, st>>>(x, scale, td, n, codes, sc);
    if (int e = check_launch("e8_encode (main)")) return e;
    // the deferred blocks are few: a grid of four CTAs per SM shares them evenly (in sweep mode it strides
    // over the whole tensor)
    const int64_t need = (n + kThreads - 1) / kThreads;
    const unsigned fgrid = (unsigned)(need < 4 * sm_count() ? (need < 1 ? 1 : need) : 4 * sm_count());
    (void)mgrid;
    if (saturate)
        k_encode_q4m2_fix<DT, MODE, true><<<fgrid, kThreads, 0, st>>>(x, scale, td, n, codes, sc);
    else
        k_encode_q4m2_fix<DT, MODE, false><<<fgrid, kThreads, 0, st>>>(x, scale, td, n, codes, sc);
    return check_launch("e8_encode (fix-up)");
}

}  // namespace

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
    if (sem != COSET_SEM_CORE && sem != COSET_SEM_CORE_LITERAL && sem != COSET_SEM_CORE_SATURATE)
        return fail(COSET_E_UNSUPPORTED, "semantics %d not available in this entry point", sem);
    if (sem == COSET_SEM_CORE_SATURATE && !(q == 4 && M == 2)) return fail(COSET_E_UNSUPPORTED, "saturating encode needs q=4, M=2");
    if (n_blocks == 0) return 0;
    if (!aligned(x, 16) || !aligned(codes, 4)) return fail(COSET_E_ALIGN, "x must be 16-byte and codes 4-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    e8::TileDiv td = e8::make_tile_div(scale_mode == COSET_SCALE_MUL_TILE ? blocks_per_tile : 1, n_blocks);
    unsigned grid = grid_for(n_blocks);
    if (q == 4 && M == 2 && sem == COSET_SEM_CORE) {
        // persistent warps: at most kEncCtasPerSm CTAs per SM of grid (4 resident at a time)
        int rc = 0;
        DISPATCH_DT(x_dtype, DT, DISPATCH_MODE(scale_mode, (rc = launch_encode_q4m2<DT, MODE>(x, scale, td, n_blocks, (uint32_t*)codes, false, st))))
        return rc;
    } else if (q == 4 && M == 2 && sem == COSET_SEM_CORE_SATURATE) {
        int rc = 0;
        DISPATCH_DT(x_dtype, DT, DISPATCH_MODE(scale_mode, (rc = launch_encode_q4m2<DT, MODE>(x, scale, td, n_blocks, (uint32_t*)codes, true, st))))
        return rc;
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
        DISPATCH_DT(x_dtype, DTI, DISPATCH_DT(out_dtype, DTO, DISPATCH_MODE(scale_mode, (k_encode_q4m2_queued<DTI, MODE, true, DTO, false><<<qgrid, kThreads, 0, st>>>(x, scale, td, n_blocks, (uint32_t*)codes_out, table, out, clip)))))
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
