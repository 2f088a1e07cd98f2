// Quantisation statistics of the q=4, M=2 E8 codec over a tensor, in one pass:
//   out[0] = sum over blocks of || x_hat - x_s ||^2   (x_s = scaled input, x_hat = decode(encode(x_s)))
//   out[1] = number of overloaded blocks: projection(x_s / q^M) != 0, the overload test of the
//            paper-faithful quantiser (ref/hnlq.py:341) evaluated with the core search
//   out[2] = number of blocks whose code is not all-zero
//   out[3] = sum over blocks of || x_s ||^2            (out[3] / out[0] is the signal-to-noise ratio)
//
// Two stages, deterministic (no atomics): every CTA reduces its blocks to one partial record in
// SCRATCH memory, then a single CTA folds the partial records in a fixed order.
#include <mutex>

#include "common.cuh"
#include "e8_fast.cuh"
#include "e8_io.cuh"
#include "e8_literal.cuh"

using namespace coset;

namespace {

constexpr int kThreads = 256;
constexpr int kBlocksPerCta = 8192;  // blocks reduced by one CTA (32 per thread)

struct Partial {
    double err2, sig2;
    unsigned long long overload, nonzero;
};

// twice the reconstruction from the code without the residual table (literal decoder per level)
__device__ __forceinline__ void decode_twice_literal(uint32_t code, float (&v2)[8]) {
    int d0[8], d1[8];
    float r0[8], r1[8];
    e8::unpack_level<2>(code & 0xffffu, d0);
    e8::unpack_level<2>(code >> 16, d1);
    e8::level_residual(d0, 4.0f, r0);
    e8::level_residual(d1, 4.0f, r1);
#pragma unroll
    for (int i = 0; i < 8; ++i) v2[i] = __fmul_rn(__fadd_rn(r0[i], __fmul_rn(4.0f, r1[i])), 2.0f);
}

template <int DT, int MODE, bool USE_TABLE = true>
__global__ void __launch_bounds__(kThreads)
k_stats_partial(const void* __restrict__ x, const float* __restrict__ scale, e8::TileDiv td, int64_t n,
                const uint2* __restrict__ table, Partial* __restrict__ partials) {
    __shared__ Partial red[kThreads / 32];
    double err2 = 0.0, sig2 = 0.0;
    unsigned long long overload = 0, nonzero = 0;
    const int64_t lo = (int64_t)blockIdx.x * kBlocksPerCta;
    const int64_t hi = lo + kBlocksPerCta < n ? lo + kBlocksPerCta : n;
    for (int64_t b = lo + threadIdx.x; b < hi; b += kThreads) {
        float v[8], xs[8], v2[8];
        e8::Row8<DT>::load(x, b, v);
        float s = 1.0f;
        if (MODE == COSET_SCALE_DIV_SCALAR) s = __ldg(scale);
        if (MODE == COSET_SCALE_MUL_TILE) s = __ldg(scale + e8::tile_of(td, b));
        float amax = 0.0f, s1 = 0.0f, e = 0.0f, g = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = MODE == COSET_SCALE_DIV_SCALAR ? __fdiv_rn(v[i], s) : (MODE == COSET_SCALE_MUL_TILE ? __fmul_rn(v[i], s) : v[i]);
            xs[i] = v[i];
            amax = fmaxf(amax, fabsf(v[i]));
            s1 += fabsf(v[i]);
        }
        uint32_t code = e8::encode_q4m2<false>(v);  // leaves v = x_s / 16
        if (USE_TABLE) e8::decode_q4m2_twice(code, table, v2); else decode_twice_literal(code, v2);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float d = __fmaf_rn(v2[i], 0.5f, -xs[i]);
            e = __fmaf_rn(d, d, e);
            g = __fmaf_rn(xs[i], xs[i], g);
        }
        bool finite = (s1 - s1) == 0.0f;
        bool over = false;
        if (!(finite && amax * 0.0625f <= 0.49f && s1 * 0.0625f <= 1.99f)) {
            float y[8];
            e8::projection(v, y);
#pragma unroll
            for (int i = 0; i < 8; ++i) over = over || (y[i] != 0.0f);
        }
        err2 += (double)e;
        sig2 += (double)g;
        overload += over ? 1ull : 0ull;
        nonzero += code != 0u ? 1ull : 0ull;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        err2 += __shfl_xor_sync(0xffffffffu, err2, o);
        sig2 += __shfl_xor_sync(0xffffffffu, sig2, o);
        overload += __shfl_xor_sync(0xffffffffu, overload, o);
        nonzero += __shfl_xor_sync(0xffffffffu, nonzero, o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = Partial{err2, sig2, overload, nonzero};
    __syncthreads();
    if (threadIdx.x == 0) {
        Partial p = red[0];
        for (int w = 1; w < kThreads / 32; ++w) {
            p.err2 += red[w].err2; p.sig2 += red[w].sig2; p.overload += red[w].overload; p.nonzero += red[w].nonzero;
        }
        partials[blockIdx.x] = p;
    }
}

__global__ void __launch_bounds__(kThreads) k_stats_final(const Partial* __restrict__ partials, int count, double* __restrict__ out) {
    __shared__ Partial red[kThreads];
    Partial p{0.0, 0.0, 0ull, 0ull};
    for (int i = threadIdx.x; i < count; i += kThreads) {
        p.err2 += partials[i].err2; p.sig2 += partials[i].sig2; p.overload += partials[i].overload; p.nonzero += partials[i].nonzero;
    }
    red[threadIdx.x] = p;
    __syncthreads();
    for (int o = kThreads / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            red[threadIdx.x].err2 += red[threadIdx.x + o].err2; red[threadIdx.x].sig2 += red[threadIdx.x + o].sig2;
            red[threadIdx.x].overload += red[threadIdx.x + o].overload; red[threadIdx.x].nonzero += red[threadIdx.x + o].nonzero;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        out[0] = red[0].err2; out[1] = (double)red[0].overload; out[2] = (double)red[0].nonzero; out[3] = red[0].sig2;
    }
}

template <bool USE_TABLE>
int launch_stats(const void* x, int x_dtype, const float* scale, int scale_mode, int64_t n_blocks, int64_t blocks_per_tile,
                 Partial* partials, double* out, cudaStream_t st) {
    const uint2* table = nullptr;
    if (USE_TABLE) {
        table = residual_table_q4(st);
        if (!table) return COSET_E_STATE;
    }
    e8::TileDiv td = e8::make_tile_div(scale_mode == COSET_SCALE_MUL_TILE ? blocks_per_tile : 1, n_blocks);
    int ctas = (int)((n_blocks + kBlocksPerCta - 1) / kBlocksPerCta);
#define STATS_CASE(DT, MODE) k_stats_partial<DT, MODE, USE_TABLE><<<ctas, kThreads, 0, st>>>(x, scale, td, n_blocks, table, partials)
    if (x_dtype == COSET_DTYPE_F32) {
        if (scale_mode == 0) STATS_CASE(0, 0); else if (scale_mode == 1) STATS_CASE(0, 1); else STATS_CASE(0, 2);
    } else {
        if (scale_mode == 0) STATS_CASE(1, 0); else if (scale_mode == 1) STATS_CASE(1, 1); else STATS_CASE(1, 2);
    }
#undef STATS_CASE
    if (int e = check_launch("e8_quant_stats (partial)")) return e;
    k_stats_final<<<1, kThreads, 0, st>>>(partials, ctas, out);
    return check_launch("e8_quant_stats (final)");
}

int check_stats_args(const void* x, int x_dtype, const float* scale, int scale_mode, int64_t n_blocks, int64_t bpt, const double* out) {
    if (n_blocks < 1) return fail(COSET_E_BADARG, "n_blocks must be >= 1");
    if (!x || !out) return fail(COSET_E_BADARG, "null pointer");
    if (x_dtype != COSET_DTYPE_F32 && x_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown x_dtype");
    if (scale_mode < 0 || scale_mode > 2 || (scale_mode != 0 && !scale)) return fail(COSET_E_BADARG, "bad scale arguments");
    if (scale_mode == COSET_SCALE_MUL_TILE && bpt < 1) return fail(COSET_E_BADARG, "blocks_per_tile must be >= 1");
    if (!aligned(x, 16) || !aligned(out, 8)) return fail(COSET_E_ALIGN, "x must be 16-byte and out 8-byte aligned");
    return 0;
}

// ---- scratch for callers that cannot allocate -------------------------------------------------
// One partial record per CTA, for at most kStaticMaxCtas CTAs (2^25 blocks).  The array lives in
// every GPU that loads the library until the process exits (128 KB).
constexpr int kStaticMaxCtas = 4096;
static __device__ __align__(256) unsigned char g_stats_scratch[kStaticMaxCtas * sizeof(Partial)];

// Device address of g_stats_scratch on the CURRENT device.  In host code the symbol's name is only
// a stand-in, not a device pointer, so the address is asked from the runtime once per device.
Partial* static_scratch_of_current_device() {
    static std::mutex mu;
    static Partial* addr[64] = {nullptr};
    int dev = 0;
    if (check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return nullptr;
    if (dev < 0 || dev >= 64) { fail(COSET_E_STATE, "device index %d out of range", dev); return nullptr; }
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void* p = nullptr;
        if (check_cuda(cudaGetSymbolAddress(&p, g_stats_scratch), "cudaGetSymbolAddress(g_stats_scratch)")) return nullptr;
        addr[dev] = (Partial*)p;
    }
    return addr[dev];
}

}  // namespace

extern "C" {

int64_t coset_e8_quant_stats_static_max_blocks(void) { return (int64_t)kStaticMaxCtas * kBlocksPerCta; }

int coset_e8_quant_stats_static(const void* x, int x_dtype, const float* scale, int scale_mode, int64_t n_blocks,
                                int64_t blocks_per_tile, double* out, void* stream) {
    if (int e = check_stats_args(x, x_dtype, scale, scale_mode, n_blocks, blocks_per_tile, out)) return e;
    if (n_blocks > coset_e8_quant_stats_static_max_blocks())
        return fail(COSET_E_UNSUPPORTED, "n_blocks = %lld exceeds the %lld blocks the built-in scratch array covers; "
                    "split the tensor or use coset_e8_quant_stats with caller-provided scratch",
                    (long long)n_blocks, (long long)coset_e8_quant_stats_static_max_blocks());
    Partial* scratch = static_scratch_of_current_device();
    if (!scratch) return COSET_E_STATE;
    return launch_stats<false>(x, x_dtype, scale, scale_mode, n_blocks, blocks_per_tile, scratch, out, (cudaStream_t)stream);
}

int64_t coset_e8_quant_stats_scratch_bytes(int64_t n_blocks) {
    if (n_blocks < 1) return 0;
    return ((n_blocks + kBlocksPerCta - 1) / kBlocksPerCta) * (int64_t)sizeof(Partial);
}

int coset_e8_quant_stats(const void* x, int x_dtype, const float* scale, int scale_mode, int64_t n_blocks,
                         int64_t blocks_per_tile, void* scratch, int64_t scratch_bytes, double* out, void* stream) {
    if (int e = check_stats_args(x, x_dtype, scale, scale_mode, n_blocks, blocks_per_tile, out)) return e;
    if (!scratch || scratch_bytes < coset_e8_quant_stats_scratch_bytes(n_blocks) || !aligned(scratch, 16))
        return fail(COSET_E_BADARG, "scratch must be 16-byte aligned and hold coset_e8_quant_stats_scratch_bytes(n_blocks) bytes");
    return launch_stats<true>(x, x_dtype, scale, scale_mode, n_blocks, blocks_per_tile, (Partial*)scratch, out, (cudaStream_t)stream);
}

}  // extern "C"
