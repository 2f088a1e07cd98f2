// Large-token code-domain matmul on the 5th-generation tensor cores (tcgen05):
//     y[T, N] = x[T, K] (bf16) * Wq^T + bias,   Wq = decode(codes) / beta  (never stored in HBM)
//
// One CTA owns a 128 (tokens) x 128 (output features) tile of y.  Per 64-wide K step
//   * the activation tile  A (128 x 64 bf16) is copied to shared memory,
//   * the weight tile      B (128 x 64 bf16) is DECODED into shared memory: one thread turns one
//     packed E8 code (4 B) plus its scale into eight bf16 weights = one 16-byte chunk,
// both in the K-major SWIZZLE_128B layout the UMMA shared-memory descriptor describes
// (8-row groups of 1024 B, 16-byte chunk c of row r stored at chunk c ^ (r & 7)); then one thread
// issues four tcgen05.mma (M=128, N=128, K=16) that accumulate into tensor memory (128 lanes x
// 128 fp32 columns) and a tcgen05.commit that releases the stage through an mbarrier.  Three
// stages let the decode of step k+1.. overlap the MMAs of step k.  The epilogue reads the
// accumulator with tcgen05.ld and writes fp32.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records an error code, still frees
// its tensor memory and returns.  No cluster features, no multicast, no peer memory.
#include <cuda_bf16.h>

#include "common.cuh"
#include "e8_fast.cuh"
#include "e8_io.cuh"

using namespace coset;

namespace {

constexpr int BM = 128, BN = 128, BK = 64, STAGES = 3, THREADS = 256;
constexpr int TILE_BYTES = BM * BK * 2;  // 16 KiB, same for A and B
constexpr uint32_t TMEM_COLS = 128;
constexpr int SMEM_BYTES = 2 * STAGES * TILE_BYTES + 1024 /*alignment slack*/ + 64 /*barriers, tmem slot*/;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// Bounded wait: false if the phase did not complete within the budget.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < (1 << 20); ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// K-major, SWIZZLE_128B operand tile: start address, LBO = 1 (unused with swizzle), SBO = 1024 B
// between 8-row groups, descriptor version 1 (sm_100), layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, N = 128, M = 128.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ uint32_t swizzled_chunk_offset(int row, int chunk) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int MODE>
__global__ void __launch_bounds__(THREADS)
k_dequant_gemm(const uint32_t* __restrict__ codes, const float* __restrict__ beta, e8::TileDiv td, int N, int K,
               const __nv_bfloat16* __restrict__ x, int64_t ldx, int T, const float* __restrict__ bias,
               const uint2* __restrict__ table, float* __restrict__ y, int64_t ldy, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;           // tiles need 1024-byte alignment for the 128B swizzle
    uint8_t* gen = smem_raw + (base - raw);                 // generic pointer to the same place
    const uint32_t a_base = base, b_base = base + STAGES * TILE_BYTES;
    const uint32_t bar_base = base + 2 * STAGES * TILE_BYTES;  // empty[STAGES], done, then the tmem slot
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + 2 * STAGES * TILE_BYTES + 8 * (STAGES + 1));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile_n = blockIdx.x, tile_m = blockIdx.y;
    const int kb_row = K / 8;  // codes per weight row

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        for (int s = 0; s <= STAGES; ++s) mbar_init(bar_base + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;
    bool ok = true;

    const int KT = K / BK;
    for (int kt = 0; kt < KT; ++kt) {
        const int s = kt % STAGES;
        if (kt >= STAGES) ok = mbar_wait(bar_base + 8 * s, (uint32_t)((kt / STAGES - 1) & 1)) && ok;
        uint8_t* a_gen = gen + s * TILE_BYTES;
        uint8_t* b_gen = gen + (STAGES + s) * TILE_BYTES;
#pragma unroll
        for (int j = 0; j < (BM * 8) / THREADS; ++j) {  // activations: 128 rows x 8 chunks of 16 B
            int idx = tid + j * THREADS, row = idx >> 3, c = idx & 7;
            int tok = tile_m * BM + row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (tok < T) v = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)tok * ldx + (int64_t)kt * BK + c * 8));
            *reinterpret_cast<uint4*>(a_gen + swizzled_chunk_offset(row, c)) = v;
        }
#pragma unroll
        for (int j = 0; j < (BN * 8) / THREADS; ++j) {  // weights: one E8 code -> one 16-byte chunk
            int idx = tid + j * THREADS, row = idx >> 3, c = idx & 7;
            int n = tile_n * BN + row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (n < N) {
                int64_t blk = (int64_t)n * kb_row + (int64_t)kt * 8 + c;
                uint32_t code = __ldg(codes + blk);
                float sc = MODE == 2 ? __ldg(beta + e8::tile_of(td, blk)) : 1.0f;
                float v2[8], w[8];
                e8::decode_q4m2_twice(code, table, v2);
                e8::scale_twice<MODE>(v2, sc, w);
                v = make_uint4(pack_bf16x2(w[0], w[1]), pack_bf16x2(w[2], w[3]), pack_bf16x2(w[4], w[5]), pack_bf16x2(w[6], w[7]));
            }
            *reinterpret_cast<uint4*>(b_gen + swizzled_chunk_offset(row, c)) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = a_base + s * TILE_BYTES, b_addr = b_base + s * TILE_BYTES;
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)  // 16 bf16 = 32 bytes along K inside the 128-byte swizzle row
                umma_f16(tmem_d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), kIdesc, (kt > 0 || k > 0) ? 1u : 0u);
            umma_commit(bar_base + 8 * s);                    // stage s may be overwritten once these MMAs retire
            if (kt == KT - 1) umma_commit(bar_base + 8 * STAGES);  // ... and the accumulator is complete
        }
    }
    ok = mbar_wait(bar_base + 8 * STAGES, 0u) && ok;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // epilogue: warp w reads TMEM lanes 32*(w%4).., columns 64*(w/4)..; thread = one token row
    {
        const int q = warp & 3, h = warp >> 2;
        const int tok = tile_m * BM + q * 32 + lane;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            uint32_t r[32];
            const int col0 = h * 64 + cc * 32;
            tmem_ld32(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)col0, r);
            if (tok < T && ok) {
                float* dst = y + (int64_t)tok * ldy + (int64_t)tile_n * BN + col0;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    int n = tile_n * BN + col0 + j;
                    if (n < N) dst[j] = __uint_as_float(r[j]) + (bias ? __ldg(bias + n) : 0.0f);
                }
            }
        }
    }
    if (!ok && tid == 0 && status) atomicExch(status, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

extern "C" int coset_e8_dequant_gemm(const void* codes, const float* beta, int64_t blocks_per_tile, int n_out, int n_in,
                                     const void* x_bf16, int64_t ldx, int T, const float* bias, float* y, int64_t ldy,
                                     int* status, void* stream) {
    if (n_out < 0 || n_in < 0 || T < 0 || (n_in % BK) != 0) return fail(COSET_E_BADARG, "bad shape (n_in must be a multiple of 64)");
    if (n_out == 0 || T == 0) return 0;
    if (!codes || !x_bf16 || !y) return fail(COSET_E_BADARG, "null pointer");
    if (ldx < n_in || ldy < n_out || (ldx % 8) != 0) return fail(COSET_E_BADARG, "leading dimensions: ldx >= n_in and a multiple of 8, ldy >= n_out");
    if (!aligned(x_bf16, 16) || !aligned(codes, 4)) return fail(COSET_E_ALIGN, "x must be 16-byte and codes 4-byte aligned");
    if (beta && blocks_per_tile < 1) return fail(COSET_E_BADARG, "blocks_per_tile must be >= 1");
    cudaStream_t st = (cudaStream_t)stream;
    const uint2* table = residual_table_q4(st);
    if (!table) return COSET_E_STATE;
    e8::TileDiv td = e8::make_tile_div(beta ? blocks_per_tile : 1, (int64_t)n_out * (n_in / 8));
    dim3 grid((n_out + BN - 1) / BN, (T + BM - 1) / BM);
    if (grid.y > 65535) return fail(COSET_E_UNSUPPORTED, "T too large");
    if (beta) {
        if (int e = check_cuda(cudaFuncSetAttribute(k_dequant_gemm<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), "cudaFuncSetAttribute")) return e;
        k_dequant_gemm<2><<<grid, THREADS, SMEM_BYTES, st>>>((const uint32_t*)codes, beta, td, n_out, n_in, (const __nv_bfloat16*)x_bf16, ldx, T, bias, table, y, ldy, status);
    } else {
        if (int e = check_cuda(cudaFuncSetAttribute(k_dequant_gemm<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), "cudaFuncSetAttribute")) return e;
        k_dequant_gemm<0><<<grid, THREADS, SMEM_BYTES, st>>>((const uint32_t*)codes, beta, td, n_out, n_in, (const __nv_bfloat16*)x_bf16, ldx, T, bias, table, y, ldy, status);
    }
    return check_launch("e8_dequant_gemm");
}
