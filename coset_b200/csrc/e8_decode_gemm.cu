// Large-token code-domain matmul, two launches:
//     Wq = clamp(decode(codes) / beta)  ->  bf16 [n_out, n_in] in a caller-provided scratch buffer
//     y[T, n_out] = x[T, n_in] (bf16) * Wq^T + bias         on the tcgen05 tensor cores
// The scratch buffer is transient: it is rewritten on every call, read by the GEMM while it is still in L2
// (32 MiB for a 4096 x 4096 layer against 126 MiB of L2), and nothing of it has to survive the call, so the
// layer keeps 4 bits per weight in HBM.  Against the single-launch kernel of e8_dequant_gemm.cu this moves the
// decode out of the GEMM's K loop: no producer warps, both operands arrive by TMA, and the results are the same
// bits.  Measured on a 4096 x 4096 layer: 1.30 PFLOP/s at 8192 tokens and 1.47 at 16384 (decode included),
// against 0.91 / 1.04 for the single-launch kernel.
//
// The GEMM runs on pairs of CTAs (a cluster of two on the two SMs of a TPC) that share one instruction
// stream of tcgen05.mma.cta_group::2: M = 256 tokens x N = 256 features x K = 16 per instruction.  CTA r of
// the pair holds
//   * in shared memory, per 64-wide K step: its own 2 x 128 token rows of x and HALF of the pair's 256 weight
//     rows, both copied by TMA in the K-major SWIZZLE_128B layout (48 KiB per stage, four stages),
//   * in tensor memory: 2 accumulators of 128 lanes (its tokens) x 256 columns (all features of the pair).
// Per instruction each SM reads 4 KiB of tokens and 4 KiB of weights out of its own shared memory for 128
// tensor cycles (the other half of the weights reaches its tensor core from the partner SM), a quarter of
// what a 128 x 128 single-CTA instruction asks of the shared-memory port per flop.
//
// Warp roles (18 warps): 0-15 epilogue; 16 TMA; 17 MMA issue (rank 0 only).  No thread forwards anything
// between the CTAs -- a cross-CTA mbarrier arrival from a thread was measured at ~1300 cycles per hop, two hops
// per stage round trip held the K loop at 1900 cycles per step against 1049 of tensor work:
//   "full"  lives in rank 0 alone and counts the bytes of BOTH CTAs' tiles: rank 1's loads are cta_group::2 TMA
//           copies that land in rank 1's shared memory and complete on rank 0's barrier;
//   "empty" (and "done") are signalled by two tcgen05.commit, one onto each CTA's barrier (the operand is a
//           shared::cluster address, rank 1's comes from mapa).
// Every wait is bounded in time; on expiry the kernel sets the status word, skips its stores, frees its tensor
// memory and returns.  No multicast of any kind: every TMA load lands in the CTA that issued it.
// Measured and not kept: persistent clusters walking over tiles, (a) with 256-token tiles and the two accumulators
// alternating so that the epilogue runs under the next tile's main loop -- 0.232 / 0.444 ms at 8192 / 16384 tokens
// against 0.207 / 0.365 here (a third more operand bytes per flop through L2), though faster below 2048 tokens,
// where 512-token tiles leave SMs idle (0.055 against 0.064 ms at 1024); (b) with this kernel's 512-token tiles
// and an epilogue of per-lane vector stores straight from registers (the stages stay busy with the next tile's
// loads, so there is no room for the transpose) -- 0.237 / 0.415 ms.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "e8_fast.cuh"
#include "e8_io.cuh"
#include "umma.cuh"

using namespace coset;
using namespace coset::umma;

namespace {

// ---------------------------------------------------------------------------------------------
// codes -> dense bf16 weights, with the arithmetic of the fused kernel's producers: twice the reconstruction
// from the residual table, one multiply by 0.5 / beta, the layer's clamp, round to bf16.
template <int MODE>
__global__ void __launch_bounds__(256)
k_decode_weights_bf16(const uint32_t* __restrict__ codes, const float* __restrict__ beta, e8::TileDiv td, int64_t n_blocks,
                      const uint2* __restrict__ table, float clip, uint4* __restrict__ wq) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += stride) {
        const uint32_t code = __ldg(codes + b);
        const float half_inv = MODE == 2 ? __fdividef(0.5f, __ldg(beta + e8::tile_of(td, b))) : 0.5f;
        float v2[8];
        e8::twice_from_entries(__ldg(table + (code & 0xffffu)), __ldg(table + (code >> 16)), v2);
#pragma unroll
        for (int i = 0; i < 8; ++i) v2[i] *= half_inv;
        if (clip > 0.0f) {  // the training layer's clamp(decode / beta, +-clip), coset/core/layers.py:463
#pragma unroll
            for (int i = 0; i < 8; ++i) v2[i] = fminf(fmaxf(v2[i], -clip), clip);
        }
        wq[b] = make_uint4(pack_bf16x2(v2[0], v2[1]), pack_bf16x2(v2[2], v2[3]), pack_bf16x2(v2[4], v2[5]), pack_bf16x2(v2[6], v2[7]));
    }
}

// ---------------------------------------------------------------------------------------------
constexpr int MSUB = 2;        // token sub-tiles of 128 per CTA
constexpr int PAIR_N = 256;    // features per pair = N of one instruction
constexpr int HALF_N = 128;    // weight rows held by one CTA
constexpr int STAGES = 4;
constexpr int STAGE_BYTES = MSUB * TILE_BYTES + HALF_N * BK * 2;  // 48 KiB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 128 /*barriers, tmem slot*/;
constexpr int EPI_WARPS = 16, TMA_WARP = 16, MMA_WARP = 17;
constexpr int THREADS = 18 * 32;
constexpr uint32_t TMEM_COLS = MSUB * PAIR_N;  // 512: the whole tensor memory of the SM
// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, N = 256, M = 256 over the pair
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PAIR_N >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
static_assert(EPI_WARPS * 32 * 33 * 4 <= STAGES * STAGE_BYTES, "epilogue scratch inside the idle stages");

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of this CTA's shared-memory location `addr` in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t peer_smem(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// TMA tile load whose completion is counted on a barrier of the pair's OTHER CTA (allowed with cta_group::2);
// the tile itself lands in this CTA.  No multicast.
__device__ __forceinline__ void tma_load_pair(uint32_t dst, const CUtensorMap* map, int k0, int row, uint32_t pair_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(k0), "r"(row), "r"(pair_bar) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The bounded wait with cluster-scope acquire, for phases that the other CTA of the pair completes.
// SLEEP: nanoseconds between polls, for warps that wait through the whole main loop.
template <int SLEEP = 0>
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {
    uint64_t t0 = 0;
    for (int it = 0; it < (1 << 24); ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (SLEEP > 0) __nanosleep(SLEEP);
        if ((it & 63) == 63) {
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > 200000000ull) return false;
        }
    }
    return false;
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <typename YT>  // float or __nv_bfloat16 result
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
k_gemm_pair(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map, int N, int K, int T,
            const float* __restrict__ bias, YT* __restrict__ y, int64_t ldy, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;  // the same offset in both CTAs: same kernel, same dynamic size
    uint8_t* gen = smem_raw + (base - raw);
    // stage s: [2 token tiles][weight half]; barriers: empty[STAGES], full[STAGES], done; tmem slot
    const uint32_t bar_base = base + STAGES * STAGE_BYTES;
    const uint32_t full_base = bar_base + 8 * STAGES, done_bar = bar_base + 16 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + STAGES * STAGE_BYTES + 16 * STAGES + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t crank = cluster_rank();
    const bool leader = crank == 0;
    const uint32_t other_base = peer_smem(base, crank ^ 1u);  // the partner's `base`; offsets carry over
    const uint32_t leader_full = peer_smem(base, 0u) + (full_base - base);
    const int tile_n = blockIdx.x >> 1, tile_m = blockIdx.y;
    const int tok0 = tile_m * (2 * MSUB * BM) + (int)crank * (MSUB * BM);  // this CTA's 2 x 128 tokens
    const int row0 = tile_n * PAIR_N + (int)crank * HALF_N;                // the 128 weight rows this CTA holds

    if (warp == 0) {  // the same warp and the same slot offset in both CTAs
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_base + 8 * s, 1);                  // empty: one commit
            mbar_init(full_base + 8 * s, 1);                 // full (used in rank 0): its TMA warp's arrive + both CTAs' bytes
        }
        mbar_init(done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();  // the partner's barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;
    bool ok = true;

    const int KT = K / BK;
    if (warp == TMA_WARP) {
        for (int kt = 0; kt < KT; ++kt) {
            const int s = kt % STAGES;
            if (kt >= STAGES) ok = ok && mbar_wait_cluster(bar_base + 8 * s, (uint32_t)((kt / STAGES - 1) & 1));
            if (lane == 0) {  // rows beyond T or N arrive as zeros
                const uint32_t stage_addr = base + s * STAGE_BYTES;
                const uint32_t bar = leader_full + 8 * s;  // rank 0's barrier, from either CTA
                if (leader) mbar_arrive_expect_tx(full_base + 8 * s, (uint32_t)(2 * STAGE_BYTES));
                for (int a = 0; a < MSUB; ++a) tma_load_pair(stage_addr + a * TILE_BYTES, &x_map, kt * BK, tok0 + a * BM, bar);
                tma_load_pair(stage_addr + MSUB * TILE_BYTES, &w_map, kt * BK, row0, bar);
            }
            __syncwarp();
        }
    } else if (warp == MMA_WARP && leader) {
        // one instruction stream for both SMs; the operand descriptors differ from the one of stage 0 / sub-tile
        // 0 / K slice 0 only in the 14-bit address field (units of 16 bytes)
        const uint64_t desc0 = umma_desc(base);
        const uint32_t desc_hi = (uint32_t)(desc0 >> 32), desc_lo0 = (uint32_t)desc0;
        for (int kt = 0; kt < KT; ++kt) {
            const int s = kt % STAGES;
            ok = ok && mbar_wait_cluster(full_base + 8 * s, (uint32_t)((kt / STAGES) & 1));
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint32_t a_lo = desc_lo0 + (uint32_t)(s * (STAGE_BYTES >> 4)), b_lo = a_lo + (uint32_t)((MSUB * TILE_BYTES) >> 4);
                const uint32_t first = kt > 0 ? 1u : 0u;
#pragma unroll
                for (int a = 0; a < MSUB; ++a) {
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)  // 16 bf16 = 32 bytes along K inside the 128-byte swizzle row
                        umma_f16_pair(tmem_d + (uint32_t)(a * PAIR_N), make_desc(a_lo + (uint32_t)(a * (TILE_BYTES >> 4) + k * 2), desc_hi),
                                      make_desc(b_lo + (uint32_t)(k * 2), desc_hi), IDESC, k > 0 ? 1u : first);
                }
                // both CTAs' stage s may be overwritten once these MMAs retire: one commit per CTA's barrier
                umma_commit_pair(bar_base + 8 * s);
                umma_commit_pair(other_base + (bar_base - base) + 8 * s);
                if (kt == KT - 1) {  // ... and the accumulators of both CTAs are complete
                    umma_commit_pair(done_bar);
                    umma_commit_pair(other_base + (done_bar - base));
                }
            }
            __syncwarp();
        }
    }
    if (!ok && status) atomicExch(status, 1);
    // always: the MMAs must have retired before the tensor memory is read or freed
    ok = mbar_wait_cluster<128>(done_bar, 0u) && ok;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // epilogue: warp w reads tensor-memory lanes 32*(w%4).. of both accumulators, 32 columns at a time (one
    // thread = one token row, 32 consecutive features), and transposes each 32 x 32 piece through shared memory
    // (the stages are idle by now) so that every global store instruction writes 128 contiguous bytes of one row
    if (warp < EPI_WARPS) {
        const int q = warp & 3, grp = warp >> 2;
        float* scr = reinterpret_cast<float*>(gen) + warp * (32 * 33);
        for (int a = 0; a < MSUB; ++a) {
            const int tok_first = tok0 + a * BM + q * 32;
            if (tok_first >= T) continue;  // warp-uniform
            for (int col0 = grp * 32; col0 < PAIR_N; col0 += 4 * 32) {
                uint32_t r[32];
                tmem_ld32(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * PAIR_N + col0), r);
#pragma unroll
                for (int j = 0; j < 32; ++j) scr[lane * 33 + j] = __uint_as_float(r[j]);
                __syncwarp();
                const int n = tile_n * PAIR_N + col0 + lane;
                const float bv = (bias && n < N) ? __ldg(bias + n) : 0.0f;
                if (ok && n < N) {
                    YT* dst = y + (int64_t)tok_first * ldy + n;
                    const int rows = T - tok_first < 32 ? T - tok_first : 32;
                    for (int rr = 0; rr < rows; ++rr) dst[(int64_t)rr * ldy] = (YT)(scr[rr * 33 + lane] + bv);
                }
                __syncwarp();
            }
        }
    }
    if (!ok) {
        if (status) atomicExch(status, 1);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // a wait gave up: leave copies still in flight time to land
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();  // neither CTA frees tensor memory or leaves while the pair's work could still touch it
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

extern "C" int64_t coset_e8_decode_gemm_scratch_bytes(int n_out, int n_in) {
    if (n_out < 0 || n_in < 0) return 0;
    return (int64_t)n_out * (int64_t)n_in * 2;
}

extern "C" int coset_e8_decode_gemm(const void* codes, const float* beta, int64_t blocks_per_tile, int n_out, int n_in,
                                    const void* x_bf16, int64_t ldx, int T, const float* bias, void* y, int y_dtype,
                                    int64_t ldy, float clip, void* scratch, int64_t scratch_bytes, int* status, void* stream) {
    if (n_out < 0 || n_in < 0 || T < 0 || (n_in % BK) != 0) return fail(COSET_E_BADARG, "bad shape (n_in must be a multiple of 64)");
    if (n_out == 0 || T == 0) return 0;
    if (!codes || !x_bf16 || !y || !scratch) return fail(COSET_E_BADARG, "null pointer");
    if (y_dtype != COSET_DTYPE_F32 && y_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown y_dtype");
    if (ldx < n_in || ldy < n_out || (ldx % 8) != 0) return fail(COSET_E_BADARG, "leading dimensions: ldx >= n_in and a multiple of 8, ldy >= n_out");
    if (!aligned(x_bf16, 16) || !aligned(codes, 4) || !aligned(scratch, 16)) return fail(COSET_E_ALIGN, "x and scratch must be 16-byte and codes 4-byte aligned");
    if (scratch_bytes < coset_e8_decode_gemm_scratch_bytes(n_out, n_in)) return fail(COSET_E_BADARG, "scratch holds fewer than n_out * n_in bf16 values");
    if (beta && blocks_per_tile < 1) return fail(COSET_E_BADARG, "blocks_per_tile must be >= 1");
    const int64_t tiles_m = ((int64_t)T + 2 * MSUB * BM - 1) / (2 * MSUB * BM);
    if (tiles_m > 65535) return fail(COSET_E_UNSUPPORTED, "T too large");
    CUtensorMap x_map, w_map;
    if (int e = make_bf16_map(&x_map, x_bf16, n_in, T, ldx)) return e;
    if (int e = make_bf16_map(&w_map, scratch, n_in, n_out, n_in)) return e;
    cudaStream_t st = (cudaStream_t)stream;
    const uint2* table = residual_table_q4(st);
    if (!table) return COSET_E_STATE;
    const int64_t n_blocks = (int64_t)n_out * (n_in / 8);
    e8::TileDiv td = e8::make_tile_div(beta ? blocks_per_tile : 1, n_blocks);
    const unsigned dgrid = (unsigned)((n_blocks + 255) / 256 < 148 * 16 ? (n_blocks + 255) / 256 : 148 * 16);
    const float c = clip > 0.0f ? clip : 0.0f;
    if (beta) k_decode_weights_bf16<2><<<dgrid, 256, 0, st>>>((const uint32_t*)codes, beta, td, n_blocks, table, c, (uint4*)scratch);
    else k_decode_weights_bf16<0><<<dgrid, 256, 0, st>>>((const uint32_t*)codes, nullptr, td, n_blocks, table, c, (uint4*)scratch);
    if (int e = check_launch("e8_decode_gemm (weights)")) return e;
    dim3 grid(2 * ((n_out + PAIR_N - 1) / PAIR_N), (unsigned)tiles_m);
    if (y_dtype == COSET_DTYPE_F32) {
        if (int e = check_cuda(cudaFuncSetAttribute(k_gemm_pair<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), "cudaFuncSetAttribute")) return e;
        k_gemm_pair<float><<<grid, THREADS, SMEM_BYTES, st>>>(x_map, w_map, n_out, n_in, T, bias, (float*)y, ldy, status);
    } else {
        if (int e = check_cuda(cudaFuncSetAttribute(k_gemm_pair<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), "cudaFuncSetAttribute")) return e;
        k_gemm_pair<__nv_bfloat16><<<grid, THREADS, SMEM_BYTES, st>>>(x_map, w_map, n_out, n_in, T, bias, (__nv_bfloat16*)y, ldy, status);
    }
    return check_launch("e8_decode_gemm");
}
