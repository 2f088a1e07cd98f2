// Large-token code-domain matmul on the 5th-generation tensor cores (tcgen05):
//     y[T, N] = x[T, K] (bf16) * Wq^T + bias,   Wq = decode(codes) / beta  (never stored in HBM)
//
// One CTA owns a 512 (tokens) x 128 (output features) tile of y: four 128 x 128 accumulators
// that fill the SM's tensor memory, so that every decoded weight tile is used by four MMAs.
// Per 64-wide K step
//   * up to four activation tiles A (128 x 64 bf16 each) are copied to shared memory by TMA
//     (cp.async.bulk.tensor.2d, one elected thread, completion counted on the stage's "full" mbarrier),
//   * the weight tile      B (128 x 64 bf16) is DECODED into shared memory: one thread turns one
//     packed E8 code (4 B) plus its scale into eight bf16 weights = one 16-byte chunk,
// both in the K-major SWIZZLE_128B layout the UMMA shared-memory descriptor describes
// (8-row groups of 1024 B, 16-byte chunk c of row r stored at chunk c ^ (r & 7)).
// Warp-specialised pipeline over 2 stages: sixteen producer warps fill a stage and arrive on its
// "full" mbarrier; the first lane of a seventeenth warp waits for "full", issues four tcgen05.mma
// (M=128, N=128, K=16) per token sub-tile that accumulate into tensor memory and a
// tcgen05.commit that signals the stage's "empty" mbarrier when those MMAs have retired.  Producer
// warps therefore run ahead of the tensor core by up to two K steps and are never in lockstep
// with each other.  The epilogue (producer warps) reads the accumulator with tcgen05.ld.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records an error code, still frees
// its tensor memory and returns.  No cluster features, no multicast, no peer memory.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "e8_fast.cuh"
#include "e8_io.cuh"
#include "umma.cuh"

using namespace coset;
using namespace coset::umma;

namespace {

constexpr int PRODUCERS = 512;            // 16 warps decode / copy tiles and run the epilogue
constexpr int THREADS = PRODUCERS + 32;   // + 1 warp whose first lane issues the MMAs
constexpr uint32_t TMEM_COLS = 512;       // MSUB accumulators of BN fp32 columns = the whole tensor memory of the SM

// CTA tile = (MSUB x 128 tokens) x BN output features over STAGES pipeline stages.  The shape in use is
// 4 x 128 tokens x 128 features with 2 stages of 80 KiB: one decoded weight tile feeds 4 MMAs, the least decode
// work per flop that 512 tensor-memory columns allow.  Its K loop is bound by the shared-memory port: every
// 128 x 128 x 16 MMA reads 8 KiB of operands for 64 tensor cycles (128 B/cycle, the whole port) while the TMA
// (64 KiB per step) and the producers (16 KiB per step) write through the same port.  Measured alternatives
// that did not beat it: 2 x 128 tokens x 256 features with 3 stages (12 KiB per 128 tensor cycles, but twice
// the decode work per flop: 0.61x); the same with the decode shared between the two CTAs of a cluster through
// st.shared::cluster (0.39x); a cta_group::2 pair (M = 256 x N = 256 per instruction, four stages, each CTA
// decoding half of the weight tile: 0.91x, bound by the issue latency of 16 producer warps per SM).
template <int MSUB_, int BN_, int STAGES_>
struct GemmCfg {
    static constexpr int MSUB = MSUB_, BN = BN_, STAGES = STAGES_;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = MSUB * TILE_BYTES + B_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 128 /*barriers, tmem slot*/;
    static constexpr int SLOTS = (BN * 8) / PRODUCERS;  // (row, 16-byte chunk) slots of the weight tile per producer thread
    // kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, N = BN, M = 128
    static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    static_assert(MSUB * BN == (int)TMEM_COLS, "the accumulators fill the tensor memory");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
    static_assert(STAGE_BYTES >= 16 * 32 * 33 * 4 || STAGES >= 2, "epilogue scratch");
};
using CfgWide = GemmCfg<4, 128, 2>;

template <int MODE, class Cfg>
__global__ void __launch_bounds__(THREADS, 1)
k_dequant_gemm(const uint32_t* __restrict__ codes, const float* __restrict__ beta, e8::TileDiv td, int N, int K,
               const __grid_constant__ CUtensorMap x_map, int T, const float* __restrict__ bias,
               const uint2* __restrict__ table, float* __restrict__ y, int64_t ldy, int* __restrict__ status, float clip) {
    constexpr int MSUB = Cfg::MSUB, BN = Cfg::BN, STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES, SLOTS = Cfg::SLOTS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;           // tiles need 1024-byte alignment for the 128B swizzle
    uint8_t* gen = smem_raw + (base - raw);                 // generic pointer to the same place
    // stage s: [MSUB activation tiles][weight tile]; barriers: empty[STAGES], full[STAGES], done; tmem slot
    const uint32_t bar_base = base + STAGES * STAGE_BYTES;
    const uint32_t full_base = bar_base + 8 * STAGES, done_bar = bar_base + 16 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + STAGES * STAGE_BYTES + 16 * STAGES + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile_n = blockIdx.x, tile_m = blockIdx.y;
    const int kb_row = K / 8;  // codes per weight row
    const int tok0 = tile_m * (MSUB * BM);
    // sub-tiles that hold tokens
    const int n_sub = tok0 >= T ? 0 : ((T - tok0 + BM - 1) / BM < MSUB ? (T - tok0 + BM - 1) / BM : MSUB);

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_base + 8 * s, 1);                  // empty: one tcgen05.commit
            mbar_init(full_base + 8 * s, PRODUCERS / 32);    // full: one arrive per producer warp
        }
        mbar_init(done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;
    bool ok = true;

    const int KT = K / BK;
    if (warp < PRODUCERS / 32) {
        // Each producer thread owns SLOTS (row, 16-byte chunk) slots of the weight tile; codes, scales and table
        // entries travel through registers.  Thread 0 also starts the TMA copies of the activations.
        // Register pipeline over K steps: codes run two steps ahead of the decode and their table entries one
        // step ahead, so neither the code load nor the dependent gathers sit between the "stage is free" wait
        // and the shared-memory stores of a step.  The K loop is unrolled by two so that the two entry sets
        // alternate by name instead of being copied.
        struct Entries {
            uint2 lo[SLOTS], hi[SLOTS];  // residual-table entries of the two level words
            float half_inv[SLOTS];       // 0.5 / scale
        };
        uint32_t code_n[SLOTS];
        float beta_n[SLOTS];
        // Per-slot constants of the K loop: block index at K step 0 (negative: the row is beyond N and holds
        // code 0 = weight 0) and the swizzled offset inside the weight tile.
        int64_t blk0[SLOTS];
        uint32_t slot_off[SLOTS];
#pragma unroll
        for (int j = 0; j < SLOTS; ++j) {
            const int idx = tid + j * PRODUCERS, row = idx >> 3, c = idx & 7, n = tile_n * BN + row;
            blk0[j] = n < N ? (int64_t)n * kb_row + c : -1;
            slot_off[j] = MSUB * TILE_BYTES + swizzled_chunk_offset(row, c);
        }
        auto fetch_codes = [&](int kt) {
#pragma unroll
            for (int j = 0; j < SLOTS; ++j) {
                code_n[j] = 0u;
                beta_n[j] = 1.0f;
                if (blk0[j] >= 0) {
                    const int64_t blk = blk0[j] + kt * 8;
                    code_n[j] = __ldg(codes + blk);
                    if (MODE == 2) beta_n[j] = __ldg(beta + e8::tile_of(td, blk));
                }
            }
        };
        auto fetch_entries = [&](Entries& e) {  // of the codes in code_n; their scales move along
#pragma unroll
            for (int j = 0; j < SLOTS; ++j) {
                e.lo[j] = __ldg(table + (code_n[j] & 0xffffu));
                e.hi[j] = __ldg(table + (code_n[j] >> 16));
                // weights are rounded to bf16, so the scale is applied as one multiply by 0.5 / beta (relative
                // error 2^-23, far below the bf16 rounding) instead of the exact IEEE division of the float32 paths
                e.half_inv[j] = MODE == 2 ? __fdividef(0.5f, beta_n[j]) : 0.5f;
            }
        };
        auto produce = [&](int kt, const Entries& e) {
            const int s = kt % STAGES;
            if (kt >= STAGES) ok = ok && mbar_wait(bar_base + 8 * s, (uint32_t)((kt / STAGES - 1) & 1));
            const uint32_t stage_addr = base + s * STAGE_BYTES;
            uint8_t* stage_gen = gen + s * STAGE_BYTES;
            if (tid == 0) {  // the stage is free: start this step's activation tiles
                mbar_expect_tx(full_base + 8 * s, (uint32_t)(n_sub * TILE_BYTES));
                for (int a = 0; a < n_sub; ++a)
                    tma_load_a(stage_addr + a * TILE_BYTES, &x_map, kt * BK, tok0 + a * BM, full_base + 8 * s);
            }
#pragma unroll
            for (int j = 0; j < SLOTS; ++j) {
                float v2[8];
                e8::twice_from_entries(e.lo[j], e.hi[j], v2);
#pragma unroll
                for (int i = 0; i < 8; ++i) v2[i] *= e.half_inv[j];
                if (clip > 0.0f) {  // the training layer's clamp(decode / beta, +-clip), coset/core/layers.py:463
#pragma unroll
                    for (int i = 0; i < 8; ++i) v2[i] = fminf(fmaxf(v2[i], -clip), clip);
                }
                uint4 v = make_uint4(pack_bf16x2(v2[0], v2[1]), pack_bf16x2(v2[2], v2[3]), pack_bf16x2(v2[4], v2[5]), pack_bf16x2(v2[6], v2[7]));
                *reinterpret_cast<uint4*>(stage_gen + slot_off[j]) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA
            __syncwarp();
            if (lane == 0) mbar_arrive(full_base + 8 * s);
        };
        Entries e0, e1;
        fetch_codes(0);
        fetch_entries(e0);
        if (KT > 1) fetch_codes(1);
        for (int kt = 0; kt < KT; kt += 2) {
            if (kt + 1 < KT) fetch_entries(e1);  // step kt+1: its codes arrived during step kt-1
            if (kt + 2 < KT) fetch_codes(kt + 2);
            produce(kt, e0);
            if (kt + 1 < KT) {
                if (kt + 2 < KT) fetch_entries(e0);
                if (kt + 3 < KT) fetch_codes(kt + 3);
                produce(kt + 1, e1);
            }
        }
    } else {
        // MMA warp: all 32 lanes follow the loop together (a lane left spinning on another barrier would share
        // this warp's issue slots with the lane that feeds the tensor core); lane 0 issues the MMAs and the
        // commits.  The issue path is kept to a few instructions per MMA: the operand descriptors differ from
        // the one of stage 0 / sub-tile 0 / K slice 0 only in the 14-bit address field (units of 16 bytes; shared
        // memory ends below 2^18), so they are one 32-bit add of a constant away from it.
        const uint64_t desc0 = umma_desc(base);
        const uint32_t desc_hi = (uint32_t)(desc0 >> 32), desc_lo0 = (uint32_t)desc0;
        for (int kt = 0; kt < KT; ++kt) {
            const int s = kt % STAGES;
            ok = ok && mbar_wait(full_base + 8 * s, (uint32_t)((kt / STAGES) & 1));
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint32_t a_lo = desc_lo0 + (uint32_t)(s * (STAGE_BYTES >> 4)), b_lo = a_lo + (uint32_t)((MSUB * TILE_BYTES) >> 4);
                const uint32_t first = kt > 0 ? 1u : 0u;
#pragma unroll
                for (int a = 0; a < MSUB; ++a) {
                    if (a < n_sub) {
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)  // 16 bf16 = 32 bytes along K inside the 128-byte swizzle row
                            umma_f16(tmem_d + (uint32_t)(a * BN), make_desc(a_lo + (uint32_t)(a * (TILE_BYTES >> 4) + k * 2), desc_hi),
                                     make_desc(b_lo + (uint32_t)(k * 2), desc_hi), Cfg::IDESC, k > 0 ? 1u : first);
                    }
                }
                umma_commit(bar_base + 8 * s);            // stage s may be overwritten once these MMAs retire
                if (kt == KT - 1) umma_commit(done_bar);  // ... and the accumulators are complete
            }
            __syncwarp();
        }
    }
    if (!ok && status) atomicExch(status, 1);
    ok = mbar_wait(done_bar, 0u) && ok;  // always: the accumulators' MMAs must have retired before the tensor memory is freed
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // epilogue: producer warp w reads TMEM lanes 32*(w%4).. of every accumulator, 32 columns at a time
    // (one thread = one token row, 32 consecutive features), and transposes each 32 x 32 piece through
    // shared memory (the pipeline stages are idle by now), so that every global store instruction
    // writes 128 contiguous bytes of one output row instead of 4 bytes of 32 different rows.
    if (warp < PRODUCERS / 32) {
        // 16 warps = 4 lane quarters x 4 groups; a group takes every fourth 32-column piece of the BN columns
        const int q = warp & 3, grp = warp >> 2;
        float* scr = reinterpret_cast<float*>(gen) + warp * (32 * 33);  // 16 warps x 4.1 KiB inside the idle stages
        for (int a = 0; a < n_sub; ++a) {
            const int tok_first = tok0 + a * BM + q * 32;
            for (int col0 = grp * 32; col0 < BN; col0 += 4 * 32) {
                uint32_t r[32];
                tmem_ld32(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN + col0), r);
#pragma unroll
                for (int j = 0; j < 32; ++j) scr[lane * 33 + j] = __uint_as_float(r[j]);
                __syncwarp();
                const int n = tile_n * BN + col0 + lane;
                const float bv = (bias && n < N) ? __ldg(bias + n) : 0.0f;
                if (ok && n < N) {
                    float* dst = y + (int64_t)tok_first * ldy + n;
                    const int rows = T - tok_first < 32 ? T - tok_first : 32;
                    for (int rr = 0; rr < rows; ++rr) dst[(int64_t)rr * ldy] = scr[rr * 33 + lane] + bv;
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
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

extern "C" int coset_e8_dequant_gemm(const void* codes, const float* beta, int64_t blocks_per_tile, int n_out, int n_in,
                                     const void* x_bf16, int64_t ldx, int T, const float* bias, float* y, int64_t ldy,
                                     float clip, int* status, void* stream) {
    if (n_out < 0 || n_in < 0 || T < 0 || (n_in % BK) != 0) return fail(COSET_E_BADARG, "bad shape (n_in must be a multiple of 64)");
    if (n_out == 0 || T == 0) return 0;
    if (!codes || !x_bf16 || !y) return fail(COSET_E_BADARG, "null pointer");
    if (ldx < n_in || ldy < n_out || (ldx % 8) != 0) return fail(COSET_E_BADARG, "leading dimensions: ldx >= n_in and a multiple of 8, ldy >= n_out");
    if (!aligned(x_bf16, 16) || !aligned(codes, 4)) return fail(COSET_E_ALIGN, "x must be 16-byte and codes 4-byte aligned");
    CUtensorMap x_map;
    if (int e = make_bf16_map(&x_map, x_bf16, n_in, T, ldx)) return e;
    if (beta && blocks_per_tile < 1) return fail(COSET_E_BADARG, "blocks_per_tile must be >= 1");
    cudaStream_t st = (cudaStream_t)stream;
    const uint2* table = residual_table_q4(st);
    if (!table) return COSET_E_STATE;
    e8::TileDiv td = e8::make_tile_div(beta ? blocks_per_tile : 1, (int64_t)n_out * (n_in / 8));
#define LAUNCH_GEMM(MODE, CFG)                                                                                              \
    do {                                                                                                                    \
        dim3 grid((n_out + CFG::BN - 1) / CFG::BN, (T + CFG::MSUB * BM - 1) / (CFG::MSUB * BM));                            \
        if (grid.y > 65535) return fail(COSET_E_UNSUPPORTED, "T too large");                                                \
        if (int e = check_cuda(cudaFuncSetAttribute(k_dequant_gemm<MODE, CFG>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                    CFG::SMEM_BYTES), "cudaFuncSetAttribute")) return e;                     \
        k_dequant_gemm<MODE, CFG><<<grid, THREADS, CFG::SMEM_BYTES, st>>>((const uint32_t*)codes, beta, td, n_out, n_in,    \
                                                                          x_map, T, bias, table, y, ldy, status,             \
                                                                          clip > 0.0f ? clip : 0.0f);                        \
    } while (0)
    if (beta) LAUNCH_GEMM(2, CfgWide);
    else LAUNCH_GEMM(0, CfgWide);
#undef LAUNCH_GEMM
    return check_launch("e8_dequant_gemm");
}
