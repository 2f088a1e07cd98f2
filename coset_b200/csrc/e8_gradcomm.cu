// Decode-and-average for the E8-quantised gradient exchange.
//
// Every rank encodes its gradient with one shared scalar scale s (x * s, then q=4, M=2 codes),
// the packed codes are all-gathered into a [W, n_blocks] array in LOCAL memory, and this kernel
// reads the W code streams once and writes
//     out = ( sum_r x_hat_r ) / (s * W)
// The sum of reconstructions is exact (half-integers, accumulated as integers), the divisor
// d = RN(s * W) is formed once in float32 and the quotient is one IEEE division, so a CPU run of
// the same recipe is bit-identical.  No pointer to another GPU's memory is ever dereferenced.
//
// Bytes per block: W * 4 read + 32 written (float32 output).
#include "common.cuh"
#include "e8_fast.cuh"
#include "e8_io.cuh"

using namespace coset;

namespace {

constexpr int kThreads = 256;

// Code streams of the ranks when they are NOT gathered into local memory first: one pointer per
// rank into that rank's own buffer (peer memory, mapped into this process), read with plain loads
// over NVLink.  first = the rank whose stream is read first (each rank starts at a different peer).
constexpr int kMaxPeers = 16;
struct PeerStreams {
    const uint32_t* p[kMaxPeers];
    int first;
};

// One thread owns kPerThread consecutive blocks (1 or 4).  With 4 it requests a 16-byte vector of codes from
// every stream before the first table lookup and writes 128 contiguous bytes; measured on local memory that
// is no faster than one block per thread (0.336 against 0.320 ms for 8 streams of 13.7 M blocks: the kernel
// is bound by the table lookups), so 1 is used.
constexpr int kPerThread = 1;

__device__ __forceinline__ void accumulate_code(uint32_t code, const uint2* __restrict__ table, uint32_t (&acc)[4]) {
    const uint2 t0 = __ldg(table + (code & 0xffffu));
    uint2 t1 = make_uint2(0x07070707u, 0x07070707u);  // all-zero top-level word: zero residual, no lookup
    if (code >> 16) t1 = __ldg(table + (code >> 16));
    const uint32_t lo = t0.x + 4u * t1.x, hi = t0.y + 4u * t1.y;  // biased bytes, each <= 90
    acc[0] += lo & 0x00ff00ffu;
    acc[1] += (lo >> 8) & 0x00ff00ffu;
    acc[2] += hi & 0x00ff00ffu;
    acc[3] += (hi >> 8) & 0x00ff00ffu;
}

template <int DT>
__device__ __forceinline__ void store_mean(const uint32_t (&acc)[4], int world, float divisor, void* __restrict__ out, int64_t b) {
    // 16-bit lanes: acc[0] = coordinates (0,2), acc[1] = (1,3), acc[2] = (4,6), acc[3] = (5,7)
    const int bias = 5 * e8::kTableBias * world;  // every rank contributes 7 + 4*7 to each lane
    int v[8];
    v[0] = (int)(acc[0] & 0xffffu) - bias; v[2] = (int)(acc[0] >> 16) - bias;
    v[1] = (int)(acc[1] & 0xffffu) - bias; v[3] = (int)(acc[1] >> 16) - bias;
    v[4] = (int)(acc[2] & 0xffffu) - bias; v[6] = (int)(acc[2] >> 16) - bias;
    v[5] = (int)(acc[3] & 0xffffu) - bias; v[7] = (int)(acc[3] >> 16) - bias;
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float sum = __fmul_rn((float)v[i], 0.5f);  // exact: |v| < 2^16
        o[i] = __fdiv_rn(sum, divisor);
    }
    e8::Row8<DT>::store(out, b, o);
}

template <int DT, bool PEERS>
__global__ void __launch_bounds__(kThreads)
k_decode_mean(const uint32_t* __restrict__ codes, PeerStreams peers, int world, int64_t n, int64_t stride, float divisor,
              const uint2* __restrict__ table, void* __restrict__ out, const int* __restrict__ status) {
    const int64_t b0 = ((int64_t)blockIdx.x * kThreads + threadIdx.x) * kPerThread;
    if (b0 >= n) return;
    // a bounded cross-rank wait before this launch gave up: the peers' streams are not known to be
    // complete, so nothing is read or written
    if (PEERS && status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
    uint32_t acc[kPerThread][4];
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0u;
    auto stream_ptr = [&](int r) -> const uint32_t* {
        if (PEERS) {
            int src = peers.first + r;
            if (src >= world) src -= world;
            return peers.p[src] + b0;
        }
        return codes + (int64_t)r * stride + b0;
    };
    // vector path when a stream's 16 bytes at b0 are aligned and inside the tensor; else (odd strides, the
    // tail of the tensor) four scalar loads
    const bool full = b0 + kPerThread <= n;
    for (int r0 = 0; r0 < world; r0 += 4) {
        uint32_t c4[4][kPerThread];
#pragma unroll
        for (int u = 0; u < 4; ++u) {  // up to four streams requested before the first table lookup
#pragma unroll
            for (int j = 0; j < kPerThread; ++j) c4[u][j] = 0u;
            if (r0 + u < world) {
                const uint32_t* p = stream_ptr(r0 + u);
                if (kPerThread == 4 && full && ((reinterpret_cast<uintptr_t>(p) & 15u) == 0)) {
                    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(p));
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < kPerThread; ++j) c4[u][j] = w[j & 3];
                } else {
#pragma unroll
                    for (int j = 0; j < kPerThread; ++j)
                        if (b0 + j < n) c4[u][j] = __ldcs(p + j);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (r0 + u >= world) break;
#pragma unroll
            for (int j = 0; j < kPerThread; ++j) accumulate_code(c4[u][j], table, acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < kPerThread; ++j)
        if (b0 + j < n) store_mean<DT>(acc[j], world, divisor, out, b0 + j);
}

}  // namespace

namespace {

// Cross-rank "everyone has arrived" with a bound.  flags[r] is rank r's own array of `world` words
// (peer / symmetric memory, mapped into this process); word s of it is written only by rank s.
// Thread t tells rank t that this rank has reached `epoch` (one release store over NVLink into
// flags[t][rank], after a system-scope fence that publishes everything this rank wrote before the
// launch) and then polls its own flags[rank][t] until rank t has said the same.  Epochs only grow, so
// the words are never cleared and a late reader of an old epoch passes at once.  The poll gives up
// after timeout_ns of the global timer: it records that in *status and returns, and the kernels that
// follow on the stream check *status before touching a peer's data.
struct PeerFlags {
    uint32_t* p[kMaxPeers];
};

__global__ void k_peer_signal_wait(PeerFlags flags, int world, int rank, uint32_t epoch, unsigned long long timeout_ns,
                                   int* __restrict__ status) {
    const int t = threadIdx.x;
    if (t >= world) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[t] + rank), "r"(epoch) : "memory");
    const uint32_t* mine = flags.p[rank] + t;
    unsigned long long start;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int32_t)(v - epoch) >= 0) break;
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - start > timeout_ns) {
            if (status != nullptr) atomicExch(status, 1 + t);  // 1 + the rank that did not arrive
            break;
        }
        __nanosleep(128);
    }
}

}  // namespace

extern "C" int coset_peer_signal_wait(void* const* rank_flags, int world, int rank, uint32_t epoch, int timeout_ms,
                                      int* status, void* stream) {
    if (world < 1 || world > kMaxPeers) return fail(COSET_E_BADARG, "world must be in 1..16");
    if (rank < 0 || rank >= world) return fail(COSET_E_BADARG, "rank outside the world");
    if (!rank_flags) return fail(COSET_E_BADARG, "null pointer");
    PeerFlags f = {};
    for (int r = 0; r < world; ++r) {
        if (!rank_flags[r] || !aligned(rank_flags[r], 4)) return fail(COSET_E_BADARG, "flag array %d is null or misaligned", r);
        f.p[r] = (uint32_t*)rank_flags[r];
    }
    const unsigned long long ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
    k_peer_signal_wait<<<1, 32, 0, (cudaStream_t)stream>>>(f, world, rank, epoch, ns, status);
    return check_launch("peer_signal_wait");
}

extern "C" int coset_e8_decode_mean(const void* codes, int world, int64_t n_blocks, int64_t rank_stride_blocks,
                                    float scale, void* out, int out_dtype, void* stream) {
    if (world < 1 || world > 512) return fail(COSET_E_BADARG, "world must be in 1..512");
    if (n_blocks < 0 || rank_stride_blocks < n_blocks) return fail(COSET_E_BADARG, "bad n_blocks / rank stride");
    if (n_blocks == 0) return 0;
    if (!codes || !out) return fail(COSET_E_BADARG, "null pointer");
    if (out_dtype != COSET_DTYPE_F32 && out_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown out_dtype");
    if (!aligned(codes, 4) || !aligned(out, 16)) return fail(COSET_E_ALIGN, "codes must be 4-byte and out 16-byte aligned");
    if (!(scale == scale) || scale == 0.0f) return fail(COSET_E_BADARG, "scale must be a non-zero number");
    cudaStream_t st = (cudaStream_t)stream;
    const uint2* table = residual_table_q4(st);
    if (!table) return COSET_E_STATE;
    float divisor = scale * (float)world;  // one float32 rounding, reproduced by the CPU recipe
    unsigned grid = (unsigned)((n_blocks + (int64_t)kThreads * kPerThread - 1) / ((int64_t)kThreads * kPerThread));
    PeerStreams none = {};
    if (out_dtype == COSET_DTYPE_F32)
        k_decode_mean<0, false><<<grid, kThreads, 0, st>>>((const uint32_t*)codes, none, world, n_blocks, rank_stride_blocks, divisor, table, out, nullptr);
    else
        k_decode_mean<1, false><<<grid, kThreads, 0, st>>>((const uint32_t*)codes, none, world, n_blocks, rank_stride_blocks, divisor, table, out, nullptr);
    return check_launch("e8_decode_mean");
}

extern "C" int coset_e8_decode_mean_peers(const void* const* rank_codes, int world, int rank, int64_t n_blocks, float scale,
                                          void* out, int out_dtype, const int* status, void* stream) {
    if (world < 1 || world > kMaxPeers) return fail(COSET_E_BADARG, "world must be in 1..16 for the peer-memory form");
    if (rank < 0 || rank >= world) return fail(COSET_E_BADARG, "rank outside the world");
    if (n_blocks < 0) return fail(COSET_E_BADARG, "n_blocks is negative");
    if (n_blocks == 0) return 0;
    if (!rank_codes || !out) return fail(COSET_E_BADARG, "null pointer");
    if (out_dtype != COSET_DTYPE_F32 && out_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown out_dtype");
    if (!aligned(out, 16)) return fail(COSET_E_ALIGN, "out must be 16-byte aligned");
    if (!(scale == scale) || scale == 0.0f) return fail(COSET_E_BADARG, "scale must be a non-zero number");
    PeerStreams peers = {};
    for (int r = 0; r < world; ++r) {
        if (!rank_codes[r] || !aligned(rank_codes[r], 4)) return fail(COSET_E_BADARG, "code stream %d is null or misaligned", r);
        peers.p[r] = (const uint32_t*)rank_codes[r];
    }
    peers.first = rank;
    cudaStream_t st = (cudaStream_t)stream;
    const uint2* table = residual_table_q4(st);
    if (!table) return COSET_E_STATE;
    float divisor = scale * (float)world;
    unsigned grid = (unsigned)((n_blocks + (int64_t)kThreads * kPerThread - 1) / ((int64_t)kThreads * kPerThread));
    if (out_dtype == COSET_DTYPE_F32)
        k_decode_mean<0, true><<<grid, kThreads, 0, st>>>(nullptr, peers, world, n_blocks, 0, divisor, table, out, status);
    else
        k_decode_mean<1, true><<<grid, kThreads, 0, st>>>(nullptr, peers, world, n_blocks, 0, divisor, table, out, status);
    return check_launch("e8_decode_mean_peers");
}
