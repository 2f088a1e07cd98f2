/*
 * coset_b200 -- C ABI of the B200 (sm_100a) implementation of coset's E8 hierarchical
 * nested-lattice quantisation (HNLQ) hot path.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its name ends in `_host`.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).  Calls only
 *     enqueue work; they never synchronise unless documented.
 *   - Return value: 0 on success, negative = bad argument (COSET_E_*), positive = cudaError_t.
 *     Nothing throws or aborts across this boundary.  coset_last_error_string() describes the
 *     last failure of the calling thread.
 *   - A "block" is one 8-vector (one E8 lattice cell).  `n_blocks` counts blocks.
 *
 * Packed code format ("fast format", additive to the reference's float32 digits)
 *   bits per digit  bpd = 2 if q <= 4 else 4   (2 <= q <= 16)
 *   level word      8 digits, digit j at bit bpd*j  -> 16 bits (q<=4) or 32 bits
 *   block code      M consecutive level words, level 0 first, little endian
 *   For q = 4, M = 2 a block code is exactly one uint32: level m, digit j at bit 16*m + 2*j.
 *   coset_e8_code_bytes(q, M) gives the bytes per block.
 *
 * Scale modes (which IEEE operation is applied, because the reference has two conventions)
 *   COSET_SCALE_NONE       x is quantised as is
 *   COSET_SCALE_DIV_SCALAR encode: x / scale[0];  decode: x_hat * scale[0]
 *                          (codec convention, coset/core/e8/codecs.py:64 and :175)
 *   COSET_SCALE_MUL_TILE   encode: x * scale[block / blocks_per_tile];  decode: x_hat / scale[...]
 *                          (layer convention, coset/core/layers.py:431-436 and :453-460;
 *                           blocks_per_tile = in_features/8 for tiling='row', 1 for 'block')
 *
 * Semantics modes
 *   COSET_SEM_CORE  bit-exact with coset.core.e8 (float32; including its g_x flip rule and its
 *                   level recurrence without re-quantisation)
 *   COSET_SEM_CORE_LITERAL  identical results to COSET_SEM_CORE by construction of the slow path:
 *                   every block runs the op-by-op restatement, none the guarded fast path; the
 *                   tests use it to cross-check the fast path on inputs too large for the CPU oracle
 *   COSET_SEM_REF   bit-exact with ref/hnlq.py (float64, tie dither, re-quantising recurrence,
 *                   overload loop); parity-only, not a timed path; served by its own entry points
 *                   coset_e8_ref_encode / coset_e8_ref_decode (it needs float64 data and a T output)
 *
 * Exactness domain of COSET_SEM_CORE: finite inputs with |scaled x| <= 2^20.  Outside it the
 * call still succeeds and never faults, but the digits are unspecified.
 */
#ifndef COSET_B200_H
#define COSET_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COSET_DTYPE_F32 0
#define COSET_DTYPE_BF16 1

#define COSET_SCALE_NONE 0
#define COSET_SCALE_DIV_SCALAR 1
#define COSET_SCALE_MUL_TILE 2

#define COSET_SEM_CORE 0
#define COSET_SEM_REF 1
#define COSET_SEM_CORE_LITERAL 2 /* same results as CORE, every block through the op-by-op search (validation) */
#define COSET_SEM_CORE_SATURATE 3 /* CORE after clamping every scaled coordinate to +-3.9 (q=4, M=2 encode only): the
                                     two-level code then never wraps around (its top level stays the origin), so an
                                     outlier costs a bounded clipping error instead of an unrelated reconstruction;
                                     identical to CORE for blocks with max|scaled x| <= 3.9.  No counterpart in the
                                     reference, whose codec wraps silently (coset/core/e8/codecs.py:63-89). */

#define COSET_E_BADARG (-1)   /* null pointer, negative size, unknown enum */
#define COSET_E_UNSUPPORTED (-2) /* q / M / dtype combination not implemented */
#define COSET_E_ALIGN (-3)    /* pointer not aligned as documented */
#define COSET_E_STATE (-4)    /* library state (context / table) unusable */

/* Library version (major*10000 + minor*100 + patch). */
int coset_version(void);
/* Message for the last non-zero return on this thread ("" if none). */
const char* coset_last_error_string(void);
/* Bytes of packed code per block; 0 if (q, M) is unsupported. */
int coset_e8_code_bytes(int q, int M);

/*
 * E8Lattice.projection (coset/core/e8/lattice.py:114-169): the reference's D8 u (D8+1/2)
 * search with its own tie rules.  x, y: [n_blocks, 8] float32.
 */
int coset_e8_projection(const float* x, int64_t n_blocks, float* y, void* stream);

/*
 * e8_encode (coset/core/e8/codecs.py:17-89): scale, then M levels of
 * encode_coords(projection(x / q^m)) (coset/core/base.py:134-154), written as packed codes.
 * x: [n_blocks, 8] of x_dtype (16-byte aligned).  codes: packed, 4-byte aligned.
  * For q = 4, M = 2 the call is two launches (main kernel + a short fix-up kernel for the blocks the
 * cheapest tier cannot prove) and uses a few MB of library-owned scratch per (device, stream), allocated
 * on the first call and when a larger tensor arrives: make the first call of a given size before a
 * stream capture begins.  Calls on one stream share the scratch (they are ordered); concurrent calls
 * on different streams have their own.
 */
int coset_e8_encode(const void* x, int x_dtype, const float* scale, int scale_mode,
                    int64_t n_blocks, int64_t blocks_per_tile, int q, int M, int sem,
                    void* codes, void* stream);

/*
 * e8_decode / E8Decoder._full_decode (coset/core/e8/codecs.py:139-218):
 * x_hat = unscale( sum_m q^m * (G b_m - q * projection(G b_m / q)) ).
 * out: [n_blocks, 8] of out_dtype (16-byte aligned).
 */
int coset_e8_decode(const void* codes, const float* scale, int scale_mode, int64_t n_blocks,
                    int64_t blocks_per_tile, int q, int M, int sem, void* out, int out_dtype,
                    void* stream);

/*
 * Fused round trip decode(encode(x)) without storing codes: e8_quantize
 * (coset/core/e8/codecs.py:221-286) when scale_mode = NONE, M = 2; with COSET_SCALE_MUL_TILE and
 * clip > 0 it is the weight path of HNLQLinearQAT._quantize_weights
 * (coset/core/layers.py:429-463): clamp(e8_quantize(W * beta) / beta, -clip, clip).
 * clip <= 0 disables the clamp.  codes_out may be NULL; if given it receives the packed codes.
 */
int coset_e8_quantize(const void* x, int x_dtype, const float* scale, int scale_mode,
                      int64_t n_blocks, int64_t blocks_per_tile, int q, int M, float clip,
                      void* out, int out_dtype, void* codes_out, void* stream);

/*
 * Compatibility views of the packed codes: the reference returns / accepts digits as float32
 * [n_blocks, M, 8] (coset/core/e8/codecs.py:83; negative zeros are not reproduced).
 */
int coset_e8_unpack_codes_f32(const void* codes, int64_t n_blocks, int q, int M, float* digits,
                              void* stream);
int coset_e8_pack_codes_f32(const float* digits, int64_t n_blocks, int q, int M, void* codes,
                            void* stream);

/*
 * Backward of the fake-quantised weight path of HNLQLinearQAT (straight-through estimator,
 * coset/core/layers.py:62-95, with torch autograd's rules for the surrounding
 * mul / div / clamp of coset/core/layers.py:429-463).  M is 2 (e8_quantize hard-wires it).
 *   grad_out : dL/dWq           [n_blocks, 8] float32 or bf16
 *   w        : weights          [n_blocks, 8] float32
 *   codes    : packed codes written by coset_e8_quantize in the forward pass
 *   beta     : per-tile scale   [ceil(n_blocks / blocks_per_tile)]
 *   grad_w   : dL/dW            [n_blocks, 8] float32
 *   grad_beta: dL/dbeta per tile (may be NULL)
 */
int coset_e8_fake_quant_bwd(const void* grad_out, int grad_dtype, const float* w, const void* codes,
                            const float* beta, int64_t n_blocks, int64_t blocks_per_tile, int q,
                            float clip, float* grad_w, float* grad_beta, void* stream);

/*
 * The layer's weight path with its scale computed on the device (coset/core/layers.py:415-470):
 *   beta[t] = beta_min[t] + sigmoid(theta[t]) * beta_range[t]        (one value per tile)
 *   out     = clamp(e8_quantize(W * beta) / beta, +-clip)            (coset_e8_quantize, M = 2)
 * coset_layer_beta is the first line alone; coset_e8_layer_fake_quant_fwd is both (two launches, one
 * call) and leaves the scales it used in `beta` and the packed codes in `codes` for the backward pass;
 * coset_e8_layer_fake_quant_bwd is coset_e8_fake_quant_bwd followed by the chain rule through the
 * sigmoid: grad_theta = (dbeta * beta_range) * (1 - s) * s, as torch autograd forms it (grad_theta may be
 * NULL when theta is not trained).
 */
int coset_layer_beta(const float* theta, const float* beta_min, const float* beta_range, int64_t n_tiles,
                     float* beta, void* stream);
int coset_e8_layer_fake_quant_fwd(const float* w, const float* theta, const float* beta_min, const float* beta_range,
                                  int64_t n_blocks, int64_t blocks_per_tile, int q, float clip, void* out,
                                  int out_dtype, void* codes, float* beta, void* stream);
int coset_e8_layer_fake_quant_bwd(const void* grad_out, int grad_dtype, const float* w, const void* codes,
                                  const float* beta, const float* theta, const float* beta_range, int64_t n_blocks,
                                  int64_t blocks_per_tile, int q, float clip, float* grad_w, float* grad_theta,
                                  void* stream);

/*
 * Host-buffer variants: the arrays live in HOST memory (page-locked for full overlap); the
 * library stages them through a context's device slots, chunk by chunk, with copies in both
 * directions overlapping the kernels.  This is the call a CPU-side caller of the reference's
 * e8_encode / e8_decode (coset/core/e8/codecs.py:17-89, 185-218) switches to.  The calls return
 * when the result is complete in host memory.  The context belongs to the device that was
 * current when it was created; one call at a time per context.
 *   chunk_blocks : blocks staged per slot (device memory held: n_slots * chunk_blocks * 68 B)
 */
typedef struct coset_host_ctx coset_host_ctx;
int coset_host_ctx_create(int64_t chunk_blocks, int n_slots, coset_host_ctx** out);
int coset_host_ctx_destroy(coset_host_ctx* ctx);
int coset_e8_encode_host(coset_host_ctx* ctx, const void* x_host, int x_dtype, const float* scale_host,
                         int scale_mode, int64_t n_blocks, int64_t blocks_per_tile, int q, int M,
                         void* codes_host);
int coset_e8_decode_host(coset_host_ctx* ctx, const void* codes_host, const float* scale_host,
                         int scale_mode, int64_t n_blocks, int64_t blocks_per_tile, int q, int M,
                         void* out_host, int out_dtype);
/*
 * Round trip over host arrays in one pass: coset_e8_quantize per chunk, so the input travels host ->
 * device while reconstructions (and, if codes_host is not NULL, the packed codes) of earlier chunks
 * travel back -- both PCIe directions are busy at once.  e8_quantize / decode(encode(x)) of
 * coset/core/e8/codecs.py:221-286 for a CPU-side caller.  Holds n_slots * chunk_blocks * 32 B more.
 */
int coset_e8_quantize_host(coset_host_ctx* ctx, const void* x_host, int x_dtype, const float* scale_host,
                           int scale_mode, int64_t n_blocks, int64_t blocks_per_tile, int q, int M,
                           float clip, void* out_host, int out_dtype, void* codes_host);

/*
 * E8-quantised gradient exchange, receive side.  The reference only plans this path
 * ("quantize gradient buckets ... decode", prompts/design_instructions.md:104-110); the recipe is:
 * every rank encodes x * scale with coset_e8_encode (q=4, M=2, COSET_SCALE_MUL_TILE with a single
 * tile), the packed codes are all-gathered into codes[world][rank_stride_blocks] in local memory,
 * and this call writes  out = (sum_r x_hat_r) / RN(scale * world)  as [n_blocks, 8].
 * The sum is exact, the division is one IEEE float32 division.
 */
int coset_e8_decode_mean(const void* codes, int world, int64_t n_blocks, int64_t rank_stride_blocks,
                         float scale, void* out, int out_dtype, void* stream);
/*
 * The same receive side WITHOUT the all-gather: rank_codes[r] (host array of `world` device pointers)
 * points at rank r's own code buffer, mapped into this process (peer / symmetric memory); the kernel
 * reads the peers' streams with plain loads over NVLink while it decodes, starting at stream `rank`.
 * The caller orders "every rank has finished encoding" before this call and "every rank has finished
 * reading" before the buffers are overwritten (coset_peer_signal_wait below, enqueued between the
 * encode and this call).  status (device int, may be NULL): when not NULL and non-zero at run time --
 * a wait before this launch gave up -- the kernel reads and writes nothing.
 * world <= 16.  Same arithmetic, bit-identical result.
 */
int coset_e8_decode_mean_peers(const void* const* rank_codes, int world, int rank, int64_t n_blocks,
                               float scale, void* out, int out_dtype, const int* status, void* stream);
/*
 * Bounded cross-rank arrival for the peer-memory paths (the exchange planned at
 * prompts/design_instructions.md:104-110 has no counterpart code in the reference).
 * rank_flags[r] (host array of `world` device pointers) is rank r's array of `world` uint32 words in
 * peer / symmetric memory, zero before first use; word s of every array is written only by rank s.
 * The one-CTA kernel publishes everything this rank wrote earlier on the stream, stores `epoch` into
 * word `rank` of every rank's array and waits until its own array holds an epoch >= `epoch` from every
 * rank.  Epochs must grow by one per call (wrap-around is handled).  The wait is bounded: after
 * timeout_ms (<= 0: 2000 ms) it stores 1 + (the first rank found missing) into *status (device int, may be
 * NULL) and returns, so a rank that died leaves its peers' streams and contexts usable.
 * world <= 16.  Every rank runs on its own GPU: two ranks that wait for each other must never share one.
 */
int coset_peer_signal_wait(void* const* rank_flags, int world, int rank, uint32_t epoch, int timeout_ms,
                           int* status, void* stream);

/*
 * Code-domain ("vLUT") product for inference, small token counts:
 *   y[T, n_out] = x[T, n_in] * Wq^T + bias,   Wq = decode(codes) / beta   (never materialised)
 * Math of the reference's one-sided vLUT inner product (coset/legacy/quant/vlut.py:72-117):
 * <x, w_hat> = sum_m 4^m <x, r(b_m)>, r(b) = G b - 4 Q(G b / 4).
 *   codes : [n_out, n_in/8] packed q=4, M=2 codes (row-major, as coset_e8_quantize emits them)
 *   beta  : per-tile scale in the layer convention (may be NULL = no scale);
 *           blocks_per_tile = n_in/8 for one scale per row, 1 for one per block
 *   x     : [T, ldx] float32 or bf16 (rows 16-byte aligned);  y: [T, ldy] float32 or bf16 (y_dtype; accumulated in
 *           float32 and rounded once on the store)
 *   clip  : > 0: every weight is clamp(decode / beta, +-clip), the layer's weight_clip_value
 *           (coset/core/layers.py:463), so that an exported layer computes what the trained one did; 0: none
 * Memory-bound on the code stream; meant for T <= ~64 (larger T: dequantise + tensor cores).
 */
int coset_e8_vlut_gemv(const void* codes, const float* beta, int64_t blocks_per_tile, int n_out, int n_in,
                       const void* x, int x_dtype, int64_t ldx, int T, const float* bias, void* y,
                       int y_dtype, int64_t ldy, float clip, void* stream);
/*
 * The same product with the result rows written into SEVERAL buffers at once: y_targets (host array of
 * n_targets <= 16 device pointers) are the places of this rank's output-feature slice in the result
 * buffer of every rank, its own and its peers' (peer / symmetric memory, plain stores over NVLink).
 * With the weight sharded along the output features this replaces the all-gather after the product;
 * the caller orders "all ranks have written" with a device-side barrier of its communication library.
 */
int coset_e8_vlut_gemv_scatter(const void* codes, const float* beta, int64_t blocks_per_tile, int n_out,
                               int n_in, const void* x, int x_dtype, int64_t ldx, int T,
                               const float* bias, float* const* y_targets, int n_targets, int64_t ldy,
                               float clip, void* stream);

/*
 * Quantisation statistics of the q=4, M=2 codec over a tensor (one pass, deterministic):
 *   out[0] = sum ||x_hat - x_s||^2   out[1] = overloaded blocks (projection(x_s / q^M) != 0, the
 *   overload test of ref/hnlq.py:341 / pub/main.tex:878-934)   out[2] = blocks with a non-zero code
 *   out[3] = sum ||x_s||^2           (x_s = scaled input, x_hat = decode(encode(x_s)), unscaled)
 * `scratch` is device memory of coset_e8_quant_stats_scratch_bytes(n_blocks) bytes (16-byte
 * aligned) holding one partial record per CTA; `out` is 4 doubles in device memory.
 */
int64_t coset_e8_quant_stats_scratch_bytes(int64_t n_blocks);
int coset_e8_quant_stats(const void* x, int x_dtype, const float* scale, int scale_mode, int64_t n_blocks,
                         int64_t blocks_per_tile, void* scratch, int64_t scratch_bytes, double* out,
                         void* stream);

/*
 * coset_e8_quant_stats for callers that must not allocate device memory.  (No counterpart in the
 * reference.)  Some hosts of this library run where cudaMalloc is off limits -- inside another
 * framework's memory pool with a fixed budget, in a plugin that is handed only its input and
 * output buffers, or on a thread that may not take the allocator's lock -- and those callers have
 * nowhere to get the scratch buffer the regular entry point asks for.  This variant keeps the
 * per-CTA partial records in a 128 KB array that is part of the library image on every GPU that
 * loads it, and reconstructs without the (allocated) residual table.  Same arguments and results
 * as coset_e8_quant_stats, minus the scratch pointer.
 *   - n_blocks above coset_e8_quant_stats_static_max_blocks() (2^25) is refused with
 *     COSET_E_UNSUPPORTED; nothing is launched.
 *   - The first call on each device looks up the array's device address (no allocation); make
 *     that first call before any stream capture begins on that device.
 *   - All calls on a device share the one array.  Every launch overwrites the records it reads,
 *     so nothing needs clearing between calls, but two calls whose kernels overlap on the GPU
 *     (different streams) race on it: serialise them.
 *   - Calls no cudaMalloc / cudaFree or any allocating library routine.
 */
int64_t coset_e8_quant_stats_static_max_blocks(void);
int coset_e8_quant_stats_static(const void* x, int x_dtype, const float* scale, int scale_mode,
                                int64_t n_blocks, int64_t blocks_per_tile, double* out, void* stream);

/*
 * COSET_SEM_REF: the paper-faithful quantiser ref/hnlq.py (HNLQ.encode, ref/hnlq.py:304-383;
 * HNLQ.decode, ref/hnlq.py:389-445; closest_point_E8 / g_x / custom_round, ref/utils.py:371-537) in
 * float64.  Parity-only.  x, out: [n_blocks, 8] float64; digits: [n_blocks, M, 8] int32;
 * T: [n_blocks] int32 (overload halvings).  dither_host: the 8 float64 added before every
 * closest-point call (the tie dither of ref/utils.py:309-324, or 8 copies of eps when the
 * reference runs with with_tie_dither=False), read on the host.
 */
int coset_e8_ref_encode(const double* x, int64_t n_blocks, double beta, double alpha, int q, int M,
                        int overload, int max_iter, const double* dither_host, int32_t* digits,
                        int32_t* T, void* stream);
int coset_e8_ref_decode(const int32_t* digits, const int32_t* T, int64_t n_blocks, double beta,
                        double alpha, int q, int M, const double* dither_host, double* out,
                        void* stream);
/*
 * HNLQ.decode_coarse_to_fine (ref/hnlq.py:447-507): reconstruction from the `depth` coarsest
 * levels only (levels M-depth .. M-1), 1 <= depth <= M; depth == M equals coset_e8_ref_decode.
 * HNLQ.decode_progressive (ref/hnlq.py:509-536) is this call for depth = 1 .. M.
 */
int coset_e8_ref_decode_coarse(const int32_t* digits, const int32_t* T, int64_t n_blocks,
                               double beta, double alpha, int q, int M, int depth,
                               const double* dither_host, double* out, void* stream);

/*
 * D4 lattice (blocks of 4 values), the reference's second lattice behind the same layer.
 *
 * coset_d4_projection: D4Lattice.projection (coset/core/d4/lattice.py:111-146; g_x at :62-109 with
 *   the same unused flip_negative mask as E8).  x, out: float32 [n_blocks, 4].
 * coset_d4_quantize: weight path of the layer built by create_d4_hnlq_linear
 *   (coset/core/d4/layers.py:15-68; coset/core/layers.py:429-463):
 *   out = clamp(projection(x * scale[tile]) / scale[tile], +-clip) for COSET_SCALE_MUL_TILE,
 *   out = clamp(projection(x), +-clip) for COSET_SCALE_NONE; clip <= 0 disables the clamp.
 *   x / out: float32 or bf16 [n_blocks, 4]; blocks_per_tile counts blocks of 4.
 * coset_d4_fake_quant_bwd: straight-through gradients of that graph (coset/core/layers.py:62-95);
 *   the unclamped forward value is recomputed from w.  grad_beta may be NULL.
 */
int coset_d4_projection(const float* x, int64_t n_blocks, float* out, void* stream);
int coset_d4_quantize(const void* x, int x_dtype, const float* scale, int scale_mode, int64_t n_blocks,
                      int64_t blocks_per_tile, float clip, void* out, int out_dtype, void* stream);
int coset_d4_fake_quant_bwd(const void* grad_out, int grad_dtype, const float* w, const float* beta,
                            int64_t n_blocks, int64_t blocks_per_tile, float clip, float* grad_w,
                            float* grad_beta, void* stream);

/*
 * Babai projection (pub/main.tex, algorithm "Babai projection onto E8"; weight path of
 * ref/qat_auto.py:120-124): z = Ginv x, z_hat = round_half_even(z / step) * step, out = G z_hat.
 * dim = 4 or 8; G_host / Ginv_host: dim x dim float32, row-major, basis vectors as columns
 * (Lattice.G / Lattice.G_inv), read on the host.  x, out: float32 [n_blocks, dim].  Products and
 * sums are rounded separately and accumulated left to right.
 */
int coset_lattice_babai(const float* x, int64_t n_blocks, int dim, const float* G_host,
                        const float* Ginv_host, float step, float* out, void* stream);

/*
 * Code-domain product for MANY tokens on the tcgen05 tensor cores: same result as
 * coset_e8_vlut_gemv (y = x * (decode(codes)/beta)^T + bias) with the weight tile decoded to bf16
 * in shared memory and multiplied by tcgen05.mma with the accumulator in tensor memory.
 *   x_bf16: [T, ldx] bf16, n_in a multiple of 64, ldx a multiple of 8;  y: [T, ldy] float32
 *   status: optional device int, set to 1 if a bounded barrier wait expired (results invalid)
 * Weights are rounded to bf16 before the product (the reference's own quantised layer would be
 * used with float32 weights; tolerance 1e-2 relative as for bf16 activations).
 */
int coset_e8_dequant_gemm(const void* codes, const float* beta, int64_t blocks_per_tile, int n_out, int n_in,
                          const void* x_bf16, int64_t ldx, int T, const float* bias, float* y, int64_t ldy,
                          float clip /* as in coset_e8_vlut_gemv; 0 = none */, int* status, void* stream);

/*
 * The same product in two launches: decode the whole weight to bf16 into `scratch`, then a TMA-fed
 * tcgen05 GEMM on pairs of CTAs (tcgen05.mma.cta_group::2, 256 x 256 x 16 per instruction).  The decode
 * leaves the GEMM's K loop; measured speed equals the fused form's up to 8192 tokens and is a few percent
 * higher beyond.  `scratch` is transient (rewritten
 * by every call, nothing in it has to survive the call); it must hold
 * coset_e8_decode_gemm_scratch_bytes(n_out, n_in) = 2 * n_out * n_in bytes and be 16-byte aligned.
 * Arguments, result and tolerance as for coset_e8_dequant_gemm (the bf16 weights are the same bits);
 * y: [T, ldy] float32 or bf16 (y_dtype), rounded once from the float32 accumulator plus bias.
 * Replaces the dense-weight matmul after a one-off dequantisation, coset/legacy/quant/vlut.py:72-117
 * (`vlut_mac_and_accumulate` over decoded rows); the reference has no tensor-core path.
 */
int64_t coset_e8_decode_gemm_scratch_bytes(int n_out, int n_in);
int coset_e8_decode_gemm(const void* codes, const float* beta, int64_t blocks_per_tile, int n_out, int n_in,
                         const void* x_bf16, int64_t ldx, int T, const float* bias, void* y, int y_dtype,
                         int64_t ldy, float clip, void* scratch, int64_t scratch_bytes, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* COSET_B200_H */
