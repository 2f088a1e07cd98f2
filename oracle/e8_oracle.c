/*
 * CPU restatement of coset's E8 hierarchical nested-lattice codec ("core" semantics).
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker for the CUDA library: it is
 * compiled to oracle/_build/libe8_oracle.so and may be loaded by tests/, by
 * __graft_entry__.smoke() and by bench.py's CPU-baseline legs -- never by the product path.
 *
 * Parity status: PINNED.  Every function below is checked bit-for-bit against the unmodified
 * reference (imported from its source tree) through the golden vectors in tests/golden/
 * (generator: tests/golden/make_golden.py).
 *
 * All arithmetic is IEEE binary32 with one rounding per operation and no fused multiply-add
 * (build with -ffp-contract=off, no -ffast-math), because the reference runs op-by-op in
 * torch float32 on the CPU.
 *
 * Reference files followed (paths inside the reference project):
 *   coset/core/base.py:134-154      Lattice.encode_coords
 *   coset/core/base.py:156-176      Lattice.decode_coords
 *   coset/core/base.py:179-202      Lattice.custom_round
 *   coset/core/e8/lattice.py:32-41  generator matrix G
 *   coset/core/e8/lattice.py:67-112 E8Lattice.g_x
 *   coset/core/e8/lattice.py:114-169 E8Lattice.projection
 *   coset/core/e8/codecs.py:63-89   e8_encode
 *   coset/core/e8/codecs.py:159-180 E8Decoder._full_decode
 *   coset/core/e8/codecs.py:245-260 e8_quantize
 *   coset/core/layers.py:415-463    HNLQLinearQAT._quantize_weights
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define E8_D 8

/* G: columns are the E8 basis vectors (coset/core/e8/lattice.py:32-41, note the .T). */
static const float G[8][8] = {
    {2, -1, 0, 0, 0, 0, 0, 0.5f},
    {0, 1, -1, 0, 0, 0, 0, 0.5f},
    {0, 0, 1, -1, 0, 0, 0, 0.5f},
    {0, 0, 0, 1, -1, 0, 0, 0.5f},
    {0, 0, 0, 0, 1, -1, 0, 0.5f},
    {0, 0, 0, 0, 0, 1, -1, 0.5f},
    {0, 0, 0, 0, 0, 0, 1, 0.5f},
    {0, 0, 0, 0, 0, 0, 0, 0.5f},
};
/* G^-1 as torch.linalg.inv returns it in float32 (exact; checked by the golden test). */
static const float GINV[8][8] = {
    {0.5f, 0.5f, 0.5f, 0.5f, 0.5f, 0.5f, 0.5f, -3.5f},
    {0, 1, 1, 1, 1, 1, 1, -6},
    {0, 0, 1, 1, 1, 1, 1, -5},
    {0, 0, 0, 1, 1, 1, 1, -4},
    {0, 0, 0, 0, 1, 1, 1, -3},
    {0, 0, 0, 0, 0, 1, 1, -2},
    {0, 0, 0, 0, 0, 0, 1, -1},
    {0, 0, 0, 0, 0, 0, 0, 2},
};

void e8o_generators(float* g_out, float* ginv_out) {
    memcpy(g_out, G, sizeof(G));
    memcpy(ginv_out, GINV, sizeof(GINV));
}

/* coset/core/base.py:179-202: y = x - sign(x)*eps32; floor(y + 0.5); two rounded adds. */
float e8o_custom_round(float x) {
    const float eps = 1.1920928955078125e-07f; /* torch.finfo(float32).eps = 2^-23 */
    float s = (x > 0.0f) ? 1.0f : ((x < 0.0f) ? -1.0f : x * 0.0f); /* sign(+-0)=0, sign(nan)=nan */
    float nudge = s * eps;
    float y = x - nudge;
    float t = y + 0.5f;
    return floorf(t);
}

/* First index of the maximum; torch.argmax treats NaN as the maximum. */
static int argmax_first(const float* v) {
    int k = 0;
    float best = v[0];
    if (best != best) return 0;
    for (int i = 1; i < E8_D; ++i) {
        if (v[i] != v[i]) return i;
        if (v[i] > best) { best = v[i]; k = i; }
    }
    return k;
}

/* coset/core/e8/lattice.py:67-112.  Only `flip_positive` selects +1; every other row gets -1. */
void e8o_g_x(const float* x, float* out) {
    float f[E8_D], delta[E8_D];
    for (int i = 0; i < E8_D; ++i) {
        f[i] = e8o_custom_round(x[i]);
        delta[i] = fabsf(x[i] - f[i]);
        out[i] = f[i];
    }
    int k = argmax_first(delta);
    int flip_positive = (x[k] >= 0.0f) && (f[k] < x[k]);
    if (flip_positive) out[k] = out[k] + 1.0f; else out[k] = out[k] - 1.0f;
}

/* torch.norm(v, dim=-1) over 8 contiguous float32: sqrt of the left-to-right float32 sum of
 * separately rounded squares (pinned by the golden vectors). */
static float norm8(const float* v) {
    float acc = 0.0f;
    for (int i = 0; i < E8_D; ++i) {
        float sq = v[i] * v[i];
        acc = acc + sq;
    }
    return sqrtf(acc);
}

/* python/torch `%` on floats: floored remainder, keeps -0.0 for negative exact multiples. */
static float floored_mod(float a, float m) {
    float r = fmodf(a, m);
    if (r != 0.0f && ((r < 0.0f) != (m < 0.0f))) r = r + m;
    return r;
}

/* coset/core/e8/lattice.py:114-169 */
void e8o_projection(const float* x, float* out) {
    float f0[E8_D], g0[E8_D], xs[E8_D], f1[E8_D], g1[E8_D], y0[E8_D], y1[E8_D], e0[E8_D], e1[E8_D];
    float sum0 = 0.0f, sum1 = 0.0f;
    for (int i = 0; i < E8_D; ++i) { f0[i] = e8o_custom_round(x[i]); sum0 = sum0 + f0[i]; }
    e8o_g_x(x, g0);
    int even0 = floored_mod(sum0, 2.0f) == 0.0f;
    for (int i = 0; i < E8_D; ++i) y0[i] = even0 ? f0[i] : g0[i];

    for (int i = 0; i < E8_D; ++i) { xs[i] = x[i] - 0.5f; f1[i] = e8o_custom_round(xs[i]); sum1 = sum1 + f1[i]; }
    e8o_g_x(xs, g1);
    int even1 = floored_mod(sum1, 2.0f) == 0.0f;
    for (int i = 0; i < E8_D; ++i) y1[i] = (even1 ? f1[i] : g1[i]) + 0.5f;

    for (int i = 0; i < E8_D; ++i) { e0[i] = x[i] - y0[i]; e1[i] = x[i] - y1[i]; }
    float d0 = norm8(e0), d1 = norm8(e1);
    int closer0 = d0 < d1;
    for (int i = 0; i < E8_D; ++i) out[i] = closer0 ? y0[i] : y1[i];
}

/* coset/core/base.py:134-154: round(G^-1 p) % q (float digits; may be -0.0). */
void e8o_encode_coords(const float* p, int q, float* out) {
    for (int j = 0; j < E8_D; ++j) {
        float acc = 0.0f;
        for (int i = 0; i < E8_D; ++i) { float t = GINV[j][i] * p[i]; acc = acc + t; }
        out[j] = floored_mod(rintf(acc), (float)q);
    }
}

/* coset/core/base.py:156-176: G b */
void e8o_decode_coords(const float* b, float* out) {
    for (int j = 0; j < E8_D; ++j) {
        float acc = 0.0f;
        for (int i = 0; i < E8_D; ++i) { float t = G[j][i] * b[i]; acc = acc + t; }
        out[j] = acc;
    }
}

/* One block of coset/core/e8/codecs.py:63-83 after scaling. codes: [M][8] float digits. */
static void encode_block(const float* xs, int q, int M, float* codes) {
    float xl[E8_D], p[E8_D];
    float qf = (float)q;
    memcpy(xl, xs, sizeof(xl));
    for (int m = 0; m < M; ++m) {
        e8o_projection(xl, p);
        e8o_encode_coords(p, q, codes + m * E8_D);
        for (int i = 0; i < E8_D; ++i) xl[i] = xl[i] / qf;
    }
}

/* One block of coset/core/e8/codecs.py:159-172 (before the final *beta). */
static void decode_block(const float* codes, int q, int M, float* xhat) {
    float qf = (float)q;
    float w = 1.0f;
    for (int i = 0; i < E8_D; ++i) xhat[i] = 0.0f;
    for (int m = 0; m < M; ++m) {
        float gb[E8_D], s[E8_D], pr[E8_D];
        e8o_decode_coords(codes + m * E8_D, gb);
        for (int i = 0; i < E8_D; ++i) s[i] = gb[i] / qf;
        e8o_projection(s, pr);
        for (int i = 0; i < E8_D; ++i) {
            float xi = gb[i] - qf * pr[i];
            xhat[i] = xhat[i] + w * xi;
        }
        w = w * qf; /* q**i is an exact python int; exact in float32 for the sizes used */
    }
}

/*
 * e8_encode (coset/core/e8/codecs.py:17-89).
 * scale_mode 0: x used as is;  1: x / beta[0] (codec convention, codecs.py:64);
 *            2: x * beta[block / blocks_per_tile] (layer convention, core/layers.py:431/435,
 *               blocks_per_tile = blocks per weight row for tiling='row', 1 for tiling='block').
 * codes: [n][M][8] float32 digits exactly as the reference returns them.
 */
void e8o_encode(const float* x, int64_t n, const float* beta, int scale_mode,
                int64_t blocks_per_tile, int q, int M, float* codes) {
    for (int64_t b = 0; b < n; ++b) {
        float xs[E8_D];
        for (int i = 0; i < E8_D; ++i) {
            float v = x[b * E8_D + i];
            if (scale_mode == 1) v = v / beta[0];
            else if (scale_mode == 2) v = v * beta[b / blocks_per_tile];
            xs[i] = v;
        }
        encode_block(xs, q, M, codes + b * M * E8_D);
    }
}

/*
 * e8_decode (coset/core/e8/codecs.py:139-180).
 * scale_mode 0: none; 1: * beta[0] (codecs.py:175); 2: / beta[tile] (core/layers.py:455/460).
 */
void e8o_decode(const float* codes, int64_t n, const float* beta, int scale_mode,
                int64_t blocks_per_tile, int q, int M, float* xhat) {
    for (int64_t b = 0; b < n; ++b) {
        float xh[E8_D];
        decode_block(codes + b * M * E8_D, q, M, xh);
        for (int i = 0; i < E8_D; ++i) {
            float v = xh[i];
            if (scale_mode == 1) v = v * beta[0];
            else if (scale_mode == 2) v = v / beta[b / blocks_per_tile];
            xhat[b * E8_D + i] = v;
        }
    }
}

/* e8_quantize (coset/core/e8/codecs.py:221-286): M is hard-wired to 2, beta to 1. */
void e8o_quantize(const float* x, int64_t n, int q, float* out) {
    for (int64_t b = 0; b < n; ++b) {
        float codes[2 * E8_D];
        encode_block(x + b * E8_D, q, 2, codes);
        decode_block(codes, q, 2, out + b * E8_D);
    }
}

/*
 * Weight fake-quantisation of HNLQLinearQAT._quantize_weights (coset/core/layers.py:429-463):
 * clamp(e8_quantize(W * beta) / beta, -clip, clip).  `unclipped` (optional) receives the value
 * before the clamp, which the backward pass needs for the clamp mask and for d/dbeta.
 */
void e8o_fake_quant(const float* w, int64_t n, const float* beta, int64_t blocks_per_tile,
                    int q, float clip, float* wq, float* unclipped) {
    for (int64_t b = 0; b < n; ++b) {
        float xs[E8_D], codes[2 * E8_D], xh[E8_D];
        float bt = beta[b / blocks_per_tile];
        for (int i = 0; i < E8_D; ++i) xs[i] = w[b * E8_D + i] * bt;
        encode_block(xs, q, 2, codes);
        decode_block(codes, q, 2, xh);
        for (int i = 0; i < E8_D; ++i) {
            float v = xh[i] / bt;
            if (unclipped) unclipped[b * E8_D + i] = v;
            float c = v < -clip ? -clip : (v > clip ? clip : v);
            if (v != v) c = v;
            wq[b * E8_D + i] = c;
        }
    }
}

/* Packed fast format of the CUDA library: 2 bits per digit, digit j of level m at bit
 * 16*m + 2*j (q <= 4, M <= 2). */
void e8o_pack_q4(const float* codes, int64_t n, int M, uint32_t* packed) {
    for (int64_t b = 0; b < n; ++b) {
        uint32_t w = 0;
        for (int m = 0; m < M; ++m)
            for (int j = 0; j < E8_D; ++j)
                w |= ((uint32_t)((int)codes[(b * M + m) * E8_D + j]) & 3u) << (16 * m + 2 * j);
        packed[b] = w;
    }
}

/* Multi-threaded wrappers over contiguous block ranges (pthreads); used to time the CPU
 * baseline on all host cores. */
#include <pthread.h>
typedef struct {
    int is_decode;
    const float* in; float* out; const float* beta;
    int scale_mode; int64_t blocks_per_tile; int q; int M; int64_t lo, hi;
} e8o_job;

static void* e8o_worker(void* arg) {
    e8o_job* j = (e8o_job*)arg;
    for (int64_t b = j->lo; b < j->hi; ++b) {
        const float* bp = j->beta;
        int64_t bpt = j->blocks_per_tile;
        if (j->scale_mode == 2) { bp = j->beta + b / j->blocks_per_tile; bpt = 1; }
        if (j->is_decode)
            e8o_decode(j->in + b * j->M * E8_D, 1, bp, j->scale_mode, bpt, j->q, j->M, j->out + b * E8_D);
        else
            e8o_encode(j->in + b * E8_D, 1, bp, j->scale_mode, bpt, j->q, j->M, j->out + b * j->M * E8_D);
    }
    return 0;
}

static void e8o_run_mt(int is_decode, const float* in, int64_t n, const float* beta, int scale_mode,
                       int64_t blocks_per_tile, int q, int M, float* out, int threads) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    pthread_t tid[256];
    e8o_job jobs[256];
    int64_t per = (n + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        int64_t lo = t * per, hi = lo + per;
        if (lo > n) lo = n;
        if (hi > n) hi = n;
        e8o_job j = {is_decode, in, out, beta, scale_mode, blocks_per_tile, q, M, lo, hi};
        jobs[t] = j;
        pthread_create(&tid[t], 0, e8o_worker, &jobs[t]);
    }
    for (int t = 0; t < threads; ++t) pthread_join(tid[t], 0);
}

void e8o_encode_mt(const float* x, int64_t n, const float* beta, int scale_mode,
                   int64_t blocks_per_tile, int q, int M, float* codes, int threads) {
    e8o_run_mt(0, x, n, beta, scale_mode, blocks_per_tile, q, M, codes, threads);
}
void e8o_decode_mt(const float* codes, int64_t n, const float* beta, int scale_mode,
                   int64_t blocks_per_tile, int q, int M, float* xhat, int threads) {
    e8o_run_mt(1, codes, n, beta, scale_mode, blocks_per_tile, q, M, xhat, threads);
}

/* =============================================================================================
 * "ref" semantics: the paper-faithful per-vector quantiser ref/hnlq.py (numpy, float64).
 * Differences from the core codec, all reproduced here: correct g_x flip rule
 * (ref/utils.py:415-455), a constant tie-dither vector added before EVERY closest-point call
 * (ref/hnlq.py:173-179, ref/utils.py:309-324), re-quantising recurrence x_l <- Q(x_l) before the
 * digits and the division (ref/hnlq.py:335-339), digits custom_round(mod(G^-1 x, q))
 * (ref/hnlq.py:337), overload loop x <- x / 2^alpha (ref/hnlq.py:369-379), reconstruction scaled
 * by 2^(alpha T) (ref/hnlq.py:445).  Parity: pinned by tests/golden/ref_mode.npz.
 * ============================================================================================= */
static double r_custom_round(double x) { /* ref/utils.py:371-412 with float64 eps */
    const double eps = 2.220446049250313e-16;
    double s = (x > 0.0) ? 1.0 : ((x < 0.0) ? -1.0 : x * 0.0);
    double y = x - s * eps;
    return floor(y + 0.5);
}

static void r_g_x(const double* x, double* out) { /* ref/utils.py:415-455 */
    double f[8], best = -1.0;
    int k = 0;
    for (int i = 0; i < 8; ++i) {
        f[i] = r_custom_round(x[i]);
        out[i] = f[i];
        double dlt = fabs(x[i] - f[i]);
        if (dlt > best) { best = dlt; k = i; }
    }
    if (x[k] >= 0.0) out[k] = (f[k] < x[k]) ? f[k] + 1.0 : f[k] - 1.0;
    else out[k] = (f[k] <= x[k]) ? f[k] + 1.0 : f[k] - 1.0;
}

static double r_fmod_floor(double a, double m) {
    double r = fmod(a, m);
    if (r != 0.0 && ((r < 0.0) != (m < 0.0))) r += m;
    return r;
}

static void r_closest_e8(const double* x, double* out) { /* ref/utils.py:494-537 */
    double f0[8], g0[8], xs[8], f1[8], g1[8], y0[8], y1[8], s0 = 0.0, s1 = 0.0, d0 = 0.0, d1 = 0.0;
    for (int i = 0; i < 8; ++i) { f0[i] = r_custom_round(x[i]); s0 += f0[i]; }
    r_g_x(x, g0);
    int e0 = r_fmod_floor(s0, 2.0) == 0.0;
    for (int i = 0; i < 8; ++i) { xs[i] = x[i] - 0.5; f1[i] = r_custom_round(xs[i]); s1 += f1[i]; }
    r_g_x(xs, g1);
    int e1 = r_fmod_floor(s1, 2.0) == 0.0;
    for (int i = 0; i < 8; ++i) {
        y0[i] = e0 ? f0[i] : g0[i];
        y1[i] = (e1 ? f1[i] : g1[i]) + 0.5;
        d0 += (x[i] - y0[i]) * (x[i] - y0[i]);
        d1 += (x[i] - y1[i]) * (x[i] - y1[i]);
    }
    int c0 = sqrt(d0) < sqrt(d1);
    for (int i = 0; i < 8; ++i) out[i] = c0 ? y0[i] : y1[i];
}

static void r_qnn(const double* x, const double* dither, double* out) { /* ref/hnlq.py:179 */
    double t[8];
    for (int i = 0; i < 8; ++i) t[i] = x[i] + dither[i];
    r_closest_e8(t, out);
}

static int r_encode_once(const double* x, double beta, int q, int M, const double* dither, int32_t* digits) {
    double xl[8], p[8];
    for (int i = 0; i < 8; ++i) xl[i] = x[i] / beta;
    for (int m = 0; m < M; ++m) { /* ref/hnlq.py:335-339 */
        r_qnn(xl, dither, p);
        for (int j = 0; j < 8; ++j) {
            double acc = 0.0;
            for (int i = 0; i < 8; ++i) acc += (double)GINV[j][i] * p[i];
            digits[m * 8 + j] = (int32_t)r_custom_round(r_fmod_floor(acc, (double)q));
        }
        for (int i = 0; i < 8; ++i) xl[i] = p[i] / (double)q;
    }
    r_qnn(xl, dither, p); /* overload test, ref/hnlq.py:341: not allclose(Q(x_l), 0, atol=1e-8) */
    int over = 0;
    for (int i = 0; i < 8; ++i) over |= !(fabs(p[i]) <= 1e-8);
    return over;
}

/* HNLQ.encode (ref/hnlq.py:344-383). x: [n][8] float64; digits: [n][M][8]; T: [n]. */
void e8o_ref_encode(const double* x, int64_t n, double beta, double alpha, int q, int M, int overload,
                    int max_iter, const double* dither, int32_t* digits, int32_t* T) {
    double scale = pow(2.0, alpha);
    for (int64_t b = 0; b < n; ++b) {
        double xv[8];
        for (int i = 0; i < 8; ++i) xv[i] = x[b * 8 + i];
        int32_t* dg = digits + b * M * 8;
        int over = r_encode_once(xv, beta, q, M, dither, dg);
        int t = 0;
        if (overload) {
            while (over && t < max_iter) {
                t += 1;
                for (int i = 0; i < 8; ++i) xv[i] = xv[i] / scale;
                over = r_encode_once(xv, beta, q, M, dither, dg);
            }
        }
        T[b] = t;
    }
}

/* HNLQ.decode_coarse_to_fine (ref/hnlq.py:447-507): the `depth` coarsest levels only, i.e. levels
 * M-depth .. M-1; depth == M is HNLQ.decode (ref/hnlq.py:389-445).  Every term is an exact multiple
 * of 1/2 far below 2^53, so the reference's summation order (coarsest first) and this one agree.
 * out: [n][8] float64. */
void e8o_ref_decode_depth(const int32_t* digits, const int32_t* T, int64_t n, double beta, double alpha, int q, int M,
                          int depth, const double* dither, double* out) {
    for (int64_t b = 0; b < n; ++b) {
        double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, w = 1.0;
        for (int m = 0; m < M; ++m) {
            if (m >= M - depth) {
                double gb[8], s[8], pr[8];
                for (int j = 0; j < 8; ++j) {
                    double a = 0.0;
                    for (int i = 0; i < 8; ++i) a += (double)G[j][i] * (double)digits[(b * M + m) * 8 + i];
                    gb[j] = a;
                    s[j] = a / (double)q;
                }
                r_qnn(s, dither, pr);
                for (int j = 0; j < 8; ++j) acc[j] = acc[j] + w * (gb[j] - (double)q * pr[j]);
            }
            w *= (double)q;
        }
        double up = pow(2.0, alpha * (double)T[b]);
        for (int j = 0; j < 8; ++j) out[b * 8 + j] = (beta * acc[j]) * up;
    }
}

/* HNLQ.decode (ref/hnlq.py:389-445). out: [n][8] float64. */
void e8o_ref_decode(const int32_t* digits, const int32_t* T, int64_t n, double beta, double alpha, int q, int M,
                    const double* dither, double* out) {
    e8o_ref_decode_depth(digits, T, n, beta, alpha, q, M, M, dither, out);
}
