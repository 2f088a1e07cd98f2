// "ref" semantics: the paper-faithful quantiser of ref/hnlq.py in float64, one thread per vector.
// Parity-only path (not tuned, not timed): correct g_x flip rule (ref/utils.py:415-455), constant
// tie dither before every closest-point call (ref/hnlq.py:173-179), re-quantising recurrence
// (ref/hnlq.py:335-339), overload loop (ref/hnlq.py:369-379), 2^(alpha T) rescale (ref/hnlq.py:445).
// Compiled without FMA contraction; every operation rounds once, as numpy does.
#include "common.cuh"

using namespace coset;

namespace {

constexpr int kThreads = 128;

struct RefParams {
    double dither[8];
    double beta, alpha, pow2alpha;
    int q, M, overload, max_iter;
};

__device__ __forceinline__ double r_custom_round(double x) {
    const double eps = 2.220446049250313e-16;
    double s = (x > 0.0) ? 1.0 : ((x < 0.0) ? -1.0 : __dmul_rn(x, 0.0));
    double y = __dsub_rn(x, __dmul_rn(s, eps));
    return floor(__dadd_rn(y, 0.5));
}

__device__ __forceinline__ double r_fmod_floor(double a, double m) {
    double r = fmod(a, m);
    if (r != 0.0 && ((r < 0.0) != (m < 0.0))) r = __dadd_rn(r, m);
    return r;
}

__device__ void r_g_x(const double (&x)[8], double (&out)[8]) {
    double best = -1.0, xk = 0.0, fk = 0.0;
    int k = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        out[i] = r_custom_round(x[i]);
        double dlt = fabs(__dsub_rn(x[i], out[i]));
        if (dlt > best) { best = dlt; k = i; xk = x[i]; fk = out[i]; }
    }
    bool up = (xk >= 0.0) ? (fk < xk) : (fk <= xk);
    double nv = up ? __dadd_rn(fk, 1.0) : __dsub_rn(fk, 1.0);
#pragma unroll
    for (int i = 0; i < 8; ++i) if (i == k) out[i] = nv;
}

__device__ void r_closest_e8(const double (&x)[8], double (&out)[8]) {
    double y0[8], y1[8], xs[8], s0 = 0.0, s1 = 0.0, d0 = 0.0, d1 = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) { y0[i] = r_custom_round(x[i]); s0 = __dadd_rn(s0, y0[i]); }
    if (r_fmod_floor(s0, 2.0) != 0.0) r_g_x(x, y0);
#pragma unroll
    for (int i = 0; i < 8; ++i) { xs[i] = __dsub_rn(x[i], 0.5); y1[i] = r_custom_round(xs[i]); s1 = __dadd_rn(s1, y1[i]); }
    if (r_fmod_floor(s1, 2.0) != 0.0) r_g_x(xs, y1);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        y1[i] = __dadd_rn(y1[i], 0.5);
        double e0 = __dsub_rn(x[i], y0[i]), e1 = __dsub_rn(x[i], y1[i]);
        d0 = __dadd_rn(d0, __dmul_rn(e0, e0));
        d1 = __dadd_rn(d1, __dmul_rn(e1, e1));
    }
    bool c0 = __dsqrt_rn(d0) < __dsqrt_rn(d1);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = c0 ? y0[i] : y1[i];
}

__device__ void r_qnn(const double (&x)[8], const RefParams& p, double (&out)[8]) {
    double t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = __dadd_rn(x[i], p.dither[i]);
    r_closest_e8(t, out);
}

// G^-1 y for the E8 generator (suffix-sum structure; exact for lattice points)
__device__ __forceinline__ void r_ginv(const double (&y)[8], double (&z)[8]) {
    double s = 0.0;
    z[7] = __dmul_rn(2.0, y[7]);
#pragma unroll
    for (int j = 6; j >= 1; --j) {
        s = __dadd_rn(s, y[j]);
        z[j] = __dsub_rn(s, __dmul_rn((double)(7 - j), y[7]));
    }
    s = __dadd_rn(s, y[0]);
    z[0] = __dmul_rn(0.5, __dsub_rn(s, __dmul_rn(7.0, y[7])));
}

__device__ bool r_encode_once(const double (&x)[8], const RefParams& p, int32_t* digits) {
    double xl[8], y[8], z[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) xl[i] = __ddiv_rn(x[i], p.beta);
    for (int m = 0; m < p.M; ++m) {
        r_qnn(xl, p, y);
        r_ginv(y, z);
#pragma unroll
        for (int j = 0; j < 8; ++j) digits[m * 8 + j] = (int32_t)r_custom_round(r_fmod_floor(z[j], (double)p.q));
#pragma unroll
        for (int i = 0; i < 8; ++i) xl[i] = __ddiv_rn(y[i], (double)p.q);
    }
    r_qnn(xl, p, y);
    bool over = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) over = over || !(fabs(y[i]) <= 1e-8);
    return over;
}

__global__ void __launch_bounds__(kThreads) k_ref_encode(const double* __restrict__ x, int64_t n, RefParams p,
                                                         int32_t* __restrict__ digits, int32_t* __restrict__ T) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    double xv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) xv[i] = x[b * 8 + i];
    int32_t* dg = digits + b * p.M * 8;
    bool over = r_encode_once(xv, p, dg);
    int t = 0;
    if (p.overload) {
        while (over && t < p.max_iter) {
            t += 1;
#pragma unroll
            for (int i = 0; i < 8; ++i) xv[i] = __ddiv_rn(xv[i], p.pow2alpha);
            over = r_encode_once(xv, p, dg);
        }
    }
    T[b] = t;
}

__global__ void __launch_bounds__(kThreads) k_ref_decode(const int32_t* __restrict__ digits, const int32_t* __restrict__ T,
                                                         int64_t n, RefParams p, int first_level,
                                                         double* __restrict__ out) {
    int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n) return;
    double acc[8], w = 1.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0;
    for (int m = 0; m < p.M; ++m) {
        if (m < first_level) {  // coarse-to-fine: the finest levels are left out, their weight still advances
            w = __dmul_rn(w, (double)p.q);
            continue;
        }
        const int32_t* d = digits + (b * p.M + m) * 8;
        double gb[8], s[8], pr[8];
        double hb = __dmul_rn(0.5, (double)d[7]);
        gb[0] = __dadd_rn((double)(2 * d[0] - d[1]), hb);
#pragma unroll
        for (int i = 1; i <= 5; ++i) gb[i] = __dadd_rn((double)(d[i] - d[i + 1]), hb);
        gb[6] = __dadd_rn((double)d[6], hb);
        gb[7] = hb;
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] = __ddiv_rn(gb[i], (double)p.q);
        r_qnn(s, p, pr);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = __dadd_rn(acc[i], __dmul_rn(w, __dsub_rn(gb[i], __dmul_rn((double)p.q, pr[i]))));
        w = __dmul_rn(w, (double)p.q);
    }
    double e = __dmul_rn(p.alpha, (double)T[b]);
    double up = (e == floor(e) && fabs(e) < 1000.0) ? scalbn(1.0, (int)e) : pow(2.0, e);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[b * 8 + i] = __dmul_rn(__dmul_rn(p.beta, acc[i]), up);
}

int fill(RefParams& p, double beta, double alpha, int q, int M, int overload, int max_iter, const double* dither_host) {
    if (q < 2 || q > 256 || M < 1 || M > 8) return fail(COSET_E_UNSUPPORTED, "ref mode needs 2 <= q <= 256, 1 <= M <= 8");
    if (!(beta > 0.0) || !(alpha > 0.0) || max_iter < 0 || !dither_host) return fail(COSET_E_BADARG, "bad beta / alpha / max_iter / dither");
    for (int i = 0; i < 8; ++i) p.dither[i] = dither_host[i];
    p.beta = beta; p.alpha = alpha; p.pow2alpha = pow(2.0, alpha);
    p.q = q; p.M = M; p.overload = overload; p.max_iter = max_iter;
    return 0;
}

}  // namespace

extern "C" {

int coset_e8_ref_encode(const double* x, int64_t n_blocks, double beta, double alpha, int q, int M, int overload,
                        int max_iter, const double* dither_host, int32_t* digits, int32_t* T, void* stream) {
    RefParams p;
    if (int e = fill(p, beta, alpha, q, M, overload, max_iter, dither_host)) return e;
    if (n_blocks < 0) return fail(COSET_E_BADARG, "n_blocks is negative");
    if (n_blocks == 0) return 0;
    if (!x || !digits || !T) return fail(COSET_E_BADARG, "null pointer");
    k_ref_encode<<<(unsigned)((n_blocks + kThreads - 1) / kThreads), kThreads, 0, (cudaStream_t)stream>>>(x, n_blocks, p, digits, T);
    return check_launch("e8_ref_encode");
}

int coset_e8_ref_decode_coarse(const int32_t* digits, const int32_t* T, int64_t n_blocks, double beta, double alpha, int q,
                               int M, int depth, const double* dither_host, double* out, void* stream) {
    RefParams p;
    if (int e = fill(p, beta, alpha, q, M, 0, 0, dither_host)) return e;
    if (depth < 1 || depth > M) return fail(COSET_E_BADARG, "depth must be between 1 and M");
    if (n_blocks < 0) return fail(COSET_E_BADARG, "n_blocks is negative");
    if (n_blocks == 0) return 0;
    if (!digits || !T || !out) return fail(COSET_E_BADARG, "null pointer");
    k_ref_decode<<<(unsigned)((n_blocks + kThreads - 1) / kThreads), kThreads, 0, (cudaStream_t)stream>>>(digits, T, n_blocks, p, M - depth, out);
    return check_launch("e8_ref_decode");
}

int coset_e8_ref_decode(const int32_t* digits, const int32_t* T, int64_t n_blocks, double beta, double alpha, int q, int M,
                        const double* dither_host, double* out, void* stream) {
    return coset_e8_ref_decode_coarse(digits, T, n_blocks, beta, alpha, q, M, M, dither_host, out, stream);
}

}  // extern "C"
