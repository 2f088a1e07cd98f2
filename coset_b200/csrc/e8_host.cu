// Host-buffer entry points: the codec over arrays that live in host memory.
//
// A context owns a small ring of device staging slots, each with its own stream.  A call cuts the
// input into chunks and issues, per chunk, host->device copy, kernel, device->host copy on the
// slot's stream, so copies of one chunk overlap the kernel and the copies of its neighbours (both
// PCIe directions busy).  Host buffers should be page-locked for the copies to be asynchronous;
// pageable memory works but serialises.  Calls return after all their work has completed.
#include <new>

#include "common.cuh"

using namespace coset;

struct coset_host_ctx {
    int device;
    int64_t chunk_blocks;
    int n_slots;
    struct Slot {
        cudaStream_t stream;
        void* x;       // chunk_blocks * 32 B  (float32 rows; bf16 uses half)
        void* codes;   // chunk_blocks * 32 B  (largest packed code: M=8, 4 B per level)
        float* scale;  // chunk_blocks * 4 B
        void* recon;   // chunk_blocks * 32 B, allocated by the first round-trip call
    } slots[8];
};

namespace {

void destroy(coset_host_ctx* c) {
    if (!c) return;
    for (int i = 0; i < c->n_slots; ++i) {
        if (c->slots[i].x) cudaFree(c->slots[i].x);
        if (c->slots[i].codes) cudaFree(c->slots[i].codes);
        if (c->slots[i].scale) cudaFree(c->slots[i].scale);
        if (c->slots[i].recon) cudaFree(c->slots[i].recon);
        if (c->slots[i].stream) cudaStreamDestroy(c->slots[i].stream);
    }
    delete c;
}

int sync_all(coset_host_ctx* c) {
    int rc = 0;
    for (int i = 0; i < c->n_slots; ++i) {
        int e = check_cuda(cudaStreamSynchronize(c->slots[i].stream), "cudaStreamSynchronize");
        if (e && !rc) rc = e;
    }
    return rc;
}

int64_t chunk_for(const coset_host_ctx* c, int scale_mode, int64_t bpt) {
    int64_t chunk = c->chunk_blocks;
    if (scale_mode == COSET_SCALE_MUL_TILE && bpt > 1) chunk -= chunk % bpt;  // chunks start on tile boundaries
    return chunk;
}

}  // namespace

extern "C" {

int coset_host_ctx_create(int64_t chunk_blocks, int n_slots, coset_host_ctx** out) {
    if (!out) return fail(COSET_E_BADARG, "out is null");
    *out = nullptr;
    if (chunk_blocks < 1 || chunk_blocks > ((int64_t)1 << 28) || n_slots < 1 || n_slots > 8)
        return fail(COSET_E_BADARG, "need 1 <= chunk_blocks <= 2^28 and 1 <= n_slots <= 8");
    coset_host_ctx* c = new (std::nothrow) coset_host_ctx();
    if (!c) return fail(COSET_E_STATE, "out of host memory");
    c->chunk_blocks = chunk_blocks;
    c->n_slots = 0;
    if (int e = check_cuda(cudaGetDevice(&c->device), "cudaGetDevice")) { delete c; return e; }
    for (int i = 0; i < n_slots; ++i) {
        coset_host_ctx::Slot& s = c->slots[i];
        s = {nullptr, nullptr, nullptr, nullptr, nullptr};
        c->n_slots = i + 1;
        cudaError_t e = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaMalloc(&s.x, (size_t)chunk_blocks * 32);
        if (e == cudaSuccess) e = cudaMalloc(&s.codes, (size_t)chunk_blocks * 32);
        if (e == cudaSuccess) e = cudaMalloc((void**)&s.scale, (size_t)chunk_blocks * 4);
        if (e != cudaSuccess) {
            destroy(c);
            return check_cuda(e, "coset_host_ctx_create");
        }
    }
    *out = c;
    return 0;
}

int coset_host_ctx_destroy(coset_host_ctx* ctx) {
    if (!ctx) return 0;
    int rc = sync_all(ctx);
    destroy(ctx);
    return rc;
}

int coset_e8_encode_host(coset_host_ctx* ctx, const void* x_host, int x_dtype, const float* scale_host, int scale_mode,
                         int64_t n_blocks, int64_t blocks_per_tile, int q, int M, void* codes_host) {
    if (!ctx) return fail(COSET_E_BADARG, "ctx is null");
    if (n_blocks < 0 || (n_blocks > 0 && (!x_host || !codes_host))) return fail(COSET_E_BADARG, "bad n_blocks or null buffer");
    int cb = coset_e8_code_bytes(q, M);
    if (!cb) return fail(COSET_E_UNSUPPORTED, "unsupported q=%d M=%d", q, M);
    if (x_dtype != COSET_DTYPE_F32 && x_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown x_dtype");
    if (scale_mode != COSET_SCALE_NONE && !scale_host) return fail(COSET_E_BADARG, "scale_host is null");
    if (scale_mode == COSET_SCALE_MUL_TILE && blocks_per_tile < 1) return fail(COSET_E_BADARG, "blocks_per_tile < 1");
    int64_t chunk = chunk_for(ctx, scale_mode, blocks_per_tile);
    if (chunk < 1) return fail(COSET_E_UNSUPPORTED, "blocks_per_tile exceeds the context's chunk size");
    const size_t row = x_dtype == COSET_DTYPE_F32 ? 32 : 16;
    int rc = 0, k = 0;
    for (int64_t lo = 0; lo < n_blocks && !rc; lo += chunk, ++k) {
        int64_t nb = n_blocks - lo < chunk ? n_blocks - lo : chunk;
        coset_host_ctx::Slot& s = ctx->slots[k % ctx->n_slots];
        rc = check_cuda(cudaMemcpyAsync(s.x, (const char*)x_host + lo * row, nb * row, cudaMemcpyHostToDevice, s.stream), "H2D x");
        if (rc) break;
        if (scale_mode == COSET_SCALE_DIV_SCALAR) {
            rc = check_cuda(cudaMemcpyAsync(s.scale, scale_host, 4, cudaMemcpyHostToDevice, s.stream), "H2D scale");
        } else if (scale_mode == COSET_SCALE_MUL_TILE) {
            int64_t t0 = lo / blocks_per_tile, t1 = (lo + nb + blocks_per_tile - 1) / blocks_per_tile;
            rc = check_cuda(cudaMemcpyAsync(s.scale, scale_host + t0, (t1 - t0) * 4, cudaMemcpyHostToDevice, s.stream), "H2D scale");
        }
        if (rc) break;
        rc = coset_e8_encode(s.x, x_dtype, s.scale, scale_mode, nb, blocks_per_tile, q, M, COSET_SEM_CORE, s.codes, s.stream);
        if (rc) break;
        rc = check_cuda(cudaMemcpyAsync((char*)codes_host + lo * cb, s.codes, nb * cb, cudaMemcpyDeviceToHost, s.stream), "D2H codes");
    }
    int rs = sync_all(ctx);
    return rc ? rc : rs;
}

int coset_e8_decode_host(coset_host_ctx* ctx, const void* codes_host, const float* scale_host, int scale_mode,
                         int64_t n_blocks, int64_t blocks_per_tile, int q, int M, void* out_host, int out_dtype) {
    if (!ctx) return fail(COSET_E_BADARG, "ctx is null");
    if (n_blocks < 0 || (n_blocks > 0 && (!out_host || !codes_host))) return fail(COSET_E_BADARG, "bad n_blocks or null buffer");
    int cb = coset_e8_code_bytes(q, M);
    if (!cb) return fail(COSET_E_UNSUPPORTED, "unsupported q=%d M=%d", q, M);
    if (out_dtype != COSET_DTYPE_F32 && out_dtype != COSET_DTYPE_BF16) return fail(COSET_E_BADARG, "unknown out_dtype");
    if (scale_mode != COSET_SCALE_NONE && !scale_host) return fail(COSET_E_BADARG, "scale_host is null");
    if (scale_mode == COSET_SCALE_MUL_TILE && blocks_per_tile < 1) return fail(COSET_E_BADARG, "blocks_per_tile < 1");
    int64_t chunk = chunk_for(ctx, scale_mode, blocks_per_tile);
    if (chunk < 1) return fail(COSET_E_UNSUPPORTED, "blocks_per_tile exceeds the context's chunk size");
    const size_t row = out_dtype == COSET_DTYPE_F32 ? 32 : 16;
    int rc = 0, k = 0;
    for (int64_t lo = 0; lo < n_blocks && !rc; lo += chunk, ++k) {
        int64_t nb = n_blocks - lo < chunk ? n_blocks - lo : chunk;
        coset_host_ctx::Slot& s = ctx->slots[k % ctx->n_slots];
        rc = check_cuda(cudaMemcpyAsync(s.codes, (const char*)codes_host + lo * cb, nb * cb, cudaMemcpyHostToDevice, s.stream), "H2D codes");
        if (rc) break;
        if (scale_mode == COSET_SCALE_DIV_SCALAR) {
            rc = check_cuda(cudaMemcpyAsync(s.scale, scale_host, 4, cudaMemcpyHostToDevice, s.stream), "H2D scale");
        } else if (scale_mode == COSET_SCALE_MUL_TILE) {
            int64_t t0 = lo / blocks_per_tile, t1 = (lo + nb + blocks_per_tile - 1) / blocks_per_tile;
            rc = check_cuda(cudaMemcpyAsync(s.scale, scale_host + t0, (t1 - t0) * 4, cudaMemcpyHostToDevice, s.stream), "H2D scale");
        }
        if (rc) break;
        rc = coset_e8_decode(s.codes, s.scale, scale_mode, nb, blocks_per_tile, q, M, COSET_SEM_CORE, s.x, out_dtype, s.stream);
        if (rc) break;
        rc = check_cuda(cudaMemcpyAsync((char*)out_host + lo * row, s.x, nb * row, cudaMemcpyDeviceToHost, s.stream), "D2H out");
    }
    int rs = sync_all(ctx);
    return rc ? rc : rs;
}

int coset_e8_quantize_host(coset_host_ctx* ctx, const void* x_host, int x_dtype, const float* scale_host, int scale_mode,
                           int64_t n_blocks, int64_t blocks_per_tile, int q, int M, float clip, void* out_host, int out_dtype,
                           void* codes_host) {
    if (!ctx) return fail(COSET_E_BADARG, "ctx is null");
    if (n_blocks < 0 || (n_blocks > 0 && (!x_host || !out_host))) return fail(COSET_E_BADARG, "bad n_blocks or null buffer");
    int cb = coset_e8_code_bytes(q, M);
    if (!cb) return fail(COSET_E_UNSUPPORTED, "unsupported q=%d M=%d", q, M);
    if ((x_dtype != COSET_DTYPE_F32 && x_dtype != COSET_DTYPE_BF16) || (out_dtype != COSET_DTYPE_F32 && out_dtype != COSET_DTYPE_BF16))
        return fail(COSET_E_BADARG, "unknown dtype");
    if (scale_mode != COSET_SCALE_NONE && !scale_host) return fail(COSET_E_BADARG, "scale_host is null");
    if (scale_mode == COSET_SCALE_MUL_TILE && blocks_per_tile < 1) return fail(COSET_E_BADARG, "blocks_per_tile < 1");
    int64_t chunk = chunk_for(ctx, scale_mode, blocks_per_tile);
    if (chunk < 1) return fail(COSET_E_UNSUPPORTED, "blocks_per_tile exceeds the context's chunk size");
    for (int i = 0; i < ctx->n_slots; ++i) {
        if (!ctx->slots[i].recon) {
            if (int e = check_cuda(cudaMalloc(&ctx->slots[i].recon, (size_t)ctx->chunk_blocks * 32), "cudaMalloc(round-trip staging)")) return e;
        }
    }
    const size_t row_in = x_dtype == COSET_DTYPE_F32 ? 32 : 16, row_out = out_dtype == COSET_DTYPE_F32 ? 32 : 16;
    int rc = 0, k = 0;
    for (int64_t lo = 0; lo < n_blocks && !rc; lo += chunk, ++k) {
        int64_t nb = n_blocks - lo < chunk ? n_blocks - lo : chunk;
        coset_host_ctx::Slot& s = ctx->slots[k % ctx->n_slots];
        rc = check_cuda(cudaMemcpyAsync(s.x, (const char*)x_host + lo * row_in, nb * row_in, cudaMemcpyHostToDevice, s.stream), "H2D x");
        if (rc) break;
        if (scale_mode == COSET_SCALE_DIV_SCALAR) {
            rc = check_cuda(cudaMemcpyAsync(s.scale, scale_host, 4, cudaMemcpyHostToDevice, s.stream), "H2D scale");
        } else if (scale_mode == COSET_SCALE_MUL_TILE) {
            int64_t t0 = lo / blocks_per_tile, t1 = (lo + nb + blocks_per_tile - 1) / blocks_per_tile;
            rc = check_cuda(cudaMemcpyAsync(s.scale, scale_host + t0, (t1 - t0) * 4, cudaMemcpyHostToDevice, s.stream), "H2D scale");
        }
        if (rc) break;
        rc = coset_e8_quantize(s.x, x_dtype, s.scale, scale_mode, nb, blocks_per_tile, q, M, clip, s.recon, out_dtype,
                               codes_host ? s.codes : nullptr, s.stream);
        if (rc) break;
        rc = check_cuda(cudaMemcpyAsync((char*)out_host + lo * row_out, s.recon, nb * row_out, cudaMemcpyDeviceToHost, s.stream), "D2H out");
        if (rc) break;
        if (codes_host)
            rc = check_cuda(cudaMemcpyAsync((char*)codes_host + lo * cb, s.codes, nb * cb, cudaMemcpyDeviceToHost, s.stream), "D2H codes");
    }
    int rs = sync_all(ctx);
    return rc ? rc : rs;
}

}  // extern "C"
