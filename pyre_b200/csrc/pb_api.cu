// C ABI: context and quantized-matrix entry points (include/pyre_b200.h).
#include "pb_formats.cuh"
#include "pb_common.cuh"
#include "pb_internal.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <new>
#include <pthread.h>

static const char* kNoCtx = "pyre_b200: null context";

int pb_enter(pb_ctx* ctx) {
    if (!ctx) return PB_ERR_ARG;
    // the reference's worker loads the model and makes every call on one thread (src/engine_qn.rs:13-17);
    // PYRE_B200_CHECK_THREAD=1 turns a call from another thread into an error instead of undefined behaviour
    if (ctx->check_thread && (unsigned long)pthread_self() != ctx->owner_thread) PB_FAIL(ctx, PB_ERR_STATE, "context used from a thread other than the one that created it");
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != ctx->device) PB_CUDA(ctx, cudaSetDevice(ctx->device));
    return PB_OK;
}

unsigned long long* pb_stamp_slot(pb_ctx* ctx, int kernel_id) {
    if (!ctx->stamps || ctx->stamp_next >= ctx->stamp_slots) return nullptr;
    ctx->stamp_ids[ctx->stamp_next] = kernel_id;
    return ctx->stamps + (size_t)PB_STAMP_WORDS * ctx->stamp_next++;
}

int pb_scratch(pb_ctx* ctx, size_t bytes, void** out) {
    if (bytes > ctx->scratch_bytes) {
        PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->scratch) cudaFree(ctx->scratch);
        ctx->scratch = nullptr; ctx->scratch_bytes = 0;
        const size_t want = (bytes + ((size_t)1 << 20)) & ~(((size_t)1 << 20) - 1);
        PB_CUDA(ctx, cudaMalloc(&ctx->scratch, want));
        ctx->scratch_bytes = want;
    }
    *out = ctx->scratch;
    return PB_OK;
}

// Synchronise the stream and turn a non-zero device status word into PB_ERR_DEVICE.
int pb_sync_check(pb_ctx* ctx, const char* who) {
    PB_CUDA(ctx, cudaMemcpyAsync(ctx->host_status, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const int st = *ctx->host_status;
    if (st) {
        cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), ctx->stream);
        cudaMemsetAsync(ctx->grid_sync, 0, 256, ctx->stream);   // a fused step that gave up leaves its barrier counter mid-way
        PB_FAIL(ctx, PB_ERR_DEVICE, "%s: a kernel reported device status %d", who, st);
    }
    return PB_OK;
}

extern "C" {

int pb_ctx_create(int device, pb_ctx** out) {
    if (!out) return PB_ERR_ARG;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) return PB_ERR_CUDA;  // no GPU: fail loudly, there is no CPU path
    if (device < 0 || device >= n) return PB_ERR_ARG;
    pb_ctx* c = new (std::nothrow) pb_ctx();
    if (!c) return PB_ERR_OOM;
    c->device = device;
    if (cudaSetDevice(device) != cudaSuccess) { delete c; return PB_ERR_CUDA; }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete c; return PB_ERR_CUDA; }
    c->sm_count = prop.multiProcessorCount;
    c->max_smem_optin = (int)prop.sharedMemPerBlockOptin;
    if (cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) != cudaSuccess) { delete c; return PB_ERR_CUDA; }
    c->stream = c->own_stream;
    if (cudaMalloc(&c->dev_status, 256) != cudaSuccess) { cudaStreamDestroy(c->own_stream); delete c; return PB_ERR_OOM; }
    cudaMemset(c->dev_status, 0, 256);
    if (cudaMalloc(&c->xh_buf, PB_XH_BYTES) != cudaSuccess) { cudaFree(c->dev_status); cudaStreamDestroy(c->own_stream); delete c; return PB_ERR_OOM; }
    if (cudaMalloc(&c->grid_sync, 256) != cudaSuccess) { cudaFree(c->xh_buf); cudaFree(c->dev_status); cudaStreamDestroy(c->own_stream); delete c; return PB_ERR_OOM; }
    cudaMemset(c->grid_sync, 0, 256);
    if (cudaMallocHost(&c->host_status, 256) != cudaSuccess) { cudaFree(c->dev_status); cudaStreamDestroy(c->own_stream); delete c; return PB_ERR_OOM; }
    *c->host_status = 0;
    c->owner_thread = (unsigned long)pthread_self();
    { const char* e = getenv("PYRE_B200_CHECK_THREAD"); c->check_thread = e && e[0] == '1'; }
    { const char* e = getenv("PYRE_B200_PDL"); if (e && e[0] == '0') c->use_pdl = false; }
    { const char* e = getenv("PYRE_B200_STEP_PDL"); c->step_pdl = c->use_pdl && !(e && e[0] == '0'); }   // PYRE_B200_STEP_PDL=0: the fused step kernel stays outside the chain   // PYRE_B200_PDL=0: plain stream order inside the token step
    *out = c;
    return PB_OK;
}

int pb_ctx_destroy(pb_ctx* ctx) {
    if (!ctx) return PB_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    pb_ep_destroy(ctx);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->stamps) cudaFree(ctx->stamps);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->xh_buf) cudaFree(ctx->xh_buf);
    if (ctx->grid_sync) cudaFree(ctx->grid_sync);
    if (ctx->host_status) cudaFreeHost(ctx->host_status);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return PB_OK;
}

const char* pb_last_error(const pb_ctx* ctx) { return ctx ? ctx->err.c_str() : kNoCtx; }

int pb_ctx_set_stream(pb_ctx* ctx, void* s) {
    if (!ctx) return PB_ERR_ARG;
    PB_TRY(pb_enter(ctx));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->stream = (cudaStream_t)s;
    return PB_OK;
}

int pb_ctx_own_stream(pb_ctx* ctx) {
    if (!ctx) return PB_ERR_ARG;
    PB_TRY(pb_enter(ctx));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->stream = ctx->own_stream;
    return PB_OK;
}

int pb_host_alloc(pb_ctx* ctx, size_t nbytes, void** out) {
    if (!ctx || !out) return PB_ERR_ARG;
    *out = nullptr;
    PB_TRY(pb_enter(ctx));
    if (cudaMallocHost(out, nbytes ? nbytes : 1) != cudaSuccess) { cudaGetLastError(); *out = nullptr; PB_FAIL(ctx, PB_ERR_OOM, "page-locked allocation of %zu bytes failed", nbytes); }
    return PB_OK;
}
int pb_host_free(pb_ctx* ctx, void* p) {
    if (!p) return PB_OK;
    if (!ctx) { if (cudaFreeHost(p) != cudaSuccess) { cudaGetLastError(); return PB_ERR_CUDA; } return PB_OK; }   // a buffer may outlive the context that made it
    PB_TRY(pb_enter(ctx));
    PB_CUDA(ctx, cudaFreeHost(p));
    return PB_OK;
}
int pb_ctx_sync(pb_ctx* ctx) {
    if (!ctx) return PB_ERR_ARG;
    PB_TRY(pb_enter(ctx));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PB_OK;
}

int pb_ctx_device_status(pb_ctx* ctx, int* status) {
    if (!ctx || !status) return PB_ERR_ARG;
    PB_TRY(pb_enter(ctx));
    PB_CUDA(ctx, cudaMemcpyAsync(status, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (*status) PB_CUDA(ctx, cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), ctx->stream));
    return PB_OK;
}

int pb_poll(pb_ctx* ctx, int* busy) {
    if (!ctx || !busy) return PB_ERR_ARG;
    PB_TRY(pb_enter(ctx));
    const cudaError_t e = cudaStreamQuery(ctx->stream);
    if (e == cudaErrorNotReady) { *busy = 1; return PB_OK; }
    *busy = 0;
    if (e != cudaSuccess) PB_FAIL(ctx, PB_ERR_CUDA, "cudaStreamQuery: %s", cudaGetErrorString(e));
    return pb_sync_check(ctx, "pb_poll");   // idle: the status word can be read without waiting
}

int pb_ctx_stamps_enable(pb_ctx* ctx, int slots) {
    if (!ctx || slots < 0) return PB_ERR_ARG;
    PB_TRY(pb_enter(ctx));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->stamps) { cudaFree(ctx->stamps); ctx->stamps = nullptr; }
    ctx->stamp_slots = 0; ctx->stamp_next = 0; ctx->stamp_ids.clear();
    if (slots == 0) return PB_OK;
    PB_CUDA(ctx, cudaMalloc(&ctx->stamps, (size_t)slots * PB_STAMP_WORDS * 8));
    PB_CUDA(ctx, cudaMemset(ctx->stamps, 0, (size_t)slots * PB_STAMP_WORDS * 8));
    ctx->stamp_slots = slots; ctx->stamp_ids.assign((size_t)slots, 0);
    return PB_OK;
}

int pb_ctx_stamps_read(pb_ctx* ctx, uint64_t* stamps_host, int32_t* kernel_ids_host, int max_slots, int* n_slots) {
    if (!ctx || !n_slots) return PB_ERR_ARG;
    PB_TRY(pb_enter(ctx));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const int n = ctx->stamp_next < max_slots ? ctx->stamp_next : max_slots;
    if (n > 0 && stamps_host) PB_CUDA(ctx, cudaMemcpy(stamps_host, ctx->stamps, (size_t)n * PB_STAMP_WORDS * 8, cudaMemcpyDeviceToHost));
    if (n > 0 && kernel_ids_host) for (int i = 0; i < n; i++) kernel_ids_host[i] = ctx->stamp_ids[i];
    *n_slots = ctx->stamp_next;
    return PB_OK;
}

int pb_type_geom(int t, int* e, int* b) { return pb_geom(t, e, b) ? PB_ERR_ARG : PB_OK; }

static int qmat_alloc(pb_ctx* ctx, int type, int64_t rows, int64_t cols, pb_qmat** out) {
    int el, bs;
    if (!ctx || !out) return PB_ERR_ARG;
    *out = nullptr;
    if (pb_geom(type, &el, &bs)) PB_FAIL(ctx, PB_ERR_ARG, "unsupported ggml type %d", type);
    if (rows <= 0 || cols <= 0 || cols % el) PB_FAIL(ctx, PB_ERR_ARG, "bad matrix shape %lld x %lld for blocks of %d", (long long)rows, (long long)cols, el);
    pb_qmat* m = new (std::nothrow) pb_qmat();
    if (!m) PB_FAIL(ctx, PB_ERR_OOM, "host allocation failed");
    m->ctx = ctx; m->type = type; m->rows = rows; m->cols = cols;
    m->row_bytes = cols / el * bs;
    m->nbytes = (size_t)rows * (size_t)m->row_bytes;
    { const int rc = pb_enter(ctx); if (rc != PB_OK) { delete m; return rc; } }
    // padded so that 16-byte-granular bulk copies of the last rows stay inside the allocation
    cudaError_t e = cudaMalloc(&m->data, m->nbytes + 256);
    if (e != cudaSuccess) { delete m; PB_FAIL(ctx, PB_ERR_OOM, "cudaMalloc(%zu): %s", m->nbytes + 256, cudaGetErrorString(e)); }
    cudaMemsetAsync(m->data + m->nbytes, 0, 256, ctx->stream);
    *out = m;
    return PB_OK;
}

// IQ3_S matrices get a second copy in the re-coded form the streaming kernels read (pb_repack.cu).
// PYRE_B200_REPACK=0 keeps only the native bytes (the kernels then decode IQ3_S itself).
static int qmat_recode(pb_ctx* ctx, pb_qmat* m) {
    static const bool on = !(getenv("PYRE_B200_REPACK") && atoi(getenv("PYRE_B200_REPACK")) == 0);
    const int64_t bpr = m->cols / 256;
    if (!on || m->type != PB_T_IQ3_S || m->cols % 256 || (bpr & 1)) return PB_OK;   // rows of the copy must stay 16-byte aligned
    m->r_row_bytes = bpr * 136;
    const size_t nb = (size_t)m->rows * (size_t)m->r_row_bytes;
    cudaError_t e = cudaMalloc(&m->rdata, nb + 256);
    if (e != cudaSuccess) { m->rdata = nullptr; PB_FAIL(ctx, PB_ERR_OOM, "cudaMalloc(%zu) for the re-coded copy: %s", nb + 256, cudaGetErrorString(e)); }
    cudaMemsetAsync(m->rdata + nb, 0, 256, ctx->stream);
    return pb_launch_repack_iq3s(ctx, m->data, m->rdata, m->rows * bpr);
}

int pb_qmat_upload(pb_ctx* ctx, int type, int64_t rows, int64_t cols, const void* bytes, size_t nbytes, pb_qmat** out) {
    if (!ctx) return PB_ERR_ARG;
    if (!bytes) PB_FAIL(ctx, PB_ERR_ARG, "pb_qmat_upload: null data");
    PB_TRY(qmat_alloc(ctx, type, rows, cols, out));
    if (nbytes != (*out)->nbytes) { size_t want = (*out)->nbytes; pb_qmat_free(*out); *out = nullptr; PB_FAIL(ctx, PB_ERR_ARG, "pb_qmat_upload: %zu bytes given, %zu expected", nbytes, want); }
    PB_CUDA(ctx, cudaMemcpyAsync((*out)->data, bytes, nbytes, cudaMemcpyHostToDevice, ctx->stream));
    int rc = qmat_recode(ctx, *out);
    if (rc != PB_OK) { pb_qmat_free(*out); *out = nullptr; return rc; }
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PB_OK;
}

int pb_qmat_synth(pb_ctx* ctx, int type, int64_t rows, int64_t cols, uint64_t seed, uint64_t tid, pb_qmat** out) {
    return pb_qmat_synth_rows(ctx, type, rows, cols, seed, tid, 0, out);
}

int pb_qmat_synth_rows(pb_ctx* ctx, int type, int64_t rows, int64_t cols, uint64_t seed, uint64_t tid, int64_t row0, pb_qmat** out) {
    if (!ctx) return PB_ERR_ARG;
    if (row0 < 0) PB_FAIL(ctx, PB_ERR_ARG, "pb_qmat_synth_rows: negative row offset");
    PB_TRY(qmat_alloc(ctx, type, rows, cols, out));
    pb_qmat* m = *out;
    int rc;
    if (type == PB_T_F32) rc = pb_launch_synth_normal_at(ctx, reinterpret_cast<float*>(m->data), rows * cols, seed, tid, row0 * cols, 0.02f);
    else { int el, bs; pb_geom(type, &el, &bs); rc = pb_launch_synth(ctx, type, m->data, rows * (cols / el), seed, tid, row0 * (cols / el)); }
    if (rc == PB_OK) rc = qmat_recode(ctx, m);
    if (rc != PB_OK) { pb_qmat_free(m); *out = nullptr; }
    return rc;
}

int pb_qmat_free(pb_qmat* m) {
    if (!m) return PB_OK;
    if (m->owns && m->data) { cudaSetDevice(m->ctx->device); cudaStreamSynchronize(m->ctx->stream); cudaFree(m->data); if (m->rdata) cudaFree(m->rdata); }
    delete m;
    return PB_OK;
}

int pb_qmat_info(const pb_qmat* m, int* type, int64_t* rows, int64_t* cols, size_t* nbytes) {
    if (!m) return PB_ERR_ARG;
    if (type) *type = m->type;
    if (rows) *rows = m->rows;
    if (cols) *cols = m->cols;
    if (nbytes) *nbytes = m->nbytes;
    return PB_OK;
}

static int check_rows(pb_ctx* ctx, const pb_qmat* m, int64_t r0, int64_t n, const char* who) {
    if (!ctx || !m) return PB_ERR_ARG;
    if (r0 < 0 || n < 0 || r0 + n > m->rows) PB_FAIL(ctx, PB_ERR_ARG, "%s: rows [%lld, %lld) outside 0..%lld", who, (long long)r0, (long long)(r0 + n), (long long)m->rows);
    return PB_OK;
}

int pb_qmat_read(pb_ctx* ctx, const pb_qmat* m, int64_t r0, int64_t n, void* bytes) {
    PB_TRY(check_rows(ctx, m, r0, n, "pb_qmat_read"));
    PB_TRY(pb_enter(ctx));
    if (!bytes) PB_FAIL(ctx, PB_ERR_ARG, "pb_qmat_read: null buffer");
    PB_CUDA(ctx, cudaMemcpyAsync(bytes, m->data + r0 * m->row_bytes, (size_t)n * m->row_bytes, cudaMemcpyDeviceToHost, ctx->stream));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PB_OK;
}

int pb_qmat_dequant_dev(pb_ctx* ctx, const pb_qmat* m, int64_t r0, int64_t n, float* out) {
    PB_TRY(check_rows(ctx, m, r0, n, "pb_qmat_dequant"));
    PB_TRY(pb_enter(ctx));
    if (!out) PB_FAIL(ctx, PB_ERR_ARG, "pb_qmat_dequant: null output");
    if ((n * m->cols) % 8) PB_FAIL(ctx, PB_UNSUPPORTED, "pb_qmat_dequant: element count must be a multiple of 8");
    if (m->type == PB_T_Q8_0 && ((r0 * m->cols) % 256)) PB_FAIL(ctx, PB_UNSUPPORTED, "pb_qmat_dequant: Q8_0 row offset must be a multiple of 256 elements");
    return pb_launch_dequant(ctx, m->type, m->data + r0 * m->row_bytes, n * m->cols / 8, out);
}

int pb_qmat_dequant(pb_ctx* ctx, const pb_qmat* m, int64_t r0, int64_t n, float* out_host) {
    PB_TRY(check_rows(ctx, m, r0, n, "pb_qmat_dequant"));
    if (!out_host) PB_FAIL(ctx, PB_ERR_ARG, "pb_qmat_dequant: null output");
    if (n == 0) return PB_OK;
    PB_TRY(pb_enter(ctx));
    void* tmp;
    const size_t bytes = (size_t)n * m->cols * 4;
    PB_TRY(pb_scratch(ctx, bytes + 1024, &tmp));
    PB_TRY(pb_qmat_dequant_dev(ctx, m, r0, n, (float*)tmp));
    PB_CUDA(ctx, cudaMemcpyAsync(out_host, tmp, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PB_OK;
}

int pb_gemv_dev(pb_ctx* ctx, const pb_qmat* m, const float* x, int t, float* y) {
    if (!ctx || !m) return PB_ERR_ARG;
    if (!x || !y) PB_FAIL(ctx, PB_ERR_ARG, "pb_gemv: null buffer");
    if (t < 0) PB_FAIL(ctx, PB_ERR_ARG, "pb_gemv: t=%d", t);
    PB_TRY(pb_enter(ctx));
    // many tokens of a re-coded IQ3_S matrix go to the tcgen05 GEMM in pieces as large as its operand buffer takes
    const bool tc = t >= pb_gemmtc_min_tokens() && m->rdata && pb_gemvq_supported(m->type, (int)m->cols) && pb_gemmtc_supported(m->type, (int)m->cols, t);   // what pb_launch_gemvq will pick
    const int piece = tc ? pb_gemmtc_max_tokens((int)m->cols) : 16;
    for (int t0 = 0; t0 < t; t0 += piece) {
        PbGemvArgs a;
        a.w = m->data; a.wr = m->rdata; a.type = m->type; a.rows = m->rows; a.cols = (int)m->cols;
        a.x = x + (int64_t)t0 * m->cols; a.ldx = m->cols; a.t = t - t0 < piece ? t - t0 : piece;
        a.y = y + (int64_t)t0 * m->rows; a.ldy = m->rows;
        PB_TRY(pb_launch_gemv(ctx, a));
    }
    return PB_OK;
}

int pb_gemv(pb_ctx* ctx, const pb_qmat* m, const float* x_host, int t, float* y_host) {
    if (!ctx || !m) return PB_ERR_ARG;
    if (!x_host || !y_host) PB_FAIL(ctx, PB_ERR_ARG, "pb_gemv: null buffer");
    if (t <= 0) return t == 0 ? PB_OK : PB_ERR_ARG;
    PB_TRY(pb_enter(ctx));
    const size_t xb = ((size_t)t * m->cols * 4 + 255) & ~(size_t)255, yb = (size_t)t * m->rows * 4;
    void* tmp;
    PB_TRY(pb_scratch(ctx, xb + yb, &tmp));
    float* xd = (float*)tmp;
    float* yd = (float*)((uint8_t*)tmp + xb);
    PB_CUDA(ctx, cudaMemcpyAsync(xd, x_host, (size_t)t * m->cols * 4, cudaMemcpyHostToDevice, ctx->stream));
    PB_TRY(pb_gemv_dev(ctx, m, xd, t, yd));
    PB_CUDA(ctx, cudaMemcpyAsync(y_host, yd, yb, cudaMemcpyDeviceToHost, ctx->stream));
    PB_TRY(pb_sync_check(ctx, "pb_gemv"));
    return PB_OK;
}

// ---------------------------------------------------------------- pb_gemv_static
// Device staging area of pb_gemv_static: a fixed array inside the library image instead of a
// cudaMalloc'd buffer.  Every GPU that loads the library carries these bytes until the
// process exits.  In host code the symbol is only a stand-in; the device address is fetched
// with cudaGetSymbolAddress once per device (with that device current) and cached.  The cache is
// filled without a lock: two threads that race on a device's slot both store the same address.
static __device__ __align__(256) unsigned char pb_static_scratch[PB_GEMV_STATIC_MAX_BYTES];
static void* g_static_scratch_addr[64] = {nullptr};

int pb_gemv_static(pb_ctx* ctx, const pb_qmat* m, const float* x_host, int t, float* y_host) {
    if (!ctx || !m) return PB_ERR_ARG;
    if (!x_host || !y_host) PB_FAIL(ctx, PB_ERR_ARG, "pb_gemv_static: null buffer");
    if (t <= 0) return t == 0 ? PB_OK : PB_ERR_ARG;
    if (ctx->device < 0 || ctx->device >= 64) PB_FAIL(ctx, PB_UNSUPPORTED, "pb_gemv_static: device index %d", ctx->device);
    const size_t xb = ((size_t)t * m->cols * 4 + 255) & ~(size_t)255, yb = (size_t)t * m->rows * 4;
    if (xb + yb > (size_t)PB_GEMV_STATIC_MAX_BYTES)
        PB_FAIL(ctx, PB_ERR_ARG, "pb_gemv_static: %zu bytes of staging needed (t * (cols + rows) floats), the built-in area holds %u; use pb_gemv", xb + yb, (unsigned)PB_GEMV_STATIC_MAX_BYTES);
    PB_TRY(pb_enter(ctx));   // the context's GPU is current on every call, not only on the first
    if (!g_static_scratch_addr[ctx->device]) {   // first call on this device: resolve the device address of the array
        void* p = nullptr;
        PB_CUDA(ctx, cudaGetSymbolAddress(&p, pb_static_scratch));
        g_static_scratch_addr[ctx->device] = p;
    }
    float* xd = (float*)g_static_scratch_addr[ctx->device];
    float* yd = (float*)((uint8_t*)xd + xb);
    PB_CUDA(ctx, cudaMemcpyAsync(xd, x_host, (size_t)t * m->cols * 4, cudaMemcpyHostToDevice, ctx->stream));
    PB_TRY(pb_gemv_dev(ctx, m, xd, t, yd));
    PB_CUDA(ctx, cudaMemcpyAsync(y_host, yd, yb, cudaMemcpyDeviceToHost, ctx->stream));
    return pb_sync_check(ctx, "pb_gemv_static");
}

}  // extern "C"
