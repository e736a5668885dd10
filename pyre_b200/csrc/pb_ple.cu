// Per-layer n-gram embeddings (PLE) of the qwen4exp loop: `ple_rows` and `ple`, src/model/qwen4exp_gguf.rs:1390-1434 of the reference.
//   pb_ple_rows_kernel   every fed token joins its sequence's id history; its context (the token and its ngram - 1 predecessors,
//                        cut at the first missing or end-of-sequence one) is hashed per n-gram size and head into a row of the table
//   pb_ple_gate_kernel   per (token, residual stream): gate = sigmoid(signed sqrt(rms(key) . rms(stream) / sqrt d)), gated = value * gate,
//                        its normalized form goes into the layer's ring of rows by position
//   pb_ple_conv_kernel   stream += gated + silu(depthwise conv over the normalized rows of this and of earlier positions)
// The table rows themselves are gathered by the embedding kernel, the key / value projections are GEMVs of the engine.
// The reference keeps the last (conv_k - 1) * ngram normalized rows in a ring that it drains and extends per token and checkpoints
// for rollbacks; here rows are addressed by position (slot = position % ring length), so a rollback only moves the position back.
#include "pb_common.cuh"
#include "pb_internal.h"

// grid (t), 32 threads.  window: the rows are consecutive positions of sequence 0 (predecessors inside the window come from `ids`),
// else row r is sequence r.  base[b] = first position of sequence b that has a history (older ones read as missing).
__global__ void __launch_bounds__(32) pb_ple_rows_kernel(PbPleHash hp, const uint32_t* __restrict__ ids, const int64_t* __restrict__ posv, int window,
                                                         uint32_t* tok_hist, int64_t max_ctx, const int64_t* __restrict__ base, uint32_t* __restrict__ rows_out) {
    const int r = blockIdx.x, lane = threadIdx.x, b = window ? 0 : r;
    const int64_t p = posv[r], b0 = base[b];
    uint32_t* th = tok_hist + (size_t)b * max_ctx;
    uint64_t ctx[8];
    ctx[0] = ids[r];
    bool cut = false;
    for (int s = 1; s < hp.ngram; s++) {
        const int64_t q = p - s;
        const bool none = cut || q < b0;
        uint32_t tk = 0;
        if (!none) tk = (window && r - s >= 0) ? ids[r - s] : th[q];
        cut = cut || none || tk == hp.eos;
        ctx[s] = cut ? hp.eos : tk;
    }
    if (lane == 0) th[p] = ids[r];
    if (lane < hp.nh) {
        const int n = 2 + lane / hp.per_gram;
        uint64_t mixed = ctx[0] * hp.mult[0];
        for (int j = 1; j < n; j++) mixed ^= ctx[j] * hp.mult[j];
        rows_out[(size_t)r * hp.nh + lane] = (uint32_t)(mixed % hp.vocab[lane] + hp.off[lane]);
    }
}

// grid (t, streams), 256 threads
__global__ void __launch_bounds__(256) pb_ple_gate_kernel(const float* __restrict__ key, int64_t ldk, const float* __restrict__ val, int64_t ldv, const float* __restrict__ x, int64_t ldx,
                                                          const float* __restrict__ nk, const float* __restrict__ nq, const float* __restrict__ nc,
                                                          float* __restrict__ gated, float* __restrict__ ring, int R, const int64_t* __restrict__ posv, int window, int d, int w, float eps) {
    __shared__ float red[4][8];
    const int r = blockIdx.x, s = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, b = window ? 0 : r;
    const int64_t p = posv[r];
    const float* k = key + (size_t)r * ldk + (size_t)s * d;
    const float* xs = x + (size_t)r * ldx + (size_t)s * d;
    const float* v = val + (size_t)r * ldv;
    const float* wk = nk + (size_t)s * d; const float* wq = nq + (size_t)s * d; const float* wc = nc + (size_t)s * d;
    float ssk = 0.f, ssx = 0.f, dkx = 0.f, sv = 0.f;
    for (int i = tid; i < d; i += 256) {
        const float a = k[i], c = xs[i], e = v[i];
        ssk = fmaf(a, a, ssk); ssx = fmaf(c, c, ssx); dkx = fmaf(a * wk[i], c * wq[i], dkx); sv = fmaf(e, e, sv);
    }
    ssk = pb_warp_sum(ssk); ssx = pb_warp_sum(ssx); dkx = pb_warp_sum(dkx); sv = pb_warp_sum(sv);
    if (lane == 0) { red[0][warp] = ssk; red[1][warp] = ssx; red[2][warp] = dkx; red[3][warp] = sv; }
    __syncthreads();
    float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) { t0 += red[0][i]; t1 += red[1][i]; t2 += red[2][i]; t3 += red[3][i]; }
    const float rk = 1.0f / sqrtf(t0 / (float)d + eps), rq = 1.0f / sqrtf(t1 / (float)d + eps);
    const float sc = t2 * rk * rq / sqrtf((float)d);
    const float g = 1.0f / (1.0f + expf(-copysignf(sqrtf(fmaxf(fabsf(sc), 1e-6f)), sc)));
    const float rg = 1.0f / sqrtf(g * g * t3 / (float)d + eps);
    float* go = gated + (size_t)r * w + (size_t)s * d;
    float* no = ring + ((size_t)b * R + (size_t)(p % R)) * w + (size_t)s * d;
    for (int i = tid; i < d; i += 256) { const float gv = v[i] * g; go[i] = gv; no[i] = gv * rg * wc[i]; }
}

// grid (t, ceil(w / 256)), 256 threads
__global__ void __launch_bounds__(256) pb_ple_conv_kernel(const float* __restrict__ gated, const float* __restrict__ ring, int R, const float* __restrict__ conv, int K, int dil,
                                                          const int64_t* __restrict__ posv, int window, const int64_t* __restrict__ base, float* __restrict__ x, int64_t ldx, int w) {
    const int r = blockIdx.x, ch = blockIdx.y * 256 + threadIdx.x, b = window ? 0 : r;
    if (ch >= w) return;
    const int64_t p = posv[r], b0 = base[b];
    const float* rb = ring + (size_t)b * R * w;
    float o = conv[(size_t)ch * K + K - 1] * rb[(size_t)(p % R) * w + ch];
    for (int k = 0; k < K - 1; k++) {
        const int64_t q = p - (int64_t)(K - 1 - k) * dil;
        if (q >= b0) o += conv[(size_t)ch * K + k] * rb[(size_t)(q % R) * w + ch];
    }
    x[(size_t)r * ldx + ch] += gated[(size_t)r * w + ch] + o / (1.0f + expf(-o));
}

int pb_launch_ple_rows(pb_ctx* ctx, const PbPleHash& hp, const uint32_t* ids, const int64_t* posv, int t, int window, uint32_t* tok_hist, int64_t max_ctx, const int64_t* base, uint32_t* rows_out) {
    pb_ple_rows_kernel<<<t, 32, 0, ctx->stream>>>(hp, ids, posv, window, tok_hist, max_ctx, base, rows_out);
    ctx->kernels_launched++; ctx->pdl_chain = false;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
int pb_launch_ple_gate(pb_ctx* ctx, const float* key, int64_t ldk, const float* val, int64_t ldv, const float* x, int64_t ldx, const float* nk, const float* nq, const float* nc,
                       float* gated, float* ring, int R, const int64_t* posv, int t, int window, int d, int streams, float eps) {
    pb_ple_gate_kernel<<<dim3(t, streams), 256, 0, ctx->stream>>>(key, ldk, val, ldv, x, ldx, nk, nq, nc, gated, ring, R, posv, window, d, streams * d, eps);
    ctx->kernels_launched++; ctx->pdl_chain = false;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
int pb_launch_ple_conv(pb_ctx* ctx, const float* gated, const float* ring, int R, const float* conv, int K, int dil, const int64_t* posv, int t, int window, const int64_t* base, float* x, int64_t ldx, int w) {
    pb_ple_conv_kernel<<<dim3(t, (w + 255) / 256), 256, 0, ctx->stream>>>(gated, ring, R, conv, K, dil, posv, window, base, x, ldx, w);
    ctx->kernels_launched++; ctx->pdl_chain = false;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
