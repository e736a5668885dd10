// Small kernels of the MTP drafter (the model's own multi-token-prediction layer used as a speculative drafter,
// src/model/mtp.rs of the reference).  The drafter's layer itself runs on the engine's attention, MoE and
// hyper-connection kernels; these are the pieces around it:
//   pb_mtp_keep_kernel    the main model's final residual rows go into a ring indexed by position (mtp_keep_r,
//                         src/model/qwen4exp_gguf.rs:2279-2285)
//   pb_mtp_input_kernel   rms(embedding) * pre_e and rms over all hc*d values of the residual * pre_h (input, mtp.rs:186-195)
//   pb_mtp_join_kernel    R'[s] = fc_hidden(h)[s] + fc_embedding(e)
//   pb_mtp_mask_kernel    the window of cells a draft step attends to, as the position mask of the attention kernels
//   pb_mtp_best_kernel    best(): arg max over the draft vocabulary and its softmax probability (mtp.rs:424-427)
#include "pb_common.cuh"
#include "pb_internal.h"

// grid (t), 256 threads: ring[(pos[j] % cap)] = x[j]
__global__ void __launch_bounds__(256) pb_mtp_keep_kernel(const float* x, int64_t ldx, const int64_t* pos, float* ring, int cap, int w) {
    const int j = blockIdx.x;
    pb_pdl_wait();
    pb_pdl_trigger();
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)j * ldx);
    float4* dst = reinterpret_cast<float4*>(ring + (size_t)(pos[j] % cap) * w);
    for (int i = threadIdx.x; i < w / 4; i += 256) dst[i] = src[i];
}

// one CTA of 1024 threads: en[d] = rms(e) * pre_e, hn[hc*d] = rms(R over hc*d) * pre_h
__global__ void __launch_bounds__(1024) pb_mtp_input_kernel(const float* e, const float* pre_e, const float* R, const float* pre_h, float* en, float* hn, int d, int w, float eps) {
    __shared__ float red[2][32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float se = 0.f, sr = 0.f;
    for (int i = tid; i < d; i += 1024) se += e[i] * e[i];
    for (int i = tid; i < w; i += 1024) sr += R[i] * R[i];
    se = pb_warp_sum(se); sr = pb_warp_sum(sr);
    if (lane == 0) { red[0][warp] = se; red[1][warp] = sr; }
    __syncthreads();
    float te = 0.f, tr = 0.f;
    for (int i = 0; i < 32; i++) { te += red[0][i]; tr += red[1][i]; }
    const float ke = 1.0f / sqrtf(te / (float)d + eps), kr = 1.0f / sqrtf(tr / (float)w + eps);
    for (int i = tid; i < d; i += 1024) en[i] = e[i] * ke * pre_e[i];
    for (int i = tid; i < w; i += 1024) hn[i] = R[i] * kr * pre_h[i];
}

// x[s][i] = h2[s][i] + e2[i]
__global__ void __launch_bounds__(256) pb_mtp_join_kernel(const float* h2, const float* e2, float* x, int d, int w) {
    for (int i = blockIdx.x * 256 + threadIdx.x; i < w; i += gridDim.x * 256) x[i] = h2[i] + e2[i % d];
}

// one CTA: bits lo .. pos set, every other bit of the words up to pos cleared; *on = 1
__global__ void __launch_bounds__(256) pb_mtp_mask_kernel(uint32_t* mask, int* on, int64_t lo, int64_t pos) {
    const int64_t nw = (pos >> 5) + 1;
    for (int64_t wd = threadIdx.x; wd < nw; wd += 256) {
        const int64_t b0 = wd * 32;
        uint32_t v = 0u;
        for (int b = 0; b < 32; b++) { const int64_t q = b0 + b; if (q >= lo && q <= pos) v |= 1u << b; }
        mask[wd] = v;
    }
    if (threadIdx.x == 0) *on = 1;
}

// one CTA of 1024 threads: out[0] = index of the largest logit (the first among equals), out[1] = bits of 1 / sum exp(l - max)
__global__ void __launch_bounds__(1024) pb_mtp_best_kernel(const float* lg, int n, uint32_t* out) {
    __shared__ float sv[32]; __shared__ int si[32]; __shared__ float bmax; __shared__ int bidx;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float v = -INFINITY; int idx = 0x7fffffff;
    for (int i = tid; i < n; i += 1024) { const float x = lg[i]; if (x > v) { v = x; idx = i; } }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o); const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if (lane == 0) { sv[warp] = v; si[warp] = idx; }
    __syncthreads();
    if (tid == 0) {
        float m = sv[0]; int mi = si[0];
        for (int i = 1; i < 32; i++) if (sv[i] > m || (sv[i] == m && si[i] < mi)) { m = sv[i]; mi = si[i]; }
        bmax = m; bidx = mi;
    }
    __syncthreads();
    float z = 0.f;
    for (int i = tid; i < n; i += 1024) z += expf(lg[i] - bmax);
    z = pb_warp_sum(z);
    __syncthreads();
    if (lane == 0) sv[warp] = z;
    __syncthreads();
    if (tid == 0) { float t = 0.f; for (int i = 0; i < 32; i++) t += sv[i]; out[0] = (uint32_t)bidx; out[1] = __float_as_uint(1.0f / t); }
}

int pb_launch_mtp_keep(pb_ctx* ctx, const float* x, int64_t ldx, const int64_t* pos, int t, float* ring, int cap, int w) {
    pb_launch_k(ctx, pb_mtp_keep_kernel, dim3(t), dim3(256), (size_t)0, x, ldx, pos, ring, cap, w);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
int pb_launch_mtp_input(pb_ctx* ctx, const float* e, const float* pre_e, const float* R, const float* pre_h, float* en, float* hn, int d, int w, float eps) {
    pb_mtp_input_kernel<<<1, 1024, 0, ctx->stream>>>(e, pre_e, R, pre_h, en, hn, d, w, eps);
    ctx->kernels_launched++; ctx->pdl_chain = false;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
int pb_launch_mtp_join(pb_ctx* ctx, const float* h2, const float* e2, float* x, int d, int w) {
    pb_mtp_join_kernel<<<(w + 255) / 256 < 64 ? (w + 255) / 256 : 64, 256, 0, ctx->stream>>>(h2, e2, x, d, w);
    ctx->kernels_launched++; ctx->pdl_chain = false;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
int pb_launch_mtp_mask(pb_ctx* ctx, uint32_t* mask, int* on, int64_t lo, int64_t pos) {
    pb_mtp_mask_kernel<<<1, 256, 0, ctx->stream>>>(mask, on, lo, pos);
    ctx->kernels_launched++; ctx->pdl_chain = false;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
int pb_launch_mtp_best(pb_ctx* ctx, const float* lg, int n, uint32_t* out) {
    pb_mtp_best_kernel<<<1, 1024, 0, ctx->stream>>>(lg, n, out);
    ctx->kernels_launched++; ctx->pdl_chain = false;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
