// Hyper-connection residual plumbing (hc >= 1): the residual stream is hc parallel copies of width d per token.
//
// Restates hc_mix and hc_combine of the reference (src/model/qwen4exp_gguf.rs:1357-1382, 1384-1388; GPU twins GHc::mix /
// k_hc_gate / k_hc_comb, src/model/qn_gpu.rs and src/model/qn_cube.rs):
//   mix      xn[s] = rms(x[s]) * norm[s];  lo = silu((down . xn) / hc);  inj = (inject . xn) / hc;  gate = up . lo;
//            mixed[i] = (sum_s xn[s][i] * sigmoid(gate[s][i])) / hc          -> the input of the mixer / MoE block
//   combine  x[s] += out * 2 * sigmoid(inj[s])                               -> after the block
// down [lr][hc*d], inject [hc][hc*d] and up [hc*d][lr] are small f32 matrices (lr = low rank, e.g. 32), so they get a
// plain warp-per-row f32 GEMV instead of the streaming kernels.
#include "pb_common.cuh"
#include "pb_internal.h"

// grid (t * hc), 256 threads: one stream of one token
__global__ void __launch_bounds__(256) pb_hc_norm_kernel(const float* __restrict__ x, const float* __restrict__ norm, float* __restrict__ xn, int d, int hc, float eps) {
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t row = blockIdx.x;
    const int s = (int)(row % hc), tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float* xr = x + row * d;
    __shared__ float red[8];
    float ss = 0.f;
    for (int i = tid; i < d; i += 256) ss = fmaf(xr[i], xr[i], ss);
    ss = pb_warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot += red[w];
    const float sc = 1.0f / sqrtf(tot / (float)d + eps);
    for (int i = tid; i < d; i += 256) xn[row * d + i] = xr[i] * sc * norm[(size_t)s * d + i];
}

// y[t][r] = post(W[r][:] . x[t][:]);  grid (ceil(rows / 8), t), warp per row.  post 0: identity; 1: silu(v / hc); 2: v / hc
__global__ void __launch_bounds__(256) pb_hc_gemv_kernel(const float* __restrict__ W, int rows, int cols, const float* __restrict__ x, int64_t ldx, float* __restrict__ y, int64_t ldy, int post, float hc) {
    pb_pdl_wait();
    pb_pdl_trigger();
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31, t = blockIdx.y;
    if (r >= rows) return;
    const float* w = W + (size_t)r * cols;
    const float* xv = x + (size_t)t * ldx;
    float acc = 0.f;
    for (int c = lane; c < cols; c += 32) acc = fmaf(w[c], xv[c], acc);
    acc = pb_warp_sum(acc);
    if (lane == 0) {
        if (post == 1) acc = pb_silu(acc / hc); else if (post == 2) acc = acc / hc;
        y[(size_t)t * ldy + r] = acc;
    }
}

// mixed[t][i] = (sum_s xn[t][s][i] * sigmoid(gate[t][s][i])) / hc, the streams added in order
__global__ void __launch_bounds__(256) pb_hc_mixdown_kernel(const float* __restrict__ xn, const float* __restrict__ gate, float* __restrict__ mixed, int d, int hc) {
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t t = blockIdx.y;
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= d) return;
    float m = 0.f;
    for (int s = 0; s < hc; s++) { const int64_t k = (t * hc + s) * d + i; m += xn[k] * pb_sigm(gate[k]); }
    mixed[t * d + i] = m / (float)hc;
}

// x[t][s][i] += out[t][i] * 2 * sigmoid(inj[t][s]);  grid (ceil(d / 256), t * hc)
__global__ void __launch_bounds__(256) pb_hc_combine_kernel(float* __restrict__ x, const float* __restrict__ out, const float* __restrict__ inj, int d, int hc) {
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t row = blockIdx.y, t = row / hc;
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= d) return;
    const float w = 2.0f * pb_sigm(inj[row]);
    x[row * d + i] += out[t * d + i] * w;
}

// x[t][s][:] = e[t][:] for every stream s (the embedding row feeds all streams, :2092)
__global__ void __launch_bounds__(256) pb_hc_spread_kernel(const float* __restrict__ e, float* __restrict__ x, int d, int hc) {
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t row = blockIdx.y, t = row / hc;
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < d) x[row * d + i] = e[t * d + i];
}

#define HC_GO(...)                        \
    do {                                  \
        pb_launch_k(ctx, __VA_ARGS__);    \
        ctx->kernels_launched++;          \
        PB_CUDA(ctx, cudaGetLastError()); \
    } while (0)

int pb_launch_hc_mix(pb_ctx* ctx, const PbHcParams& p, const float* x, int t, float* mixed) {
    const int d = p.d, hc = p.hc, w = hc * d;
    HC_GO(pb_hc_norm_kernel, dim3(t * hc), dim3(256), (size_t)0, x, p.norm, p.xn, d, hc, p.eps);
    HC_GO(pb_hc_gemv_kernel, dim3((p.lr + 7) / 8, t), dim3(256), (size_t)0, p.down, p.lr, w, (const float*)p.xn, (int64_t)w, p.lo, (int64_t)p.lr, 1, (float)hc);
    if (p.inject) HC_GO(pb_hc_gemv_kernel, dim3((hc + 7) / 8, t), dim3(256), (size_t)0, p.inject, hc, w, (const float*)p.xn, (int64_t)w, p.inj, (int64_t)hc, 2, (float)hc);
    else PB_CUDA(ctx, cudaMemsetAsync(p.inj, 0, (size_t)t * hc * 4, ctx->stream));
    HC_GO(pb_hc_gemv_kernel, dim3((w + 7) / 8, t), dim3(256), (size_t)0, p.up, w, p.lr, (const float*)p.lo, (int64_t)p.lr, p.gate, (int64_t)w, 0, (float)hc);
    HC_GO(pb_hc_mixdown_kernel, dim3((d + 255) / 256, t), dim3(256), (size_t)0, (const float*)p.xn, (const float*)p.gate, mixed, d, hc);
    return PB_OK;
}
int pb_launch_hc_combine(pb_ctx* ctx, const PbHcParams& p, float* x, const float* out, int t) {
    HC_GO(pb_hc_combine_kernel, dim3((p.d + 255) / 256, t * p.hc), dim3(256), (size_t)0, x, out, (const float*)p.inj, p.d, p.hc);
    return PB_OK;
}
int pb_launch_hc_spread(pb_ctx* ctx, const float* e, float* x, int t, int d, int hc) {
    HC_GO(pb_hc_spread_kernel, dim3((d + 255) / 256, t * hc), dim3(256), (size_t)0, e, x, d, hc);
    return PB_OK;
}
