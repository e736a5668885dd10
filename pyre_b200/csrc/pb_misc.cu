// Small kernels of the token loop: embedding row dequantization, greedy argmax, position advance.
#include "pb_formats.cuh"
#include "pb_internal.h"

#include <stdio.h>

// x[b] = dequant(token_embd row ids[b])  (forward_inner, src/model/qwen4exp_gguf.rs:2092); grid (steps, t)
template <int FMT>
__global__ void __launch_bounds__(32) pb_embed_kernel(const uint8_t* __restrict__ w, int64_t rows, int row_bytes, const uint32_t* __restrict__ ids, float* __restrict__ out, int64_t ldo) {
    using F = PbFmt<FMT>;
    const int lane = threadIdx.x, step = blockIdx.x, b = blockIdx.y;
    pb_pdl_wait();
    pb_pdl_trigger();
    uint32_t id = ids[b];
    if (id >= rows) id = 0;   // out-of-range token ids read row 0 instead of faulting
    PbTables T;
    T.iq3s = PB_IQ3S_GRID; T.iq2xs = PB_IQ2XS_GRID; T.ksigns = PB_KSIGNS_IQ2XS;
    T.iq3xxs = PB_IQ3XXS_GRID; T.iq2s = PB_IQ2S_GRID; T.kvalues = PB_KVALUES_IQ4NL; T.iq2xxs = PB_IQ2XXS_GRID; T.iq1s = PB_IQ1S_GRID;
    PbUnit u;
    F::unit(w + (size_t)id * row_bytes + (size_t)step * F::STEP_BYTES, lane, T, u);
    float* o = out + (size_t)b * ldo + step * 256;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float v = __fmul_rn(j < 4 ? u.sa : u.sb, u.w[j]);
        if (F::HAS_MIN) v = __fsub_rn(v, j < 4 ? u.ma : u.mb);
        o[F::pos(lane, j)] = v;
    }
}

int pb_launch_embed(pb_ctx* ctx, int type, const uint8_t* w, int64_t rows, int cols, const uint32_t* ids, int t, float* out, int64_t ldo) {
    int el, bs;
    if (pb_geom(type, &el, &bs) || cols % 256) PB_FAIL(ctx, PB_UNSUPPORTED, "embed: type %d cols %d", type, cols);
    const int row_bytes = cols / el * bs;
    const dim3 grid(cols / 256, t);
#define LAUNCH() pb_launch_k(ctx, pb_embed_kernel<FMT>, grid, dim3(32), (size_t)0, w, rows, row_bytes, ids, out, ldo)
    PB_DISPATCH_FMT(type, LAUNCH);
#undef LAUNCH
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

// sampler::argmax, src/sampler.rs:142-148: first index of the maximum.  grid (blocks, t): every CTA
// scans a slice and folds its best (value, index) into one 64-bit key per sequence with atomicMax;
// the key orders by value first and by lower index second, NaN counts as the lowest value.
__device__ __forceinline__ unsigned long long pb_argmax_key(float v, int i) {
    uint32_t u = __float_as_uint(v);
    u = (v != v) ? 0u : ((u & 0x80000000u) ? ~u : (u | 0x80000000u));
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
}
__global__ void __launch_bounds__(256) pb_argmax_kernel(const float* __restrict__ logits, int64_t ld, int n, unsigned long long* __restrict__ keys) {
    pb_pdl_wait();
    pb_pdl_trigger();
    const float* v = logits + (size_t)blockIdx.y * ld;
    unsigned long long best = 0;
    for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256) { const unsigned long long k = pb_argmax_key(v[i], i); best = k > best ? k : best; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o); best = ok > best ? ok : best; }
    __shared__ unsigned long long sk[8];
    if ((threadIdx.x & 31) == 0) sk[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) best = sk[w] > best ? sk[w] : best;
        atomicMax(keys + blockIdx.y, best);
    }
}

int pb_launch_argmax(pb_ctx* ctx, const float* logits, int64_t ld, int n, int t, unsigned long long* keys) {
    int blocks = (n + 2047) / 2048;
    if (blocks > 148) blocks = 148;
    pb_launch_k(ctx, pb_argmax_kernel, dim3(dim3(blocks, t)), dim3(256), (size_t)(0), logits, ld, n, keys);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

// end of a decode step: decode the argmax keys into token ids (and clear them for the next step),
// pos += 1, feed the chosen tokens back as the next inputs and log them
__global__ void pb_advance_kernel(int64_t* pos, int t, unsigned long long* keys, uint32_t* next, uint32_t* ids, uint32_t* trace, int64_t* trace_len, int64_t trace_cap,
                                  unsigned long long* ep_seq, unsigned long long ep_seq_step) {
    const int b = threadIdx.x;
    pb_pdl_wait();
    pb_pdl_trigger();
    if (b < t) {
        const unsigned long long k = keys[b];
        const uint32_t tok = k ? 0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull) : 0u;
        keys[b] = 0;
        pos[b] += 1;
        next[b] = tok;
        ids[b] = tok;
        const int64_t j = *trace_len;
        if (j < trace_cap) trace[j * t + b] = tok;
    }
    __syncthreads();
    if (b == 0) *trace_len += 1;
    if (b == 0 && ep_seq) *ep_seq += ep_seq_step;   // the next step's peer exchanges carry new sequence numbers
}

int pb_launch_advance(pb_ctx* ctx, int64_t* pos, int t, unsigned long long* keys, uint32_t* next, uint32_t* ids, uint32_t* trace, int64_t* trace_len, int64_t trace_cap,
                      unsigned long long* ep_seq, unsigned long long ep_seq_step) {
    pb_launch_k(ctx, pb_advance_kernel, dim3(1), dim3((t + 31) & ~31), (size_t)(0), pos, t, keys, next, ids, trace, trace_len, trace_cap, ep_seq, ep_seq_step);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

// Rollback of a verify window: every DeltaNet layer's conv ring and recurrent state go back to the checkpoint taken after token
// `idx` of the window.  tab[(li * stride + idx) * 2 + {0, 1}] = checkpoint of layer li (conv, ssm), live[li * 2 + {0, 1}] = the live
// buffers.  grid (n_lin, 32), 256 threads; one launch instead of two copies per layer.
__global__ void __launch_bounds__(256) pb_ck_restore_kernel(const float* const* __restrict__ tab, float* const* __restrict__ live, int stride, int idx, int64_t conv_n, int64_t ssm_n) {
    const int li = blockIdx.x;
    const float4* cs = reinterpret_cast<const float4*>(tab[((size_t)li * stride + idx) * 2]);
    const float4* ss = reinterpret_cast<const float4*>(tab[((size_t)li * stride + idx) * 2 + 1]);
    float4* cd = reinterpret_cast<float4*>(live[li * 2]);
    float4* sd = reinterpret_cast<float4*>(live[li * 2 + 1]);
    const int64_t step = (int64_t)gridDim.y * 256, i0 = (int64_t)blockIdx.y * 256 + threadIdx.x;
    for (int64_t i = i0; i < conv_n / 4; i += step) cd[i] = cs[i];
    for (int64_t i = i0; i < ssm_n / 4; i += step) sd[i] = ss[i];
}
int pb_launch_ck_restore(pb_ctx* ctx, const float* const* tab, float* const* live, int n_lin, int stride, int idx, int64_t conv_n, int64_t ssm_n) {
    if (conv_n % 4 || ssm_n % 4) PB_FAIL(ctx, PB_UNSUPPORTED, "checkpoint restore: state sizes %lld / %lld are not multiples of four", (long long)conv_n, (long long)ssm_n);
    pb_ck_restore_kernel<<<dim3(n_lin, 32), 256, 0, ctx->stream>>>(tab, live, stride, idx, conv_n, ssm_n);
    ctx->kernels_launched++; ctx->pdl_chain = false;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

// Window bookkeeping of a batch-1 state: advance == 0: wpos[j] = pos[0] + j for j < t; advance == 1: pos[0] += t.
__global__ void pb_window_pos_kernel(int64_t* pos, int64_t* wpos, int t, int advance) {
    pb_pdl_wait();
    pb_pdl_trigger();
    if (advance) { if (threadIdx.x == 0) pos[0] += t; }
    else for (int j = threadIdx.x; j < t; j += blockDim.x) wpos[j] = pos[0] + j;
}
int pb_launch_window_pos(pb_ctx* ctx, int64_t* pos, int64_t* wpos, int t, int advance) {
    pb_launch_k(ctx, pb_window_pos_kernel, dim3(1), dim3(256), (size_t)0, pos, wpos, t, advance);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
