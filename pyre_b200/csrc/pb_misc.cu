// Small kernels of the token loop: embedding row dequantization, greedy argmax, position advance.
#include "pb_formats.cuh"
#include "pb_internal.h"

#include <stdio.h>

// x[b] = dequant(token_embd row ids[b])  (forward_inner, src/model/qwen4exp_gguf.rs:2092); grid (steps, t)
template <int FMT>
__global__ void __launch_bounds__(32) pb_embed_kernel(const uint8_t* __restrict__ w, int64_t rows, int row_bytes, const uint32_t* __restrict__ ids, float* __restrict__ out, int64_t ldo) {
    using F = PbFmt<FMT>;
    const int lane = threadIdx.x, step = blockIdx.x, b = blockIdx.y;
    uint32_t id = ids[b];
    if (id >= rows) id = 0;   // out-of-range token ids read row 0 instead of faulting
    PbTables T;
    T.iq3s = PB_IQ3S_GRID; T.iq2xs = PB_IQ2XS_GRID; T.ksigns = PB_KSIGNS_IQ2XS;
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
#define LAUNCH() pb_embed_kernel<FMT><<<grid, 32, 0, ctx->stream>>>(w, rows, row_bytes, ids, out, ldo)
    PB_DISPATCH_FMT(type, LAUNCH);
#undef LAUNCH
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

// sampler::argmax, src/sampler.rs:142-148: first index of the maximum.  grid (t), 1024 threads
__global__ void __launch_bounds__(1024) pb_argmax_kernel(const float* __restrict__ logits, int64_t ld, int n, uint32_t* __restrict__ out) {
    const float* v = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += 1024) { const float x = v[i]; if (x > best || (x == best && i < bi)) { best = x; bi = i; } }
    __shared__ float sv[32]; __shared__ int si[32];
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sv[threadIdx.x]; bi = si[threadIdx.x];
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0u : (uint32_t)bi;   // all-NaN row: index 0, like the reference loop
    }
}

int pb_launch_argmax(pb_ctx* ctx, const float* logits, int64_t ld, int n, int t, uint32_t* out) {
    pb_argmax_kernel<<<t, 1024, 0, ctx->stream>>>(logits, ld, n, out);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

// end of a decode step: pos += 1; optionally feed the chosen tokens back as the next inputs and log them
__global__ void pb_advance_kernel(int64_t* pos, int t, const uint32_t* next, uint32_t* ids, uint32_t* trace, int64_t* trace_len, int64_t trace_cap) {
    const int b = threadIdx.x;
    if (b >= t) return;
    pos[b] += 1;
    if (next && ids) ids[b] = next[b];
    if (next && trace && trace_len) { const int64_t k = *trace_len; if (k < trace_cap) trace[k * t + b] = next[b]; }
    __syncthreads();
    if (b == 0 && trace_len && next && trace) *trace_len += 1;
}

int pb_launch_advance(pb_ctx* ctx, int64_t* pos, int t, const uint32_t* next, uint32_t* ids, uint32_t* trace, int64_t* trace_len, int64_t trace_cap) {
    pb_advance_kernel<<<1, t < 32 ? 32 : ((t + 31) & ~31), 0, ctx->stream>>>(pos, t, next, ids, trace, trace_len, trace_cap);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
