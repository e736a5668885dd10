// Bit-exact dequantization to f32 and the seeded synthetic-weight generator.
//
// dequant: restates dequant(), src/model/gguf_q.rs:67-166 of the reference, one warp per
// 256-weight step (lane = one 8-weight unit, see pb_formats.cuh).
// synth: benchmark weights generated in place on the GPU.  The byte stream is specified
// in terms of splitmix64 only (no libm), so a host program can reproduce any block.
#include "pb_formats.cuh"
#include "pb_internal.h"

#include <stdio.h>

template <int FMT>
__global__ void __launch_bounds__(256) pb_dequant_kernel(const uint8_t* __restrict__ w, int64_t n_units, float* __restrict__ out) {
    using F = PbFmt<FMT>;
    const int lane = threadIdx.x & 31;
    const int64_t step = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (step * 32 >= n_units) return;
    if (step * 32 + (FMT == PB_T_Q4_K ? 0 : lane) >= n_units) return;  // ragged tail (formats with 32-wide blocks)
    PbTables T;
    T.iq3s = PB_IQ3S_GRID; T.iq2xs = PB_IQ2XS_GRID; T.ksigns = PB_KSIGNS_IQ2XS; T.iq3xxs = PB_IQ3XXS_GRID; T.iq2s = PB_IQ2S_GRID; T.kvalues = PB_KVALUES_IQ4NL; T.iq2xxs = PB_IQ2XXS_GRID; T.iq1s = PB_IQ1S_GRID;
    PbUnit u;
    F::unit(w + step * F::STEP_BYTES, lane, T, u);
    float* o = out + step * 256;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float s = j < 4 ? u.sa : u.sb;
        float v = __fmul_rn(s, u.w[j]);
        if (F::HAS_MIN) v = __fsub_rn(v, j < 4 ? u.ma : u.mb);
        o[F::pos(lane, j)] = v;
    }
}

int pb_launch_dequant(pb_ctx* ctx, int type, const uint8_t* w, int64_t n_units, float* out) {
    if (n_units <= 0) return PB_OK;
    const int64_t steps = (n_units + 31) / 32;
    const unsigned grid = (unsigned)((steps + 7) / 8);
#define LAUNCH() pb_dequant_kernel<FMT><<<grid, 256, 0, ctx->stream>>>(w, n_units, out)
    PB_DISPATCH_FMT(type, LAUNCH);
#undef LAUNCH
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

// ---------------------------------------------------------------------------------------
// Synthetic tensors.
//   sm64(x)    = splitmix64 finaliser of x + 0x9E3779B97F4A7C15
//   tkey       = sm64(sm64(seed) ^ tensor_id)
//   bkey(b)    = sm64(tkey ^ (b * 0xD1342543DE82EF95))      b = block (or f32 element) index
//   word(b, j) = sm64(bkey(b) + j)
//   normal     = (sum of the twelve 16-bit fields of three words - 393210) / 65536
//   scale      = f16(|normal| * 0.02)                       i.e. d ~ |N(0, 0.02)|
// Q8_0: d = scale(words 0-2), q[j] = byte j of words 3-6, mod 255, minus 127 (uniform -127..127)
// Q4_K: d = scale(0-2), dmin = scale(3-5), the 140 payload bytes = words 6..
// IQ2_XS / IQ3_S: d = scale(0-2), the 72 / 108 payload bytes = words 3..  (uniform bytes give
// uniform sub-scales, grid indices and sign bits)
// f32: element i = normal(words 0-2 of bkey(i)) * sigma
__host__ __device__ static inline uint64_t pb_sm64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__device__ static inline float pb_synth_normal(uint64_t bkey, int j0) {
    int s = 0;
#pragma unroll
    for (int j = 0; j < 3; j++) {
        const uint64_t w = pb_sm64(bkey + (uint64_t)(j0 + j));
        s += (int)(w & 0xFFFF) + (int)((w >> 16) & 0xFFFF) + (int)((w >> 32) & 0xFFFF) + (int)(w >> 48);
    }
    return __fmul_rn((float)(s - 393210), 1.0f / 65536.0f);
}
__device__ static inline uint16_t pb_synth_scale(uint64_t bkey, int j0) {
    return __half_as_ushort(__float2half_rn(__fmul_rn(fabsf(pb_synth_normal(bkey, j0)), 0.02f)));
}

template <int FMT>
__global__ void __launch_bounds__(256) pb_synth_kernel(uint8_t* __restrict__ w, int64_t nblocks, uint64_t tkey, int64_t block0) {
    constexpr int BS = FMT == PB_T_Q8_0 ? 34 : (FMT == PB_T_IQ4_NL || FMT == PB_T_Q2_0 || FMT == PB_T_Q4_0 ? 18 : (FMT == PB_T_Q5_0 ? 22 : PbFmt<FMT>::STEP_BYTES));
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const uint64_t k = pb_sm64(tkey ^ ((uint64_t)(block0 + b) * 0xD1342543DE82EF95ull));
    uint16_t* o = reinterpret_cast<uint16_t*>(w + b * BS);  // every block size is even
    o[0] = pb_synth_scale(k, 0);
    int j0 = 3, off = 1, payload = BS - 2;
    if (FMT == PB_T_Q4_K || FMT == PB_T_Q5_K) { o[1] = pb_synth_scale(k, 3); j0 = 6; off = 2; payload = FMT == PB_T_Q4_K ? 140 : 172; }
    if (FMT == PB_T_Q3_K) { off = 0; payload = 108; }   // the f16 scale closes the block
    if (FMT == PB_T_Q6_K) { off = 0; payload = 208; }   // the f16 scale closes the block
    if (FMT == PB_T_IQ1_M) { off = 0; payload = 56; }   // no scale of its own at the front
    for (int i = 0; i < payload; i += 8) {
        const uint64_t v = pb_sm64(k + (uint64_t)(j0 + i / 8));
#pragma unroll
        for (int h = 0; h < 4; h++) {
            if (i + 2 * h >= payload) break;
            uint32_t two = (uint32_t)(v >> (16 * h)) & 0xFFFF;
            if (FMT == PB_T_Q8_0) {
                const uint32_t lo = (uint32_t)(int8_t)((int)((two & 0xFF) % 255) - 127) & 0xFF;
                const uint32_t hi = (uint32_t)(int8_t)((int)((two >> 8) % 255) - 127) & 0xFF;
                two = lo | (hi << 8);
            }
            o[off + i / 2 + h] = (uint16_t)two;
        }
    }
    if (FMT == PB_T_Q3_K) o[54] = pb_synth_scale(k, 0);
    if (FMT == PB_T_IQ1_M) {   // the f16 scale goes, a nibble each, into the top of the four scale words
        const uint32_t d = pb_synth_scale(k, 0);
        for (int i = 0; i < 4; i++) o[24 + i] = (uint16_t)((o[24 + i] & 0x0FFF) | (((d >> (4 * i)) & 0xF) << 12));
    }
    if (FMT == PB_T_Q6_K) {   // sub-block scales kept to -8..7
        for (int i = 96; i < 104; i++) {
            const uint32_t two = o[i];
            o[i] = (uint16_t)(((uint32_t)((int)(two & 15) - 8) & 0xFF) | (((uint32_t)((int)((two >> 8) & 15) - 8) & 0xFF) << 8));
        }
        o[104] = pb_synth_scale(k, 0);
    }
}

__global__ void __launch_bounds__(256) pb_synth_normal_kernel(float* __restrict__ out, int64_t n, uint64_t tkey, float sigma, int64_t i0) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t k = pb_sm64(tkey ^ ((uint64_t)(i0 + i) * 0xD1342543DE82EF95ull));
    out[i] = __fmul_rn(pb_synth_normal(k, 0), sigma);
}

int pb_launch_synth(pb_ctx* ctx, int type, uint8_t* w, int64_t nblocks, uint64_t seed, uint64_t tid, int64_t block0) {
    const uint64_t tkey = pb_sm64(pb_sm64(seed) ^ tid);
    const unsigned grid = (unsigned)((nblocks + 255) / 256);
    switch (type) {
        case PB_T_Q8_0: pb_synth_kernel<PB_T_Q8_0><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_Q4_K: pb_synth_kernel<PB_T_Q4_K><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_IQ2_XS: pb_synth_kernel<PB_T_IQ2_XS><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_IQ3_S: pb_synth_kernel<PB_T_IQ3_S><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_IQ3_XXS: pb_synth_kernel<PB_T_IQ3_XXS><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_IQ2_S: pb_synth_kernel<PB_T_IQ2_S><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_IQ4_NL: pb_synth_kernel<PB_T_IQ4_NL><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_IQ4_XS: pb_synth_kernel<PB_T_IQ4_XS><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_Q2_0: pb_synth_kernel<PB_T_Q2_0><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_IQ2_XXS: pb_synth_kernel<PB_T_IQ2_XXS><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_Q6_K: pb_synth_kernel<PB_T_Q6_K><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_IQ1_M: pb_synth_kernel<PB_T_IQ1_M><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_Q4_0: pb_synth_kernel<PB_T_Q4_0><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_Q5_0: pb_synth_kernel<PB_T_Q5_0><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_Q3_K: pb_synth_kernel<PB_T_Q3_K><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        case PB_T_Q5_K: pb_synth_kernel<PB_T_Q5_K><<<grid, 256, 0, ctx->stream>>>(w, nblocks, tkey, block0); break;
        default: PB_FAIL(ctx, PB_ERR_ARG, "pb_qmat_synth: no generator for ggml type %d", type);
    }
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

int pb_launch_synth_normal(pb_ctx* ctx, float* out, int64_t n, uint64_t seed, uint64_t tid, float sigma) {
    return pb_launch_synth_normal_at(ctx, out, n, seed, tid, 0, sigma);
}

// elements i0 .. i0+n of the synthetic f32 tensor (seed, tid)
int pb_launch_synth_normal_at(pb_ctx* ctx, float* out, int64_t n, uint64_t seed, uint64_t tid, int64_t i0, float sigma) {
    if (n <= 0) return PB_OK;
    const uint64_t tkey = pb_sm64(pb_sm64(seed) ^ tid);
    pb_synth_normal_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(out, n, tkey, sigma, i0);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
