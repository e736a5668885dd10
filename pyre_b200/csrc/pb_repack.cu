// IQ3_S -> PB_T_IQ3S_N4: a lossless re-coding done once when a matrix arrives on the device.
//
// An IQ3_S weight is  d * (1 + 2 s) * sign * g  (dequant, gguf_q.rs:141-151) where g is one byte of a
// codebook entry.  All 2048 codebook bytes are odd numbers 1..15, so sign * g is one of the sixteen values
// -15, -13, .. 15 = 2 c - 15 with a 4-bit code c.  The re-coded block keeps d and the 4-bit sub-scales
// unchanged and stores c for every weight: 136 bytes per 256 weights instead of 110.  The streaming kernels
// then spend two logic operations per eight weights on decoding instead of a codebook walk with sign
// arithmetic, which is what kept the native format at a third of the HBM roofline; the values they
// multiply are bit-identical.
#include "pb_internal.h"
#include "pb_formats.cuh"

// one thread per output word (8 weights); 32 threads per block of 256 weights
__global__ void __launch_bounds__(256) pb_repack_iq3s_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t nblocks, int* bad) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t blk = i >> 5;
    const int m = (int)(i & 31);
    if (blk >= nblocks) return;
    const uint8_t* p = src + blk * 110;
    uint8_t* q = dst + blk * 136;
    if (m == 0) {
        q[0] = p[0]; q[1] = p[1]; q[2] = 0; q[3] = 0;
        q[4] = p[106]; q[5] = p[107]; q[6] = p[108]; q[7] = p[109];
    }
    // word m = weights 8m .. 8m+7 = codebook entries 2m and 2m+1, sign byte m
    const uint32_t qh = p[66 + (m >> 2)] >> (2 * (m & 3));
    const uint32_t g0 = PB_IQ3S_GRID[p[2 + 2 * m] | ((qh & 1) << 8)];
    const uint32_t g1 = PB_IQ3S_GRID[p[3 + 2 * m] | ((qh & 2) << 7)];
    const uint32_t sg = p[74 + m];
    uint32_t w = 0;
    bool odd = true;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int a = (int)((g0 >> (8 * j)) & 0xFF), b = (int)((g1 >> (8 * j)) & 0xFF);
        odd = odd && (a & 1) && a <= 15 && (b & 1) && b <= 15;
        const int va = (sg >> j) & 1 ? -a : a, vb = (sg >> (4 + j)) & 1 ? -b : b;
        w |= (uint32_t)(((va + 15) >> 1) & 0xF) << (8 * j);
        w |= (uint32_t)(((vb + 15) >> 1) & 0xF) << (8 * j + 4);
    }
    if (!odd) atomicExch(bad, PB_DEV_BAD_INDEX);   // cannot happen with the IQ3_S codebook; checked rather than assumed
    reinterpret_cast<uint32_t*>(q + 8)[m] = w;
}

int pb_launch_repack_iq3s(pb_ctx* ctx, const uint8_t* src, uint8_t* dst, int64_t nblocks) {
    if (nblocks <= 0) return PB_OK;
    const int64_t threads = nblocks * 32;
    pb_repack_iq3s_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, ctx->stream>>>(src, dst, nblocks, ctx->dev_status);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
