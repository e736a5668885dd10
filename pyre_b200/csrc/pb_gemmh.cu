// Batched dequant-GEMM for 4..16 activation columns on the tensor cores (IQ3_S weights).
//
//   y[b][yoff_s + r] (+)= sum_c W_s[r][c] * act(x)[b][c]        b = 0 .. t-1 (t <= 16)
//
// Used where one weight matrix meets several tokens at once (batched decode, verify windows):
// the weight bytes are streamed and decoded ONCE for all columns, instead of once per column
// as in the dp4a GEMV.  Same streaming skeleton (persistent CTAs, producer warp, 1-D bulk
// copies into a 4-stage ring, bounded mbarrier waits); the arithmetic is
// mma.sync.m16n8k16 (f16 x f16 -> f32):
//   - A = 16 rows of decoded weights.  The codebook lives in shared memory as four f16 per
//     entry; the sub-block multiplier (1 + 2*s <= 31) is folded in exactly (|w| <= 465), the f16
//     block scale d is applied in f32 once per 256-weight block.
//   - B = activations split into f16 high and low parts (x = hi + lo, 22 significant bits),
//     laid out in shared memory in fragment order; an n-tile holds 4 tokens x (hi, lo), so a
//     thread owns both halves of its tokens and adds them itself.
//   - the contraction index inside a block is permuted so that thread q of a quad owns the 64
//     consecutive weights of quarter q (one decode per lane, as in the GEMV); A and B use the
//     same permutation, so the sum is unchanged.
// A chunk is 16 rows; the eight consumer warps split its blocks (K) and meet in shared memory.
// Replaces the reference's batched GEMV / prefill GEMM (k_gemv4*, k_gemm_pf / k_gemm_tc,
// src/model/qn_cube.rs:71-233, 293-1159) for IQ3_S; other formats keep the dp4a kernel.
#include "pb_stream.cuh"
#include "pb_internal.h"

#include <cuda_fp16.h>
#include <stdio.h>

#define GH_CONSUMERS 8
#define GH_THREADS ((GH_CONSUMERS + 1) * 32)
#define GH_ROWS 16

__device__ __forceinline__ void pb_mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One quarter (64 weights) of an IQ3_S block as 32 half2 words with the sub-block multiplier and
// the signs applied; returns the block scale d.  tab_h: this lane's copy of the f16 codebook (512 x 4 f16,
// four interleaved copies: entry i of copy c at (4 i + c) * 8 bytes, so lanes of different copies never share a bank).
__device__ __forceinline__ float pb_iq3s_quarter_h(uint32_t p, int qt, uint32_t tab_h, uint32_t (&h)[32]) {
    const float d = pb_h2f((uint16_t)pb_lds16(p));
    uint32_t qs[4], sg[2];
    pb_ld_u32x<4>(p + 2 + 16 * qt, qs);
    pb_ld_u32x<2>(p + 74 + 8 * qt, sg);
    const uint32_t qh = pb_lds16(p + 66 + 2 * qt);
    const uint32_t sc = pb_lds8(p + 106 + qt);
    const __half2 m0 = __half2half2(__int2half_rn(1 + 2 * (int)(sc & 0xF))), m1 = __half2half2(__int2half_rn(1 + 2 * (int)(sc >> 4)));
#pragma unroll
    for (int u = 0; u < 8; u++) {
        const uint32_t hb = pb_spread4((qh >> (4 * (u >> 1))) & 0xF);
        const uint32_t i0 = (u & 1) ? pb_iq3s_index<2>(qs[u >> 1], hb) : pb_iq3s_index<0>(qs[u >> 1], hb);
        const uint32_t i1 = (u & 1) ? pb_iq3s_index<3>(qs[u >> 1], hb) : pb_iq3s_index<1>(qs[u >> 1], hb);
        const uint2 g0 = pb_lds64(tab_h + i0 * 32), g1 = pb_lds64(tab_h + i1 * 32);
        // f16 sign bits by arithmetic: bit k of a nibble -> 0x80 in byte k, then into bytes 1 and 3 of two words
        const uint32_t sb = sg[u >> 2] >> (8 * (u & 3));
        const uint32_t ca = ((sb & 0xF) * 0x10204080u) & 0x80808080u, cb = (((sb >> 4) & 0xF) * 0x10204080u) & 0x80808080u;
        const uint32_t s00 = __byte_perm(ca, 0, 0x1404), s01 = __byte_perm(ca, 0, 0x3424);
        const uint32_t s10 = __byte_perm(cb, 0, 0x1404), s11 = __byte_perm(cb, 0, 0x3424);
        const __half2 mm = u < 4 ? m0 : m1;
        __half2 a;
        a = __hmul2(*reinterpret_cast<const __half2*>(&g0.x), mm); h[4 * u + 0] = *reinterpret_cast<uint32_t*>(&a) ^ s00;
        a = __hmul2(*reinterpret_cast<const __half2*>(&g0.y), mm); h[4 * u + 1] = *reinterpret_cast<uint32_t*>(&a) ^ s01;
        a = __hmul2(*reinterpret_cast<const __half2*>(&g1.x), mm); h[4 * u + 2] = *reinterpret_cast<uint32_t*>(&a) ^ s10;
        a = __hmul2(*reinterpret_cast<const __half2*>(&g1.y), mm); h[4 * u + 3] = *reinterpret_cast<uint32_t*>(&a) ^ s11;
    }
    return d;
}

// The same 32 half2 words from a block re-coded into 4-bit codes (PB_T_IQ3S_N4, weight = 2 c - 15): a byte
// permute puts two codes into the mantissas of two f16 with the exponent of 1024 (0x6400 | c = 1024 + c,
// exact), one subtraction leaves c, one fused multiply-add makes (2 c - 15) * multiplier -- all exact in
// f16, so the words equal those of pb_iq3s_quarter_h bit for bit.
__device__ __forceinline__ float pb_n4_quarter_h(uint32_t p, int qt, uint32_t (&h)[32]) {
    const float d = pb_h2f((uint16_t)(pb_lds32(p) & 0xFFFF));
    const uint32_t sc = pb_lds8(p + 4 + qt);
    const float f0 = (float)(1 + 2 * (int)(sc & 0xF)), f1 = (float)(1 + 2 * (int)(sc >> 4));
    const __half2 a0 = __float2half2_rn(2.0f * f0), b0 = __float2half2_rn(-15.0f * f0);
    const __half2 a1 = __float2half2_rn(2.0f * f1), b1 = __float2half2_rn(-15.0f * f1);
    const __half2 k1024 = __float2half2_rn(1024.0f);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint2 c = pb_lds64(p + 8 + 32 * qt + 8 * i);
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int u = 2 * i + j;
            const uint32_t w = j ? c.y : c.x;
            const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
            const uint32_t r[4] = {pb_prmt(lo, 0x64006400u, 0x7150u), pb_prmt(lo, 0x64006400u, 0x7352u), pb_prmt(hi, 0x64006400u, 0x7150u), pb_prmt(hi, 0x64006400u, 0x7352u)};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const __half2 v = __hfma2(__hsub2(*reinterpret_cast<const __half2*>(&r[e]), k1024), u < 4 ? a0 : a1, u < 4 ? b0 : b1);
                h[4 * u + e] = *reinterpret_cast<const uint32_t*>(&v);
            }
        }
    }
    return d;
}

// byte offset of the 8-byte B-fragment slot of (block blk, entry j, n-tile nt, token-in-tile tq, level lv, quarter q).
// The slots of n-tiles 2p and 2p+1 of one lane are adjacent, so one 128-bit load feeds two mma.
__device__ __forceinline__ uint32_t pb_xh_off(int blk, int j, int nt, int NT, int tq, int lv, int q) {
    const int lane = (2 * tq + lv) * 4 + q;
    if (NT == 1) return (uint32_t)(((blk * 16 + j) * 32 + lane) * 8);
    return (uint32_t)(((((blk * 16 + j) * (NT / 2) + (nt >> 1)) * 32 + lane) * 2 + (nt & 1)) * 8);
}

// store 4 consecutive activations (elements c .. c+3, c % 4 == 0) of token b as f16 hi / lo fragments
__device__ __forceinline__ void pb_xh_store(uint8_t* xh, int NT, int b, int c, float4 v) {
    const int blk = c >> 8, q = (c >> 6) & 3, j = (c >> 2) & 15, nt = b >> 2, tq = b & 3;
    const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
    const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
    const __half2 l01 = __floats2half2_rn(v.x - f01.x, v.y - f01.y), l23 = __floats2half2_rn(v.z - f23.x, v.w - f23.y);
    *reinterpret_cast<uint2*>(xh + pb_xh_off(blk, j, nt, NT, tq, 0, q)) = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
    *reinterpret_cast<uint2*>(xh + pb_xh_off(blk, j, nt, NT, tq, 1, q)) = make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
}

// Activations of all t tokens of a GEMM -> f16 high / low parts in B-fragment order, written once to
// global memory for all CTAs of all its launches.  The tokens are cut into tiles of `tile` (16 or 8);
// a tile of tt tokens uses NT = 1 / 2 / 4 n-tiles (4 * NT token slots, the unused ones zero) and lives at
// xbuf + tile_index * tile_stride: 256 bytes of per-token prescale inverses, then the fragments.
// grid = number of tiles * tile CTAs (one token slot each), 256 threads.  PLAIN columns get an exact
// power-of-two prescale into [0.5, 1) (f16 neither overflows nor loses small columns).
__global__ void __launch_bounds__(256) pb_xh_prep_kernel(const PbGemvQParams p, uint8_t* __restrict__ xbuf, int tile, size_t tile_stride) {
    constexpr int CT = 256;
    const int ti = (int)blockIdx.x / tile, b = (int)blockIdx.x - ti * tile;   // tile, slot inside the tile
    const int tt = min(tile, p.t - ti * tile);                                  // tokens of this tile
    const int NT = tt <= 4 ? 1 : (tt <= 8 ? 2 : 4);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cols = p.bpr * 256;
    __shared__ float red0[8];
    pb_pdl_wait();
    pb_pdl_trigger();
    if (b >= 4 * NT) return;
    const bool live = b < tt;
    const float* x = p.x + (size_t)(ti * tile + b) * p.ldx;
    const float* z = p.z ? p.z + (size_t)(ti * tile + b) * p.ldz : nullptr;
    uint8_t* xh = xbuf + (size_t)ti * tile_stride + 256;
    float* xinv = reinterpret_cast<float*>(xbuf + (size_t)ti * tile_stride);
    if (tid == 0 && blockIdx.y == 0) xinv[b] = 1.0f;
    if (p.mode == PB_ACT_GNORM) {
        const int nheads = cols / p.head_dim;   // head_dim == 128 (checked on the host); the heads are spread over grid.y
        for (int h = warp + 8 * (int)blockIdx.y; h < nheads; h += 8 * (int)gridDim.y) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live) {
                v = *reinterpret_cast<const float4*>(x + h * p.head_dim + 4 * lane);
                const float ss = pb_warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
                const float s = 1.0f / sqrtf(ss / (float)p.head_dim + p.eps);
                const float4 w = *reinterpret_cast<const float4*>(p.norm_w + 4 * lane);
                const float4 zz = *reinterpret_cast<const float4*>(z + h * p.head_dim + 4 * lane);
                v.x = v.x * (s * w.x) * pb_sigm(zz.x); v.y = v.y * (s * w.y) * pb_sigm(zz.y); v.z = v.z * (s * w.z) * pb_sigm(zz.z); v.w = v.w * (s * w.w) * pb_sigm(zz.w);
            }
            pb_xh_store(xh, NT, b, h * p.head_dim + 4 * lane, v);
        }
        return;
    }
    // one CTA-wide reduction: sum of squares (NORM) or largest magnitude (PLAIN)
    float r = 0.f;
    if (live) for (int c = tid; c < cols; c += CT) { const float v = x[c]; r = p.mode == PB_ACT_NORM ? r + v * v : fmaxf(r, fabsf(v)); }
    r = p.mode == PB_ACT_NORM ? pb_warp_sum(r) : pb_warp_max(r);
    if (lane == 0) red0[warp] = r;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot = p.mode == PB_ACT_NORM ? tot + red0[i] : fmaxf(tot, red0[i]);
    float s = 1.0f;
    if (p.mode == PB_ACT_NORM) s = 1.0f / sqrtf(tot / (float)cols + p.eps);
    else if (tot > 0.f && tot <= 3.0e38f) {
        int e; (void)frexpf(tot, &e);
        s = ldexpf(1.0f, -e);
        if (tid == 0) xinv[b] = ldexpf(1.0f, e);
    }
    for (int c = tid * 4; c < cols; c += CT * 4) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            v = *reinterpret_cast<const float4*>(x + c);
            if (p.mode == PB_ACT_NORM) { const float4 w = *reinterpret_cast<const float4*>(p.norm_w + c); v.x = v.x * s * w.x; v.y = v.y * s * w.y; v.z = v.z * s * w.z; v.w = v.w * s * w.w; }
            else { v.x *= s; v.y *= s; v.z *= s; v.w *= s; }
        }
        pb_xh_store(xh, NT, b, c, v);
    }
}

// NST = stages of the ring (4; 2 for rows wider than 2048 columns, whose fragments leave less room)
// RC: the weights are the re-coded copy (136-byte blocks, no codebook table)
template <int NT, int NST, bool RC>
__global__ void __launch_bounds__(GH_THREADS, 1) pb_gemmh_iq3s_kernel(const PbGemvQParams p) {
    constexpr int NB = 4 * NT;
    extern __shared__ __align__(128) uint8_t smem[];
    PbRing ring;
    ring.full = reinterpret_cast<uint64_t*>(smem);
    ring.empty = ring.full + NST;
    float* red0 = reinterpret_cast<float*>(smem + 64);            // GH_CONSUMERS floats
    float* xinv = reinterpret_cast<float*>(smem + 128);           // per token: inverse of the power-of-two prescale
    uint64_t* xbar = reinterpret_cast<uint64_t*>(smem + 192);     // completion of the fragment copies
    uint8_t* tab = smem + 256;                                    // f16 codebook, four interleaved copies (16 KB)
    const int cols = p.bpr * 256;
    uint8_t* xh = tab + (RC ? 0 : 16384);                         // B fragments: cols * NB * 4 bytes
    float* red = reinterpret_cast<float*>(xh + (size_t)cols * NB * 4);   // [2][GH_CONSUMERS][16 rows][NB]
    ring.stages = reinterpret_cast<uint8_t*>(red) + 2 * GH_CONSUMERS * GH_ROWS * NB * 4;
    ring.stage_bytes = p.stage_bytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pb_pdl_trigger();
    if (tid == 0) {
        for (int s = 0; s < NST; s++) { pb_mbar_init(&ring.full[s], 1); pb_mbar_init(&ring.empty[s], GH_CONSUMERS); }
        pb_mbar_init(xbar, 1);
        pb_fence_barrier_init();
    }
    __syncthreads();
    const int my_chunks = p.nchunks > (int)blockIdx.x ? (p.nchunks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (warp == GH_CONSUMERS) {
        if (lane == 0) {
            int k = 0;
            bool x_issued = false;
            for (; k < my_chunks; k++) {
                if (k == NST && !x_issued) {
                    // the ring is full of weights (which no earlier kernel writes): now wait for the kernel
                    // that made the fragments and bring them in, in pieces of 16 KB
                    pb_pdl_wait();
                    const uint32_t xbytes = (uint32_t)cols * NB * 4;
                    pb_mbar_expect_tx(xbar, xbytes);
                    for (uint32_t o = 0; o < xbytes; o += 16384) pb_bulk_g2s(xh + o, p.xh_in + o, min(16384u, xbytes - o), xbar);
                    x_issued = true;
                }
                const int chunk = (int)blockIdx.x + k * (int)gridDim.x;
                int s = 0;
                while (s + 1 < p.nseg && chunk >= p.seg[s + 1].chunk0) s++;
                const int r0 = (chunk - p.seg[s].chunk0) * GH_ROWS;
                const int nr = min(GH_ROWS, p.seg[s].rows - r0);
                const uint32_t bytes = ((uint32_t)nr * (uint32_t)p.row_bytes + 15u) & ~15u;
                const int st = k % NST;
                if (k >= NST && !pb_mbar_wait_relaxed(&ring.empty[st], ((k / NST) - 1) & 1, p.status, PB_DEV_WAIT_EMPTY_TIMEOUT)) break;
                pb_mbar_expect_tx(&ring.full[st], bytes);
                pb_bulk_g2s(ring.stages + (size_t)st * ring.stage_bytes, p.seg[s].w + (size_t)r0 * p.row_bytes, bytes, &ring.full[st]);
            }
            if (!x_issued) {
                pb_pdl_wait();
                const uint32_t xbytes = (uint32_t)cols * NB * 4;
                pb_mbar_expect_tx(xbar, xbytes);
                for (uint32_t o = 0; o < xbytes; o += 16384) pb_bulk_g2s(xh + o, p.xh_in + o, min(16384u, xbytes - o), xbar);
            }
            // error path: give the copies in flight a bounded chance to land before the CTA may exit
            if (k < my_chunks) {
                for (int j = max(0, k - NST); j < k; j++) pb_mbar_wait(&ring.full[j % NST], (j / NST) & 1, nullptr, 0);
                pb_mbar_wait(xbar, 0, nullptr, 0);
            }
        }
        return;
    }

    // ---- consumers: tables ----
    constexpr int CT = GH_CONSUMERS * 32;
    if (!RC) {   // the re-coded form needs no codebook (and the fragments start where the table would be)
        uint2* gh = reinterpret_cast<uint2*>(tab);
        for (int i = tid; i < 512; i += CT) {
            const uint32_t g = PB_IQ3S_GRID[i];
            const __half2 a = __floats2half2_rn((float)(g & 0xFF), (float)((g >> 8) & 0xFF)), b = __floats2half2_rn((float)((g >> 16) & 0xFF), (float)(g >> 24));
            const uint2 e = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
            gh[4 * i] = e; gh[4 * i + 1] = e; gh[4 * i + 2] = e; gh[4 * i + 3] = e;
        }
    }
    const uint32_t tab_h = pb_smem_u32(tab) + (lane & 3) * 8;
    if (tid < NB) xinv[tid] = 1.0f;
    pb_named_barrier(2, CT);
    pb_pdl_wait();
    // ---- f16 hi/lo fragments and prescales made by pb_xh_prep_kernel: wait for the producer's bulk copies ----
    if (tid < NB) xinv[tid] = p.xinv_in[tid];
    if (!pb_mbar_wait(xbar, 0, p.status, PB_DEV_WAIT_FULL_TIMEOUT)) return;
    pb_named_barrier(1, CT);

    const int g = lane >> 2, q = lane & 3;
    const uint32_t xh_s = pb_smem_u32(xh);
    for (int k = 0; k < my_chunks; k++) {
        if (!pb_mbar_wait(&ring.full[k % NST], (k / NST) & 1, p.status, PB_DEV_WAIT_FULL_TIMEOUT)) return;
        const int chunk = (int)blockIdx.x + k * (int)gridDim.x;
        int s = 0;
        while (s + 1 < p.nseg && chunk >= p.seg[s + 1].chunk0) s++;
        const int r0 = (chunk - p.seg[s].chunk0) * GH_ROWS;
        const int nr = min(GH_ROWS, p.seg[s].rows - r0);
        const uint32_t base = pb_smem_u32(ring.stages + (size_t)(k % NST) * ring.stage_bytes);
        float tot[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) { tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.f; }
        for (int blk = warp; blk < p.bpr; blk += GH_CONSUMERS) {   // K split: this warp's blocks of the 16 rows
            uint32_t ha[32], hb[32];
            // rows g and g + 8 (rows past the end of the matrix decode stale bytes of the stage; never stored)
            const float da = RC ? pb_n4_quarter_h(base + (uint32_t)g * p.row_bytes + blk * 136, q, ha) : pb_iq3s_quarter_h(base + (uint32_t)g * p.row_bytes + blk * 110, q, tab_h, ha);
            const float db = RC ? pb_n4_quarter_h(base + (uint32_t)(g + 8) * p.row_bytes + blk * 136, q, hb) : pb_iq3s_quarter_h(base + (uint32_t)(g + 8) * p.row_bytes + blk * 110, q, tab_h, hb);
            float acc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
#pragma unroll
            for (int j = 0; j < 16; j++) {
                if (NT == 1) {
                    const uint2 bx = pb_lds64(xh_s + (uint32_t)(((blk * 16 + j) * 32 + lane) * 8));
                    pb_mma_f16(acc[0], ha[2 * j], hb[2 * j], ha[2 * j + 1], hb[2 * j + 1], bx.x, bx.y);
                } else {
#pragma unroll
                    for (int np = 0; np < NT / 2; np++) {
                        const uint4 bx = pb_lds128(xh_s + (uint32_t)((((blk * 16 + j) * (NT / 2) + np) * 32 + lane) * 16));
                        pb_mma_f16(acc[2 * np], ha[2 * j], hb[2 * j], ha[2 * j + 1], hb[2 * j + 1], bx.x, bx.y);
                        pb_mma_f16(acc[2 * np + 1], ha[2 * j], hb[2 * j], ha[2 * j + 1], hb[2 * j + 1], bx.z, bx.w);
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                tot[nt][0] = fmaf(da, acc[nt][0], tot[nt][0]); tot[nt][1] = fmaf(da, acc[nt][1], tot[nt][1]);
                tot[nt][2] = fmaf(db, acc[nt][2], tot[nt][2]); tot[nt][3] = fmaf(db, acc[nt][3], tot[nt][3]);
            }
        }
        __syncwarp();
        if (lane == 0) pb_mbar_arrive(&ring.empty[k % NST]);
        // this warp's partial [16 rows][NB tokens]: thread (g, q) owns rows g, g+8 and token 4*nt + q (hi + lo columns)
        float* mine = red + (size_t)((k & 1) * GH_CONSUMERS + warp) * GH_ROWS * NB;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            mine[g * NB + 4 * nt + q] = tot[nt][0] + tot[nt][1];
            mine[(g + 8) * NB + 4 * nt + q] = tot[nt][2] + tot[nt][3];
        }
        pb_named_barrier(1, CT);
        // 256 threads <-> 16 rows x up to 16 tokens
        for (int o = tid; o < GH_ROWS * NB; o += CT) {
            const int r = o / NB, b = o - r * NB;
            if (r < nr && b < p.t) {
                const float* src = red + (size_t)(k & 1) * GH_CONSUMERS * GH_ROWS * NB + o;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < GH_CONSUMERS; w++) v += src[(size_t)w * GH_ROWS * NB];
                v *= xinv[b];
                float* dst = p.y + b * p.ldy + p.seg[s].yoff + r0 + r;
                *dst = p.accumulate ? *dst + v : v;
            }
        }
        // the buffer of parity k & 1 is rewritten two chunks later, after the barrier of chunk k + 1
    }
}

template <int NT, int NST, bool RC>
static int launch_h(pb_ctx* ctx, const PbGemvQArgs& a, const uint8_t* tile_buf) {
    constexpr int NB = 4 * NT;
    PbGemvQParams p;
    memset(&p, 0, sizeof p);
    p.row_bytes = a.cols / 256 * (RC ? 136 : 110); p.bpr = a.cols / 256; p.nseg = a.nseg;
    p.x = a.x; p.ldx = a.ldx; p.t = a.t; p.y = a.y; p.ldy = a.ldy; p.status = ctx->dev_status;
    p.mode = a.mode; p.norm_w = a.norm_w; p.z = a.z; p.ldz = a.ldz; p.head_dim = a.head_dim; p.eps = a.eps; p.accumulate = a.accumulate;
    p.rows_per_chunk = GH_ROWS;
    int nchunks = 0;
    for (int s = 0; s < a.nseg; s++) {
        p.seg[s].w = RC ? a.seg[s].wr : a.seg[s].w; p.seg[s].rows = (int)a.seg[s].rows; p.seg[s].yoff = (int)a.seg[s].yoff; p.seg[s].chunk0 = nchunks;
        nchunks += (int)((a.seg[s].rows + GH_ROWS - 1) / GH_ROWS);
    }
    p.nchunks = nchunks;
    p.stage_bytes = (uint32_t)(((size_t)GH_ROWS * p.row_bytes + 16 + 127) & ~(size_t)127);
    const size_t smem = 256 + (RC ? 0 : 16384) + (size_t)a.cols * NB * 4 + 2 * GH_CONSUMERS * GH_ROWS * NB * 4 + (size_t)NST * p.stage_bytes;
    if (smem > (size_t)ctx->max_smem_optin) PB_FAIL(ctx, PB_UNSUPPORTED, "gemm: %zu bytes of shared memory needed for cols=%d t=%d", smem, a.cols, a.t);
    p.xh_in = tile_buf + 256; p.xinv_in = reinterpret_cast<const float*>(tile_buf);
    auto kern = pb_gemmh_iq3s_kernel<NT, NST, RC>;
    PB_TRY(pb_ensure_smem(ctx, kern, smem));
    const int grid = nchunks < ctx->sm_count ? nchunks : ctx->sm_count;
    pb_launch_k(ctx, kern, dim3(grid), dim3(GH_THREADS), smem, p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

bool pb_gemmh_supported(int type, int cols, int t) { return type == PB_T_IQ3_S && t >= 3 && cols % 256 == 0 && cols >= 256 && cols <= 4096; }

int pb_launch_gemmh(pb_ctx* ctx, const PbGemvQArgs& a) {
    if (!pb_gemmh_supported(a.type, a.cols, a.t)) PB_FAIL(ctx, PB_UNSUPPORTED, "gemm: type %d cols %d t %d", a.type, a.cols, a.t);
    if (a.mode == PB_ACT_PREQ) PB_FAIL(ctx, PB_UNSUPPORTED, "gemm: pre-split activations are not accepted");
    if (a.mode == PB_ACT_GNORM && a.head_dim != 128) PB_FAIL(ctx, PB_UNSUPPORTED, "gemm: gated norm over heads of %d (128 is built)", a.head_dim);
    if (((uintptr_t)a.x & 15) || (a.ldx & 3)) PB_FAIL(ctx, PB_ERR_ARG, "gemm: activations must be 16-byte aligned");
    // columns per launch: 16 with a 4-stage ring up to 2048 weight columns, 8 with a 2-stage ring above
    const bool wide = a.cols > 2048;
    const int tile = wide ? 8 : 16;
    const int ntiles = (a.t + tile - 1) / tile;
    const size_t tile_stride = 256 + (size_t)a.cols * tile * 4;
    if (ntiles * tile_stride > PB_XH_BYTES) PB_FAIL(ctx, PB_UNSUPPORTED, "gemm: %d tokens of %d columns exceed the %d-byte fragment buffer", a.t, a.cols, (int)PB_XH_BYTES);
    {   // fragments of all tokens, made once for all launches and CTAs of this GEMM
        PbGemvQParams p;
        memset(&p, 0, sizeof p);
        p.bpr = a.cols / 256; p.x = a.x; p.ldx = a.ldx; p.t = a.t; p.mode = a.mode; p.norm_w = a.norm_w; p.z = a.z; p.ldz = a.ldz; p.head_dim = a.head_dim; p.eps = a.eps;
        pb_launch_k(ctx, pb_xh_prep_kernel, dim3(ntiles * tile, p.mode == PB_ACT_GNORM ? 4 : 1), dim3(256), (size_t)0, p, ctx->xh_buf, tile, tile_stride);
        ctx->kernels_launched++;
        PB_CUDA(ctx, cudaGetLastError());
    }
    bool recoded = true;   // every segment has a re-coded copy
    for (int sg = 0; sg < a.nseg && sg < 4; sg++) recoded = recoded && a.seg[sg].wr != nullptr;
    int rc = PB_OK;
    for (int ti = 0; ti < ntiles && rc == PB_OK; ti++) {
        const int t0 = ti * tile;
        PbGemvQArgs s = a;
        s.t = a.t - t0 < tile ? a.t - t0 : tile;
        s.x = a.x + (int64_t)t0 * a.ldx; s.y = a.y + (int64_t)t0 * a.ldy; s.z = a.z ? a.z + (int64_t)t0 * a.ldz : nullptr;
        const uint8_t* tb = ctx->xh_buf + (size_t)ti * tile_stride;
        if (recoded) {
            if (wide) rc = s.t <= 4 ? launch_h<1, 2, true>(ctx, s, tb) : launch_h<2, 2, true>(ctx, s, tb);
            else rc = s.t <= 4 ? launch_h<1, 4, true>(ctx, s, tb) : (s.t <= 8 ? launch_h<2, 4, true>(ctx, s, tb) : launch_h<4, 4, true>(ctx, s, tb));
        } else if (wide) rc = s.t <= 4 ? launch_h<1, 2, false>(ctx, s, tb) : launch_h<2, 2, false>(ctx, s, tb);
        else rc = s.t <= 4 ? launch_h<1, 4, false>(ctx, s, tb) : (s.t <= 8 ? launch_h<2, 4, false>(ctx, s, tb) : launch_h<4, 4, false>(ctx, s, tb));
    }
    return rc;
}
