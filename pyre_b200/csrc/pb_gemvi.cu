// Dequant-GEMV for two tokens (one on request) on the integer tensor cores (re-coded IQ3_S weights).
//
//   y[b][yoff_s + r] (+)= sum_c W_s[r][c] * act(x)[b][c]        b = 0 .. t-1 (t <= 2)
//
// Persistent CTAs of up to twelve warps.  A warp (rows of up to 1024 columns) or a team of two warps (2048 columns,
// half a row each) owns a tile of 16 rows over all of K: it fetches its part of the tile with one bulk copy per row
// into one of its two private buffers (mbarrier per buffer, bounded wait) while it works on the other, so no warp
// waits for another except the two of a team, which meet once per tile to add their halves in a fixed order.  The dot:
//   - the activations of a token are split into PB_XLEVELS int8 levels with ONE scale per 256 values
//     and level, x = S1 q1 + S2 q2 + S3 q3 + e, |e| <= max|x| / (2 * 254^2 * 127).  The levels of the
//     tokens are the columns of the B operand of mma.sync.m16n8k32 (s8 x s8 -> s32): one instruction
//     multiplies 16 rows x 32 weights with all levels of two tokens, where the dp4a kernel issues
//     PB_XLEVELS instructions per row, token and 4 weights;
//   - a weight is 2 c - 15 with a 4-bit code c.  The code goes into the HIGH nibble of an s8 with its top
//     bit flipped, which reads as 16 (c - 8); with 8 * (sum of the level over the 32 weights) as the
//     accumulator input the instruction returns 8 * sum (2 c - 15) q exactly.  Unpacking eight codes
//     costs three logic operations;
//   - the sub-block multiplier 1 + 2 n (one per 32 weights and row) multiplies the integer result,
//     the f16 block scale and the level scale are applied once per 256 weights in f32.
// Rows lie in a buffer with a padded stride, so that the eight rows a load instruction touches fall into
// different shared-memory banks.
// Replaces QMat::matmul (src/model/gguf_q.rs:217-242) and the k_gemv* kernels (src/model/qn_cube.rs:257-2331)
// of the reference for two tokens of IQ3_S weights.
#include "pb_stream.cuh"
#include "pb_internal.h"
#include <stdlib.h>
#include <stdio.h>

#define GI_NCOL 8       // columns of the mma: two tokens x three levels, two idle
#define GI_SMAX 8       // 256-weight blocks per row at most (2048 columns)
#define GI_WARPS 12      // at most; the launch takes as many (an even number) as shared memory holds
#define GI_SBW 4        // 256-weight blocks of a row one warp takes (rows of 2048 columns are shared by two warps)
#define GI_THREADS (GI_WARPS * 32)
#define GI_OFF_PAIR 256
#define GI_OFF_S (GI_OFF_PAIR + 2 * GI_WARPS * 32 * 4)
#define GI_OFF_QS (GI_OFF_S + GI_NCOL * GI_SMAX * 4)

struct PbGemvIParams {
    PbGemvQParams q;    // seg[].chunk0 = first 16-row tile of the segment, nchunks = tiles in all
    int stride;         // bytes between rows of a tile in shared memory
    int sbw, ks;        // blocks per warp and row, warps per tile (bpr = sbw * ks)
    int xstride;        // bytes between the level arrays of two columns
    uint32_t buf_bytes; // one tile buffer
    uint32_t off_qs, off_xq, off_bufs;
};

__device__ __forceinline__ void pb_mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, int c0, int c1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
}

// One 256-value block of one token, held by a warp (lane l: values 8 l .. 8 l + 7): PB_XLEVELS int8 levels with one
// scale per level.  Writes the levels (bytes 8 l .. of the block in the column's level array), 8 * the sum of
// each level over every 32 values (the accumulator input) and the scales (already divided by that 8).
__device__ __forceinline__ void pb_split_block256(float (&r)[8], int lane, int sb, int b, uint8_t* xq, int xstride, int* qs, float* S) {
    const float kMagic = 12582912.0f;   // 1.5 * 2^23: adding it rounds to the nearest integer (ties to even)
#pragma unroll
    for (int l = 0; l < PB_XLEVELS; l++) {
        float m = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) m = fmaxf(m, fabsf(r[j]));
        m = pb_warp_max(m);
        const float s = m > 1e-30f && isfinite(m) ? m * (1.0f / 127.f) : 0.f;
        const float inv = s > 0.f ? __fdividef(1.0f, s) : 0.f;
        uint32_t pa[2] = {0u, 0u};
        int as = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float t = s > 0.f ? fminf(fmaxf(r[j] * inv, -127.f), 127.f) : 0.f;
            const float tm = t + kMagic;
            const int a = __float_as_int(tm) - 0x4B400000;
            r[j] = s > 0.f ? fmaf(-s, tm - kMagic, r[j]) : 0.f;
            pa[j >> 2] |= (uint32_t)(a & 0xFF) << (8 * (j & 3));
            as += a;
        }
        const int col = PB_XLEVELS * b + l;
        *reinterpret_cast<uint2*>(xq + (size_t)col * xstride + 256 * sb + 8 * lane) = make_uint2(pa[0], pa[1]);
        as += __shfl_xor_sync(0xffffffffu, as, 1); as += __shfl_xor_sync(0xffffffffu, as, 2);
        if ((lane & 3) == 0) qs[(8 * sb + (lane >> 2)) * GI_NCOL + col] = 8 * as;
        if (lane == 0) S[sb * GI_NCOL + col] = s * 0.125f;
    }
}

template <int NB, int SBW>
__global__ void __launch_bounds__(GI_THREADS, 1) pb_gemvi_kernel(const PbGemvIParams pi) {
    const PbGemvQParams& p = pi.q;
    const int nwarps = (int)blockDim.x >> 5, nthreads = (int)blockDim.x;
    extern __shared__ __align__(128) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem);                 // GI_WARPS floats
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 64);     // 2 x GI_WARPS: "buffer b of warp w is full"
    float* pairbuf = reinterpret_cast<float*>(smem + GI_OFF_PAIR);   // 2 x GI_WARPS x 2 x 16 partial results of the second warp of a pair
    float* S = reinterpret_cast<float*>(smem + GI_OFF_S);            // GI_SMAX x GI_NCOL level scales / 8
    int* qs = reinterpret_cast<int*>(smem + pi.off_qs);          // (cols / 32) x GI_NCOL accumulator inputs
    uint8_t* xq = smem + pi.off_xq;                              // 3 NB level arrays and one of zeros
    const int cols = p.bpr * 256;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t buf0 = pb_smem_u32(smem + pi.off_bufs) + (uint32_t)warp * pi.buf_bytes;   // first buffers of all warps, then the second ones
    const uint32_t buf1 = buf0 + (uint32_t)nwarps * pi.buf_bytes;
    float* xs = reinterpret_cast<float*>(smem + pi.off_bufs + (size_t)nwarps * pi.buf_bytes);      // prologue only: NB x cols prepared activations

    const bool st_first = tid == 0 && blockIdx.x == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1;
    pb_stamp(p.stamps, 0, st_first); pb_stamp(p.stamps, 6, st_last);
    pb_pdl_trigger();

    // a team of pi.ks warps owns a tile of 16 rows; warp `part` of the team takes blocks part * SBW .. of every row.
    // Tiles of a team: slot, slot + nslots, ...
    const int team = warp / pi.ks, part = warp - team * pi.ks, nteams = nwarps / pi.ks;
    const int nslots = (int)gridDim.x * nteams, slot = team * (int)gridDim.x + (int)blockIdx.x;
    const int my_tiles = p.nchunks > slot ? (p.nchunks - 1 - slot) / nslots + 1 : 0;
    auto locate = [&](int n, int& s, int& r0, int& nr) {
        const int tile = slot + n * nslots;
        s = 0;
        while (s + 1 < p.nseg && tile >= p.seg[s + 1].chunk0) s++;
        r0 = (tile - p.seg[s].chunk0) * 16;
        nr = min(16, p.seg[s].rows - r0);
    };
    // lane 0 starts one bulk copy per row for the warp's part of tile n, to the padded rows of buffer b; the bytes are
    // counted on the buffer's barrier
    const uint32_t mybars = pb_smem_u32(bars) + 16u * (uint32_t)warp;
    auto issue = [&](int n, int b) {
        if (n < my_tiles && lane == 0) {
            int s, r0, nr;
            locate(n, s, r0, nr);
            const uint8_t* src = p.seg[s].w + (size_t)r0 * p.row_bytes + (size_t)part * (SBW * 136);
            uint32_t dst = b ? buf1 : buf0;
            const uint32_t bar = mybars + 8u * (uint32_t)b;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)nr * (SBW * 136u)) : "memory");
            for (int r = 0; r < nr; r++) {
                asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(SBW * 136u), "r"(bar) : "memory");
                src += p.row_bytes; dst += (uint32_t)pi.stride;
            }
        }
    };
    if (tid == 0) {
        for (int i = 0; i < 2 * nwarps; i++) pb_mbar_init(&bars[i], 1);
        pb_fence_barrier_init();
    }
    __syncthreads();
    issue(0, 0);        // the weights do not depend on the activations
    pb_stamp(p.stamps, 1, st_first);

    // ---- activations -> levels ----
    for (int i = tid; i < (int)(pi.off_bufs - GI_OFF_PAIR) / 4; i += nthreads) reinterpret_cast<uint32_t*>(smem + GI_OFF_PAIR)[i] = 0u;   // partial results, scales, inputs, levels
    pb_pdl_wait();
    pb_stamp(p.stamps, 2, st_first);
    if (p.mode == PB_ACT_GNORM) {
        // per head: rms_inplace(o, norm, eps) then * sigmoid(z)  (linear_core, qwen4exp_gguf.rs:1667)
        const int nheads = cols / p.head_dim;
        for (int i = warp; i < p.t * nheads; i += nwarps) {
            const int b = i / nheads, h = i - b * nheads;
            float4 v = *reinterpret_cast<const float4*>(p.x + b * p.ldx + h * p.head_dim + 4 * lane);
            const float4 z = *reinterpret_cast<const float4*>(p.z + b * p.ldz + h * p.head_dim + 4 * lane);
            const float4 sg = make_float4(pb_sigm(z.x), pb_sigm(z.y), pb_sigm(z.z), pb_sigm(z.w));
            v = pb_gnorm_vec(v, *reinterpret_cast<const float4*>(p.norm_w + 4 * lane), sg, p.head_dim, p.eps);
            *reinterpret_cast<float4*>(xs + (size_t)b * cols + h * p.head_dim + 4 * lane) = v;
        }
    } else {
        for (int b = 0; b < p.t; b++) {
            float s = 1.0f;
            if (p.mode == PB_ACT_NORM) {  // rms(): x * s * w  (qwen4exp_gguf.rs:209)
                float ss = pb_warp_sum(pb_strided_ss(p.x + b * p.ldx, cols, tid, nthreads));
                __syncthreads();
                if (lane == 0) red[warp] = ss;
                __syncthreads();
                ss = 0.f;
                for (int i = 0; i < nwarps; i++) ss += red[i];
                s = 1.0f / sqrtf(ss / (float)cols + p.eps);
            }
            for (int c = 4 * tid; c < cols; c += 4 * nthreads) {
                float4 v = *reinterpret_cast<const float4*>(p.x + b * p.ldx + c);
                if (p.mode == PB_ACT_NORM) v = pb_norm_vec(v, s, *reinterpret_cast<const float4*>(p.norm_w + c));
                *reinterpret_cast<float4*>(xs + (size_t)b * cols + c) = v;
            }
        }
    }
    __syncthreads();
    for (int i = warp; i < p.t * p.bpr; i += nwarps) {
        const int b = i / p.bpr, sb = i - b * p.bpr;
        const float4 v0 = *reinterpret_cast<const float4*>(xs + (size_t)b * cols + 256 * sb + 8 * lane);
        const float4 v1 = *reinterpret_cast<const float4*>(xs + (size_t)b * cols + 256 * sb + 8 * lane + 4);
        float r[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        pb_split_block256(r, lane, sb, b, xq, pi.xstride, qs, S);
    }
    __syncthreads();    // levels ready; the activations in the second buffers are no longer needed
    pb_stamp(p.stamps, 3, st_first);

    // thread -> rows g and g + 8 of the tile, word t of every 16-byte group, columns 2 t and 2 t + 1 of the result
    const int g = lane >> 2, t = lane & 3, sb0 = part * SBW;
    const uint32_t xb = pb_smem_u32(xq) + (uint32_t)min(g, PB_XLEVELS * NB) * (uint32_t)pi.xstride + 8u * (uint32_t)t + 256u * (uint32_t)sb0;   // idle columns read the zeros
    const uint32_t cb = pb_smem_u32(qs) + 8u * (uint32_t)t + (uint32_t)sb0 * (8 * GI_NCOL * 4), sbase = pb_smem_u32(S) + 8u * (uint32_t)t + (uint32_t)sb0 * (GI_NCOL * 4);
    const uint32_t rowoff = (uint32_t)g * (uint32_t)pi.stride + 4u * (uint32_t)t;

    bool dead = false;
    for (int n = 0; n < my_tiles; n++) {
        issue(n + 1, (n + 1) & 1);
        // a wait that runs out is recorded in the status word; the warp then finishes its tiles without waiting (its
        // results are void, the host reports the status), so that the other warp of its team is never left at a barrier
        if (!dead && !pb_mbar_wait(&bars[2 * warp + (n & 1)], (uint32_t)(n >> 1) & 1u, p.status, PB_DEV_WAIT_FULL_TIMEOUT)) dead = true;
        if (n == 0) pb_stamp(p.stamps, 4, st_first);
        const uint32_t pa = ((n & 1) ? buf1 : buf0) + rowoff, pb = pa + 8u * (uint32_t)pi.stride;
        float f[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int sb = 0; sb < SBW; sb++) {
            const uint2 ha = pb_lds64(pa + 136u * sb - 4u * (uint32_t)t), hb = pb_lds64(pb + 136u * sb - 4u * (uint32_t)t);      // [d f16][pad][eight 4-bit multipliers]
            // multipliers 1 + 2 n as bytes: even groups in one word, odd groups in the other
            const uint32_t mae = (ha.y & 0x0F0F0F0Fu) * 2u + 0x01010101u, mao = ((ha.y >> 4) & 0x0F0F0F0Fu) * 2u + 0x01010101u;
            const uint32_t mbe = (hb.y & 0x0F0F0F0Fu) * 2u + 0x01010101u, mbo = ((hb.y >> 4) & 0x0F0F0F0Fu) * 2u + 0x01010101u;
            int acc[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t wa = pb_lds32(pa + 136u * sb + 8 + 16 * j), wb = pb_lds32(pb + 136u * sb + 8 + 16 * j);
                const uint2 bv = pb_lds64(xb + 256u * sb + 32 * j), cv = pb_lds64(cb + (8u * sb + j) * (GI_NCOL * 4));
                // 16 (c - 8) as s8: the code in the high nibble, top bit flipped
                const uint32_t a0 = ((wa << 4) & 0xF0F0F0F0u) ^ 0x80808080u, a1 = ((wb << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                const uint32_t a2 = (wa & 0xF0F0F0F0u) ^ 0x80808080u, a3 = (wb & 0xF0F0F0F0u) ^ 0x80808080u;
                int d[4];
                pb_mma_s8(d, a0, a1, a2, a3, bv.x, bv.y, (int)cv.x, (int)cv.y);
                const int ma = (int)__byte_perm((j & 1) ? mao : mae, 0u, 0x4440 + (j >> 1));
                const int mb = (int)__byte_perm((j & 1) ? mbo : mbe, 0u, 0x4440 + (j >> 1));
                acc[0] += d[0] * ma; acc[1] += d[1] * ma; acc[2] += d[2] * mb; acc[3] += d[3] * mb;
            }
            const float da = pb_h2f((uint16_t)(ha.x & 0xFFFF)), db = pb_h2f((uint16_t)(hb.x & 0xFFFF));
            const uint2 sv = pb_lds64(sbase + (uint32_t)sb * (GI_NCOL * 4));
            const float s0 = __uint_as_float(sv.x), s1 = __uint_as_float(sv.y);
            f[0] = fmaf((float)acc[0], da * s0, f[0]); f[1] = fmaf((float)acc[1], da * s1, f[1]);
            f[2] = fmaf((float)acc[2], db * s0, f[2]); f[3] = fmaf((float)acc[3], db * s1, f[3]);
        }
        // columns 0 1 | 2 3 | 4 5 of a row sit in lanes t = 0, 1, 2: token 0 = (c2 + c1) + c0, token 1 = (c5 + c4) + c3
        float ya, yb;      // rows g and g + 8
        {
            const float n0a = __shfl_down_sync(0xffffffffu, f[0], 1), n0b = __shfl_down_sync(0xffffffffu, f[2], 1);   // column 2 t + 2
            const float n1a = __shfl_down_sync(0xffffffffu, f[1], 1), n1b = __shfl_down_sync(0xffffffffu, f[3], 1);   // column 2 t + 3
            ya = t == 0 ? (n0a + f[1]) + f[0] : (n1a + n0a) + f[1];
            yb = t == 0 ? (n0b + f[3]) + f[2] : (n1b + n0b) + f[3];
        }
        if (pi.ks == 2) {
            // the second warp of the team hands its half over; the first adds it after its own (fixed order)
            float* pbuf = pairbuf + ((size_t)(n & 1) * GI_WARPS + team) * 32;
            if (part == 1 && t < NB) { pbuf[t * 16 + g] = ya; pbuf[t * 16 + g + 8] = yb; }
            pb_named_barrier(1 + team, 64);
            if (part == 0 && t < NB) { ya += pbuf[t * 16 + g]; yb += pbuf[t * 16 + g + 8]; }
        }
        int s, r0, nr;
        locate(n, s, r0, nr);
        if (part == 0 && t < NB && t < p.t) {
            float* dst = p.y + t * p.ldy + p.seg[s].yoff + r0;
            if (g < nr) dst[g] = p.accumulate ? dst[g] + ya : ya;
            if (g + 8 < nr) dst[g + 8] = p.accumulate ? dst[g + 8] + yb : yb;
        }
        __syncwarp();   // every lane has left this buffer before the next copies into it are issued
    }
    if (dead && my_tiles > 0) {
        // copies that may still be on their way get a bounded chance to land before the CTA can exit
        const int last = my_tiles - 1;
        pb_mbar_wait(&bars[2 * warp + (last & 1)], (uint32_t)(last >> 1) & 1u, nullptr, 0);
        if (last > 0) pb_mbar_wait(&bars[2 * warp + ((last - 1) & 1)], (uint32_t)((last - 1) >> 1) & 1u, nullptr, 0);
    }
    pb_stamp(p.stamps, 5, st_first); pb_stamp(p.stamps, 7, st_last);
}

// One token stays on the dp4a kernel: on the 151936 x 2048 lm-head this kernel takes 50 us with one token and 56 us
// with two, the dp4a kernel 43 us and 126 us.  About 40 instructions still surround every mma (the per-row copies,
// the unpacking, the multipliers), so one token does not pay.  PYRE_B200_IMMA_MIN=1 sends one token here too,
// PYRE_B200_IMMA=0 switches the kernel off.
static int pb_gemvi_min_tokens() {
    static const int v = getenv("PYRE_B200_IMMA_MIN") ? atoi(getenv("PYRE_B200_IMMA_MIN")) : 2;
    return v < 1 ? 1 : v;
}
bool pb_gemvi_supported(int type, int cols, int t) {
    static const bool on = !(getenv("PYRE_B200_IMMA") && atoi(getenv("PYRE_B200_IMMA")) == 0);
    const int bpr = cols / 256;
    return on && (type == PB_T_IQ3_S || type == PB_T_IQ3S_N4) && cols % 256 == 0 && (bpr == 2 || bpr == 4 || bpr == 8) && t >= pb_gemvi_min_tokens() && t <= 2;
}

// a.seg[].wr (or a.seg[].w when a.type is the re-coded type) holds the re-coded rows
int pb_launch_gemvi(pb_ctx* ctx, const PbGemvQArgs& a) {
    if (!pb_gemvi_supported(a.type, a.cols, a.t) || a.mode == PB_ACT_PREQ) PB_FAIL(ctx, PB_UNSUPPORTED, "gemvi: type %d cols %d t %d mode %d", a.type, a.cols, a.t, a.mode);
    if (a.nseg < 1 || a.nseg > 4) PB_FAIL(ctx, PB_ERR_ARG, "gemv: %d segments", a.nseg);
    if (a.mode == PB_ACT_GNORM && a.head_dim != 128) PB_FAIL(ctx, PB_UNSUPPORTED, "gemv: gated norm over heads of %d (128 is built)", a.head_dim);
    if (((uintptr_t)a.x & 15) || (a.ldx & 3)) PB_FAIL(ctx, PB_ERR_ARG, "gemv: activations must be 16-byte aligned");
    PbGemvIParams pi;
    memset(&pi, 0, sizeof pi);
    PbGemvQParams& p = pi.q;
    p.bpr = a.cols / 256; p.row_bytes = p.bpr * 136; p.nseg = a.nseg;
    p.x = a.x; p.ldx = a.ldx; p.t = a.t; p.y = a.y; p.ldy = a.ldy; p.status = ctx->dev_status;
    p.mode = a.mode; p.norm_w = a.norm_w; p.z = a.z; p.ldz = a.ldz; p.head_dim = a.head_dim; p.eps = a.eps;
    p.accumulate = a.accumulate;
    p.stamps = pb_stamp_slot(ctx, PB_K_GEMVQ);
    p.rows_per_chunk = 16;
    pi.sbw = p.bpr < GI_SBW ? p.bpr : GI_SBW; pi.ks = p.bpr / pi.sbw;
    // padded row stride: the eight rows of a load must start in eight different groups of four banks
    int pad = 16;
    while ((((pi.sbw * 136 + pad) / 4) % 32) % 8 != 4) pad += 16;
    pi.stride = pi.sbw * 136 + pad;
    pi.xstride = a.cols + 32;
    pi.off_qs = GI_OFF_QS;
    pi.off_xq = pi.off_qs + (uint32_t)(a.cols / 32) * GI_NCOL * 4;
    pi.off_bufs = (pi.off_xq + (uint32_t)(PB_XLEVELS * a.t + 1) * pi.xstride + 127u) & ~127u;
    pi.buf_bytes = (uint32_t)((16 * pi.stride + 127) & ~127);
    int nwarps = GI_WARPS;
    while (nwarps > 2 && pi.off_bufs + (size_t)2 * nwarps * pi.buf_bytes > (size_t)ctx->max_smem_optin) nwarps -= 2;
    const size_t smem = pi.off_bufs + (size_t)2 * nwarps * pi.buf_bytes;
    if ((size_t)a.t * a.cols * 4 > (size_t)nwarps * pi.buf_bytes || smem > (size_t)ctx->max_smem_optin)
        PB_FAIL(ctx, PB_UNSUPPORTED, "gemvi: %zu bytes of shared memory needed for cols=%d t=%d", smem, a.cols, a.t);
    int ntiles = 0;
    for (int s = 0; s < a.nseg; s++) {
        const uint8_t* w = a.type == PB_T_IQ3S_N4 ? a.seg[s].w : a.seg[s].wr;
        if (!w || ((uintptr_t)w & 15)) PB_FAIL(ctx, PB_ERR_ARG, "gemvi: segment %d has no 16-byte aligned re-coded copy", s);
        p.seg[s].w = w; p.seg[s].rows = (int)a.seg[s].rows; p.seg[s].yoff = (int)a.seg[s].yoff; p.seg[s].chunk0 = ntiles;
        ntiles += (int)((a.seg[s].rows + 15) / 16);
    }
    p.nchunks = ntiles;
    const int nteams = nwarps / pi.ks;
    const int want = (ntiles + nteams - 1) / nteams;
    const int grid = want < ctx->sm_count ? want : ctx->sm_count;
    if (grid <= 0) return PB_OK;
#define GI_LAUNCH(NB, SBW) { auto kern = pb_gemvi_kernel<NB, SBW>; PB_TRY(pb_ensure_smem(ctx, kern, smem)); pb_launch_k(ctx, kern, dim3(grid), dim3(nwarps * 32), smem, pi); }
    if (a.t == 1) { if (pi.sbw == 2) GI_LAUNCH(1, 2) else GI_LAUNCH(1, 4) }
    else { if (pi.sbw == 2) GI_LAUNCH(2, 2) else GI_LAUNCH(2, 4) }
#undef GI_LAUNCH
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
