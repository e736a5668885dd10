// Dequant-GEMV for two tokens (one on request) on the integer tensor cores (re-coded IQ3_S weights).
//
//   y[b][yoff_s + r] (+)= sum_c W_s[r][c] * act(x)[b][c]        b = 0 .. t-1 (t <= 2)
//
// Persistent CTAs of sixteen warps stream the rows through a four-stage shared-memory ring; every thread copies its
// share of a stage with cp.async (16-byte pieces, commit groups), one CTA barrier per stage.  The dot:
//   - the activations of a token are split into PB_XLEVELS int8 levels with ONE scale per 256 values
//     and level, x = S1 q1 + S2 q2 + S3 q3 + e, |e| <= max|x| / (2 * 254^2 * 127).  The levels of the
//     tokens are the columns of the B operand of mma.sync.m16n8k32 (s8 x s8 -> s32): one instruction
//     multiplies 16 rows x 32 weights with all levels of two tokens, where the dp4a kernel issues
//     PB_XLEVELS instructions per row and 4 weights;
//   - a weight is 2 c - 15 with a 4-bit code c.  The code goes into the HIGH nibble of an s8 with its top
//     bit flipped, which reads as 16 (c - 8); with 8 * (sum of the level over the 32 weights) as the
//     accumulator input the instruction returns 8 * sum (2 c - 15) q exactly.  Unpacking eight codes
//     costs three logic operations;
//   - the sub-block multiplier 1 + 2 n (one per 32 weights and row) multiplies the integer result,
//     the f16 block scale and the level scale are applied once per 256 weights in f32;
//   - a warp owns one 256-weight block column of a 16-row tile for the whole kernel, so its B operand,
//     accumulator inputs and level scales stay in registers; the warps of a tile meet in shared memory
//     and one thread per output adds the block columns in a fixed order.
// Rows lie in a stage with a padded stride, so that the eight rows a load instruction touches fall into
// different shared-memory banks; that is why the copies are pieces issued by all threads (one bulk copy per
// row serialises in the issuing warp, and so do the pieces when one warp issues them all).
// Replaces QMat::matmul (src/model/gguf_q.rs:217-242) and the k_gemv* kernels (src/model/qn_cube.rs:257-2331)
// of the reference for one and two tokens of IQ3_S weights.
#include "pb_stream.cuh"
#include "pb_internal.h"
#include <stdlib.h>
#include <stdio.h>

#define GI_NCOL 8       // columns of the mma: two tokens x three levels, two idle
#define GI_SMAX 16      // 256-weight blocks per row at most (4096 columns)

struct PbGemvIParams {
    PbGemvQParams q;
    int stride;         // bytes between rows of a stage
    int kslices;        // warps that share a 16-row tile (= blocks per row)
    int xstride;        // bytes between the level arrays of two columns
    uint32_t off_qs, off_xq, off_red, off_stages;
};

__device__ __forceinline__ void pb_mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, int c0, int c1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
}

// One 256-value block of one token, held by a warp (lane l: values 8 l .. 8 l + 7): PB_XLEVELS int8 levels with one
// scale per level.  Writes the levels (bytes 8 l .. of the block in the column's level array), 8 * the sum of
// each level over every 32 values (the accumulator input) and the scales.
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
        if (lane == 0) S[col * GI_SMAX + sb] = s;
    }
}

#define GI_THREADS 512
#define GI_WARPS 16
#define GI_STAGES 4

template <int NB>
__global__ void __launch_bounds__(GI_THREADS, 1) pb_gemvi_kernel(const PbGemvIParams pi) {
    const PbGemvQParams& p = pi.q;
    extern __shared__ __align__(128) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem + 64);            // GI_WARPS floats
    float* S = reinterpret_cast<float*>(smem + 192);             // GI_NCOL x GI_SMAX level scales
    int* qs = reinterpret_cast<int*>(smem + pi.off_qs);          // (cols / 32) x GI_NCOL accumulator inputs
    uint8_t* xq = smem + pi.off_xq;                              // GI_NCOL level arrays
    float* xs = reinterpret_cast<float*>(smem + pi.off_red);     // prologue: NB x cols prepared activations ...
    float* red2 = xs;                                            // ... then 2 x GI_WARPS x 16 x GI_NCOL partial sums
    const uint32_t stages = pb_smem_u32(smem + pi.off_stages);
    const int cols = p.bpr * 256;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool st_first = tid == 0 && blockIdx.x == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1;
    pb_stamp(p.stamps, 0, st_first); pb_stamp(p.stamps, 6, st_last);
    pb_pdl_trigger();

    const int my_chunks = p.nchunks > (int)blockIdx.x ? (p.nchunks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    // chunk k of this CTA -> its segment, first row and row count
    auto locate = [&](int k, int& s, int& r0, int& nr) {
        const int chunk = (int)blockIdx.x + k * (int)gridDim.x;
        s = 0;
        while (s + 1 < p.nseg && chunk >= p.seg[s + 1].chunk0) s++;
        r0 = (chunk - p.seg[s].chunk0) * p.rows_per_chunk;
        nr = min(p.rows_per_chunk, p.seg[s].rows - r0);
    };
    // every thread copies its share of chunk k (16-byte pieces) to the padded rows of stage k % GI_STAGES; one
    // commit group per call, also when there is nothing left to copy, so that the group counts stay aligned
    const int gpr = p.row_bytes / 16;
    const int q0 = tid % gpr, row0 = tid / gpr, dq = GI_THREADS % gpr, drow = GI_THREADS / gpr;
    auto issue = [&](int k) {
        if (k < my_chunks) {
            int s, r0, nr;
            locate(k, s, r0, nr);
            const uint8_t* src = p.seg[s].w + (size_t)r0 * p.row_bytes;
            const uint32_t dst = stages + (uint32_t)(k % GI_STAGES) * p.stage_bytes;
            const int total = nr * gpr;
            int row = row0, q = q0;
            for (int i = tid; i < total; i += GI_THREADS) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)row * (uint32_t)pi.stride + 16u * (uint32_t)q), "l"(src + 16 * (size_t)i) : "memory");
                q += dq; row += drow;
                if (q >= gpr) { q -= gpr; row++; }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // the weights do not depend on the activations: the first stages are on their way before anything else
    for (int k = 0; k < GI_STAGES - 1; k++) issue(k);
    pb_stamp(p.stamps, 1, st_first);

    // ---- activations -> levels ----
    constexpr int CT = GI_THREADS;
    for (int i = tid; i < (int)(pi.off_red - 128) / 4; i += CT) reinterpret_cast<uint32_t*>(smem + 128)[i] = 0u;   // scales, inputs, levels
    pb_pdl_wait();
    pb_stamp(p.stamps, 2, st_first);
    if (p.mode == PB_ACT_GNORM) {
        // per head: rms_inplace(o, norm, eps) then * sigmoid(z)  (linear_core, qwen4exp_gguf.rs:1667)
        const int nheads = cols / p.head_dim;
        for (int i = warp; i < p.t * nheads; i += GI_WARPS) {
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
                float ss = pb_strided_ss(p.x + b * p.ldx, cols, tid, CT);
                ss = pb_consumer_sum(ss, red, warp, lane);
                s = 1.0f / sqrtf(ss / (float)cols + p.eps);
            }
            for (int c = 4 * tid; c < cols; c += 4 * CT) {
                float4 v = *reinterpret_cast<const float4*>(p.x + b * p.ldx + c);
                if (p.mode == PB_ACT_NORM) v = pb_norm_vec(v, s, *reinterpret_cast<const float4*>(p.norm_w + c));
                *reinterpret_cast<float4*>(xs + (size_t)b * cols + c) = v;
            }
        }
    }
    __syncthreads();
    for (int i = warp; i < p.t * p.bpr; i += GI_WARPS) {
        const int b = i / p.bpr, sb = i - b * p.bpr;
        const float4 v0 = *reinterpret_cast<const float4*>(xs + (size_t)b * cols + 256 * sb + 8 * lane);
        const float4 v1 = *reinterpret_cast<const float4*>(xs + (size_t)b * cols + 256 * sb + 8 * lane + 4);
        float r[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        pb_split_block256(r, lane, sb, b, xq, pi.xstride, qs, S);
    }
    __syncthreads();
    pb_stamp(p.stamps, 3, st_first);

    // warp -> (tile of 16 rows, block column); thread -> (row g and g + 8, word t of every 16-byte group)
    const int tile = warp / pi.kslices, sb = warp - tile * pi.kslices;
    const int g = lane >> 2, t = lane & 3;
    uint32_t breg[8][2];
    int creg[8][2];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const uint2 bv = *reinterpret_cast<const uint2*>(xq + (size_t)g * pi.xstride + 256 * sb + 32 * j + 8 * t);
        breg[j][0] = bv.x; breg[j][1] = bv.y;
        const int2 cv = *reinterpret_cast<const int2*>(qs + (8 * sb + j) * GI_NCOL + 2 * t);
        creg[j][0] = cv.x; creg[j][1] = cv.y;
    }
    const float s0 = S[(2 * t) * GI_SMAX + sb] * 0.125f, s1 = S[(2 * t + 1) * GI_SMAX + sb] * 0.125f;
    const uint32_t rowoff = (uint32_t)(16 * tile + g) * (uint32_t)pi.stride + (uint32_t)sb * 136u;
    const int nout = p.rows_per_chunk * NB;
    // one thread per output of chunk kk adds the block columns in a fixed order
    auto reduce = [&](int kk) {
        if (tid < nout) {
            int s, r0, nr;
            locate(kk, s, r0, nr);
            const int b = tid / p.rows_per_chunk, r = tid - b * p.rows_per_chunk;
            if (r < nr && b < p.t) {
                const float* src = red2 + ((size_t)((kk & 1) * GI_WARPS + (r >> 4) * pi.kslices) * 16 + (r & 15)) * GI_NCOL + PB_XLEVELS * b;
                float v = 0.f;
                for (int ks = 0; ks < pi.kslices; ks++) {
                    const float* e = src + (size_t)ks * 16 * GI_NCOL;
                    v += (e[2] + e[1]) + e[0];       // smallest level first
                }
                float* dst = p.y + b * p.ldy + p.seg[s].yoff + r0 + r;
                *dst = p.accumulate ? *dst + v : v;
            }
        }
    };

    for (int k = 0; k < my_chunks; k++) {
        // this thread's pieces of chunk k have landed; after the barrier everyone's have, and every warp has left chunk k - 1
        asm volatile("cp.async.wait_group %0;" ::"n"(GI_STAGES - 2) : "memory");
        __syncthreads();
        if (k == 0) pb_stamp(p.stamps, 4, st_first);
        if (k > 0) reduce(k - 1);
        issue(k + GI_STAGES - 1);       // into the stage chunk k - 1 has just left
        const uint32_t pa = stages + (uint32_t)(k % GI_STAGES) * p.stage_bytes + rowoff, pb = pa + 8u * (uint32_t)pi.stride;
        const uint2 ha = pb_lds64(pa), hb = pb_lds64(pb);      // [d f16][pad][eight 4-bit multipliers]
        // multipliers 1 + 2 n as bytes: even groups in one word, odd groups in the other
        const uint32_t mae = (ha.y & 0x0F0F0F0Fu) * 2u + 0x01010101u, mao = ((ha.y >> 4) & 0x0F0F0F0Fu) * 2u + 0x01010101u;
        const uint32_t mbe = (hb.y & 0x0F0F0F0Fu) * 2u + 0x01010101u, mbo = ((hb.y >> 4) & 0x0F0F0F0Fu) * 2u + 0x01010101u;
        int acc[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t wa = pb_lds32(pa + 8 + 16 * j + 4 * t), wb = pb_lds32(pb + 8 + 16 * j + 4 * t);
            // 16 (c - 8) as s8: the code in the high nibble, top bit flipped
            const uint32_t a0 = ((wa << 4) & 0xF0F0F0F0u) ^ 0x80808080u, a1 = ((wb << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
            const uint32_t a2 = (wa & 0xF0F0F0F0u) ^ 0x80808080u, a3 = (wb & 0xF0F0F0F0u) ^ 0x80808080u;
            int d[4];
            pb_mma_s8(d, a0, a1, a2, a3, breg[j][0], breg[j][1], creg[j][0], creg[j][1]);
            const int ma = (int)__byte_perm((j & 1) ? mao : mae, 0u, 0x4440 + (j >> 1));
            const int mb = (int)__byte_perm((j & 1) ? mbo : mbe, 0u, 0x4440 + (j >> 1));
            acc[0] += d[0] * ma; acc[1] += d[1] * ma; acc[2] += d[2] * mb; acc[3] += d[3] * mb;
        }
        const float da = pb_h2f((uint16_t)(ha.x & 0xFFFF)), db = pb_h2f((uint16_t)(hb.x & 0xFFFF));
        float* rp = red2 + ((size_t)((k & 1) * GI_WARPS + warp) * 16) * GI_NCOL;
        *reinterpret_cast<float2*>(rp + g * GI_NCOL + 2 * t) = make_float2((float)acc[0] * (da * s0), (float)acc[1] * (da * s1));
        *reinterpret_cast<float2*>(rp + (g + 8) * GI_NCOL + 2 * t) = make_float2((float)acc[2] * (db * s0), (float)acc[3] * (db * s1));
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    if (my_chunks > 0) reduce(my_chunks - 1);
    pb_stamp(p.stamps, 5, st_first); pb_stamp(p.stamps, 7, st_last);
}

// One token stays on the dp4a kernel: on the 151936 x 2048 lm-head this kernel takes 60 us with one token or two, the
// dp4a kernel 43 us with one and 127 us with two.  Its sixteen warps meet at a barrier after every stage and each
// issues only eight mma per stage, so issue slots are half idle (barrier, pipe-throttle and dependency stalls) while
// the integer tensor pipe is 8 % busy.  PYRE_B200_IMMA_MIN=1 sends one token here too, PYRE_B200_IMMA=0 switches
// the kernel off.
static int pb_gemvi_min_tokens() {
    static const int v = getenv("PYRE_B200_IMMA_MIN") ? atoi(getenv("PYRE_B200_IMMA_MIN")) : 2;
    return v < 1 ? 1 : v;
}
bool pb_gemvi_supported(int type, int cols, int t) {
    static const bool on = !(getenv("PYRE_B200_IMMA") && atoi(getenv("PYRE_B200_IMMA")) == 0);
    const int bpr = cols / 256;
    return on && (type == PB_T_IQ3_S || type == PB_T_IQ3S_N4) && cols % 256 == 0 && (bpr == 2 || bpr == 4 || bpr == 8 || bpr == 16) && t >= pb_gemvi_min_tokens() && t <= 2;
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
    pi.kslices = p.bpr;
    p.rows_per_chunk = 16 * (GI_WARPS / pi.kslices);
    // padded row stride: the eight rows of a load must start in eight different groups of four banks
    int pad = 16;
    while ((((p.row_bytes + pad) / 4) % 32) % 8 != 4) pad += 16;
    pi.stride = p.row_bytes + pad;
    pi.xstride = a.cols + 32;
    pi.off_qs = 192 + GI_NCOL * GI_SMAX * 4;
    pi.off_xq = pi.off_qs + (uint32_t)(a.cols / 32) * GI_NCOL * 4;
    pi.off_red = (pi.off_xq + (uint32_t)GI_NCOL * pi.xstride + 127u) & ~127u;
    size_t red_bytes = (size_t)2 * GI_WARPS * 16 * GI_NCOL * 4, xs_bytes = (size_t)a.t * a.cols * 4;
    pi.off_stages = (uint32_t)((pi.off_red + (red_bytes > xs_bytes ? red_bytes : xs_bytes) + 127) & ~(size_t)127);
    p.stage_bytes = (uint32_t)(((size_t)p.rows_per_chunk * pi.stride + 127) & ~(size_t)127);
    const size_t smem = pi.off_stages + (size_t)GI_STAGES * p.stage_bytes;
    if (smem > (size_t)ctx->max_smem_optin) PB_FAIL(ctx, PB_UNSUPPORTED, "gemvi: %zu bytes of shared memory needed for cols=%d t=%d", smem, a.cols, a.t);
    int nchunks = 0;
    for (int s = 0; s < a.nseg; s++) {
        const uint8_t* w = a.type == PB_T_IQ3S_N4 ? a.seg[s].w : a.seg[s].wr;
        if (!w || ((uintptr_t)w & 15)) PB_FAIL(ctx, PB_ERR_ARG, "gemvi: segment %d has no 16-byte aligned re-coded copy", s);
        p.seg[s].w = w; p.seg[s].rows = (int)a.seg[s].rows; p.seg[s].yoff = (int)a.seg[s].yoff; p.seg[s].chunk0 = nchunks;
        nchunks += (int)((a.seg[s].rows + p.rows_per_chunk - 1) / p.rows_per_chunk);
    }
    p.nchunks = nchunks;
    const int grid = nchunks < ctx->sm_count ? nchunks : ctx->sm_count;
    if (grid <= 0) return PB_OK;
#define GI_LAUNCH(NB) { auto kern = pb_gemvi_kernel<NB>; PB_TRY(pb_ensure_smem(ctx, kern, smem)); pb_launch_k(ctx, kern, dim3(grid), dim3(GI_THREADS), smem, pi); }
    if (a.t == 1) GI_LAUNCH(1) else GI_LAUNCH(2)
#undef GI_LAUNCH
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
