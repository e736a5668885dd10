// Dequant-GEMV for the quantized block formats (IQ3_S, IQ2_XS, Q4_K, Q8_0), integer core.
//
//   y[b][r] = sum_c W[r][c] * x[b][c]
//
// Same streaming skeleton as the generic kernel in pb_gemv.cu (persistent CTAs, one
// producer warp issuing 1-D bulk copies of whole row chunks into a 4-stage shared-memory
// ring, mbarrier full/empty hand-off, bounded waits) with a cheaper arithmetic core:
//   - the CTA first splits the activations into two int8 levels per 32 values (pb_qdot.cuh);
//   - a lane owns a quarter super-step (64 weights) of a row, so the fields of a block are
//     fetched once per 64 weights; a warp covers 2048 columns of one row per pass (or
//     several shorter rows side by side);
//   - codebook entries are used as packed int8 directly (SWAR sign, dp4a), no float
//     conversion; the IQ3_S / IQ2_XS codebook is replicated once per shared-memory bank for
//     large matrices so that random lookups never conflict (64 KB of the 227 KB per SM).
// Replaces QMat::matmul (src/model/gguf_q.rs:217-242) and the k_gemv* / k_gemv_iq4* kernels
// (src/model/qn_cube.rs:257-2102) of the reference.
#include "pb_qdot.cuh"
#include "pb_internal.h"

#include <stdio.h>

#define GQ_CONSUMERS 16
#define GQ_THREADS ((GQ_CONSUMERS + 1) * 32)
#define GQ_STAGES 4

struct GemvQParams {
    const uint8_t* w;
    int64_t rows;
    int row_bytes;
    int bpr;            // 256-weight super-steps per row
    int rows_per_chunk;
    int nchunks;
    uint32_t stage_bytes;
    uint32_t tab_bytes;
    int rep;            // codebook replication (1, or 32 for u32 entries / 16 for u64 entries)
    const float* x;
    int64_t ldx;
    int t;
    float* y;
    int64_t ldy;
    int* status;
};

__device__ __forceinline__ void pb_named_barrier(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }

// word offset of quad i (4 words) of quarter qi inside one level array of NQ quarters
__device__ __forceinline__ int pb_xq_off(int qi, int i, int nq) { return (i * nq + qi) * 4; }

__device__ __forceinline__ void pb_load_xquarter(const uint32_t* xcol, int cols, int qi, PbXQuarter& o) {
    const int nq = cols / 64, ng = cols / 32;
    const uint32_t* q1 = xcol;
    const uint32_t* q2 = xcol + cols / 4;
    const float* sc = reinterpret_cast<const float*>(xcol + cols / 2);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint4 a = *reinterpret_cast<const uint4*>(q1 + pb_xq_off(qi, i, nq));
        const uint4 b = *reinterpret_cast<const uint4*>(q2 + pb_xq_off(qi, i, nq));
        o.q1[4 * i] = (int)a.x; o.q1[4 * i + 1] = (int)a.y; o.q1[4 * i + 2] = (int)a.z; o.q1[4 * i + 3] = (int)a.w;
        o.q2[4 * i] = (int)b.x; o.q2[4 * i + 1] = (int)b.y; o.q2[4 * i + 2] = (int)b.z; o.q2[4 * i + 3] = (int)b.w;
    }
    o.s1[0] = sc[2 * qi]; o.s1[1] = sc[2 * qi + 1];
    o.s2[0] = sc[ng + 2 * qi]; o.s2[1] = sc[ng + 2 * qi + 1];
    o.sum[0] = sc[2 * ng + 2 * qi]; o.sum[1] = sc[2 * ng + 2 * qi + 1];
}

template <int FMT, int NB, int PASSES>
__global__ void __launch_bounds__(GQ_THREADS, 1) pb_gemvq_kernel(const GemvQParams p) {
    using D = PbQDec<FMT>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + GQ_STAGES;
    uint2* sign16 = reinterpret_cast<uint2*>(smem + 128);
    uint8_t* tab = smem + 256;
    const int cols = p.bpr * 256;
    uint32_t* xq = reinterpret_cast<uint32_t*>(tab + p.tab_bytes);
    const int xw = pb_xq_words(cols);
    uint8_t* stages = reinterpret_cast<uint8_t*>(xq) + (((size_t)NB * xw * 4 + 127) & ~(size_t)127);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < GQ_STAGES; s++) { pb_mbar_init(&full[s], 1); pb_mbar_init(&empty[s], GQ_CONSUMERS); }
        pb_fence_barrier_init();
    }
    __syncthreads();

    const int my_chunks = p.nchunks > (int)blockIdx.x ? (p.nchunks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (warp == GQ_CONSUMERS) {
        // ---------------- producer: weights do not depend on the activations, start streaming now ----------------
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int k = 0; k < my_chunks; k++) {
                const int s = k % GQ_STAGES;
                if (k >= GQ_STAGES) ok = pb_mbar_wait(&empty[s], ((k / GQ_STAGES) - 1) & 1, p.status, PB_DEV_WAIT_EMPTY_TIMEOUT);
                if (!ok) break;
                const int64_t r0 = ((int64_t)blockIdx.x + (int64_t)k * gridDim.x) * p.rows_per_chunk;
                const int nr = (int)min((int64_t)p.rows_per_chunk, p.rows - r0);
                const uint32_t bytes = ((uint32_t)nr * (uint32_t)p.row_bytes + 15u) & ~15u;
                pb_mbar_expect_tx(&full[s], bytes);
                pb_bulk_g2s(stages + (size_t)s * p.stage_bytes, p.w + r0 * p.row_bytes, bytes, &full[s]);
                issued = k + 1;
            }
            if (!ok)  // give copies in flight a bounded chance to land before the CTA can exit
                for (int k = max(0, issued - GQ_STAGES); k < issued; k++) pb_mbar_wait(&full[k % GQ_STAGES], (k / GQ_STAGES) & 1, nullptr, 0);
        }
        return;
    }

    // ---------------- consumers: tables, activation split ----------------
    constexpr int CT = GQ_CONSUMERS * 32;
    if (tid < 16) {
        uint32_t m = 0;
        for (int j = 0; j < 4; j++) if (tid & (1 << j)) m |= 0xFFu << (8 * j);
        sign16[tid] = make_uint2(m, m & 0x01010101u);
    }
    PbQTabs T;
    T.sign16 = sign16; T.grid3 = reinterpret_cast<const uint32_t*>(tab); T.grid2 = reinterpret_cast<const uint64_t*>(tab); T.rep3 = T.rep2 = p.rep;
    if (FMT == PB_T_IQ3_S) {
        uint32_t* g = reinterpret_cast<uint32_t*>(tab);
        for (int i = tid; i < 512 * p.rep; i += CT) g[i] = PB_IQ3S_GRID[i / p.rep];
    }
    if (FMT == PB_T_IQ2_XS) {
        uint64_t* g = reinterpret_cast<uint64_t*>(tab);
        for (int i = tid; i < 512 * p.rep; i += CT) g[i] = PB_IQ2XS_GRID[i / p.rep];
    }
    {
        const int ng = cols / 32, nq = cols / 64;
        for (int i = warp; i < NB * ng; i += GQ_CONSUMERS) {
            const int b = i / ng, g = i - b * ng;
            const float v = b < p.t ? p.x[b * p.ldx + 32 * g + lane] : 0.f;
            uint32_t* col = xq + (size_t)b * xw;
            float* sc = reinterpret_cast<float*>(col + cols / 2);
            // group g = words 8*(g&1) .. +7 of quarter g/2, i.e. its quads 2*(g&1) and 2*(g&1)+1
            const float m1 = pb_warp_max(fabsf(v));
            const float s1 = m1 > 0.f && isfinite(m1) ? m1 / 127.f : 0.f;
            const int a = s1 > 0.f ? __float2int_rn(v / s1) : 0;
            const float r = s1 > 0.f ? fmaf(-s1, (float)a, v) : 0.f;
            const float m2 = pb_warp_max(fabsf(r));
            const float s2 = m2 > 0.f ? m2 / 127.f : 0.f;
            const int bq = s2 > 0.f ? __float2int_rn(r / s2) : 0;
            const float sum = pb_warp_sum(v);
            uint32_t pa = (uint32_t)(a & 0xFF) << (8 * (lane & 3)), pq = (uint32_t)(bq & 0xFF) << (8 * (lane & 3));
            pa |= __shfl_xor_sync(0xffffffffu, pa, 1); pa |= __shfl_xor_sync(0xffffffffu, pa, 2);
            pq |= __shfl_xor_sync(0xffffffffu, pq, 1); pq |= __shfl_xor_sync(0xffffffffu, pq, 2);
            if ((lane & 3) == 0) {
                const int k = lane >> 2;                       // word 0..7 of the group
                const int off = pb_xq_off(g >> 1, 2 * (g & 1) + (k >> 2), nq) + (k & 3);
                col[off] = pa; col[cols / 4 + off] = pq;
            }
            if (lane == 0) { sc[g] = s1; sc[ng + g] = s2; sc[2 * ng + g] = sum; }
        }
    }
    pb_named_barrier(1, CT);

    // lane -> (row sub-index, quarter) mapping
    const int nquarters = 4 * p.bpr;
    const int lpr = nquarters < 32 ? nquarters : 32;   // lanes per row (a power of two for bpr in {1,2,4,8,..})
    const int rpw = 32 / lpr;                           // rows handled side by side by one warp
    const int sub = lane / lpr, ql = lane - sub * lpr;

    PbXQuarter xr[NB == 1 ? PASSES : 1];
    if (NB == 1) {
#pragma unroll
        for (int ps = 0; ps < PASSES; ps++) {
            const int qi = ps * 32 + ql;
            if (qi < nquarters) pb_load_xquarter(xq, cols, qi, xr[ps]);
        }
    }

    for (int k = 0; k < my_chunks; k++) {
        const int s = k % GQ_STAGES;
        if (!pb_mbar_wait(&full[s], (k / GQ_STAGES) & 1, p.status, PB_DEV_WAIT_FULL_TIMEOUT)) return;
        const int64_t r0 = ((int64_t)blockIdx.x + (int64_t)k * gridDim.x) * p.rows_per_chunk;
        const int nr = (int)min((int64_t)p.rows_per_chunk, p.rows - r0);
        const uint8_t* base = stages + (size_t)s * p.stage_bytes;
        for (int rb = warp * rpw; rb < nr; rb += GQ_CONSUMERS * rpw) {
            const int r = rb + sub;
            const bool valid = r < nr;
            float acc[NB];
#pragma unroll
            for (int b = 0; b < NB; b++) acc[b] = 0.f;
            if (valid) {
                const uint8_t* rowp = base + (size_t)r * p.row_bytes;
#pragma unroll
                for (int ps = 0; ps < PASSES; ps++) {
                    const int qi = ps * 32 + ql;
                    if (qi < nquarters) {
                        PbQuarter wq;
                        D::quarter(rowp + (qi >> 2) * D::STEP_BYTES, qi & 3, lane, T, wq);
                        if (NB == 1) {
                            acc[0] += pb_quarter_dot<FMT>(wq, xr[ps]);
                        } else {
#pragma unroll 1
                            for (int b = 0; b < NB; b++) {
                                PbXQuarter xv;
                                pb_load_xquarter(xq + (size_t)b * xw, cols, qi, xv);
                                acc[b] += pb_quarter_dot<FMT>(wq, xv);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float v = acc[b];
                for (int o = lpr >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (ql == 0 && valid && b < p.t) p.y[b * p.ldy + r0 + r] = v;
            }
        }
        __syncwarp();
        if (lane == 0) pb_mbar_arrive(&empty[s]);
    }
}

template <int FMT, int NB, int PASSES>
static int launch_q(pb_ctx* ctx, const PbGemvArgs& a, int row_bytes) {
    GemvQParams p;
    p.w = a.w; p.rows = a.rows; p.row_bytes = row_bytes; p.bpr = a.cols / 256;
    p.x = a.x; p.ldx = a.ldx; p.t = a.t; p.y = a.y; p.ldy = a.ldy; p.status = ctx->dev_status;
    const int grid_max = ctx->sm_count;
    const size_t wbytes = (size_t)a.rows * row_bytes;
    // replicate the codebook per bank only when the matrix is large enough to amortise the fill
    const bool has_tab = FMT == PB_T_IQ3_S || FMT == PB_T_IQ2_XS;
    const int entry = FMT == PB_T_IQ3_S ? 4 : 8;
    p.rep = has_tab && wbytes >= ((size_t)8 << 20) ? 128 / entry : 1;
    p.tab_bytes = has_tab ? 512 * entry * p.rep : 0;
    const size_t xbytes = ((size_t)NB * pb_xq_words(a.cols) * 4 + 127) & ~(size_t)127;
    const size_t fixed = 256 + p.tab_bytes + xbytes;
    int align_rows = 1;
    while ((align_rows * row_bytes) % 16) align_rows *= 2;
    if (fixed + (size_t)GQ_STAGES * (align_rows * row_bytes + 144) > (size_t)ctx->max_smem_optin)
        PB_FAIL(ctx, PB_UNSUPPORTED, "gemv: cols=%d with %d columns does not fit shared memory", a.cols, a.t);
    size_t stage_cap = ((size_t)ctx->max_smem_optin - fixed) / GQ_STAGES;
    if (stage_cap > 32768) stage_cap = 32768;
    const int lpr = 4 * p.bpr < 32 ? 4 * p.bpr : 32;
    const int step_rows = GQ_CONSUMERS * (32 / lpr);   // rows one sweep of the consumer warps covers
    int rpc = step_rows * 2;
    while (rpc > step_rows && (a.rows + rpc - 1) / rpc < 4 * (int64_t)grid_max) rpc /= 2;
    while ((size_t)rpc * row_bytes + 144 > stage_cap && rpc > 1) rpc /= 2;
    rpc = ((rpc + align_rows - 1) / align_rows) * align_rows;
    p.rows_per_chunk = rpc;
    p.nchunks = (int)((a.rows + rpc - 1) / rpc);
    p.stage_bytes = (uint32_t)(((size_t)rpc * row_bytes + 16 + 127) & ~(size_t)127);
    const size_t smem = fixed + (size_t)GQ_STAGES * p.stage_bytes;
    if (smem > (size_t)ctx->max_smem_optin) PB_FAIL(ctx, PB_UNSUPPORTED, "gemv: %zu bytes of shared memory needed for cols=%d t=%d", smem, a.cols, a.t);
    auto kern = pb_gemvq_kernel<FMT, NB, PASSES>;
    PB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int grid = p.nchunks < grid_max ? p.nchunks : grid_max;
    kern<<<grid, GQ_THREADS, smem, ctx->stream>>>(p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

template <int FMT, int NB>
static int launch_q_passes(pb_ctx* ctx, const PbGemvArgs& a, int row_bytes) {
    return a.cols <= 2048 ? launch_q<FMT, NB, 1>(ctx, a, row_bytes) : launch_q<FMT, NB, 2>(ctx, a, row_bytes);
}

template <int FMT>
static int launch_q_fmt(pb_ctx* ctx, const PbGemvArgs& a, int row_bytes) {
    if (a.t == 1) return launch_q_passes<FMT, 1>(ctx, a, row_bytes);
    if (a.t <= 2) return launch_q_passes<FMT, 2>(ctx, a, row_bytes);
    if (a.t <= 4) return launch_q_passes<FMT, 4>(ctx, a, row_bytes);
    if (a.t <= 8) return launch_q_passes<FMT, 8>(ctx, a, row_bytes);
    return launch_q_passes<FMT, 16>(ctx, a, row_bytes);
}

int pb_launch_gemv_f32(pb_ctx* ctx, const PbGemvArgs& a);

int pb_launch_gemv(pb_ctx* ctx, const PbGemvArgs& a) {
    int el, bs;
    if (pb_geom(a.type, &el, &bs)) PB_FAIL(ctx, PB_ERR_ARG, "gemv: unsupported ggml type %d", a.type);
    const bool quant = a.type == PB_T_IQ3_S || a.type == PB_T_IQ2_XS || a.type == PB_T_Q4_K || a.type == PB_T_Q8_0;
    const int bpr = a.cols / 256;
    const bool pow2 = bpr > 0 && (bpr & (bpr - 1)) == 0;
    if (!quant || a.cols % 256 || !pow2 || a.cols > 4096) return pb_launch_gemv_f32(ctx, a);
    if (a.t < 1 || a.t > 16) PB_FAIL(ctx, PB_ERR_ARG, "gemv: t=%d outside 1..16", a.t);
    if (a.rows <= 0) return PB_OK;
    if (((uintptr_t)a.w & 15) || ((uintptr_t)a.x & 3)) PB_FAIL(ctx, PB_ERR_ARG, "gemv: weight pointer must be 16-byte aligned");
    const int row_bytes = a.cols / el * bs;
    switch (a.type) {
        case PB_T_IQ3_S: return launch_q_fmt<PB_T_IQ3_S>(ctx, a, row_bytes);
        case PB_T_IQ2_XS: return launch_q_fmt<PB_T_IQ2_XS>(ctx, a, row_bytes);
        case PB_T_Q4_K: return launch_q_fmt<PB_T_Q4_K>(ctx, a, row_bytes);
        default: return launch_q_fmt<PB_T_Q8_0>(ctx, a, row_bytes);
    }
}
