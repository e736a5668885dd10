// Dequant-GEMV for the quantized block formats (IQ3_S, IQ2_XS, Q4_K, Q8_0), integer core.
//
//   y[b][yoff_s + r] (+)= sum_c W_s[r][c] * act(x)[b][c]      for up to four matrices W_s
//
// Streaming skeleton (pb_stream.cuh): persistent CTAs, one producer warp issuing 1-D bulk
// (TMA) copies of whole row chunks into a 4-stage shared-memory ring, mbarrier full/empty
// hand-off with bounded waits, sixteen consumer warps.  Arithmetic core (pb_qdot.cuh):
//   - the CTA prepares the activations once: optional RMSNorm (plain or per-head gated), then
//     a split into PB_XLEVELS int8 levels per 32 values;
//   - a lane owns a quarter super-step (64 weights) of a row, so block fields are fetched
//     once per 64 weights; a warp covers 2048 columns of a row per pass (or several
//     shorter rows side by side);
//   - codebook entries are used as packed int8 directly (dp4a); IQ3_S indices are built with prmt and
//     its signs applied by arithmetic (xor 0xFE negates the odd grid values), because table reads
//     made shared-memory wavefronts the bound; for large matrices the IQ3_S / IQ2_XS codebook is
//     replicated once per shared-memory bank so that random lookups never conflict (64 KB of the
//     227 KB per SM);
//   - three or more columns of IQ3_S weights go to the tensor-core kernel of pb_gemmh.cu instead.
// Replaces QMat::matmul (src/model/gguf_q.rs:217-242), the k_gemv* / k_gemv_iq4* kernels and
// the k_rms* prologues (src/model/qn_cube.rs:257-2331) of the reference.
#include "pb_stream.cuh"
#include "pb_internal.h"
#include <stdlib.h>

#include <stdio.h>

template <int FMT, int NB, int PASSES>
__global__ void __launch_bounds__(PB_KTHREADS, 1) pb_gemvq_kernel(const PbGemvQParams p) {
    using D = PbQDec<FMT>;
    extern __shared__ __align__(128) uint8_t smem[];
    PbRing ring;
    ring.full = reinterpret_cast<uint64_t*>(smem);
    ring.empty = ring.full + PB_STAGES;
    float* red = reinterpret_cast<float*>(smem + 64);            // PB_CONSUMERS floats
    uint8_t* tab = smem + 256;
    const int cols = p.bpr * 256;
    uint32_t* xq = reinterpret_cast<uint32_t*>(tab + p.tab_bytes);
    const int xw = pb_xq_words(cols);
    ring.stages = reinterpret_cast<uint8_t*>(xq) + (((size_t)NB * xw * 4 + 127) & ~(size_t)127);
    ring.stage_bytes = p.stage_bytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool st_first = tid == 0 && blockIdx.x == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1;
    pb_stamp(p.stamps, 0, st_first); pb_stamp(p.stamps, 6, st_last);
    pb_pdl_trigger();   // the next kernel may start its own set-up and weight stream
    pb_ring_init(ring, tid);
    __syncthreads();
    pb_stamp(p.stamps, 1, st_first);

    const int my_chunks = p.nchunks > (int)blockIdx.x ? (p.nchunks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (warp == PB_CONSUMERS) {
        // ---- producer: the weights do not depend on the activations, so streaming starts at once ----
        if (lane == 0) {
            int k = 0;
            for (; k < my_chunks; k++) {
                const int chunk = (int)blockIdx.x + k * (int)gridDim.x;
                int s = 0;
                while (s + 1 < p.nseg && chunk >= p.seg[s + 1].chunk0) s++;
                const int r0 = (chunk - p.seg[s].chunk0) * p.rows_per_chunk;
                const int nr = min(p.rows_per_chunk, p.seg[s].rows - r0);
                const uint32_t bytes = ((uint32_t)nr * (uint32_t)p.row_bytes + 15u) & ~15u;
                if (!pb_ring_acquire(ring, k, bytes, p.status)) break;
                pb_ring_copy(ring, k, 0, p.seg[s].w + (size_t)r0 * p.row_bytes, bytes);
            }
            if (k < my_chunks) pb_ring_drain(ring, k);
        }
        return;
    }

    // ---- consumers: codebooks, activations ----
    constexpr int CT = PB_CONSUMERS * 32;
    const PbQTabs T = pb_fill_qtabs<FMT>(tab, p.rep, tid, CT, lane);
    pb_pdl_wait();      // activations (and the residual this kernel may add to) come from earlier kernels
    pb_stamp(p.stamps, 2, st_first);
    const int ng = cols / 32;
    if (p.mode == PB_ACT_PREQ) {
        for (int i = tid; i < NB * xw; i += CT) { const int b = i / xw; xq[i] = b < p.t ? p.xq_in[(size_t)b * xw + (i - b * xw)] : 0u; }
    } else if (p.mode == PB_ACT_GNORM) {
        // per head: rms_inplace(o, norm, eps) then * sigmoid(z)  (linear_core, qwen4exp_gguf.rs:1667).
        // A warp takes one head of 128 (= four groups) per pass: lane l owns elements 4l..4l+3.
        const int nheads = cols / p.head_dim;
        for (int i = warp; i < NB * nheads; i += PB_CONSUMERS) {
            const int b = i / nheads, h = i - b * nheads;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f), sg = make_float4(1.f, 1.f, 1.f, 1.f);
            if (b < p.t) {
                v = *reinterpret_cast<const float4*>(p.x + b * p.ldx + h * p.head_dim + 4 * lane);
                const float4 z = *reinterpret_cast<const float4*>(p.z + b * p.ldz + h * p.head_dim + 4 * lane);
                sg = make_float4(pb_sigm(z.x), pb_sigm(z.y), pb_sigm(z.z), pb_sigm(z.w));
            }
            v = pb_gnorm_vec(v, *reinterpret_cast<const float4*>(p.norm_w + 4 * lane), sg, p.head_dim, p.eps);
            pb_split_groups4(v, lane, h * 4, cols, xq + (size_t)b * xw);
        }
    } else {
        for (int b = 0; b < NB; b++) {
            // the values this warp splits (its first two passes: rows of up to 4096 columns) are requested before the sum of
            // squares is formed, so that the two walks over the row share one trip to L2
            float4 vp0 = make_float4(0.f, 0.f, 0.f, 0.f), vp1 = vp0;
            if (b < p.t) {
                if (warp * 4 < ng) vp0 = *reinterpret_cast<const float4*>(p.x + b * p.ldx + 32 * (warp * 4) + 4 * lane);
                if ((warp + PB_CONSUMERS) * 4 < ng) vp1 = *reinterpret_cast<const float4*>(p.x + b * p.ldx + 32 * ((warp + PB_CONSUMERS) * 4) + 4 * lane);
            }
            float s = 1.0f;
            if (p.mode == PB_ACT_NORM && b < p.t) {  // rms(): x * s * w  (qwen4exp_gguf.rs:209)
                float ss = pb_strided_ss(p.x + b * p.ldx, cols, tid, CT);
                ss = pb_consumer_sum(ss, red, warp, lane);
                s = 1.0f / sqrtf(ss / (float)cols + p.eps);
            }
            int pass = 0;
            for (int g0 = warp * 4; g0 < ng; g0 += PB_CONSUMERS * 4, pass++) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (b < p.t) v = pass == 0 ? vp0 : (pass == 1 ? vp1 : *reinterpret_cast<const float4*>(p.x + b * p.ldx + 32 * g0 + 4 * lane));
                if (p.mode == PB_ACT_NORM) v = pb_norm_vec(v, s, *reinterpret_cast<const float4*>(p.norm_w + 32 * g0 + 4 * lane));
                pb_split_groups4(v, lane, g0, cols, xq + (size_t)b * xw);
            }
        }
    }
    pb_named_barrier(1, CT);
    pb_stamp(p.stamps, 3, st_first);

    // lane -> (row sub-index, quarter)
    const int nquarters = 4 * p.bpr;
    const int lpr = nquarters < 32 ? nquarters : 32;   // lanes per row
    const int rpw = 32 / lpr;                           // rows one warp handles side by side
    const int sub = lane / lpr, ql = lane - sub * lpr;

    PbXQuarter xr[NB == 1 ? PASSES : 1];
    if (NB == 1) {
#pragma unroll
        for (int ps = 0; ps < PASSES; ps++) {
            const int qi = ps * 32 + ql;
            if (qi < nquarters) pb_load_xquarter<PbQDec<FMT>::AFFINE>(xq, cols, qi, xr[ps]);
        }
    }

    for (int k = 0; k < my_chunks; k++) {
        if (!pb_ring_wait(ring, k, p.status)) return;
        if (k == 0) pb_stamp(p.stamps, 4, st_first);
        const int chunk = (int)blockIdx.x + k * (int)gridDim.x;
        int s = 0;
        while (s + 1 < p.nseg && chunk >= p.seg[s + 1].chunk0) s++;
        const int r0 = (chunk - p.seg[s].chunk0) * p.rows_per_chunk;
        const int nr = min(p.rows_per_chunk, p.seg[s].rows - r0);
        const uint32_t base = pb_smem_u32(pb_ring_stage(ring, k));
        if ((FMT == PB_T_IQ3_S || FMT == PB_T_IQ3S_N4) && NB == 1 && PASSES == 1 && lpr == 32) {
            // one column, full-width rows: two rows per iteration, so that the two independent decode
            // chains overlap each other's shared-memory latency (a row past nr decodes stale bytes of the
            // stage and is not stored)
            float* ybase = p.y + p.seg[s].yoff + r0;
            for (int ra = warp; ra < nr; ra += 2 * PB_CONSUMERS) {
                const int rc = ra + PB_CONSUMERS;
                const bool two = rc < p.rows_per_chunk;
                float v0 = pb_decode_dot<FMT>(base + (uint32_t)ra * (uint32_t)p.row_bytes + (ql >> 2) * D::STEP_BYTES, ql & 3, T, xr[0]);
                float v1 = pb_decode_dot<FMT>(base + (uint32_t)(two ? rc : ra) * (uint32_t)p.row_bytes + (ql >> 2) * D::STEP_BYTES, ql & 3, T, xr[0]);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) { v0 += __shfl_xor_sync(0xffffffffu, v0, o); v1 += __shfl_xor_sync(0xffffffffu, v1, o); }
                if (lane == 0) {
                    ybase[ra] = p.accumulate ? ybase[ra] + v0 : v0;
                    if (two && rc < nr) ybase[rc] = p.accumulate ? ybase[rc] + v1 : v1;
                }
            }
            pb_ring_release(ring, k, lane);
            continue;
        }
        for (int rb = warp * rpw; rb < nr; rb += PB_CONSUMERS * rpw) {
            const int r = rb + sub;
            const bool valid = r < nr;
            float acc[NB];
#pragma unroll
            for (int b = 0; b < NB; b++) acc[b] = 0.f;
            if (valid) {
                const uint32_t rowp = base + (uint32_t)r * (uint32_t)p.row_bytes;
#pragma unroll
                for (int ps = 0; ps < PASSES; ps++) {
                    const int qi = ps * 32 + ql;
                    if (qi < nquarters) {
                        if (FMT == PB_T_IQ3_S && NB == 1) {
                            acc[0] += pb_iq3s_quarter_dot(rowp + (qi >> 2) * D::STEP_BYTES, qi & 3, T, xr[ps]);
                            continue;
                        }
                        PbQuarter wq;
                        D::quarter(rowp + (qi >> 2) * D::STEP_BYTES, qi & 3, T, wq);
                        if (NB == 1) {
                            acc[0] += pb_quarter_dot<FMT>(wq, xr[ps]);
                        } else {
#pragma unroll 1
                            for (int b = 0; b < NB; b++) {
                                PbXQuarter xv;
                                pb_load_xquarter<PbQDec<FMT>::AFFINE>(xq + (size_t)b * xw, cols, qi, xv);
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
                if (ql == 0 && valid && b < p.t) {
                    float* dst = p.y + b * p.ldy + p.seg[s].yoff + r0 + r;
                    *dst = p.accumulate ? *dst + v : v;
                }
            }
        }
        pb_ring_release(ring, k, lane);
    }
    pb_stamp(p.stamps, 5, st_first); pb_stamp(p.stamps, 7, st_last);
}

template <int FMT, int NB, int PASSES>
static int launch_q(pb_ctx* ctx, const PbGemvQArgs& a, int row_bytes) {
    PbGemvQParams p;
    memset(&p, 0, sizeof p);
    p.row_bytes = row_bytes; p.bpr = a.cols / 256; p.nseg = a.nseg;
    p.x = a.x; p.ldx = a.ldx; p.t = a.t; p.y = a.y; p.ldy = a.ldy; p.status = ctx->dev_status;
    p.mode = a.mode; p.norm_w = a.norm_w; p.z = a.z; p.ldz = a.ldz; p.head_dim = a.head_dim; p.eps = a.eps;
    p.xq_in = a.xq_in; p.accumulate = a.accumulate;
    p.stamps = pb_stamp_slot(ctx, PB_K_GEMVQ);
    const int grid_max = ctx->sm_count;
    int64_t total_rows = 0;
    for (int s = 0; s < a.nseg; s++) total_rows += a.seg[s].rows;
    const size_t wbytes = (size_t)total_rows * row_bytes;
    // replicate the codebook per bank only when the matrix is large enough to amortise the fill
    constexpr int entry = pb_tab_entry_bytes<FMT>();
    p.rep = entry && wbytes >= ((size_t)8 << 20) ? pb_tab_rep_max<FMT>() : 1;
    p.tab_bytes = pb_tab_bytes<FMT>(p.rep);
    const size_t xbytes = ((size_t)NB * pb_xq_words(a.cols) * 4 + 127) & ~(size_t)127;
    const size_t fixed = 256 + p.tab_bytes + xbytes;
    int align_rows = 1;
    while ((align_rows * row_bytes) % 16) align_rows *= 2;
    if (fixed + (size_t)PB_STAGES * (align_rows * row_bytes + 144) > (size_t)ctx->max_smem_optin)
        PB_FAIL(ctx, PB_UNSUPPORTED, "gemv: cols=%d with %d columns does not fit shared memory", a.cols, a.t);
    size_t stage_cap = ((size_t)ctx->max_smem_optin - fixed) / PB_STAGES;
    // the re-coded format needs no tables and little arithmetic: larger stages keep more bytes in flight
    const size_t cap_max = FMT == PB_T_IQ3S_N4 ? 53248 : 32768;
    if (stage_cap > cap_max) stage_cap = cap_max;
    const int lpr = 4 * p.bpr < 32 ? 4 * p.bpr : 32;
    const int step_rows = PB_CONSUMERS * (32 / lpr);   // rows one sweep of the consumer warps covers
    int rpc = step_rows * 2;
    while (rpc > step_rows && (total_rows + rpc - 1) / rpc < 4 * (int64_t)grid_max) rpc /= 2;
    while ((size_t)rpc * row_bytes + 144 > stage_cap && rpc > 1) rpc /= 2;
    rpc = ((rpc + align_rows - 1) / align_rows) * align_rows;
    p.rows_per_chunk = rpc;
    int nchunks = 0;
    for (int s = 0; s < a.nseg; s++) {
        if (((uintptr_t)a.seg[s].w & 15)) PB_FAIL(ctx, PB_ERR_ARG, "gemv: weight pointer must be 16-byte aligned");
        p.seg[s].w = a.seg[s].w; p.seg[s].rows = (int)a.seg[s].rows; p.seg[s].yoff = (int)a.seg[s].yoff; p.seg[s].chunk0 = nchunks;
        nchunks += (int)((a.seg[s].rows + rpc - 1) / rpc);
    }
    p.nchunks = nchunks;
    p.stage_bytes = (uint32_t)(((size_t)rpc * row_bytes + 16 + 127) & ~(size_t)127);
    const size_t smem = fixed + (size_t)PB_STAGES * p.stage_bytes;
    if (smem > (size_t)ctx->max_smem_optin) PB_FAIL(ctx, PB_UNSUPPORTED, "gemv: %zu bytes of shared memory needed for cols=%d t=%d", smem, a.cols, a.t);
    auto kern = pb_gemvq_kernel<FMT, NB, PASSES>;
    PB_TRY(pb_ensure_smem(ctx, kern, smem));
    const int grid = nchunks < grid_max ? nchunks : grid_max;
    pb_launch_k(ctx, kern, dim3(grid), dim3(PB_KTHREADS), (size_t)(smem), p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

template <int FMT, int NB>
static int launch_q_passes(pb_ctx* ctx, const PbGemvQArgs& a, int row_bytes) {
    return a.cols <= 2048 ? launch_q<FMT, NB, 1>(ctx, a, row_bytes) : launch_q<FMT, NB, 2>(ctx, a, row_bytes);
}

template <int FMT>
static int launch_q_fmt(pb_ctx* ctx, const PbGemvQArgs& a, int row_bytes) {
    if (a.t == 1) return launch_q_passes<FMT, 1>(ctx, a, row_bytes);
    if (a.t <= 2) return launch_q_passes<FMT, 2>(ctx, a, row_bytes);
    if (a.t <= 4) return launch_q_passes<FMT, 4>(ctx, a, row_bytes);
    if (a.t <= 8) return launch_q_passes<FMT, 8>(ctx, a, row_bytes);
    return launch_q_passes<FMT, 16>(ctx, a, row_bytes);
}

bool pb_gemvq_supported(int type, int cols) {
    const bool quant = type == PB_T_IQ3_S || type == PB_T_IQ3S_N4 || type == PB_T_IQ2_XS || type == PB_T_Q4_K || type == PB_T_Q8_0 ||
                       type == PB_T_IQ3_XXS || type == PB_T_IQ2_S || type == PB_T_IQ4_NL || type == PB_T_IQ4_XS ||
                       type == PB_T_Q2_0 || type == PB_T_IQ2_XXS || type == PB_T_Q6_K || type == PB_T_IQ1_M ||
                       type == PB_T_Q4_0 || type == PB_T_Q5_0 || type == PB_T_Q3_K || type == PB_T_Q5_K;
    const int bpr = cols / 256;
    return quant && cols % 256 == 0 && bpr > 0 && (bpr & (bpr - 1)) == 0 && cols <= 4096;
}

static int launch_gemvq_dp4a(pb_ctx* ctx, const PbGemvQArgs& a, int el, int bs);
int pb_launch_gemvq(pb_ctx* ctx, const PbGemvQArgs& a) {
    int el, bs;
    if (pb_geom(a.type, &el, &bs) || !pb_gemvq_supported(a.type, a.cols)) PB_FAIL(ctx, PB_UNSUPPORTED, "gemvq: type %d cols %d not supported by the integer kernel", a.type, a.cols);
    if (!a.exact && a.mode != PB_ACT_PREQ && pb_gemmtc_supported(a.type, a.cols, a.t) && a.t <= pb_gemmtc_max_tokens(a.cols)) {
        // tcgen05 from pb_gemmtc_min_tokens() tokens on (PYRE_B200_TC=0 keeps the warp-level kernel below)
        static const bool use_tc = !(getenv("PYRE_B200_TC") && atoi(getenv("PYRE_B200_TC")) == 0);
        bool all = true;
        for (int s = 0; s < a.nseg && s < 4; s++) all = all && a.seg[s].wr != nullptr;
        if (use_tc && all && a.t >= pb_gemmtc_min_tokens()) return pb_launch_gemmtc(ctx, a);
    }
    if (a.mode != PB_ACT_PREQ && pb_gemvi_supported(a.type, a.cols, a.t)) {
        bool all = true;
        int64_t rows = 0;
        for (int s = 0; s < a.nseg && s < 4; s++) { all = all && (a.type == PB_T_IQ3S_N4 ? a.seg[s].w : a.seg[s].wr) != nullptr; rows += a.seg[s].rows; }
        // measured: from about ten million weights on it beats the dp4a kernel with two tokens, below that they tie
        static const int64_t min_weights = getenv("PYRE_B200_IMMA_MIN_WEIGHTS") ? atoll(getenv("PYRE_B200_IMMA_MIN_WEIGHTS")) : ((int64_t)10 << 20);
        if (all && rows * a.cols >= min_weights) return pb_launch_gemvi(ctx, a);
    }
    if (a.mode != PB_ACT_PREQ && pb_gemmh_supported(a.type, a.cols, a.t)) {
        static const bool use_mma = !(getenv("PYRE_B200_MMA") && atoi(getenv("PYRE_B200_MMA")) == 0);
        if (use_mma) return pb_launch_gemmh(ctx, a);
    }
    PbGemvQArgs b = a;
    if (a.type == PB_T_IQ3_S) {
        // every segment has a re-coded copy: stream that one
        bool all = true;
        for (int s = 0; s < a.nseg && s < 4; s++) all = all && a.seg[s].wr != nullptr;
        if (all) { b.type = PB_T_IQ3S_N4; for (int s = 0; s < a.nseg && s < 4; s++) b.seg[s].w = a.seg[s].wr; pb_geom(b.type, &el, &bs); }
    }
    return launch_gemvq_dp4a(ctx, b, el, bs);
}

static int launch_gemvq_dp4a(pb_ctx* ctx, const PbGemvQArgs& a, int el, int bs) {
    if (a.t < 1 || a.t > 16) PB_FAIL(ctx, PB_ERR_ARG, "gemv: t=%d outside 1..16", a.t);
    if (a.nseg < 1 || a.nseg > 4) PB_FAIL(ctx, PB_ERR_ARG, "gemv: %d segments", a.nseg);
    if (a.mode == PB_ACT_GNORM && a.head_dim != 128) PB_FAIL(ctx, PB_UNSUPPORTED, "gemv: gated norm over heads of %d (128 is built)", a.head_dim);
    if (((uintptr_t)a.x & 15) || (a.ldx & 3)) PB_FAIL(ctx, PB_ERR_ARG, "gemv: activations must be 16-byte aligned");
    const int row_bytes = a.cols / el * bs;
    // column tiles: the int8-split activations of one launch must fit in ~96 KB of shared memory
    int tile = 16;
    while (tile > 1 && (size_t)tile * pb_xq_words(a.cols) * 4 > 98304) tile /= 2;
    int rc = PB_OK;
    for (int t0 = 0; t0 < a.t && rc == PB_OK; t0 += tile) {
        PbGemvQArgs s = a;
        s.t = a.t - t0 < tile ? a.t - t0 : tile;
        s.x = a.x ? a.x + (int64_t)t0 * a.ldx : nullptr; s.y = a.y + (int64_t)t0 * a.ldy; s.z = a.z ? a.z + (int64_t)t0 * a.ldz : nullptr;
        s.xq_in = a.xq_in ? a.xq_in + (size_t)t0 * pb_xq_words(a.cols) : nullptr;
        switch (a.type) {
            case PB_T_IQ3_S: rc = launch_q_fmt<PB_T_IQ3_S>(ctx, s, row_bytes); break;
            case PB_T_IQ3S_N4: rc = launch_q_fmt<PB_T_IQ3S_N4>(ctx, s, row_bytes); break;
            case PB_T_IQ2_XS: rc = launch_q_fmt<PB_T_IQ2_XS>(ctx, s, row_bytes); break;
            case PB_T_Q4_K: rc = launch_q_fmt<PB_T_Q4_K>(ctx, s, row_bytes); break;
            case PB_T_IQ3_XXS: rc = launch_q_fmt<PB_T_IQ3_XXS>(ctx, s, row_bytes); break;
            case PB_T_IQ2_S: rc = launch_q_fmt<PB_T_IQ2_S>(ctx, s, row_bytes); break;
            case PB_T_IQ4_NL: rc = launch_q_fmt<PB_T_IQ4_NL>(ctx, s, row_bytes); break;
            case PB_T_IQ4_XS: rc = launch_q_fmt<PB_T_IQ4_XS>(ctx, s, row_bytes); break;
            case PB_T_Q2_0: rc = launch_q_fmt<PB_T_Q2_0>(ctx, s, row_bytes); break;
            case PB_T_IQ2_XXS: rc = launch_q_fmt<PB_T_IQ2_XXS>(ctx, s, row_bytes); break;
            case PB_T_Q6_K: rc = launch_q_fmt<PB_T_Q6_K>(ctx, s, row_bytes); break;
            case PB_T_IQ1_M: rc = launch_q_fmt<PB_T_IQ1_M>(ctx, s, row_bytes); break;
            case PB_T_Q4_0: rc = launch_q_fmt<PB_T_Q4_0>(ctx, s, row_bytes); break;
            case PB_T_Q5_0: rc = launch_q_fmt<PB_T_Q5_0>(ctx, s, row_bytes); break;
            case PB_T_Q3_K: rc = launch_q_fmt<PB_T_Q3_K>(ctx, s, row_bytes); break;
            case PB_T_Q5_K: rc = launch_q_fmt<PB_T_Q5_K>(ctx, s, row_bytes); break;
            default: rc = launch_q_fmt<PB_T_Q8_0>(ctx, s, row_bytes); break;
        }
    }
    return rc;
}

int pb_launch_gemv_f32(pb_ctx* ctx, const PbGemvArgs& a);

// Plain y = W x for any supported type (the pb_gemv entry points).
int pb_launch_gemv(pb_ctx* ctx, const PbGemvArgs& a) {
    if (!pb_gemvq_supported(a.type, a.cols)) return pb_launch_gemv_f32(ctx, a);
    if (a.rows <= 0) return PB_OK;
    PbGemvQArgs q;
    memset(&q, 0, sizeof q);
    q.type = a.type; q.cols = a.cols; q.nseg = 1; q.seg[0].w = a.w; q.seg[0].wr = a.wr; q.seg[0].rows = a.rows; q.seg[0].yoff = 0;
    q.x = a.x; q.ldx = a.ldx; q.t = a.t; q.y = a.y; q.ldy = a.ldy; q.mode = PB_ACT_PLAIN;
    return pb_launch_gemvq(ctx, q);
}
