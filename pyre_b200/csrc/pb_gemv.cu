// Dequant-GEMV on native GGUF blocks:  y[b][r] = sum_c W[r][c] * x[b][c],  f32 accumulate.
// Replaces QMat::matmul (src/model/gguf_q.rs:217-242 of the reference) and the CubeCL
// k_gemv* family (src/model/qn_cube.rs:257-1159).
//
// Shape of the kernel (HBM-bound byte streaming):
//   - persistent CTAs; each walks chunks of R consecutive rows, i.e. R*row_bytes
//     contiguous bytes of the matrix, strided by the grid;
//   - one producer warp streams chunks into a ring of shared-memory stages with 1-D bulk
//     (TMA) copies completing on mbarriers; eight consumer warps decode from shared memory
//     (codebooks staged in shared memory) and release stages through "empty" barriers;
//   - a consumer warp owns one row at a time: lane l decodes 8 weights of every 256-wide
//     step, multiplies by the activations (registers for one column, shared memory for
//     2..16 columns) and the row sum is a warp-shuffle reduction.
// Every barrier wait is bounded (pb_mbar_wait) and reports through the status word.
#include "pb_formats.cuh"
#include "pb_internal.h"

#include <stdio.h>

#define GEMV_CONSUMERS 8
#define GEMV_THREADS ((GEMV_CONSUMERS + 1) * 32)
#define GEMV_STAGES 4
#define GEMV_MAX_STEPS_REG 8  // activations of up to 8 steps (2048 columns) live in registers

struct GemvParams {
    const uint8_t* w;
    int64_t rows;
    int row_bytes;
    int steps;        // cols / 256
    int rows_per_chunk;
    int nchunks;
    uint32_t stage_bytes;
    const float* x;
    int64_t ldx;
    int t;
    float* y;
    int64_t ldy;
    int* status;
};

template <int FMT, int NB>
__global__ void __launch_bounds__(GEMV_THREADS, 1) pb_gemv_f32_kernel(const GemvParams p) {
    using F = PbFmt<FMT>;
    constexpr bool XREG = (NB == 1);
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + GEMV_STAGES;
    uint8_t* tab = smem + 128;
    float4* xs = reinterpret_cast<float4*>(smem + 128 + ((PB_TABLE_BYTES + 127) & ~127));
    const int xs_bytes = XREG && p.steps <= GEMV_MAX_STEPS_REG ? 0 : NB * p.steps * 1024;
    uint8_t* stages = reinterpret_cast<uint8_t*>(xs) + ((xs_bytes + 127) & ~127);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < GEMV_STAGES; s++) { pb_mbar_init(&full[s], 1); pb_mbar_init(&empty[s], GEMV_CONSUMERS); }
        pb_fence_barrier_init();
    }
    const PbTables T = pb_load_tables<FMT>(tab, tid, GEMV_THREADS);
    // activations -> shared memory in lane-major order (quad k of a step stored at F::perm(k))
    if (xs_bytes) {
        const int quads = p.steps * 64;
        for (int i = tid; i < NB * quads; i += GEMV_THREADS) {
            const int b = i / quads, q = i - b * quads;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (b < p.t) v = *reinterpret_cast<const float4*>(p.x + b * p.ldx + 4 * q);
            xs[b * quads + (q & ~63) + F::perm(q & 63)] = v;
        }
    }
    __syncthreads();

    const int my_chunks = p.nchunks > (int)blockIdx.x ? (p.nchunks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (warp == GEMV_CONSUMERS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int k = 0; k < my_chunks && ok; k++) {
                const int s = k % GEMV_STAGES;
                if (k >= GEMV_STAGES) ok = pb_mbar_wait_relaxed(&empty[s], ((k / GEMV_STAGES) - 1) & 1, p.status, PB_DEV_WAIT_EMPTY_TIMEOUT);
                if (!ok) break;
                const int64_t chunk = (int64_t)blockIdx.x + (int64_t)k * gridDim.x;
                const int64_t r0 = chunk * p.rows_per_chunk;
                const int nr = (int)min((int64_t)p.rows_per_chunk, p.rows - r0);
                const uint32_t bytes = ((uint32_t)nr * (uint32_t)p.row_bytes + 15u) & ~15u;
                pb_mbar_expect_tx(&full[s], bytes);
                pb_bulk_g2s(stages + (size_t)s * p.stage_bytes, p.w + r0 * p.row_bytes, bytes, &full[s]);
                issued = k + 1;
            }
            if (!ok) {
                // give the copies already in flight a bounded chance to land before the CTA exits
                for (int k = max(0, issued - GEMV_STAGES); k < issued; k++) pb_mbar_wait(&full[k % GEMV_STAGES], (k / GEMV_STAGES) & 1, nullptr, 0);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    float xr[XREG ? GEMV_MAX_STEPS_REG * 8 : 1];
    const bool xin_regs = XREG && p.steps <= GEMV_MAX_STEPS_REG;
    if (xin_regs) {
#pragma unroll
        for (int s = 0; s < GEMV_MAX_STEPS_REG; s++) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
            if (s < p.steps) {
                a = *reinterpret_cast<const float4*>(p.x + s * 256 + 4 * F::xa(lane));
                b = *reinterpret_cast<const float4*>(p.x + s * 256 + 4 * F::xb(lane));
            }
            xr[8 * s + 0] = a.x; xr[8 * s + 1] = a.y; xr[8 * s + 2] = a.z; xr[8 * s + 3] = a.w;
            xr[8 * s + 4] = b.x; xr[8 * s + 5] = b.y; xr[8 * s + 6] = b.z; xr[8 * s + 7] = b.w;
        }
    }
    const int quads = p.steps * 64;

    for (int k = 0; k < my_chunks; k++) {
        const int s = k % GEMV_STAGES;
        if (!pb_mbar_wait(&full[s], (k / GEMV_STAGES) & 1, p.status, PB_DEV_WAIT_FULL_TIMEOUT)) return;
        const int64_t chunk = (int64_t)blockIdx.x + (int64_t)k * gridDim.x;
        const int64_t r0 = chunk * p.rows_per_chunk;
        const int nr = (int)min((int64_t)p.rows_per_chunk, p.rows - r0);
        const uint8_t* base = stages + (size_t)s * p.stage_bytes;
        for (int r = warp; r < nr; r += GEMV_CONSUMERS) {
            const uint8_t* rowp = base + (size_t)r * p.row_bytes;
            float acc[NB];
#pragma unroll
            for (int b = 0; b < NB; b++) acc[b] = 0.f;
            if (xin_regs) {
#pragma unroll
                for (int st = 0; st < GEMV_MAX_STEPS_REG; st++) {
                    if (st < p.steps) {
                        PbUnit u;
                        F::unit(rowp + st * F::STEP_BYTES, lane, T, u);
                        float pa = 0.f, pb = 0.f;
#pragma unroll
                        for (int j = 0; j < 4; j++) { pa = fmaf(xr[8 * st + j], u.w[j], pa); pb = fmaf(xr[8 * st + 4 + j], u.w[4 + j], pb); }
                        acc[0] = fmaf(u.sa, pa, acc[0]);
                        acc[0] = fmaf(u.sb, pb, acc[0]);
                        if (F::HAS_MIN) {
                            const float sa = (xr[8 * st] + xr[8 * st + 1]) + (xr[8 * st + 2] + xr[8 * st + 3]);
                            const float sb = (xr[8 * st + 4] + xr[8 * st + 5]) + (xr[8 * st + 6] + xr[8 * st + 7]);
                            acc[0] = fmaf(-u.ma, sa, acc[0]);
                            acc[0] = fmaf(-u.mb, sb, acc[0]);
                        }
                    }
                }
            } else {
                for (int st = 0; st < p.steps; st++) {
                    PbUnit u;
                    F::unit(rowp + st * F::STEP_BYTES, lane, T, u);
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const float4 xa = xs[b * quads + st * 64 + lane], xb = xs[b * quads + st * 64 + 32 + lane];
                        float pa = xa.x * u.w[0]; pa = fmaf(xa.y, u.w[1], pa); pa = fmaf(xa.z, u.w[2], pa); pa = fmaf(xa.w, u.w[3], pa);
                        float pb = xb.x * u.w[4]; pb = fmaf(xb.y, u.w[5], pb); pb = fmaf(xb.z, u.w[6], pb); pb = fmaf(xb.w, u.w[7], pb);
                        acc[b] = fmaf(u.sa, pa, acc[b]);
                        acc[b] = fmaf(u.sb, pb, acc[b]);
                        if (F::HAS_MIN) {
                            acc[b] = fmaf(-u.ma, (xa.x + xa.y) + (xa.z + xa.w), acc[b]);
                            acc[b] = fmaf(-u.mb, (xb.x + xb.y) + (xb.z + xb.w), acc[b]);
                        }
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float v = pb_warp_sum(acc[b]);
                if (lane == 0 && b < p.t) p.y[b * p.ldy + r0 + r] = v;
            }
        }
        __syncwarp();
        if (lane == 0) pb_mbar_arrive(&empty[s]);
    }
}

template <int FMT, int NB>
static int launch_one_f32(pb_ctx* ctx, const PbGemvArgs& a, int row_bytes) {
    GemvParams p;
    p.w = a.w; p.rows = a.rows; p.row_bytes = row_bytes; p.steps = a.cols / 256;
    p.x = a.x; p.ldx = a.ldx; p.t = a.t; p.y = a.y; p.ldy = a.ldy; p.status = ctx->dev_status;
    // rows per chunk: keep chunk bytes a multiple of 16 (bulk-copy rule) and aim for at least
    // four chunks per CTA so the stage ring stays full; at most ~32 KB per stage.
    int align_rows = 1;
    while ((align_rows * row_bytes) % 16) align_rows *= 2;
    const int grid_max = ctx->sm_count;
    const bool xin_regs = NB == 1 && p.steps <= GEMV_MAX_STEPS_REG;
    const size_t xs_bytes = xin_regs ? 0 : (size_t)NB * p.steps * 1024;
    const size_t fixed = 128 + ((PB_TABLE_BYTES + 127) & ~127) + ((xs_bytes + 127) & ~(size_t)127);
    if (fixed + (size_t)GEMV_STAGES * align_rows * row_bytes > (size_t)ctx->max_smem_optin)
        PB_FAIL(ctx, PB_UNSUPPORTED, "gemv: cols=%d with %d columns does not fit shared memory", a.cols, a.t);
    size_t stage_cap = ((size_t)ctx->max_smem_optin - fixed) / GEMV_STAGES;
    if (stage_cap > 32768) stage_cap = 32768;
    int rpc = GEMV_CONSUMERS * 4;
    while (rpc > GEMV_CONSUMERS && (a.rows + rpc - 1) / rpc < 4 * (int64_t)grid_max) rpc /= 2;
    while ((size_t)rpc * row_bytes + 144 > stage_cap && rpc > 1) rpc /= 2;
    rpc = ((rpc + align_rows - 1) / align_rows) * align_rows;
    p.rows_per_chunk = rpc;
    p.nchunks = (int)((a.rows + rpc - 1) / rpc);
    p.stage_bytes = (uint32_t)(((size_t)rpc * row_bytes + 16 + 127) & ~(size_t)127);
    const size_t smem = fixed + (size_t)GEMV_STAGES * p.stage_bytes;
    if (smem > (size_t)ctx->max_smem_optin) PB_FAIL(ctx, PB_UNSUPPORTED, "gemv: %zu bytes of shared memory needed for cols=%d t=%d", smem, a.cols, a.t);
    auto kern = pb_gemv_f32_kernel<FMT, NB>;
    PB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int grid = p.nchunks < grid_max ? p.nchunks : grid_max;
    kern<<<grid, GEMV_THREADS, smem, ctx->stream>>>(p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

template <int FMT>
static int launch_fmt_f32(pb_ctx* ctx, const PbGemvArgs& a, int row_bytes) {
    if (a.t == 1) return launch_one_f32<FMT, 1>(ctx, a, row_bytes);
    if (a.t <= 4) return launch_one_f32<FMT, 4>(ctx, a, row_bytes);
    if (a.t <= 8) return launch_one_f32<FMT, 8>(ctx, a, row_bytes);
    return launch_one_f32<FMT, 16>(ctx, a, row_bytes);
}

int pb_launch_gemv_f32(pb_ctx* ctx, const PbGemvArgs& a) {
    int el, bs;
    if (pb_geom(a.type, &el, &bs)) PB_FAIL(ctx, PB_ERR_ARG, "gemv: unsupported ggml type %d", a.type);
    if (a.cols <= 0 || a.cols % 256) PB_FAIL(ctx, PB_UNSUPPORTED, "gemv: cols=%d is not a multiple of 256", a.cols);
    if (a.t < 1 || a.t > 16) PB_FAIL(ctx, PB_ERR_ARG, "gemv: t=%d outside 1..16", a.t);
    if (a.rows <= 0) return PB_OK;
    if (((uintptr_t)a.w & 15) || ((uintptr_t)a.x & 15)) PB_FAIL(ctx, PB_ERR_ARG, "gemv: weight and activation pointers must be 16-byte aligned");
    const int row_bytes = a.cols / el * bs;
    // column tiles: the activations of one launch must fit in ~128 KB of shared memory
    int tile = 16;
    while (tile > 1 && (size_t)tile * a.cols * 4 > 131072) tile /= 2;
    int rc = PB_OK;
    for (int t0 = 0; t0 < a.t && rc == PB_OK; t0 += tile) {
        PbGemvArgs s = a;
        s.x = a.x + (int64_t)t0 * a.ldx; s.y = a.y + (int64_t)t0 * a.ldy; s.t = a.t - t0 < tile ? a.t - t0 : tile;
        rc = PB_ERR_ARG;
#define LAUNCH() rc = launch_fmt_f32<FMT>(ctx, s, row_bytes)
        PB_DISPATCH_FMT(a.type, LAUNCH);
#undef LAUNCH
    }
    return rc;
}
