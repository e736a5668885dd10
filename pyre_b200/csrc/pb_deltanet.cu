// Gated DeltaNet decode step: depthwise causal conv1d + SiLU, q/k L2 norm, decay / beta gates,
// delta-rule state update and readout, fused in one kernel.
//
// Restates linear_core of the reference (src/model/qwen4exp_gguf.rs:1624-1673; GPU twins
// k_conv / k_delta, src/model/qn_cube.rs:2753-2839).  The gated RMSNorm that follows the
// readout (:1667) needs the whole 128-wide head, so it lives in the prologue of the output
// projection (PB_ACT_GNORM in pb_gemvq.cu).
//
// Work split: one CTA per (sequence, V head, slice of 32 state columns).  The f32 state
// S[h][i][j] (dk x dv per head, 64 KB) is read once and written once; a warp owns 16 rows i,
// a lane one column j, so every row access is a coalesced 128-byte line and the two
// reductions over i (S^T k and S^T q) are 16 FMAs per lane plus a sum across the 8 warps in
// shared memory.  The conv history is a 4-slot ring ([slot][channel], slot = position mod
// conv_k), so no CTA ever writes a slot another CTA reads in the same step.
#include "pb_deltanet.cuh"

#include <stdio.h>

struct PbDeltaCtaPolicy {
    __device__ static __forceinline__ void sync() { __syncthreads(); }
    __device__ __forceinline__ void wait_inputs() {}   // the kernel waited for its predecessor before anything was read
};

// grid (nv * dv / (DN_COLS * NS), batch).  NS = column slices of 32 one CTA walks in turn (1: most CTAs, shortest
// latency; dv / 32: the conv, norm and gate phases run once per head instead of once per slice, which pays when
// there are thousands of CTAs)
template <int RPW, int NS>
__global__ void __launch_bounds__(DN_THREADS) pb_deltanet_kernel(const PbDeltaParams p) {
    const int splits = p.dv / (DN_COLS * NS);
    const int h = blockIdx.x / splits, j0 = (blockIdx.x % splits) * DN_COLS * NS;
    const int b = blockIdx.y, tid = threadIdx.x;
    const bool st_first = tid == 0 && blockIdx.x == 0 && blockIdx.y == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1;
    pb_stamp(p.stamps, 0, st_first); pb_stamp(p.stamps, 6, st_last);
    pb_pdl_wait();
    pb_pdl_trigger();
    extern __shared__ float sm[];
    __shared__ float nrm[2];
    PbDeltaCtaPolicy pol;
    // (requesting the state early pays only with few sequences: with thousands of CTAs the SM already overlaps them,
    // and holding the slice through the first phases costs more than it hides)
    pb_deltanet_unit<RPW, NS>(p, p.pos[b], h, j0, b, tid, gridDim.y <= 4, sm, nrm, pol, p.stamps, st_first);
    pb_stamp(p.stamps, 5, st_first); pb_stamp(p.stamps, 7, st_last);
}

// A run of T consecutive tokens of ONE sequence (a prefill chunk): the recurrence is sequential in the tokens, so the
// CTA of (V head, 32 state columns) keeps its slice of S in registers for the whole run instead of one launch, one
// read and one write of the state per token (the reference loops the tokens inside k_delta_m the same way,
// src/model/qn_cube.rs:2839-2913).  Token j reads row j of proj (row stride ldp) and writes row j of out (stride ldo);
// p.pos[0] is the position of token 0.  The conv history of in-window tokens comes from the earlier rows of proj, that
// of the tokens before the window from the ring; the arithmetic per token is that of pb_deltanet_unit.
template <int RPW>
__global__ void __launch_bounds__(DN_THREADS) pb_deltanet_seq_kernel(const PbDeltaParams p, int T, const PbDeltaCk ck) {
    constexpr int K = 4;                                    // conv taps (checked by the launcher)
    const int nk = p.nk, nv = p.nv, dk = p.dk, dv = p.dv;
    const int splits = dv / DN_COLS;
    const int h = blockIdx.x / splits, j0 = (blockIdx.x % splits) * DN_COLS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ch = 2 * nk * dk + nv * dv, kh = h % nk;
    extern __shared__ float sm[];
    __shared__ float nrm[2];
    float* qs = sm; float* ks = sm + dk; float* vs = sm + 2 * dk; float* red = sm + 2 * dk + DN_COLS;
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t pos0 = p.pos[0];
    float* S = p.ssm + ((size_t)h * dk) * dv + j0 + lane;
    float s[RPW];
#pragma unroll
    for (int r = 0; r < RPW; r++) s[r] = S[(size_t)(warp * RPW + r) * dv];
    // this thread's channels (at most two), their conv weights and the history before the window (oldest first)
    const int nel = 2 * dk + DN_COLS;
    float cw[2][K], hist[2][K - 1];
    int cidx[2]; bool own[2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int i = tid + e * DN_THREADS;
        int c = 0;
        if (i < nel) {
            if (i < dk) c = kh * dk + i;
            else if (i < 2 * dk) c = nk * dk + kh * dk + (i - dk);
            else c = 2 * nk * dk + h * dv + j0 + (i - 2 * dk);
#pragma unroll
            for (int k = 0; k < K; k++) cw[e][k] = p.conv_w[c * K + k];
#pragma unroll
            for (int k = 0; k < K - 1; k++) hist[e][k] = p.conv[(size_t)((int)(pos0 % K) + 1 + k) % K * ch + c];
        }
        cidx[e] = c;
        own[e] = i < nel && (i >= 2 * dk || (h == kh && j0 == 0));
    }
    const float dt_h = p.dt[h], a_h = p.a[h];
    // inputs of token 0; those of token j + 1 are requested while token j is computed
    float cur[2] = {0.f, 0.f}, alpha, beta;
#pragma unroll
    for (int e = 0; e < 2; e++) if (tid + e * DN_THREADS < nel) cur[e] = __ldcg(p.proj + cidx[e]);
    alpha = __ldcg(p.proj + ch + nv * dv + nv + h); beta = __ldcg(p.proj + ch + nv * dv + h);
    for (int j = 0; j < T; j++) {
        float ncur[2] = {0.f, 0.f}, nalpha = 0.f, nbeta = 0.f;
        if (j + 1 < T) {
            const float* pn = p.proj + (size_t)(j + 1) * p.ldp;
#pragma unroll
            for (int e = 0; e < 2; e++) if (tid + e * DN_THREADS < nel) ncur[e] = __ldcg(pn + cidx[e]);
            nalpha = __ldcg(pn + ch + nv * dv + nv + h); nbeta = __ldcg(pn + ch + nv * dv + h);
        }
        // 1) conv + SiLU (:1645), history shifted by one
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int i = tid + e * DN_THREADS;
            if (i < nel) {
                float o = cw[e][K - 1] * cur[e];
#pragma unroll
                for (int k = 0; k < K - 1; k++) o = fmaf(cw[e][k], hist[e][k], o);
                const float co = pb_silu(o);
                if (i < dk) qs[i] = co; else if (i < 2 * dk) ks[i - dk] = co; else vs[i - 2 * dk] = co;
#pragma unroll
                for (int k = 0; k + 1 < K - 1; k++) hist[e][k] = hist[e][k + 1];
                hist[e][K - 2] = cur[e];
                if (own[e] && j + K > T) p.conv[(size_t)((pos0 + j) % K) * ch + cidx[e]] = cur[e];   // the ring keeps the last K inputs
            }
        }
        __syncthreads();
        // 2) L2 norms (:1650-1651)
        if (warp < 2) {
            const float* src = warp == 0 ? qs : ks;
            float ss = 0.f;
            for (int i = lane; i < dk; i += 32) ss = fmaf(src[i], src[i], ss);
            ss = pb_warp_sum(ss);
            if (lane == 0) nrm[warp] = 1.0f / sqrtf(ss + 1e-6f) * (warp == 0 ? 1.0f / sqrtf((float)dk) : 1.0f);
        }
        __syncthreads();
        for (int i = tid; i < 2 * dk; i += DN_THREADS) sm[i] *= nrm[i < dk ? 0 : 1];
        __syncthreads();
        // 3) gates (:1660), 4) state update and readout (:1663)
        const float g = expf(pb_softplus(alpha + dt_h) * a_h);
        const float bt = pb_sigm(beta);
        float mem = 0.f;
#pragma unroll
        for (int r = 0; r < RPW; r++) {
            const int i = warp * RPW + r;
            s[r] *= g;
            mem = fmaf(s[r], ks[i], mem);
        }
        red[warp * DN_COLS + lane] = mem;
        __syncthreads();
        mem = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) mem += red[w * DN_COLS + lane];
        const float delta = (vs[lane] - mem) * bt;
        __syncthreads();
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < RPW; r++) {
            const int i = warp * RPW + r;
            s[r] = fmaf(ks[i], delta, s[r]);
            o = fmaf(s[r], qs[i], o);
        }
        red[warp * DN_COLS + lane] = o;
        __syncthreads();
        if (warp == 0) {
            o = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) o += red[w * DN_COLS + lane];
            p.out[(size_t)j * p.ldo + h * dv + j0 + lane] = o;
        }
        __syncthreads();   // red and the q / k / v vectors are rewritten by the next token
        // rollback checkpoint after token j (k_delta_m writes them from registers too, src/model/qn_cube.rs:2839-2913): the
        // state slice, and the K - 1 inputs the next token's conv reads, at their ring slots
        if (j < 8 && j + 1 < T && ck.ssm[j]) {
            float* C = ck.ssm[j] + ((size_t)h * dk) * dv + j0 + lane;
#pragma unroll
            for (int r = 0; r < RPW; r++) C[(size_t)(warp * RPW + r) * dv] = s[r];
#pragma unroll
            for (int e = 0; e < 2; e++)
                if (own[e])
#pragma unroll
                    for (int k = 0; k < K - 1; k++) ck.conv[j][(size_t)((pos0 + j - (K - 2) + k + K) % K) * ch + cidx[e]] = hist[e][k];
        }
        cur[0] = ncur[0]; cur[1] = ncur[1]; alpha = nalpha; beta = nbeta;
    }
#pragma unroll
    for (int r = 0; r < RPW; r++) S[(size_t)(warp * RPW + r) * dv] = s[r];
}

// T consecutive tokens of sequence 0 in one launch; false when the shape is outside what the kernel is built for
bool pb_deltanet_seq_supported(const PbDeltaParams& p) { return p.conv_k == 4 && p.dv % DN_COLS == 0 && (p.dk == 128 || p.dk == 64 || p.dk == 32) && 2 * p.dk + DN_COLS <= 2 * DN_THREADS; }
int pb_launch_deltanet_seq(pb_ctx* ctx, const PbDeltaParams& p, int T, const PbDeltaCk* ckp) {
    if (!pb_deltanet_seq_supported(p)) PB_FAIL(ctx, PB_UNSUPPORTED, "deltanet run: dk=%d dv=%d conv_k=%d not supported", p.dk, p.dv, p.conv_k);
    PbDeltaCk ck; memset(&ck, 0, sizeof ck);
    if (ckp) ck = *ckp;
    const dim3 grid(p.nv * (p.dv / DN_COLS));
    const size_t smem = (size_t)(2 * p.dk + DN_COLS + 8 * DN_COLS) * 4;
    if (p.dk == 128) pb_launch_k(ctx, pb_deltanet_seq_kernel<16>, grid, dim3(DN_THREADS), smem, p, T, ck);
    else if (p.dk == 64) pb_launch_k(ctx, pb_deltanet_seq_kernel<8>, grid, dim3(DN_THREADS), smem, p, T, ck);
    else pb_launch_k(ctx, pb_deltanet_seq_kernel<4>, grid, dim3(DN_THREADS), smem, p, T, ck);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

int pb_launch_deltanet(pb_ctx* ctx, const PbDeltaParams& p0) {
    PbDeltaParams p = p0;
    p.stamps = pb_stamp_slot(ctx, PB_K_DELTANET);
    if (p.dv % DN_COLS || (p.dk != 128 && p.dk != 64 && p.dk != 32) || p.conv_k < 2 || p.conv_k > 8)
        PB_FAIL(ctx, PB_UNSUPPORTED, "deltanet: dk=%d dv=%d conv_k=%d not supported", p.dk, p.dv, p.conv_k);
    // many sequences: a CTA walks all slices of its head (conv / norm / gates once per head)
    const bool whole = p.batch >= 8 && p.dv == 4 * DN_COLS;
    const dim3 grid(p.nv * (whole ? 1 : p.dv / DN_COLS), p.batch);
    const size_t smem = (size_t)(2 * p.dk + DN_COLS * (whole ? 4 : 1) + 8 * DN_COLS) * 4;
#define GO(R)                                                                                             \
    if (whole) pb_launch_k(ctx, pb_deltanet_kernel<R, 4>, dim3(grid), dim3(DN_THREADS), (size_t)(smem), p); \
    else pb_launch_k(ctx, pb_deltanet_kernel<R, 1>, dim3(grid), dim3(DN_THREADS), (size_t)(smem), p);
    if (p.dk == 128) { GO(16) } else if (p.dk == 64) { GO(8) } else { GO(4) }
#undef GO
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
