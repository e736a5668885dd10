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
#include "pb_common.cuh"
#include "pb_internal.h"

#include <stdio.h>

#define DN_THREADS 256
#define DN_COLS 32   // state columns per CTA

// NS = column slices of 32 one CTA walks in turn (1: most CTAs, shortest latency; dv / 32: the conv, norm and gate
// phases run once per head instead of once per slice, which pays when there are thousands of CTAs)
template <int RPW, int NS>
__global__ void __launch_bounds__(DN_THREADS) pb_deltanet_kernel(const PbDeltaParams p) {
    const int nk = p.nk, nv = p.nv, dk = p.dk, dv = p.dv, K = p.conv_k;
    const int ch = 2 * nk * dk + nv * dv;
    const int splits = dv / (DN_COLS * NS);
    const int h = blockIdx.x / splits, j0 = (blockIdx.x % splits) * DN_COLS * NS;
    const int b = blockIdx.y;
    const int kh = h % nk;                                  // V head h reads K head h % nk (:1655)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool st_first = tid == 0 && blockIdx.x == 0 && blockIdx.y == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1;
    pb_stamp(p.stamps, 0, st_first); pb_stamp(p.stamps, 6, st_last);
    pb_pdl_wait();
    pb_pdl_trigger();
    pb_stamp(p.stamps, 2, st_first);
    const float* proj = p.proj + (size_t)b * p.ldp;        // [qkv (ch) | z | beta | alpha]
    float* ring = p.conv + (size_t)b * K * ch;             // [K slots][ch]
    const int64_t pos = p.pos[b];
    const int wslot = (int)(pos % K);                       // slot that receives the current input

    // the state slice is requested first: rows i in [warp*rpw, (warp+1)*rpw), column j0 + lane; its DRAM
    // latency then overlaps the conv / norm / gate phases below, which do not depend on it
    constexpr int rpw = RPW;   // rows per warp = dk / 8 (16 for dk = 128)
    float* S = p.ssm + (((size_t)b * nv + h) * dk) * dv + j0 + lane;
    float s[RPW];
    // (only with few sequences: with thousands of CTAs the SM already overlaps them, and holding the slice
    // through the first phases costs more than it hides)
    const bool early = gridDim.y <= 4;
    if (early) {
#pragma unroll
        for (int r = 0; r < rpw; r++) s[r] = S[(size_t)(warp * rpw + r) * dv];
    }

    extern __shared__ float sm[];
    float* qs = sm;              // [dk] normalized q
    float* ks = sm + dk;         // [dk] normalized k
    float* vs = sm + 2 * dk;     // [DN_COLS * NS]
    float* red = sm + 2 * dk + DN_COLS * NS;   // [8 warps][DN_COLS]
    __shared__ float nrm[2];

    // 1) conv + SiLU for the channels this CTA needs: q and k of head kh, v columns j0..j0+31 of head h
    //    o = w[c*K + K-1] * cur + sum_{k < K-1} w[c*K + k] * hist[k]  (hist oldest first)   (:1645)
    for (int i = tid; i < 2 * dk + DN_COLS * NS; i += DN_THREADS) {
        int c;
        if (i < dk) c = kh * dk + i;
        else if (i < 2 * dk) c = nk * dk + kh * dk + (i - dk);
        else c = 2 * nk * dk + h * dv + j0 + (i - 2 * dk);
        const float cur = proj[c];
        float o = p.conv_w[c * K + K - 1] * cur;
        for (int k = 0; k < K - 1; k++) o += p.conv_w[c * K + k] * ring[(size_t)((pos + 1 + k) % K) * ch + c];
        const float co = pb_silu(o);
        if (i < dk) qs[i] = co; else if (i < 2 * dk) ks[i - dk] = co; else vs[i - 2 * dk] = co;
        // the history slot of this step: q/k channels are written by the first V head that maps
        // to K head kh (slice 0); v channels by their own CTA
        const bool owner = i >= 2 * dk || (h == kh && j0 == 0);
        if (owner) ring[(size_t)wslot * ch + c] = cur;
    }
    __syncthreads();
    // 2) L2 norms: x * (1/sqrt(sum x^2 + 1e-6)) * scale, q scaled by 1/sqrt(dk)  (:1650-1651)
    if (warp < 2) {
        const float* src = warp == 0 ? qs : ks;
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) ss += src[i] * src[i];
        ss = pb_warp_sum(ss);
        if (lane == 0) nrm[warp] = 1.0f / sqrtf(ss + 1e-6f) * (warp == 0 ? 1.0f / sqrtf((float)dk) : 1.0f);
    }
    __syncthreads();
    for (int i = tid; i < 2 * dk; i += DN_THREADS) sm[i] *= nrm[i < dk ? 0 : 1];
    __syncthreads();

    pb_stamp(p.stamps, 3, st_first);   // conv and norms done
    // 3) gates (:1660)
    const float alpha = proj[ch + nv * dv + nv + h], beta = proj[ch + nv * dv + h];
    const float g = expf(pb_softplus(alpha + p.dt[h]) * p.a[h]);
    const float bt = pb_sigm(beta);

    // 4) state slices (the first one was requested at the top when `early`)
#pragma unroll 1
    for (int sl = 0; sl < NS; sl++) {
        float* Ss = S + sl * DN_COLS;
        float mem = 0.f;
#pragma unroll
        for (int r = 0; r < rpw; r++) {
            const int i = warp * rpw + r;
            s[r] = ((early && sl == 0) ? s[r] : Ss[(size_t)i * dv]) * g;   // S *= g
            mem = fmaf(s[r], ks[i], mem);           // mem_j = sum_i S[i][j] k_i
        }
        if (sl > 0) __syncthreads();                // the previous slice's readers of red are done
        red[warp * DN_COLS + lane] = mem;
        __syncthreads();
        mem = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) mem += red[w * DN_COLS + lane];
        const float delta = (vs[sl * DN_COLS + lane] - mem) * bt;  // (:1663)
        __syncthreads();
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < rpw; r++) {
            const int i = warp * rpw + r;
            s[r] = fmaf(ks[i], delta, s[r]);        // S[i][j] += k_i * delta_j
            o = fmaf(s[r], qs[i], o);                // o_j = sum_i S[i][j] q_i
            Ss[(size_t)i * dv] = s[r];
        }
        red[warp * DN_COLS + lane] = o;
        __syncthreads();
        if (warp == 0) {
            o = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) o += red[w * DN_COLS + lane];
            p.out[(size_t)b * p.ldo + h * dv + j0 + sl * DN_COLS + lane] = o;   // readout before the gated norm
        }
    }
    pb_stamp(p.stamps, 5, st_first); pb_stamp(p.stamps, 7, st_last);
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
