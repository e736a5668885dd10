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
