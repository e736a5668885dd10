// Fused MoE block of the decode path: router + top-k + grouped expert SwiGLU + shared expert.
//
// Restates ffn / routed / top_k of the reference (src/model/qwen4exp_gguf.rs:1675-1684,
// 1721-1793 f32 branch, 3121-3139) and replaces its host-side routing (route_sel :2164-2174,
// behind a per-layer device->host readback) and the k_xgu* / k_xdown* / k_xgr_topk kernels
// (src/model/qn_cube.rs:3482-5419, 5210-5256).  Nothing leaves the device:
//   1. pb_router_kernel   RMSNorm (optional) + f32 router GEMV + shared-gate logit; also emits
//                         the normalized activations split into int8 levels for the experts
//   2. pb_route_tokens    (last router CTA of each group of 8 tokens) per token top-k (descending logit, ties to the
//                         lower id, NaN -> -inf), softmax over the selection, selection sorted by expert id;
//      pb_route_lists     (last of those CTAs) the list of distinct local experts with their (token, slot) entries
//   3. pb_expert_gu_kernel   h = silu(gate_e x) * (up_e x) for every (expert, token) entry and the
//                         shared expert; weights streamed once per expert
//   4. pb_split_h_kernel  (several tokens) the hidden vectors of all entries split into int8 levels once
//   5. pb_expert_down_kernel part[token][slot] = w * (down_e h); shared expert unweighted
//   6. pb_moe_combine_kernel y = sigmoid(shared gate) * shared + sum over slots in ascending
//                         expert id (fixed order: deterministic, independent of the GPU count)
//   One token on one GPU replaces 4-6 by pb_expert_down_rows_kernel, which cuts the work by output rows
//   and forms the same ordered sum inside each CTA.
#include "pb_stream.cuh"
#include "pb_internal.h"
#include "pb_topk.cuh"
#include "pb_router.cuh"
#include "pb_ep.cuh"

#include <stdio.h>

// ------------------------------------------------------------------------------------ routing

// Tokens [b_lo, b_hi) by the 256 threads of one CTA (the last router CTA of the tokens' group), warp per token.
// Everything stays in registers: lane l holds experts l, l+32, ... of the token.
__device__ __forceinline__ void pb_route_tokens(const PbRouteParams& p, int b_lo, int b_hi) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int b = b_lo + warp; b < b_hi; b += 8) {
        const float* lg = p.logits + (size_t)b * p.ldl;
        // lane j keeps the j-th pick, its softmax weight and its rank by expert id (pb_topk.cuh)
        int my_e, rank; float w;
        pb_route_token(lg, p.n_exp, p.top_k, lane, my_e, w, rank);
        if (lane < p.top_k) { p.sel_e[b * p.top_k + rank] = my_e; p.sel_w[b * p.top_k + rank] = w; }
    }
}

// One token routed by all 256 threads of the CTA (the last router CTA), the scheme of the fused step kernel's routing: every logit
// becomes a 64-bit key (pb_topk.cuh); pass 1: each warp ranks its own keys (n_exp / 8 of them) by counting the greater ones and
// passes on its top_k; pass 2: the 8 * top_k candidates are ranked the same way, the counting of each cut over several threads;
// rank j < top_k is the j-th pick, and warp 0 finishes as pb_route_token does (same picks, same weights, same order).  One warp
// alone spends top_k rounds of a warp-wide maximum on this.  sm = 2048 ints of shared memory; n_exp <= 512, top_k <= 16.
__device__ __forceinline__ void pb_route_token_cta(const PbRouteParams& p, int b, int* sm) {
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(sm);      // [8 warps][32 * kpt]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kpt = (p.n_exp + 255) / 256, gsz = 32 * kpt, top_k = p.top_k;   // kpt <= 2
    unsigned long long* cand = keys + 8 * gsz;                                  // [8][top_k]
    unsigned long long* pick = cand + 8 * 16;                                   // [top_k]
    int* crank = reinterpret_cast<int*>(pick + 16);                             // [8 * top_k]
    const float* lg = p.logits + (size_t)b * p.ldl;
    if (tid < 8 * 16) crank[tid] = 0;
    unsigned long long mine[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        mine[j] = 0;
        if (j < kpt) {
            const int e = tid + 256 * j;
            mine[j] = e < p.n_exp ? pb_topk_key(__ldcg(lg + e), e) : (unsigned long long)(0xFFFFFFFFu - (unsigned)e);   // slots past n_exp: distinct keys below every real one
            keys[warp * gsz + j * 32 + lane] = mine[j];
        }
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; j++) {
        if (j < kpt) {
            int rk = 0;
            for (int i = 0; i < gsz; i++) rk += keys[warp * gsz + i] > mine[j] ? 1 : 0;
            if (rk < top_k) cand[warp * top_k + rk] = mine[j];
        }
    }
    __syncthreads();
    const int ncand = 8 * top_k, parts = 256 / ncand;   // parts >= 2: ncand <= 128
    if (tid < ncand * parts) {
        const int ci = tid % ncand, part = tid / ncand;
        const int i0 = part * ncand / parts, i1 = (part + 1) * ncand / parts;
        const unsigned long long key = cand[ci];
        int rk = 0;
#pragma unroll 4
        for (int i = i0; i < i1; i++) rk += cand[i] > key ? 1 : 0;
        if (rk) atomicAdd(&crank[ci], rk);
    }
    __syncthreads();
    if (warp == 0) {
        for (int i = lane; i < ncand; i += 32) { const int rk = crank[i]; if (rk < top_k) pick[rk] = cand[i]; }
        __syncwarp();
        int my_e, rank; float w;
        pb_route_finish(lane < top_k ? pick[lane] : 0ull, top_k, lane, my_e, w, rank);
        if (lane < top_k) { p.sel_e[b * top_k + rank] = my_e; p.sel_w[b * top_k + rank] = w; }
    }
    __syncthreads();
}

// Runs in ONE CTA of 256 threads (the last router CTA to finish) once every token is routed: the list of distinct local
// experts with their (token, slot) entries.  rsm = 2048 ints of shared memory.
__device__ __forceinline__ void pb_route_lists(const PbRouteParams& p, int* rsm) {
    int* cnt = rsm;                 // [1024] entries per expert (local experts only)
    int* cursor = rsm + 1024;       // [1024] start offset of the expert's entries, then a fill cursor
    __shared__ int wsum[2][8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int e = tid; e < 1024; e += 256) { cnt[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int i = tid; i < p.t * p.top_k; i += 256) {
        const int e = __ldcg(p.sel_e + i);
        if (e >= p.e_lo && e < p.e_hi) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    // distinct local experts in ascending id with entry offsets: block-wide exclusive scans of
    // (used flag, entry count) over expert ids; thread t owns experts 4t .. 4t+3
    int c4[4], f = 0, c = 0;
#pragma unroll
    for (int q = 0; q < 4; q++) { const int e = 4 * tid + q; c4[q] = e < p.n_exp ? cnt[e] : 0; f += c4[q] > 0; c += c4[q]; }
    int fi = f, ci = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int a = __shfl_up_sync(0xffffffffu, fi, o), d = __shfl_up_sync(0xffffffffu, ci, o); if (lane >= o) { fi += a; ci += d; } }
    if (lane == 31) { wsum[0][warp] = fi; wsum[1][warp] = ci; }
    __syncthreads();
    int fb = 0, cb = 0;
    for (int w2 = 0; w2 < warp; w2++) { fb += wsum[0][w2]; cb += wsum[1][w2]; }
    int n = fb + fi - f, off = cb + ci - c;   // exclusive prefixes for expert 4 * tid
#pragma unroll
    for (int q = 0; q < 4; q++) if (c4[q] > 0) { const int e = 4 * tid + q; p.used_e[n] = e; p.used_off[n] = off; cursor[e] = off; n++; off += c4[q]; }
    if (tid == 255) { p.used_off[n] = off; *p.n_used = n; }
    __syncthreads();
    for (int i = tid; i < p.t * p.top_k; i += 256) {
        const int e = __ldcg(p.sel_e + i);
        if (e >= p.e_lo && e < p.e_hi) { const int pos = atomicAdd(&cursor[e], 1); p.ent_tok[pos] = i / p.top_k; p.ent_slot[pos] = i % p.top_k; p.ent_w[pos] = __ldcg(p.sel_w + i); }
    }
}

// ------------------------------------------------------------------------------------ router

// grid: ceil((n_exp + 1) / 8) CTAs of 256 threads; warp per router row (row n_exp = shared-gate vector).
// CTA j additionally splits groups 4j..4j+3 of every token's normalized activations into int8
// levels for the expert kernels, so that work is spread over the grid.
#define PB_ROUTER_TPG 8   // tokens per router CTA (one warp each for the RMS scales)
#define PB_ROUTER_TICKETS 8   // ticket[0 .. 8): whole-launch counters (router, expert kernels); ticket[8 + g]: token group g of the router
__global__ void __launch_bounds__(256) pb_router_kernel(const PbRouterParams p, const PbRouteParams rp, unsigned int* ticket) {
    extern __shared__ float rs[];   // 2048 ints for the routing pass, then scale[t]
    float* scale = rs + 2048;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool st_first = tid == 0 && blockIdx.x == 0 && blockIdx.y == 0;
    pb_stamp(p.stamps, 0, st_first);
    // the warp's router row (times the norm weight) is model data: it is fetched before the wait for the previous kernel, so its
    // trip to DRAM overlaps that kernel's tail
    const int row = blockIdx.x * 8 + warp;
    const float* wrow = p.phase != 2 && row <= p.n_exp ? (row < p.n_exp ? p.router + (size_t)row * p.cols : p.sh_gate_inp) : nullptr;
    PbRouterRow2048 rr;
    if (p.cols == 2048 && wrow) rr.load(wrow, p.norm_w, lane);
    pb_pdl_wait();
    pb_pdl_trigger();
    pb_stamp(p.stamps, 2, st_first);
    if (p.zero && p.phase != 1) {
        // expert parallelism: the partial-row buffer must be zero where other ranks' experts write; cleared
        // here instead of by a memset node between the launches (which would also end the dependent-launch chain)
        float4* z = reinterpret_cast<float4*>(p.zero);
        const int64_t n4 = p.zero_n / 4, nthreads = (int64_t)gridDim.x * gridDim.y * 256;
        for (int64_t i = ((int64_t)blockIdx.y * gridDim.x + blockIdx.x) * 256 + tid; i < n4; i += nthreads) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // grid.y cuts the tokens into groups of PB_ROUTER_TPG: this CTA handles tokens [b_lo, b_hi)
    const int b_lo = (int)blockIdx.y * PB_ROUTER_TPG, b_hi = min(p.t, b_lo + PB_ROUTER_TPG);
    if (p.t == 1 && p.cols == 2048 && p.phase == 0 && p.norm_w && !p.exch) {
        // One token on one GPU: every warp fetches the activation row once, in the layout that the RMS scale, the row product and
        // (for the CTAs that split a piece of it) the split all use, instead of one trip to L2 for each of the three.  Same arithmetic
        // as pb_row_rms_scale, PbRouterRow2048::dot and the general loops below.
        float4 xv[16];
#pragma unroll
        for (int k = 0; k < 16; k++) xv[k] = *reinterpret_cast<const float4*>(p.x + lane * 4 + 128 * k);
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 16; k++) ss += fmaf(xv[k].x, xv[k].x, fmaf(xv[k].y, xv[k].y, fmaf(xv[k].z, xv[k].z, __fmul_rn(xv[k].w, xv[k].w))));
        ss = pb_warp_sum(ss);
        const float s = 1.0f / sqrtf(ss / (float)p.cols + p.eps);
        if (warp == 0 && (int)blockIdx.x < 16) {   // groups 4 j .. 4 j + 3 of CTA j are elements 128 j + 4 lane ..: the lane's xv[j]
            float4 v = xv[0];
#pragma unroll
            for (int k = 1; k < 16; k++) if (k == (int)blockIdx.x) v = xv[k];
            const int g0 = (int)blockIdx.x * 4;
            const float4 n = *reinterpret_cast<const float4*>(p.norm_w + 32 * g0 + 4 * lane);
            v.x = v.x * s * n.x; v.y = v.y * s * n.y; v.z = v.z * s * n.z; v.w = v.w * s * n.w;
            pb_split_groups4(v, lane, g0, p.cols, p.xq_out);
        }
        pb_stamp(p.stamps, 3, st_first);
        if (wrow) {
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int k = 0; k < 16; k++) { a0 = fmaf(rr.wr[k].x, xv[k].x, a0); a1 = fmaf(rr.wr[k].y, xv[k].y, a1); a2 = fmaf(rr.wr[k].z, xv[k].z, a2); a3 = fmaf(rr.wr[k].w, xv[k].w, a3); }
            const float acc = pb_warp_sum((a0 + a1) + (a2 + a3)) * s;
            if (lane == 0) p.logits[row] = acc;
        }
    } else {
    // per-token RMS scale (rms(): 1 / sqrt(mean(x^2) + eps), qwen4exp_gguf.rs:209); one warp per token
    for (int b = b_lo + warp; b < b_hi; b += 8) {
        const float s = p.norm_w ? pb_row_rms_scale(p.x + b * p.ldx, p.cols, p.eps, lane) : 1.0f;
        if (lane == 0) scale[b] = s;
    }
    __syncthreads();
    const int ng = p.cols / 32;
    for (int g0 = blockIdx.x * 4; g0 < ng; g0 += gridDim.x * 4) {
        for (int b = b_lo + warp; b < b_hi; b += 8) {
            float4 v = *reinterpret_cast<const float4*>(p.x + b * p.ldx + 32 * g0 + 4 * lane);
            if (p.phase == 1) {   // raw row for the gather: the local copy, and with a peer exchange every rank's gathered buffer
                *reinterpret_cast<float4*>(p.xcopy + b * p.ldl + 32 * g0 + 4 * lane) = v;
                if (p.exch) for (int q = 0; q < p.exch->world; q++) *reinterpret_cast<float4*>(p.exch->peer_xg[q] + p.peer_off + b * p.ldl + 32 * g0 + 4 * lane) = v;
                continue;
            }
            if (p.norm_w) {
                const float4 n = *reinterpret_cast<const float4*>(p.norm_w + 32 * g0 + 4 * lane);
                const float s = scale[b];
                v.x = v.x * s * n.x; v.y = v.y * s * n.y; v.z = v.z * s * n.z; v.w = v.w * s * n.w;
            }
            pb_split_groups4(v, lane, g0, p.cols, p.xq_out + (size_t)b * pb_xq_words(p.cols));
        }
    }
    pb_stamp(p.stamps, 3, st_first);   // activations split
    if (p.phase != 2 && row <= p.n_exp) {
        if (p.cols == 2048 && wrow) {
            // the row, times the norm weight, stays in registers for all tokens
#pragma unroll 2
            for (int b = b_lo; b < b_hi; b++) {
                const float acc = rr.dot(p.x + b * p.ldx, scale[b], lane);
                if (lane == 0) p.logits[b * p.ldl + row] = acc;
                if (p.exch && lane < p.exch->world) p.exch->peer_xg[lane][p.peer_off + b * p.ldl + p.cols + row] = acc;
            }
        } else
        for (int b = b_lo; b < b_hi; b++) {
            const float acc = wrow ? pb_router_row_dot(wrow, p.norm_w, p.x + b * p.ldx, scale[b], p.cols, lane) : 0.f;
            if (lane == 0) p.logits[b * p.ldl + row] = acc;
            if (p.exch && lane < p.exch->world) p.exch->peer_xg[lane][p.peer_off + b * p.ldl + p.cols + row] = acc;
        }
    }
    }
    if (p.phase == 1) {
        if (!p.exch) return;
        // peer exchange: every CTA fences its stores into peer memory and takes a ticket; the last one announces the
        // exchange to every rank and waits for theirs (one thread per rank)
        __shared__ int last1;
        __threadfence_system();
        __syncthreads();
        if (tid == 0) last1 = atomicAdd(ticket, 1u) == gridDim.x * gridDim.y - 1;
        __syncthreads();
        if (!last1) return;
        if (tid == 0) *ticket = 0;
        if (tid < p.exch->world) pb_ep_handshake(*p.exch, tid, 0, *p.exch->seq_base + (unsigned long long)p.exch_idx + 1);
        return;
    }
    // two levels of the last-block pattern (fence, ticket, the last one reads what the others wrote): the last CTA of a
    // token group (grid.y) routes the group's tokens, so the groups are routed in parallel; the last of those CTAs
    // builds the expert lists from all selections.  The tickets are reset for the next launch.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    pb_stamp(p.stamps, 5, st_first);   // this CTA's logits stored
    if (tid == 0) is_last = atomicAdd(ticket + PB_ROUTER_TICKETS + blockIdx.y, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    if (tid == 0) ticket[PB_ROUTER_TICKETS + blockIdx.y] = 0;
    __threadfence();
    pb_stamp(p.stamps, 6, tid == 0 && blockIdx.y == 0);   // the routing pass of the first group starts (its logits are in)
    if (b_hi - b_lo == 1 && rp.top_k <= 16 && rp.n_exp >= rp.top_k && rp.n_exp <= 512) pb_route_token_cta(rp, b_lo, reinterpret_cast<int*>(rs));   // 512 experts: its keys and candidates fit the 8 KB
    else pb_route_tokens(rp, b_lo, b_hi);
    if (gridDim.y > 1) {
        __threadfence();
        __syncthreads();
        if (tid == 0) is_last = atomicAdd(ticket, 1u) == gridDim.y - 1;
        __syncthreads();
        if (!is_last) return;
        if (tid == 0) *ticket = 0;
        __threadfence();
    } else __syncthreads();   // one group: this CTA routed every token itself
    if (rp.t == 1 && rp.top_k <= 32) {
        // one token: its selection, already in ascending expert id, IS the list of distinct experts, one entry each (what
        // pb_route_lists would build with its counting pass over all expert ids)
        if (warp == 0) {
            const int e = lane < rp.top_k ? __ldcg(rp.sel_e + lane) : -1;
            const bool local = e >= rp.e_lo && e < rp.e_hi;
            const unsigned m = __ballot_sync(0xffffffffu, local);
            const int n = __popc(m & ((1u << lane) - 1u));
            if (local) { rp.used_e[n] = e; rp.used_off[n] = n; rp.ent_tok[n] = 0; rp.ent_slot[n] = lane; rp.ent_w[n] = __ldcg(rp.sel_w + lane); }
            if (lane == 0) { const int tot = __popc(m); rp.used_off[tot] = tot; *rp.n_used = tot; }
        }
    } else pb_route_lists(rp, reinterpret_cast<int*>(rs));
    __syncthreads();
    pb_stamp(p.stamps, 7, tid == 0);
}

// ------------------------------------------------------------------------------------ expert gate/up

#define PB_SH_GROUP 4   // tokens per virtual shared expert (see pb_expert_gu_kernel)

template <int FMT, int PASSES>
__global__ void __launch_bounds__(PB_KTHREADS, 1) pb_expert_gu_kernel(const PbExpertParams p) {
    using D = PbQDec<FMT>;
    extern __shared__ __align__(128) uint8_t smem[];
    PbRing ring;
    ring.full = reinterpret_cast<uint64_t*>(smem);
    ring.empty = ring.full + PB_STAGES;
    uint8_t* tab = smem + 256;
    ring.stages = tab + p.tab_bytes;
    ring.stage_bytes = p.stage_bytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool st_first = tid == 0 && blockIdx.x == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1;
    pb_stamp(p.stamps, 0, st_first); pb_stamp(p.stamps, 6, st_last);
    pb_pdl_trigger();
    pb_ring_init(ring, tid);
    __syncthreads();
    pb_stamp(p.stamps, 1, st_first);
    pb_pdl_wait();   // the expert lists come from the routing kernel
    pb_stamp(p.stamps, 2, st_first);

    const int cols = p.bpr * 256;
    const int n_used = *p.n_used;
    const int cpe = p.rows_e / p.rows_per_chunk;                       // chunks per routed expert
    // the shared expert serves every token: its tokens are cut into groups of PB_SH_GROUP, each group a
    // virtual expert with its own chunks, so that no chunk carries 32 tokens' worth of dots (those chunks
    // used to finish last and left most SMs idle)
    const int cps1 = p.has_shared ? p.rows_sh / p.rows_per_chunk : 0;   // row chunks of the shared expert
    const int cps = cps1 * ((p.sh_ntok + PB_SH_GROUP - 1) / PB_SH_GROUP);
    const int nchunks = n_used * cpe + cps;
    const int my_chunks = nchunks > (int)blockIdx.x ? (nchunks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const uint32_t half = (uint32_t)p.rows_per_chunk * p.row_bytes;   // a multiple of 16 by construction
    const uint32_t xbytes = (uint32_t)pb_xq_words(p.bpr * 256) * 4;   // one token's activation levels (a multiple of 16)

    // chunk headers {first row, first entry, end entry, shared flag}, one per stage, written by the producer:
    // the consumers start a chunk without a division or a dependent chain of global loads
    int4* hdr = reinterpret_cast<int4*>(smem + 128);
    if (warp == PB_CONSUMERS) {
        // the whole warp looks up the metadata of 32 chunks at a time (expert id, entry range, first token: up
        // to three dependent global loads each, in parallel over the lanes); lane 0 then issues the copies
        int k = 0; bool ok = true;
        for (int k0 = 0; k0 < my_chunks && ok; k0 += 32) {
            const int kk = k0 + lane;
            int m_e = 0, m_r0 = 0, m_e0 = 0, m_e1 = 0, m_tok0 = 0, m_tok1 = 0, m_sh = 0;
            if (kk < my_chunks) {
                const int chunk = (int)blockIdx.x + kk * (int)gridDim.x;
                if (chunk < n_used * cpe) {
                    const int s = chunk / cpe;
                    m_r0 = (chunk - s * cpe) * p.rows_per_chunk;
                    m_e = p.used_e[s]; m_e0 = p.used_off[s]; m_e1 = p.used_off[s + 1];
                    const bool in = m_e0 >= 0 && m_e0 < p.t * p.top_k;
                    m_tok0 = in ? p.ent_tok[m_e0] : -1;
                    m_tok1 = in && m_e1 - m_e0 > 1 && m_e0 + 1 < p.t * p.top_k ? p.ent_tok[m_e0 + 1] : 0;
                } else {
                    const int sc = chunk - n_used * cpe;
                    m_sh = 1; m_r0 = (sc % cps1) * p.rows_per_chunk;
                    m_e0 = (sc / cps1) * PB_SH_GROUP; m_e1 = min(p.sh_ntok, m_e0 + PB_SH_GROUP);
                    m_tok0 = p.sh_tok0 + m_e0; m_tok1 = m_tok0 + 1;
                }
            }
            const int nk = min(32, my_chunks - k0);
            for (int j = 0; j < nk; j++, k++) {
                const int e = __shfl_sync(0xffffffffu, m_e, j), r0 = __shfl_sync(0xffffffffu, m_r0, j), e0 = __shfl_sync(0xffffffffu, m_e0, j);
                const int e1 = __shfl_sync(0xffffffffu, m_e1, j), sh = __shfl_sync(0xffffffffu, m_sh, j);
                int good = 1;
                if (lane == 0) {
                    if (!sh && (e < 0 || e >= p.n_exp)) { atomicExch(p.status, PB_DEV_BAD_INDEX); good = 0; }
                    else if (!pb_ring_acquire_wait(ring, k, p.status)) good = 0;
                    else {
                        const uint8_t *g, *u;
                        if (!sh) { const size_t off = ((size_t)(e - p.e_base) * p.rows_e + r0) * p.row_bytes; g = p.w_a + off; u = p.w_b + off; }
                        else { const size_t off = (size_t)r0 * p.row_bytes; g = p.sh_a + off; u = p.sh_b + off; }
                        hdr[k % PB_STAGES] = make_int4(r0, e0, e1, sh);
                        pb_ring_announce(ring, k, 2 * half + xbytes * (uint32_t)min(p.nx, max(1, e1 - e0)));
                        pb_ring_copy(ring, k, 0, g, half);
                        pb_ring_copy(ring, k, half, u, half);
                    }
                }
                good = __shfl_sync(0xffffffffu, good, 0);
                if (!good) { ok = false; break; }
                // the activation levels of the chunk's first entries (p.nx of them, at most two) ride along, so that the
                // consumers read them from shared memory instead of waiting for L2 after the decode.  The tokens come
                // from a second dependent load, awaited only here, after the weights are on their way.
                int tok0 = __shfl_sync(0xffffffffu, m_tok0, j), tok1 = __shfl_sync(0xffffffffu, m_tok1, j);
                if (lane == 0) {
                    if (tok0 < 0 || tok0 >= p.t) { atomicExch(p.status, PB_DEV_BAD_INDEX); tok0 = 0; }   // the announced bytes must still arrive
                    pb_ring_copy(ring, k, 2 * half, p.xq + (size_t)tok0 * pb_xq_words(p.bpr * 256), xbytes);
                    if (p.nx > 1 && e1 - e0 > 1) {
                        if (tok1 < 0 || tok1 >= p.t) { atomicExch(p.status, PB_DEV_BAD_INDEX); tok1 = 0; }
                        pb_ring_copy(ring, k, 2 * half + xbytes, p.xq + (size_t)tok1 * pb_xq_words(p.bpr * 256), xbytes);
                    }
                }
            }
        }
        if (!ok && lane == 0) pb_ring_drain(ring, k);
        return;
    }

    constexpr int CT = PB_CONSUMERS * 32;
    const PbQTabs T = pb_fill_qtabs<FMT>(tab, p.rep, tid, CT, lane);
    pb_named_barrier(1, CT);
    const int nquarters = 4 * p.bpr;
    const int lpr = nquarters < 32 ? nquarters : 32, rpw = 32 / lpr;
    const int sub = lane / lpr, ql = lane - sub * lpr;
    const int xw = pb_xq_words(cols);
    pb_stamp(p.stamps, 3, st_first);

    for (int k = 0; k < my_chunks; k++) {
        if (!pb_ring_wait(ring, k, p.status)) return;
        if (k == 0) pb_stamp(p.stamps, 4, st_first);
        const int4 hd = hdr[k % PB_STAGES];
        const int r0 = hd.x, e0 = hd.y, e1 = hd.z;
        const bool shared = hd.w != 0;
        // tokens of the entries after the first, one per lane, requested before the decode
        const bool lanes_hold = e1 - e0 <= 33;
        int l_tok = 0;
        if (!shared && lanes_hold && e0 + 1 + lane < e1) l_tok = p.ent_tok[e0 + 1 + lane];
        const uint32_t base = pb_smem_u32(pb_ring_stage(ring, k));
        for (int rb = warp * rpw; rb < p.rows_per_chunk; rb += PB_CONSUMERS * rpw) {
            const int r = rb + sub;
            PbQuarter wg[PASSES], wu[PASSES];
#pragma unroll
            for (int ps = 0; ps < PASSES; ps++) {
                const int qi = ps * 32 + ql;
                if (qi < nquarters) {
                    D::quarter(base + (uint32_t)r * p.row_bytes + (qi >> 2) * D::STEP_BYTES, qi & 3, T, wg[ps]);
                    D::quarter(base + half + (uint32_t)r * p.row_bytes + (qi >> 2) * D::STEP_BYTES, qi & 3, T, wu[ps]);
                }
            }
            for (int en = e0; en < e1; en++) {
                int tok = 0;
                if (shared) tok = p.sh_tok0 + en;
                else if (en > e0) tok = lanes_hold ? __shfl_sync(0xffffffffu, l_tok, en - e0 - 1) : p.ent_tok[en];
                const uint32_t* xcol = en - e0 < p.nx ? reinterpret_cast<const uint32_t*>(pb_ring_stage(ring, k) + 2 * half + (uint32_t)(en - e0) * xbytes) : p.xq + (size_t)tok * xw;
                float g = 0.f, u = 0.f;
#pragma unroll
                for (int ps = 0; ps < PASSES; ps++) {
                    const int qi = ps * 32 + ql;
                    if (qi < nquarters) {
                        PbXQuarter xv;
                        pb_load_xquarter<PbQDec<FMT>::AFFINE>(xcol, cols, qi, xv);
                        g += pb_quarter_dot<FMT>(wg[ps], xv);
                        u += pb_quarter_dot<FMT>(wu[ps], xv);
                    }
                }
                for (int o = lpr >> 1; o > 0; o >>= 1) { g += __shfl_xor_sync(0xffffffffu, g, o); u += __shfl_xor_sync(0xffffffffu, u, o); }
                if (ql == 0) {
                    // hidden = silu(gate . x) * (up . x)   (routed :1781-1783, ffn :1680)
                    float* dst = shared ? p.h_sh + (size_t)tok * p.rows_sh : p.h + (size_t)en * p.rows_e;
                    dst[r0 + r] = pb_silu(g) * u;
                }
            }
        }
        pb_ring_release(ring, k, lane);
    }
    pb_stamp(p.stamps, 5, st_first); pb_stamp(p.stamps, 7, st_last);
}

// y[tok][r] = sigmoid(shared-gate logit) * shared[tok][r] + sum_j part[tok][j][r]  (ascending expert id),
// then either stored (layer-level call) or added to the residual stream.  One output element.
__device__ __forceinline__ void pb_combine_one(const PbCombineParams& p, int64_t i, bool bypass_l1) {
    const int tok = (int)(i / p.d), r = (int)(i - (int64_t)tok * p.d);
    float y = 0.f;
    if (p.part_sh) y = (bypass_l1 ? __ldcg(p.part_sh + i) : p.part_sh[i]) * pb_sigm(p.logits[(size_t)tok * p.ldl + p.n_exp]);   // routed :1723
    float o = 0.f;
    for (int j = 0; j < p.top_k; j++) { const float* q = p.part + ((size_t)tok * p.top_k + j) * p.d + r; o += bypass_l1 ? __ldcg(q) : *q; }
    y += o;
    float* dst = p.y + (size_t)tok * p.ldy + r;
    *dst = p.accumulate ? *dst + y : y;
}

// ------------------------------------------------------------------------------------ expert down

// Hidden vectors of all (expert, token) entries and of the shared expert -> int8 levels, once, for the
// down kernel of a multi-token step.  grid = t * top_k + t CTAs (entry slots past the number of local
// entries return), one warp per four 32-value groups.
__global__ void __launch_bounds__(128) pb_split_h_kernel(const PbExpertParams p) {
    pb_pdl_wait();
    pb_pdl_trigger();
    const int cols = p.bpr * 256, xw = pb_xq_words(cols), ne = p.t * p.top_k;
    const int slot = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* src;
    if (slot < ne) { if (slot >= p.used_off[*p.n_used]) return; src = p.h + (size_t)slot * cols; }
    else { const int tok = slot - ne; if (!p.has_shared || tok < p.sh_tok0 || tok >= p.sh_tok0 + p.sh_ntok) return; src = p.h_sh + (size_t)tok * cols; }
    uint32_t* dst = p.hq + (size_t)slot * xw;
    for (int g0 = warp * 4; g0 < cols / 32; g0 += 16) pb_split_groups4(*reinterpret_cast<const float4*>(src + 32 * g0 + 4 * lane), lane, g0, cols, dst);
}

template <int FMT, int PASSES>
__global__ void __launch_bounds__(PB_KTHREADS, 1) pb_expert_down_kernel(const PbExpertParams p, const PbCombineParams cp, unsigned int* ticket) {
    using D = PbQDec<FMT>;
    extern __shared__ __align__(128) uint8_t smem[];
    PbRing ring;
    ring.full = reinterpret_cast<uint64_t*>(smem);
    ring.empty = ring.full + PB_STAGES;
    uint8_t* tab = smem + 256;
    const int cols = p.bpr * 256;   // = expert intermediate size
    const int xw = pb_xq_words(cols);
    uint32_t* xq = reinterpret_cast<uint32_t*>(tab + p.tab_bytes);
    ring.stages = reinterpret_cast<uint8_t*>(xq) + (((size_t)xw * 4 + 127) & ~(size_t)127);
    ring.stage_bytes = p.stage_bytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pb_pdl_trigger();
    pb_ring_init(ring, tid);
    __syncthreads();
    pb_pdl_wait();   // the expert lists and hidden vectors come from earlier kernels

    const int n_used = *p.n_used;
    const int cpe = p.rows_e / p.rows_per_chunk;   // output rows (= model width) per expert / rows per chunk
    const int cps1 = p.has_shared ? cpe : 0;   // shared expert: token groups as in pb_expert_gu_kernel
    const int cps = cps1 * ((p.sh_ntok + PB_SH_GROUP - 1) / PB_SH_GROUP);
    const int nchunks = n_used * cpe + cps;
    const int my_chunks = nchunks > (int)blockIdx.x ? (nchunks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const uint32_t bytes = (uint32_t)p.rows_per_chunk * p.row_bytes;
    const uint32_t hbytes = (uint32_t)xw * 4;   // levels of one hidden vector (a multiple of 16)

    int4* hdr = reinterpret_cast<int4*>(smem + 128);   // chunk headers as in pb_expert_gu_kernel
    if (warp == PB_CONSUMERS) {
        int k = 0; bool ok = true;
        for (int k0 = 0; k0 < my_chunks && ok; k0 += 32) {
            const int kk = k0 + lane;
            int m_e = 0, m_r0 = 0, m_e0 = 0, m_e1 = 0, m_sh = 0;
            if (kk < my_chunks) {
                const int chunk = (int)blockIdx.x + kk * (int)gridDim.x;
                if (chunk < n_used * cpe) {
                    const int s = chunk / cpe;
                    m_r0 = (chunk - s * cpe) * p.rows_per_chunk;
                    m_e = p.used_e[s]; m_e0 = p.used_off[s]; m_e1 = p.used_off[s + 1];
                } else {
                    const int sc = chunk - n_used * cpe;
                    m_sh = 1; m_r0 = (sc % cps1) * p.rows_per_chunk;
                    m_e0 = (sc / cps1) * PB_SH_GROUP; m_e1 = min(p.sh_ntok, m_e0 + PB_SH_GROUP);
                }
            }
            const int nk = min(32, my_chunks - k0);
            for (int j = 0; j < nk; j++, k++) {
                const int e = __shfl_sync(0xffffffffu, m_e, j), r0 = __shfl_sync(0xffffffffu, m_r0, j), e0 = __shfl_sync(0xffffffffu, m_e0, j);
                const int e1 = __shfl_sync(0xffffffffu, m_e1, j), sh = __shfl_sync(0xffffffffu, m_sh, j);
                int good = 1;
                if (lane == 0) {
                    if (!sh && (e < 0 || e >= p.n_exp || e0 < 0 || e0 >= p.t * p.top_k)) { atomicExch(p.status, PB_DEV_BAD_INDEX); good = 0; }
                    else if (!pb_ring_acquire_wait(ring, k, p.status)) good = 0;
                    else {
                        const uint8_t* src = sh ? p.sh_a + (size_t)r0 * p.row_bytes : p.w_a + ((size_t)(e - p.e_base) * p.rows_e + r0) * p.row_bytes;
                        hdr[k % PB_STAGES] = make_int4(r0, e0, e1, sh);
                        if (p.hq) {
                            // several tokens: the levels of the chunk's first hidden vector ride along with the weights
                            // (the hidden vectors of an expert's entries, and of consecutive tokens, are adjacent in hq)
                            const size_t slot = sh ? (size_t)p.t * p.top_k + p.sh_tok0 + e0 : (size_t)e0;
                            const uint32_t hb = hbytes * (uint32_t)min(p.nx, max(1, e1 - e0));
                            pb_ring_announce(ring, k, bytes + hb);
                            pb_ring_copy(ring, k, 0, src, bytes);
                            pb_ring_copy(ring, k, bytes, p.hq + slot * xw, hb);
                        } else {
                            pb_ring_announce(ring, k, bytes);
                            pb_ring_copy(ring, k, 0, src, bytes);
                        }
                    }
                }
                good = __shfl_sync(0xffffffffu, good, 0);
                if (!good) { ok = false; break; }
            }
        }
        if (!ok && lane == 0) pb_ring_drain(ring, k);
        return;
    }

    constexpr int CT = PB_CONSUMERS * 32;
    const PbQTabs T = pb_fill_qtabs<FMT>(tab, p.rep, tid, CT, lane);
    pb_named_barrier(1, CT);
    const int nquarters = 4 * p.bpr;
    const int lpr = nquarters < 32 ? nquarters : 32, rpw = 32 / lpr;
    const int sub = lane / lpr, ql = lane - sub * lpr;
    const int ng = cols / 32;

    for (int k = 0; k < my_chunks; k++) {
        if (!pb_ring_wait(ring, k, p.status)) return;
        const int4 hd = hdr[k % PB_STAGES];
        const int r0 = hd.x, e0 = hd.y, e1 = hd.z;
        const bool shared = hd.w != 0;
        const uint32_t base = pb_smem_u32(pb_ring_stage(ring, k));
        if (p.hq) {
            // several tokens: the hidden vectors were split by pb_split_h_kernel; decode each row once
            // and walk the entries of the expert with their levels read from global memory
            // entry bookkeeping of the chunk (token, slot, weight), one entry per lane, requested before the decode:
            // read inside the entry loop each of these global loads would stall the store that ends an entry
            const bool lanes_hold = !shared && e1 - e0 <= 32;
            int l_tok = 0, l_slot = 0; float l_w = 0.f;
            if (lanes_hold && e0 + lane < e1) { l_tok = p.ent_tok[e0 + lane]; l_slot = p.ent_slot[e0 + lane]; l_w = p.ent_w[e0 + lane]; }
            for (int rb = warp * rpw; rb < p.rows_per_chunk; rb += PB_CONSUMERS * rpw) {
                const int r = rb + sub;
                PbQuarter wq[PASSES];
#pragma unroll
                for (int ps = 0; ps < PASSES; ps++) {
                    const int qi = ps * 32 + ql;
                    if (qi < nquarters) D::quarter(base + (uint32_t)r * p.row_bytes + (qi >> 2) * D::STEP_BYTES, qi & 3, T, wq[ps]);
                }
                for (int en = e0; en < e1; en++) {
                    int tok, slot = 0; float wgt = 1.0f;
                    if (lanes_hold) { tok = __shfl_sync(0xffffffffu, l_tok, en - e0); slot = __shfl_sync(0xffffffffu, l_slot, en - e0); wgt = __shfl_sync(0xffffffffu, l_w, en - e0); }
                    else if (shared) tok = p.sh_tok0 + en;
                    else { tok = p.ent_tok[en]; slot = p.ent_slot[en]; wgt = p.ent_w[en]; }
                    const uint32_t* xcol = en - e0 < p.nx ? reinterpret_cast<const uint32_t*>(pb_ring_stage(ring, k) + bytes + (uint32_t)(en - e0) * hbytes) : p.hq + (size_t)(shared ? p.t * p.top_k + tok : en) * xw;
                    float acc = 0.f;
#pragma unroll
                    for (int ps = 0; ps < PASSES; ps++) {
                        const int qi = ps * 32 + ql;
                        if (qi < nquarters) { PbXQuarter xv; pb_load_xquarter<PbQDec<FMT>::AFFINE>(xcol, cols, qi, xv); acc += pb_quarter_dot<FMT>(wq[ps], xv); }
                    }
                    for (int o = lpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    if (ql == 0) {
                        if (shared) p.part_sh[(size_t)tok * p.rows_e + r0 + r] = acc;
                        else if (p.part_tok) p.part_tok[tok][(size_t)slot * p.rows_e + r0 + r] = wgt * acc;   // straight into the owner's memory
                        else p.part[((size_t)tok * p.top_k + slot) * p.rows_e + r0 + r] = wgt * acc;
                    }
                }
            }
        } else
        for (int en = e0; en < e1; en++) {
            const int tok = shared ? p.sh_tok0 + en : p.ent_tok[en];
            const float* hv = shared ? p.h_sh + (size_t)tok * cols : p.h + (size_t)en * cols;
            // split this entry's hidden vector into int8 levels (all consumer warps, one group each)
            pb_named_barrier(1, CT);
            for (int g0 = warp * 4; g0 < ng; g0 += PB_CONSUMERS * 4) pb_split_groups4(*reinterpret_cast<const float4*>(hv + 32 * g0 + 4 * lane), lane, g0, cols, xq);
            pb_named_barrier(1, CT);
            float* dst; float wgt = 1.0f;
            if (shared) dst = p.part_sh + (size_t)tok * p.rows_e;
            else { dst = p.part_tok ? p.part_tok[tok] + (size_t)p.ent_slot[en] * p.rows_e : p.part + ((size_t)tok * p.top_k + p.ent_slot[en]) * p.rows_e; wgt = p.ent_w[en]; }
            for (int rb = warp * rpw; rb < p.rows_per_chunk; rb += PB_CONSUMERS * rpw) {
                const int r = rb + sub;
                float acc = 0.f;
#pragma unroll
                for (int ps = 0; ps < PASSES; ps++) {
                    const int qi = ps * 32 + ql;
                    if (qi < nquarters) {
                        PbQuarter wq; PbXQuarter xv;
                        D::quarter(base + (uint32_t)r * p.row_bytes + (qi >> 2) * D::STEP_BYTES, qi & 3, T, wq);
                        pb_load_xquarter<PbQDec<FMT>::AFFINE>(xq, cols, qi, xv);
                        acc += pb_quarter_dot<FMT>(wq, xv);
                    }
                }
                for (int o = lpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (ql == 0) dst[r0 + r] = wgt * acc;   // routed :1786: o += w * dot
            }
        }
        pb_ring_release(ring, k, lane);
    }
    // optional fused combine (small token counts, single GPU): the last CTA whose consumers get here
    // sums the partial rows of all CTAs -- last-block pattern: fence, ticket, fence, L1-bypassing reads
    if (!ticket) return;
    __shared__ int is_last;
    __threadfence();
    pb_named_barrier(1, CT);
    if (tid == 0) is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    pb_named_barrier(1, CT);
    if (!is_last) return;
    if (tid == 0) *ticket = 0;
    __threadfence();
    for (int64_t i = tid; i < (int64_t)cp.t * cp.d; i += CT) pb_combine_one(cp, i, true);
}

// ------------------------------------------------------------------------------------ expert down, one token

// One token on one GPU: the work is cut by OUTPUT ROWS instead of by expert.  CTA c owns rows
// [16 c, 16 c + 16) of every selected expert and of the shared expert, so the weighted sum over the
// experts (ascending expert id, then the shared expert as in pb_combine_one) is formed inside the CTA
// and written straight to y: no partial-row buffer, no combine pass, no per-chunk barriers.  All
// row slices (<= 16 x 16 rows) are requested up front; the hidden vectors of all entries are split into
// int8 levels once per CTA.
#define PB_DR_ROWS 16
#define PB_DR_MAXE 16
template <int FMT>
__global__ void __launch_bounds__(PB_KTHREADS, 1) pb_expert_down_rows_kernel(const PbExpertParams p, const PbCombineParams cp) {
    using D = PbQDec<FMT>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);                       // [PB_DR_MAXE]
    float* res = reinterpret_cast<float*>(smem + 128);                        // [PB_DR_MAXE][16 rows]
    uint8_t* tab = smem + 128 + PB_DR_MAXE * PB_DR_ROWS * 4;
    const int cols = p.bpr * 256, xw = pb_xq_words(cols);
    uint32_t* xq = reinterpret_cast<uint32_t*>(tab + p.tab_bytes);            // [n_used + 1][xw]
    const uint32_t slice = (uint32_t)PB_DR_ROWS * p.row_bytes;                // bytes of one expert's 16 rows
    uint8_t* stages = reinterpret_cast<uint8_t*>(xq) + (((size_t)PB_DR_MAXE * xw * 4 + 127) & ~(size_t)127);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool st_first = tid == 0 && blockIdx.x == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1;
    pb_stamp(p.stamps, 0, st_first); pb_stamp(p.stamps, 6, st_last);
    pb_pdl_trigger();
    if (tid == 0) {
        for (int i = 0; i < PB_DR_MAXE; i++) pb_mbar_init(&full[i], 1);
        pb_fence_barrier_init();
    }
    __syncthreads();
    pb_stamp(p.stamps, 1, st_first);
    pb_pdl_wait();   // expert lists and hidden vectors come from earlier kernels
    pb_stamp(p.stamps, 2, st_first);
    const int n_used = *p.n_used;
    const int nsl = n_used + (p.has_shared ? 1 : 0);   // slices: the used experts in ascending id, then the shared expert
    const int r0 = (int)blockIdx.x * PB_DR_ROWS;
    if (nsl > PB_DR_MAXE) { if (tid == 0) atomicExch(p.status, PB_DEV_BAD_INDEX); return; }

    if (warp == PB_CONSUMERS) {
        if (lane == 0) {
            int k = 0;
            for (; k < nsl; k++) {
                const uint8_t* src;
                if (k < n_used) {
                    const int e = p.used_e[k];
                    if (e < 0 || e >= p.n_exp) { atomicExch(p.status, PB_DEV_BAD_INDEX); break; }
                    src = p.w_a + ((size_t)(e - p.e_base) * p.rows_e + r0) * p.row_bytes;
                } else src = p.sh_a + (size_t)r0 * p.row_bytes;
                pb_mbar_expect_tx(&full[k], slice);
                pb_bulk_g2s(stages + (size_t)k * slice, src, slice, &full[k]);
            }
            // a slice that was not requested is completed by hand so that no consumer waits for it
            for (int j = k; j < nsl; j++) pb_mbar_arrive(&full[j]);
        }
        return;
    }

    constexpr int CT = PB_CONSUMERS * 32;
    const PbQTabs T = pb_fill_qtabs<FMT>(tab, p.rep, tid, CT, lane);
    // int8 levels of every entry's hidden vector (entry k of expert slice k: one token), four groups per warp pass
    const int gpe = cols / 128;   // warp passes per entry
    for (int i = warp; i < nsl * gpe; i += PB_CONSUMERS) {
        const int k = i / gpe, g0 = (i - k * gpe) * 4;
        const float* hv = k < n_used ? p.h + (size_t)p.used_off[k] * cols : p.h_sh + (size_t)p.sh_tok0 * cols;
        pb_split_groups4(*reinterpret_cast<const float4*>(hv + 32 * g0 + 4 * lane), lane, g0, cols, xq + (size_t)k * xw);
    }
    pb_named_barrier(1, CT);
    pb_stamp(p.stamps, 3, st_first);

    const int nquarters = 4 * p.bpr;                    // <= 32 (checked on the host)
    const int rpw = 32 / nquarters, sub = lane / nquarters, ql = lane - sub * nquarters;
    const int ppe = PB_DR_ROWS / rpw;                   // warp passes per slice
    for (int i = warp; i < nsl * ppe; i += PB_CONSUMERS) {
        const int k = i / ppe, r = (i - k * ppe) * rpw + sub;
        if (!pb_mbar_wait(&full[k], 0, p.status, PB_DEV_WAIT_FULL_TIMEOUT)) break;
        if (i == 0) pb_stamp(p.stamps, 4, st_first);
        PbQuarter wq; PbXQuarter xv;
        D::quarter(pb_smem_u32(stages + (size_t)k * slice) + (uint32_t)r * p.row_bytes + (ql >> 2) * D::STEP_BYTES, ql & 3, T, wq);
        pb_load_xquarter<PbQDec<FMT>::AFFINE>(xq + (size_t)k * xw, cols, ql, xv);
        float acc = pb_quarter_dot<FMT>(wq, xv);
        for (int o = nquarters >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (ql == 0) res[k * PB_DR_ROWS + r] = acc;
    }
    pb_named_barrier(1, CT);
    if (tid < PB_DR_ROWS) {
        // pb_combine_one for token sh_tok0: sigmoid(gate) * shared + sum over slots in ascending expert id
        float y = 0.f;
        if (p.has_shared) y = __fmul_rn(res[n_used * PB_DR_ROWS + tid], pb_sigm(cp.logits[(size_t)p.sh_tok0 * cp.ldl + cp.n_exp]));
        float o = 0.f;
        // product rounded, then added (no fused multiply-add): the bits of the partial-row path
        for (int k = 0; k < n_used; k++) o = __fadd_rn(o, __fmul_rn(p.ent_w[p.used_off[k]], res[k * PB_DR_ROWS + tid]));
        y = __fadd_rn(y, o);
        float* dst = cp.y + (size_t)p.sh_tok0 * cp.ldy + r0 + tid;
        *dst = cp.accumulate ? *dst + y : y;
    }
    pb_stamp(p.stamps, 5, st_first); pb_stamp(p.stamps, 7, st_last);
}

// ------------------------------------------------------------------------------------ combine

// y[tok][r] = sigmoid(shared-gate logit) * shared[tok][r] + sum_j part[tok][j][r]  (ascending expert id),
// then either stored (layer-level call) or added to the residual stream.
__global__ void __launch_bounds__(256) pb_moe_combine_kernel(const PbCombineParams p) {
    pb_pdl_wait();      // with a peer exchange: this rank's expert rows are stored in their owners' memory
    pb_pdl_trigger();
    if (p.exch) {
        // CTA 0 announces, every CTA waits for all ranks (one thread per rank); the barrier hands the acquired view on
        if ((int)threadIdx.x < p.exch->world) {
            const unsigned long long seq = *p.exch->seq_base + (unsigned long long)p.exch_idx + 1;
            if (blockIdx.x == 0) pb_ep_handshake(*p.exch, threadIdx.x, 1, seq);
            else pb_ep_wait(*p.exch, threadIdx.x, 1, seq);
        }
        __syncthreads();
    }
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < (int64_t)p.t * p.d) pb_combine_one(p, i, false);
}

// ------------------------------------------------------------------------------------ launchers

int pb_launch_router(pb_ctx* ctx, const PbRouterParams& p, const PbRouteParams& rp, unsigned int* ticket) {
    if (p.cols % 128) PB_FAIL(ctx, PB_UNSUPPORTED, "router: width %d is not a multiple of 128", p.cols);
    if (rp.top_k > PB_MAX_TOPK || rp.n_exp > 1024) PB_FAIL(ctx, PB_UNSUPPORTED, "route: top_k %d / n_exp %d beyond %d / 1024", rp.top_k, rp.n_exp, PB_MAX_TOPK);
    const int grid = p.phase == 2 ? (p.cols / 128 > 0 ? p.cols / 128 : 1) : (p.n_exp + 1 + 7) / 8;   // phase 2 only splits (4 groups of 32 per CTA) and routes
    const size_t smem = (size_t)(2048 + ((p.t + 31) & ~31)) * 4;
    PbRouterParams ps = p;
    ps.stamps = pb_stamp_slot(ctx, PB_K_ROUTER);
    pb_launch_k(ctx, pb_router_kernel, dim3(grid, (p.t + PB_ROUTER_TPG - 1) / PB_ROUTER_TPG), dim3(256), smem, ps, rp, ticket);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

template <int FMT, int PASSES, bool DOWN>
static int launch_expert(pb_ctx* ctx, PbExpertParams p, int cols, const PbCombineParams* cp, unsigned int* ticket) {
    int el, bs;
    pb_geom(FMT, &el, &bs);
    p.row_bytes = cols / el * bs; p.bpr = cols / 256;
    // a few MB per launch at one or two tokens: the plain codebook; many tokens select most experts
    // (hundreds of MB), where the per-bank replicated form of pb_gemvq.cu pays for its fill
    constexpr int entry = pb_tab_entry_bytes<FMT>();
    p.rep = entry && p.t >= 4 ? pb_tab_rep_max<FMT>() : 1;
    p.tab_bytes = pb_tab_bytes<FMT>(p.rep);
    const int lpr = 4 * p.bpr < 32 ? 4 * p.bpr : 32;
    int rpc = PB_CONSUMERS * (32 / lpr);
    while ((rpc * p.row_bytes) % 16) rpc *= 2;
    if (p.rows_e % rpc || (p.has_shared && !DOWN && p.rows_sh % rpc)) PB_FAIL(ctx, PB_UNSUPPORTED, "expert kernel: %d rows per expert is not a multiple of the %d-row chunk", p.rows_e, rpc);
    p.rows_per_chunk = rpc;
    const size_t xbytes = DOWN ? (((size_t)pb_xq_words(cols) * 4 + 127) & ~(size_t)127) : 0;
    // a stage = the chunk's rows + the activation levels of its first nx entries: two (gate/up) or four (down) where
    // shared memory allows (formats without tables), else one
    p.nx = p.t == 1 ? 1 : (DOWN ? 4 : 2);   // one token: one entry per expert, and smaller stages start sooner
    p.stage_bytes = (uint32_t)((((size_t)rpc * p.row_bytes * (DOWN ? 1 : 2)) + (size_t)p.nx * pb_xq_words(cols) * 4 + 16 + 127) & ~(size_t)127);
    if (256 + p.tab_bytes + xbytes + (size_t)PB_STAGES * p.stage_bytes > (size_t)ctx->max_smem_optin) {
        p.nx = 1;
        p.stage_bytes = (uint32_t)((((size_t)rpc * p.row_bytes * (DOWN ? 1 : 2)) + (size_t)pb_xq_words(cols) * 4 + 16 + 127) & ~(size_t)127);
    }
    // wide rows (Q8_0 at 2048 columns: 2176 bytes): fewer rows per chunk than consumer warps, the other warps sit the chunk out
    while (256 + p.tab_bytes + xbytes + (size_t)PB_STAGES * p.stage_bytes > (size_t)ctx->max_smem_optin && rpc > 32 / lpr && ((rpc / 2) * p.row_bytes) % 16 == 0) {
        rpc /= 2;
        p.rows_per_chunk = rpc;
        p.stage_bytes = (uint32_t)((((size_t)rpc * p.row_bytes * (DOWN ? 1 : 2)) + (size_t)pb_xq_words(cols) * 4 + 16 + 127) & ~(size_t)127);
    }
    const size_t smem = 256 + p.tab_bytes + xbytes + (size_t)PB_STAGES * p.stage_bytes;
    if (smem > (size_t)ctx->max_smem_optin) PB_FAIL(ctx, PB_UNSUPPORTED, "expert kernel needs %zu bytes of shared memory", smem);
    p.status = ctx->dev_status;
    p.stamps = pb_stamp_slot(ctx, DOWN ? PB_K_EXPERT_DOWN : PB_K_EXPERT_GU);
    if (DOWN && cp && p.t == 1 && p.top_k + 1 <= PB_DR_MAXE && p.rows_e % PB_DR_ROWS == 0 && 4 * p.bpr <= 32 && PB_DR_ROWS % (32 / (4 * p.bpr)) == 0 && PASSES == 1) {
        // one token, combine requested: the row-partitioned kernel writes y directly
        const size_t xbytes1 = (((size_t)PB_DR_MAXE * pb_xq_words(cols) * 4 + 127) & ~(size_t)127);
        const size_t smem1 = 128 + PB_DR_MAXE * PB_DR_ROWS * 4 + p.tab_bytes + xbytes1 + (size_t)PB_DR_MAXE * PB_DR_ROWS * p.row_bytes;
        if (smem1 <= (size_t)ctx->max_smem_optin) {
            auto kern = pb_expert_down_rows_kernel<FMT>;
            PB_TRY(pb_ensure_smem(ctx, kern, smem1));
            pb_launch_k(ctx, kern, dim3(p.rows_e / PB_DR_ROWS), dim3(PB_KTHREADS), smem1, p, *cp);
            ctx->kernels_launched++;
            PB_CUDA(ctx, cudaGetLastError());
            return PB_OK;
        }
    }
    if (DOWN) {
        if (p.hq) {
            pb_launch_k(ctx, pb_split_h_kernel, dim3(p.t * p.top_k + p.t), dim3(128), (size_t)0, p);
            ctx->kernels_launched++;
            PB_CUDA(ctx, cudaGetLastError());
        }
        auto kern = pb_expert_down_kernel<FMT, PASSES>;
        PB_TRY(pb_ensure_smem(ctx, kern, smem));
        PbCombineParams c0; memset(&c0, 0, sizeof c0);
        pb_launch_k(ctx, kern, dim3(ctx->sm_count), dim3(PB_KTHREADS), (size_t)(smem), p, cp ? *cp : c0, cp ? ticket : (unsigned int*)nullptr);
    } else {
        auto kern = pb_expert_gu_kernel<FMT, PASSES>;
        PB_TRY(pb_ensure_smem(ctx, kern, smem));
        pb_launch_k(ctx, kern, dim3(ctx->sm_count), dim3(PB_KTHREADS), (size_t)(smem), p);
    }
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

template <bool DOWN>
static int launch_expert_type(pb_ctx* ctx, const PbExpertParams& p, int type, int cols, const PbCombineParams* cp = nullptr, unsigned int* ticket = nullptr) {
    if (!pb_gemvq_supported(type, cols)) PB_FAIL(ctx, PB_UNSUPPORTED, "expert kernel: ggml type %d with %d columns is not supported", type, cols);
#define GO(F) return cols <= 2048 ? launch_expert<F, 1, DOWN>(ctx, p, cols, cp, ticket) : launch_expert<F, 2, DOWN>(ctx, p, cols, cp, ticket)
    switch (type) {
        case PB_T_IQ3_S: GO(PB_T_IQ3_S);
        case PB_T_IQ3S_N4: GO(PB_T_IQ3S_N4);
        case PB_T_IQ2_XS: GO(PB_T_IQ2_XS);
        case PB_T_Q4_K: GO(PB_T_Q4_K);
        case PB_T_IQ3_XXS: GO(PB_T_IQ3_XXS);
        case PB_T_IQ2_S: GO(PB_T_IQ2_S);
        case PB_T_IQ4_NL: GO(PB_T_IQ4_NL);
        case PB_T_IQ4_XS: GO(PB_T_IQ4_XS);
        case PB_T_Q2_0: GO(PB_T_Q2_0);
        case PB_T_IQ2_XXS: GO(PB_T_IQ2_XXS);
        case PB_T_Q6_K: GO(PB_T_Q6_K);
        case PB_T_IQ1_M: GO(PB_T_IQ1_M);
        case PB_T_Q4_0: GO(PB_T_Q4_0);
        case PB_T_Q5_0: GO(PB_T_Q5_0);
        case PB_T_Q3_K: GO(PB_T_Q3_K);
        case PB_T_Q5_K: GO(PB_T_Q5_K);
        default: GO(PB_T_Q8_0);
    }
#undef GO
}

int pb_launch_expert_gu(pb_ctx* ctx, const PbExpertParams& p, int type, int cols) { return launch_expert_type<false>(ctx, p, type, cols); }
// cp != null: the last CTA also performs the combine (see pb_expert_down_kernel)
int pb_launch_expert_down(pb_ctx* ctx, const PbExpertParams& p, int type, int cols, const PbCombineParams* cp, unsigned int* ticket) { return launch_expert_type<true>(ctx, p, type, cols, cp, ticket); }

int pb_launch_moe_combine(pb_ctx* ctx, const PbCombineParams& p) {
    const int64_t n = (int64_t)p.t * p.d;
    pb_launch_k(ctx, pb_moe_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)(0), p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
