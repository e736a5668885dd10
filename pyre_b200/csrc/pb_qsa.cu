// QSA block-sparse attention: the indexer that decides which key positions a query attends to.
//
// Restates the indexer part of attn_core (src/model/qwen4exp_gguf.rs:1565-1599; the reference's GPU form is
// qsa_pool / attn_qsa, :992-1012).  Tokens are grouped in blocks of `ratio`.  Every token leaves a raw index key
// (a projection of the layer input); a complete block has a pooled key: the mean of its raw keys, RMS-normed with
// the index key norm, roped at the block's first position.  A query that sees more than budget + ratio - 1 tokens
// scores every complete block with  sum over index heads of relu(q_h . pooled_b) / sqrt(idx_hd)  (q_h: raw index
// query head, RMS-normed, roped at the query's position) and attends to the budget / ratio best blocks plus the
// incomplete tail; equal scores go to the lower block.  The result is a bit mask over positions that the attention
// kernels (pb_attn.cu) read: tiles without a set bit are never fetched, unselected positions inside a fetched tile
// get a score of minus infinity.
//
//   pb_qsa_append_kernel  one CTA per sequence: store the token's raw key, pool the block it completes
//   pb_qsa_score_kernel   tiles of pooled keys in shared memory, a thread per block: the block scores, dots accumulated
//                         in the order of the reference's dot (32 partial sums, dot_avx2 in src/model/gguf_q.rs:176-197)
//   pb_qsa_pick_kernel    one CTA per sequence: the budget / ratio-th largest (score, lower block first) key by a
//                         radix select over 64-bit keys, then the mask
#include "pb_common.cuh"
#include "pb_internal.h"

#include <stdio.h>

#define QSA_MAX_HD 256

// sine and cosine (times the YaRN mscale) of this lane's rope angles at `pos`: dims lane and lane + 32 (rotary halves of up to 64)
struct PbQsaAngles { float sn[2], co[2]; };
__device__ __forceinline__ PbQsaAngles pb_qsa_angles(const float* rope_inv, int n_rot, int64_t pos, int lane) {
    PbQsaAngles a;
    const int half = n_rot / 2;
    const float ms = rope_inv[half];
#pragma unroll
    for (int k = 0; k < 2; k++) {
        a.sn[k] = 0.f; a.co[k] = 1.f;
        const int i = lane + 32 * k;
        if (i < half) {
            sincosf((float)pos * rope_inv[i], &a.sn[k], &a.co[k]);
            if (ms != 1.0f) { a.co[k] *= ms; a.sn[k] *= ms; }
        }
    }
    return a;
}
// rms_inplace(x, w) then rope over the first n_rot dims (n_rot <= 128) with the lane's angles, for a vector held by a warp
// (lane l: dims l, l + 32, ...)
__device__ __forceinline__ void pb_qsa_norm_rope_a(float* v, const float* w, int n, int n_rot, float eps, const PbQsaAngles& a, int lane) {
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) ss += v[i] * v[i];
    ss = pb_warp_sum(ss);
    const float s = 1.0f / sqrtf(ss / (float)n + eps);
    __syncwarp();
    for (int i = lane; i < n; i += 32) v[i] *= s * w[i];
    __syncwarp();
    const int half = n_rot / 2;
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const int i = lane + 32 * k;
        if (i < half) {
            const float x0 = v[i], x1 = v[i + half];
            v[i] = x0 * a.co[k] - x1 * a.sn[k]; v[i + half] = x1 * a.co[k] + x0 * a.sn[k];
        }
    }
    __syncwarp();
}
__device__ __forceinline__ void pb_qsa_norm_rope(float* v, const float* w, const float* rope_inv, int n, int n_rot, float eps, int64_t pos, int lane) {
    pb_qsa_norm_rope_a(v, w, n, n_rot, eps, pb_qsa_angles(rope_inv, n_rot, pos, lane), lane);
}

// pooled key of block `blk` of one sequence from its raw keys (one warp)
__device__ __forceinline__ void pb_qsa_pool_block(const PbQsaParams& p, const float* ik, float* ib, int64_t blk, float* tmp, int lane) {
    for (int i = lane; i < p.ihd; i += 32) {
        float a = 0.f;
        for (int64_t q = blk * p.ratio; q < (blk + 1) * p.ratio; q++) a += ik[q * p.ihd + i];
        tmp[i] = a / (float)p.ratio;
    }
    __syncwarp();
    pb_qsa_norm_rope(tmp, p.ikn, p.rope_inv, p.ihd, p.n_rot, p.eps, blk * p.ratio, lane);
    for (int i = lane; i < p.ihd; i += 32) ib[blk * p.ihd + i] = tmp[i];
}

// grid (batch), 32 threads
__global__ void __launch_bounds__(32) pb_qsa_append_kernel(const PbQsaParams p) {
    const int b = blockIdx.x, lane = threadIdx.x;
    __shared__ float tmp[QSA_MAX_HD];
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t pos = p.pos[b];
    const int sb = p.shared_seq ? 0 : b;
    float* ik = p.ik + (size_t)sb * p.max_ctx * p.ihd;
    float* ib = p.ib + (size_t)sb * p.nb_cap * p.ihd;
    const float* src = p.iproj + (size_t)b * p.ldi + (size_t)p.inh * p.ihd;
    for (int i = lane; i < p.ihd; i += 32) ik[pos * p.ihd + i] = src[i];
    __syncwarp();
    if ((pos + 1) % p.ratio == 0) pb_qsa_pool_block(p, ik, ib, pos / p.ratio, tmp, lane);
}

// grid (blocks to pool, sequences), 32 threads: pools blocks [0, nblk) of every sequence (after a restore or a fill)
__global__ void __launch_bounds__(32) pb_qsa_pool_kernel(const PbQsaParams p, int64_t nblk) {
    const int b = blockIdx.y, lane = threadIdx.x;
    __shared__ float tmp[QSA_MAX_HD];
    for (int64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x)
        pb_qsa_pool_block(p, p.ik + (size_t)b * p.max_ctx * p.ihd, p.ib + (size_t)b * p.nb_cap * p.ihd, blk, tmp, lane);
}

// grid (tiles, batch), 64 threads.  A CTA stages a tile of consecutive pooled keys in shared memory (coalesced loads, rows
// padded by one word so that a column walk is conflict-free), then thread i scores block i of the tile against every
// query head with the 32 running sums of the reference's dot (dot_avx2, src/model/gguf_q.rs:176-197: dims i, i + 32, ...
// go to sum i mod 32), combined in its order: (s0 + s1) + (s2 + s3) per lane of eight, the eight added one after the other.
#define QSA_TILE 64
// IHD > 0: the head dim is known at compile time and the thread keeps its block's key in registers, so that only the
// queries are read again for every head (as 128-bit broadcasts); IHD = 0: any head dim, everything from shared memory
template <int IHD>
__global__ void __launch_bounds__(QSA_TILE) pb_qsa_score_kernel(const PbQsaParams p, int tile_rows) {
    const int b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    extern __shared__ __align__(16) float qsm[];     // [inh][ihd] normed, roped index queries, then two tiles [tile_rows][ihd + 4]
    pb_pdl_wait();
    pb_pdl_trigger();
    const int ihd = IHD > 0 ? IHD : p.ihd;
    const int64_t pos = p.pos[b], n = pos + 1;
    if (n <= (int64_t)p.budget + p.ratio - 1) return;       // dense range (dense_n, :1555)
    const int64_t nb = n / p.ratio;
    if ((int64_t)blockIdx.x * tile_rows >= nb) return;
    const float* iq = p.iproj + (size_t)b * p.ldi;
    for (int i = tid; i < p.inh * ihd; i += QSA_TILE) qsm[i] = iq[i];
    __syncthreads();
    {   // the heads share the position: one pair of sincosf per lane for all of them
        const PbQsaAngles ang = pb_qsa_angles(p.rope_inv, p.n_rot, pos, lane);
        for (int h = warp; h < p.inh; h += QSA_TILE / 32) pb_qsa_norm_rope_a(qsm + h * ihd, p.iqn, ihd, p.n_rot, p.eps, ang, lane);
    }
    float* tile = qsm + p.inh * ihd;
    const int ld = ihd + 4;                                 // rows stay 16-byte aligned; eight rows fall into eight groups of four banks
    const int sb = p.shared_seq ? 0 : b;
    const float* ibase = p.ib + (size_t)sb * p.nb_cap * ihd;
    const float iscale = 1.0f / sqrtf((float)ihd);
    // two tile buffers: the next tile is on its way (cp.async) while this one is scored
    const int64_t t_step = (int64_t)gridDim.x * tile_rows;
    auto fetch = [&](int64_t t0, float* buf) {
        const int rows = (int)(nb - t0 < tile_rows ? nb - t0 : tile_rows);
        const float* src = ibase + t0 * ihd;
        for (int e = tid; e < rows * ihd / 4; e += QSA_TILE) {
            const int row = (4 * e) / ihd, col = 4 * e - row * ihd;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(pb_smem_u32(buf + row * ld + col)), "l"(src + 4 * e) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float* bufs[2] = {tile, tile + (size_t)tile_rows * ld};
    int cur = 0;
    fetch((int64_t)blockIdx.x * tile_rows, bufs[0]);
    for (int64_t t0 = (int64_t)blockIdx.x * tile_rows; t0 < nb; t0 += t_step, cur ^= 1) {
        const int rows = (int)(nb - t0 < tile_rows ? nb - t0 : tile_rows);
        if (t0 + t_step < nb) { fetch(t0 + t_step, bufs[cur ^ 1]); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                    // the tile (and, the first time, the queries) are ready
        tile = bufs[cur];
        if (tid < rows) {
            const float* kb = tile + tid * ld;
            float s = 0.f;
            if (IHD > 0) {
                float4 kr[IHD > 0 ? IHD / 4 : 1];
#pragma unroll
                for (int i = 0; i < IHD / 4; i++) kr[i] = *reinterpret_cast<const float4*>(kb + 4 * i);
                for (int h = 0; h < p.inh; h++) {
                    const float4* qh = reinterpret_cast<const float4*>(qsm + h * IHD);
                    float acc[32];
#pragma unroll
                    for (int j = 0; j < 32; j++) acc[j] = 0.f;
#pragma unroll
                    for (int i = 0; i < IHD / 4; i++) {
                        const float4 qv = qh[i];
                        const int j = (4 * i) & 31;
                        acc[j] = fmaf(qv.x, kr[i].x, acc[j]); acc[j + 1] = fmaf(qv.y, kr[i].y, acc[j + 1]);
                        acc[j + 2] = fmaf(qv.z, kr[i].z, acc[j + 2]); acc[j + 3] = fmaf(qv.w, kr[i].w, acc[j + 3]);
                    }
                    float r = 0.f;
#pragma unroll
                    for (int l = 0; l < 8; l++) r += (acc[l] + acc[8 + l]) + (acc[16 + l] + acc[24 + l]);
                    s += r > 0.f ? r : 0.f;
                }
            } else {
                for (int h = 0; h < p.inh; h++) {
                    const float* qh = qsm + h * ihd;
                    float acc[32];
#pragma unroll
                    for (int j = 0; j < 32; j++) acc[j] = 0.f;
                    for (int i = 0; i < ihd; i += 32) {
#pragma unroll
                        for (int j = 0; j < 32; j++) acc[j] = fmaf(qh[i + j], kb[i + j], acc[j]);
                    }
                    float r = 0.f;
#pragma unroll
                    for (int l = 0; l < 8; l++) r += (acc[l] + acc[8 + l]) + (acc[16 + l] + acc[24 + l]);
                    s += r > 0.f ? r : 0.f;
                }
            }
            p.scores[(size_t)b * p.nb_cap + t0 + tid] = s * iscale;
        }
        __syncthreads();                                    // everyone has left this buffer before the next fetch refills it
    }
}

// grid (batch), 1024 threads
__global__ void __launch_bounds__(1024) pb_qsa_pick_kernel(const PbQsaParams p) {
    const int b = blockIdx.x, tid = threadIdx.x;
    __shared__ unsigned int hist[256];
    __shared__ unsigned long long prefix_s;
    __shared__ int want_s, all_s;
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t pos = p.pos[b], n = pos + 1;
    if (n <= (int64_t)p.budget + p.ratio - 1) { if (tid == 0) p.sparse[b] = 0; return; }
    const int64_t nb = n / p.ratio;
    const int kk = p.budget / p.ratio;                 // nb > kk here: n >= budget + ratio
    const float* sc = p.scores + (size_t)b * p.nb_cap;
    // key: score bits (scores are >= 0, so their bit patterns order like the values), then the complement of the
    // block index, so that the larger key is the better block and no two keys are equal
    auto key = [&](int64_t blk) -> unsigned long long { return ((unsigned long long)__float_as_uint(sc[blk]) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)blk); };
    if (tid == 0) { prefix_s = 0ull; want_s = kk; }
    __syncthreads();
    // radix select, most significant byte first: the byte of the kk-th largest key among those that share the prefix
    for (int shift = 56; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0u;
        __syncthreads();
        const unsigned long long prefix = prefix_s;
        const unsigned long long himask = shift == 56 ? 0ull : ~0ull << (shift + 8);
        for (int64_t blk = tid; blk < nb; blk += 1024) {
            const unsigned long long k = key(blk);
            if ((k & himask) == prefix) atomicAdd(&hist[(unsigned int)(k >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid < 32) {
            // the bin that holds the want-th largest: lane l owns bins 8 l .. 8 l + 7; `above` = keys in the bins of higher lanes
            const int want = want_s;
            unsigned int c[8], mine = 0u;
#pragma unroll
            for (int j = 0; j < 8; j++) { c[j] = hist[8 * tid + j]; mine += c[j]; }
            unsigned int incl = mine;                    // inclusive suffix sum over lanes tid .. 31
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const unsigned int v = __shfl_down_sync(0xffffffffu, incl, o); if (tid + o < 32) incl += v; }
            const unsigned int above = incl - mine;
            if ((int)above < want && want <= (int)incl) {
                int w = want - (int)above, j = 7;
                for (; j > 0; j--) { if ((int)c[j] >= w) break; w -= (int)c[j]; }
                prefix_s = prefix | ((unsigned long long)(8 * tid + j) << shift);
                want_s = w;
                all_s = (int)c[j] == w;                 // every key that shares the prefix so far is wanted
            }
        }
        __syncthreads();
        if (shift == 32 && all_s) break;                // no tie at the cut: the block index bits need not be searched
    }
    const unsigned long long thr = prefix_s;            // the kk-th largest key (its low half zero when the search stopped early): exactly kk keys are >= thr
    uint32_t* mask = p.mask + (size_t)b * p.mask_ld;
    const int64_t nwords = (n + 31) / 32;
    for (int64_t w = tid; w < nwords; w += 1024) mask[w] = 0u;
    __syncthreads();
    for (int64_t blk = tid; blk < nb; blk += 1024) {
        if (key(blk) >= thr)
            for (int64_t q = blk * p.ratio; q < (blk + 1) * p.ratio; q++) atomicOr(&mask[q >> 5], 1u << (q & 31));
    }
    for (int64_t q = nb * p.ratio + tid; q < n; q += 1024) atomicOr(&mask[q >> 5], 1u << (q & 31));   // the incomplete tail
    if (tid == 0) p.sparse[b] = 1;
}

int pb_launch_qsa_append(pb_ctx* ctx, const PbQsaParams& p) {
    if (p.ihd > QSA_MAX_HD || p.ihd % 8 || p.n_rot > p.ihd || p.n_rot > 128) PB_FAIL(ctx, PB_UNSUPPORTED, "indexer head dim %d (a multiple of 8, at least the rope width %d <= 128, at most %d)", p.ihd, p.n_rot, QSA_MAX_HD);
    pb_launch_k(ctx, pb_qsa_append_kernel, dim3(p.batch), dim3(32), (size_t)0, p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

int pb_launch_qsa_select(pb_ctx* ctx, const PbQsaParams& p) {
    if (p.ihd % 32 || p.n_rot > 128) PB_FAIL(ctx, PB_UNSUPPORTED, "indexer head dim %d (a multiple of 32), rope width %d (at most 128)", p.ihd, p.n_rot);
    int tile_rows = QSA_TILE;
    auto need = [&](int rows) { return ((size_t)p.inh * p.ihd + (size_t)2 * rows * (p.ihd + 4)) * 4; };
    while (need(tile_rows) > 96 * 1024 && tile_rows > 8) tile_rows /= 2;
    const size_t smem = need(tile_rows);
    if (smem > 96 * 1024) PB_FAIL(ctx, PB_UNSUPPORTED, "indexer with %d heads of %d does not fit shared memory", p.inh, p.ihd);
    int64_t gx = (p.nb_cap + tile_rows - 1) / tile_rows;
    const int64_t cap = p.batch >= 4 ? 32 : 256;     // enough CTAs to fill the GPU
    if (gx > cap) gx = cap;
    const dim3 grid((unsigned)gx, p.batch);
    if (p.ihd == 128) { PB_TRY(pb_ensure_smem(ctx, pb_qsa_score_kernel<128>, smem)); pb_launch_k(ctx, pb_qsa_score_kernel<128>, grid, dim3(QSA_TILE), smem, p, tile_rows); }
    else if (p.ihd == 64) { PB_TRY(pb_ensure_smem(ctx, pb_qsa_score_kernel<64>, smem)); pb_launch_k(ctx, pb_qsa_score_kernel<64>, grid, dim3(QSA_TILE), smem, p, tile_rows); }
    else { PB_TRY(pb_ensure_smem(ctx, pb_qsa_score_kernel<0>, smem)); pb_launch_k(ctx, pb_qsa_score_kernel<0>, grid, dim3(QSA_TILE), smem, p, tile_rows); }
    pb_launch_k(ctx, pb_qsa_pick_kernel, dim3(p.batch), dim3(1024), (size_t)0, p);
    ctx->kernels_launched += 2;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

int pb_launch_qsa_pool_all(pb_ctx* ctx, const PbQsaParams& p, int64_t nblk) {
    if (nblk <= 0) return PB_OK;
    if (p.ihd > QSA_MAX_HD || p.n_rot > p.ihd || p.n_rot > 128) PB_FAIL(ctx, PB_UNSUPPORTED, "indexer head dim %d, rope width %d (at most 128)", p.ihd, p.n_rot);
    const unsigned gx = (unsigned)(nblk < 1024 ? nblk : 1024);
    pb_qsa_pool_kernel<<<dim3(gx, p.batch), 32, 0, ctx->stream>>>(p, nblk);
    ctx->kernels_launched++;
    ctx->pdl_chain = false;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
