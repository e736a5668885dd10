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
//   pb_qsa_score_kernel   grid (blocks / 128, sequences): the block scores, dots accumulated in the order of the
//                         reference's dot (32 partial sums, dot_avx2 in src/model/gguf_q.rs:176-197)
//   pb_qsa_pick_kernel    one CTA per sequence: the budget / ratio-th largest (score, lower block first) key by a
//                         radix select over 64-bit keys, then the mask
#include "pb_common.cuh"
#include "pb_internal.h"

#include <stdio.h>

#define QSA_MAX_HD 256

// rms_inplace(x, w) then rope at `pos` over the first n_rot dims, for a vector held by a warp (lane l: dims l, l + 32, ...)
__device__ __forceinline__ void pb_qsa_norm_rope(float* v, const float* w, const float* rope_inv, int n, int n_rot, float eps, int64_t pos, int lane) {
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) ss += v[i] * v[i];
    ss = pb_warp_sum(ss);
    const float s = 1.0f / sqrtf(ss / (float)n + eps);
    __syncwarp();
    for (int i = lane; i < n; i += 32) v[i] *= s * w[i];
    __syncwarp();
    const int half = n_rot / 2;
    const float ms = rope_inv[half];
    for (int i = lane; i < half; i += 32) {
        float sn, co;
        sincosf((float)pos * rope_inv[i], &sn, &co);
        if (ms != 1.0f) { co *= ms; sn *= ms; }
        const float x0 = v[i], x1 = v[i + half];
        v[i] = x0 * co - x1 * sn; v[i + half] = x1 * co + x0 * sn;
    }
    __syncwarp();
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

// grid (ceil(nb_cap / 128), batch), 128 threads
__global__ void __launch_bounds__(128) pb_qsa_score_kernel(const PbQsaParams p) {
    const int b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    extern __shared__ float qsm[];     // [inh][ihd] normed, roped index queries
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t pos = p.pos[b], n = pos + 1;
    if (n <= (int64_t)p.budget + p.ratio - 1) return;       // dense range (dense_n, :1555)
    const int64_t nb = n / p.ratio;
    if ((int64_t)blockIdx.x * 128 >= nb) return;
    const float* iq = p.iproj + (size_t)b * p.ldi;
    for (int i = tid; i < p.inh * p.ihd; i += 128) qsm[i] = iq[i];
    __syncthreads();
    for (int h = warp; h < p.inh; h += 4) pb_qsa_norm_rope(qsm + h * p.ihd, p.iqn, p.rope_inv, p.ihd, p.n_rot, p.eps, pos, lane);
    __syncthreads();
    const int64_t blk = (int64_t)blockIdx.x * 128 + tid;
    if (blk >= nb) return;
    const int sb = p.shared_seq ? 0 : b;
    const float* kb = p.ib + ((size_t)sb * p.nb_cap + blk) * p.ihd;
    const float iscale = 1.0f / sqrtf((float)p.ihd);
    float s = 0.f;
    for (int h = 0; h < p.inh; h++) {
        const float* q = qsm + h * p.ihd;
        // dot in the order of the reference: four groups of eight running sums over strides of 32, then
        // (s0 + s1) + (s2 + s3) per lane, lanes added in order
        float a[4][8];
#pragma unroll
        for (int k = 0; k < 4; k++)
#pragma unroll
            for (int l = 0; l < 8; l++) a[k][l] = 0.f;
        int i = 0;
        for (; i + 32 <= p.ihd; i += 32) {
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float4 k0 = *reinterpret_cast<const float4*>(kb + i + 8 * k), k1 = *reinterpret_cast<const float4*>(kb + i + 8 * k + 4);
                a[k][0] = fmaf(q[i + 8 * k + 0], k0.x, a[k][0]); a[k][1] = fmaf(q[i + 8 * k + 1], k0.y, a[k][1]);
                a[k][2] = fmaf(q[i + 8 * k + 2], k0.z, a[k][2]); a[k][3] = fmaf(q[i + 8 * k + 3], k0.w, a[k][3]);
                a[k][4] = fmaf(q[i + 8 * k + 4], k1.x, a[k][4]); a[k][5] = fmaf(q[i + 8 * k + 5], k1.y, a[k][5]);
                a[k][6] = fmaf(q[i + 8 * k + 6], k1.z, a[k][6]); a[k][7] = fmaf(q[i + 8 * k + 7], k1.w, a[k][7]);
            }
        }
        for (; i + 8 <= p.ihd; i += 8)
#pragma unroll
            for (int l = 0; l < 8; l++) a[0][l] = fmaf(q[i + l], kb[i + l], a[0][l]);
        float r = 0.f;
#pragma unroll
        for (int l = 0; l < 8; l++) r += (a[0][l] + a[1][l]) + (a[2][l] + a[3][l]);
        for (; i < p.ihd; i++) r += q[i] * kb[i];
        s += r > 0.f ? r : 0.f;
    }
    p.scores[(size_t)b * p.nb_cap + blk] = s * iscale;
}

// grid (batch), 1024 threads
__global__ void __launch_bounds__(1024) pb_qsa_pick_kernel(const PbQsaParams p) {
    const int b = blockIdx.x, tid = threadIdx.x;
    __shared__ unsigned int hist[256];
    __shared__ unsigned long long prefix_s;
    __shared__ int want_s;
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
        if (tid == 0) {
            int want = want_s, byte = 255;
            for (; byte > 0; byte--) { if ((int)hist[byte] >= want) break; want -= (int)hist[byte]; }
            prefix_s = prefix | ((unsigned long long)byte << shift);
            want_s = want;
        }
        __syncthreads();
    }
    const unsigned long long thr = prefix_s;            // the kk-th largest key: exactly kk keys are >= thr
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
    if (p.ihd > QSA_MAX_HD || p.ihd % 8 || p.n_rot > p.ihd) PB_FAIL(ctx, PB_UNSUPPORTED, "indexer head dim %d (a multiple of 8, at least the rope width %d, at most %d)", p.ihd, p.n_rot, QSA_MAX_HD);
    pb_launch_k(ctx, pb_qsa_append_kernel, dim3(p.batch), dim3(32), (size_t)0, p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

int pb_launch_qsa_select(pb_ctx* ctx, const PbQsaParams& p) {
    const size_t smem = (size_t)p.inh * p.ihd * 4;
    if (smem > 48 * 1024) PB_FAIL(ctx, PB_UNSUPPORTED, "indexer with %d heads of %d", p.inh, p.ihd);
    pb_launch_k(ctx, pb_qsa_score_kernel, dim3((unsigned)((p.nb_cap + 127) / 128), p.batch), dim3(128), smem, p);
    pb_launch_k(ctx, pb_qsa_pick_kernel, dim3(p.batch), dim3(1024), (size_t)0, p);
    ctx->kernels_launched += 2;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

int pb_launch_qsa_pool_all(pb_ctx* ctx, const PbQsaParams& p, int64_t nblk) {
    if (nblk <= 0) return PB_OK;
    const unsigned gx = (unsigned)(nblk < 1024 ? nblk : 1024);
    pb_qsa_pool_kernel<<<dim3(gx, p.batch), 32, 0, ctx->stream>>>(p, nblk);
    ctx->kernels_launched++;
    ctx->pdl_chain = false;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
