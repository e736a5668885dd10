// Gated-attention decode with a 4-bit KV cache dequantized in the kernel.
//
// Restates attn_core (dense branch) and the KV layout rule of kv_push of the reference
// (src/model/qwen4exp_gguf.rs:1558-1615, 1517-1534), rope (:1436-1439, :529-533) and kv4
// pack/get (src/model/kv4.rs:12-42); replaces k_attn_prep / k_attn3 / k_attn3sc8 / k_attn3r8
// (src/model/qn_cube.rs:5419-5655, 7394-7500).
//
// Cache layout per attention layer (head-major, so the positions of one KV head are one
// contiguous stream): packed words kw[b][kvh][pos][hd/8] (8 nibbles per u32, low nibble =
// element 0) with one f32 scale per 32 values ks[b][kvh][pos][hd/32]; positions older than
// the packed boundary q4n live there, the newest ones in an f32 ring kr[b][kvh][slot][hd],
// slot = pos mod ring capacity.  q4n = ((len - recent) / 64) * 64, the reference's rule.
//
//   pb_kv_append_kernel    RMSNorm(k) * kn, partial RoPE, append K and V at the position,
//                          move the packed boundary (packs whole multiples of 64 positions)
//   pb_attn_partial_kernel split-KV flash-decode: grid (split, KV head, sequence); the 8 query
//                          heads of a GQA group share every K/V byte that is read
//   pb_attn_combine_kernel merges the splits, normalizes, applies the sigmoid output gate
#include "pb_common.cuh"
#include "pb_internal.h"

#include <stdio.h>

#define AT_THREADS 256
#define AT_WARPS 8
#define AT_MAXG 8       // query heads per KV head handled by one CTA
#define AT_TILE 32      // positions per warp tile

// Sum N per-lane values over the warp so that the totals end up spread over the lanes:
// N >= 32: lane l holds totals of indices l*N/32 .. in v[0 .. N/32); N < 32: index lane >> log2(32/N) in v[0].
template <int N>
__device__ __forceinline__ void pb_transpose_reduce(float (&v)[N], int lane) {
    int n = N / 2;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        if (n >= 1) {
            const bool up = lane & off;
#pragma unroll
            for (int i = 0; i < N / 2; i++) {
                if (i < n) {
                    const float send = up ? v[i] : v[i + n];
                    const float keep = up ? v[i + n] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            n >>= 1;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
        }
    }
}

__device__ __forceinline__ float pb_kv4_dequant(uint32_t w, int j, float s) {
    const int q = ((int)(w << (28 - 4 * j))) >> 28;   // sign-extended nibble j
    return (float)q * s;
}

// one warp packs one 32-value block: lane = element.  kv4::pack, src/model/kv4.rs:12-32
__device__ __forceinline__ void pb_kv4_pack_block(float v, int lane, uint32_t* words4, float* scale) {
    const float m = pb_warp_max(fabsf(v));
    const float s = (m > 0.f && isfinite(m)) ? m / 7.0f : 0.f;
    int q = 0;
    if (s > 0.f) { float r = roundf(v / s); r = fminf(fmaxf(r, -7.f), 7.f); q = (int)r; }
    uint32_t u = ((uint32_t)q & 0xF) << (4 * (lane & 7));
    u |= __shfl_xor_sync(0xffffffffu, u, 1); u |= __shfl_xor_sync(0xffffffffu, u, 2); u |= __shfl_xor_sync(0xffffffffu, u, 4);
    if ((lane & 7) == 0) words4[lane >> 3] = u;
    if (lane == 0) *scale = s;
}

// generic packer: x [n] f32 -> words [n/8], scales [n/32]; one warp per block
__global__ void __launch_bounds__(256) pb_kv4_pack_kernel(const float* __restrict__ x, int64_t nblocks, uint32_t* __restrict__ w, float* __restrict__ sc) {
    const int64_t blk = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (blk >= nblocks) return;
    pb_kv4_pack_block(x[blk * 32 + (threadIdx.x & 31)], threadIdx.x & 31, w + blk * 4, sc + blk);
}
__global__ void __launch_bounds__(256) pb_kv4_unpack_kernel(const uint32_t* __restrict__ w, const float* __restrict__ sc, int64_t n, float* __restrict__ x) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = pb_kv4_dequant(w[i / 8], (int)(i % 8), sc[i / 32]);
}

// ------------------------------------------------------------------------------------ append

// grid (batch), 256 threads
__global__ void __launch_bounds__(AT_THREADS) pb_kv_append_kernel(const PbAttnParams p) {
    const int b = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = p.hd, nkv = p.n_kv, half = p.n_rot / 2;
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t pos = p.pos[b];
    const float* proj = p.proj + (size_t)b * p.ldp;
    const float* kraw = proj + (size_t)p.n_head * 2 * hd;
    const float* vraw = kraw + (size_t)nkv * hd;
    const int64_t slot = pos % p.ring_cap;
    __shared__ float sc[8];
    for (int h = warp; h < nkv; h += AT_WARPS) {
        float ss = 0.f;
        for (int i = lane; i < hd; i += 32) { const float v = kraw[h * hd + i]; ss += v * v; }
        ss = pb_warp_sum(ss);
        if (lane == 0) sc[h & 7] = 1.0f / sqrtf(ss / (float)hd + p.eps);
        __syncwarp();
        const float s = sc[h & 7];
        float* kd = p.kr + (((size_t)b * nkv + h) * p.ring_cap + slot) * hd;
        float* vd = p.vr + (((size_t)b * nkv + h) * p.ring_cap + slot) * hd;
        for (int i = lane; i < hd; i += 32) {
            // rms_inplace: x *= s * w  (:210); rope rotates dims i and i + n_rot/2 for i < n_rot/2 (:1436-1439)
            float x = kraw[h * hd + i] * (s * p.kn[i]);
            if (i < p.n_rot) {
                const int j = i < half ? i : i - half;
                const float other = kraw[h * hd + (i < half ? i + half : i - half)] * (s * p.kn[i < half ? i + half : i - half]);
                float sn, co;
                sincosf((float)pos * p.rope_inv[j], &sn, &co);
                x = i < half ? x * co - other * sn : x * co + other * sn;
            }
            kd[i] = x;
            vd[i] = vraw[h * hd + i];
        }
    }
    if (p.kv_bits != 4) return;
    __syncthreads();
    // packed boundary for len = pos + 1 rows (kv_push :1520): whole multiples of 64 positions
    const int64_t len = pos + 1, have = p.q4n[b];
    const int64_t want = len > p.kv_recent ? ((len - p.kv_recent) / 64) * 64 : 0;
    if (want <= have) return;
    const int bpp = hd / 32;                                  // blocks per position per head
    const int64_t nblk = (want - have) * nkv * bpp;
    for (int64_t i = warp; i < nblk; i += AT_WARPS) {
        const int blk = (int)(i % bpp); const int h = (int)((i / bpp) % nkv); const int64_t pp = have + i / ((int64_t)bpp * nkv);
        const size_t src = (((size_t)b * nkv + h) * p.ring_cap + (pp % p.ring_cap)) * hd + blk * 32 + lane;
        const size_t row = ((size_t)b * nkv + h) * p.max_ctx + pp;
        pb_kv4_pack_block(p.kr[src], lane, p.kw + row * (hd / 8) + blk * 4, p.ks + row * bpp + blk);
        pb_kv4_pack_block(p.vr[src], lane, p.vw + row * (hd / 8) + blk * 4, p.vs + row * bpp + blk);
    }
    __syncthreads();
    if (tid == 0) p.q4n[b] = want;
}

// ------------------------------------------------------------------------------------ partial

// grid (nsplit, n_kv, batch), 256 threads.  Lane l of a warp owns dims 8l..8l+7 of the head
// (one packed word, or two float4 of an f32 row); a warp walks tiles of 32 positions.
template <int G>
__global__ void __launch_bounds__(AT_THREADS, 1) pb_attn_partial_kernel(const PbAttnParams p) {
    const int sp = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = p.hd, half = p.n_rot / 2;
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t pos = p.pos[b], n = pos + 1, q4n = p.kv_bits == 4 ? p.q4n[b] : 0;
    const float* proj = p.proj + (size_t)b * p.ldp;

    extern __shared__ float asm_[];
    float* qs = asm_;                         // [G][hd] normalized, roped, scaled queries
    float* prob = asm_ + G * hd;              // [AT_WARPS][AT_TILE][G] tile probabilities
    float* mrg = prob + AT_WARPS * AT_TILE * G;   // [AT_WARPS][G][2 + hd] merge buffer

    // queries of this GQA group: rms_inplace(q, qn), rope, times 1/sqrt(hd)  (:1603-1606)
    for (int g = warp; g < G; g += AT_WARPS) {
        const int h = kvh * G + g;
        const float* qraw = proj + (size_t)h * 2 * hd;
        float ss = 0.f;
        for (int i = lane; i < hd; i += 32) ss += qraw[i] * qraw[i];
        ss = pb_warp_sum(ss);
        const float s = 1.0f / sqrtf(ss / (float)hd + p.eps);
        const float scale = 1.0f / sqrtf((float)hd);
        for (int i = lane; i < hd; i += 32) {
            float x = qraw[i] * (s * p.qn[i]);
            if (i < p.n_rot) {
                const int j = i < half ? i : i - half;
                const int oi = i < half ? i + half : i - half;
                const float other = qraw[oi] * (s * p.qn[oi]);
                float sn, co;
                sincosf((float)pos * p.rope_inv[j], &sn, &co);
                x = i < half ? x * co - other * sn : x * co + other * sn;
            }
            qs[g * hd + i] = x * scale;
        }
    }
    __syncthreads();

    // this lane's 8 query dims for every head of the group (hd = 256 -> one 8-dim slice per lane)
    float q[G][8];
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int j = 0; j < 8; j++) q[g][j] = qs[g * hd + 8 * lane + j];

    float m_run[G], l_run[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; g++) { m_run[g] = -INFINITY; l_run[g] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) acc[g][j] = 0.f; }

    const int64_t ntiles = (n + AT_TILE - 1) / AT_TILE;
    // tiles are dealt round-robin to (split, warp) so that the slower f32 tiles of the recent window
    // are spread over all CTAs instead of landing on the last splits
    const size_t hrow = (size_t)b * p.n_kv + kvh;
    const uint32_t* kw = p.kw + hrow * p.max_ctx * (hd / 8);
    const uint32_t* vw = p.vw + hrow * p.max_ctx * (hd / 8);
    const float* ks = p.ks + hrow * p.max_ctx * (hd / 32);
    const float* vs = p.vs + hrow * p.max_ctx * (hd / 32);
    const float* kr = p.kr + hrow * p.ring_cap * hd;
    const float* vr = p.vr + hrow * p.ring_cap * hd;
    float* pw = prob + warp * AT_TILE * G;
    // per-warp staging of one packed tile: K/V words [32 pos][hd/8] and scales [32 pos][hd/32]
    uint32_t* tkw = reinterpret_cast<uint32_t*>(mrg + (size_t)AT_WARPS * G * (2 + hd)) + (size_t)warp * 2 * (AT_TILE * (hd / 8) + AT_TILE * (hd / 32));
    float* tks = reinterpret_cast<float*>(tkw + AT_TILE * (hd / 8));
    uint32_t* tvw = reinterpret_cast<uint32_t*>(tks + AT_TILE * (hd / 32));
    float* tvs = reinterpret_cast<float*>(tvw + AT_TILE * (hd / 8));

    for (int64_t t = (int64_t)warp * gridDim.x + sp; t < ntiles; t += (int64_t)AT_WARPS * gridDim.x) {
        const int64_t pbase = t * AT_TILE;
        // q4n is a multiple of 64 and tiles start at multiples of 32: a tile is entirely packed or entirely f32
        const bool packed = pbase < q4n;
        if (packed) {
            // coalesced 16-byte loads of the whole tile (contiguous in the head-major layout), all issued up front
            const uint4* gk = reinterpret_cast<const uint4*>(kw + pbase * (hd / 8));
            const uint4* gv = reinterpret_cast<const uint4*>(vw + pbase * (hd / 8));
            const uint4* gks = reinterpret_cast<const uint4*>(ks + pbase * (hd / 32));
            const uint4* gvs = reinterpret_cast<const uint4*>(vs + pbase * (hd / 32));
            uint4 a[8], c[8];
#pragma unroll
            for (int i = 0; i < 8; i++) { a[i] = gk[i * 32 + lane]; c[i] = gv[i * 32 + lane]; }
            const uint4 sa0 = gks[lane], sa1 = gks[32 + lane], sc0 = gvs[lane], sc1 = gvs[32 + lane];
#pragma unroll
            for (int i = 0; i < 8; i++) { reinterpret_cast<uint4*>(tkw)[i * 32 + lane] = a[i]; reinterpret_cast<uint4*>(tvw)[i * 32 + lane] = c[i]; }
            reinterpret_cast<uint4*>(tks)[lane] = sa0; reinterpret_cast<uint4*>(tks)[32 + lane] = sa1;
            reinterpret_cast<uint4*>(tvs)[lane] = sc0; reinterpret_cast<uint4*>(tvs)[32 + lane] = sc1;
            __syncwarp();
        }
        // ---- scores of the 32 positions of the tile, 8 positions at a time: every lane holds the
        //      partial dots of its 8 dims for (8 positions x G heads); a transposed butterfly sums
        //      them over the warp, leaving the totals spread over the lanes, which go through
        //      shared memory to the "lane = position" layout of the softmax
        float sc[G];
#pragma unroll
        for (int g = 0; g < G; g++) sc[g] = -INFINITY;
        for (int i0 = 0; i0 < AT_TILE; i0 += 8) {
            if (pbase + i0 >= n) break;
            float part[8 * G];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int64_t pp = pbase + i0 + i;
                float kv[8];
                if (packed) {
                    const uint32_t w = tkw[(i0 + i) * (hd / 8) + lane];
                    const float s = tks[(i0 + i) * (hd / 32) + (lane >> 2)];
#pragma unroll
                    for (int j = 0; j < 8; j++) kv[j] = pb_kv4_dequant(w, j, s);
                } else if (pp < n) {
                    const float4* src = reinterpret_cast<const float4*>(kr + (size_t)(pp % p.ring_cap) * hd + 8 * lane);
                    const float4 a = src[0], c = src[1];
                    kv[0] = a.x; kv[1] = a.y; kv[2] = a.z; kv[3] = a.w; kv[4] = c.x; kv[5] = c.y; kv[6] = c.z; kv[7] = c.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++) kv[j] = 0.f;
                }
#pragma unroll
                for (int g = 0; g < G; g++) {
                    float d = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; j++) d = fmaf(q[g][j], kv[j], d);
                    part[i * G + g] = d;
                }
            }
            pb_transpose_reduce<8 * G>(part, lane);
            constexpr int PER = (8 * G) / 32 > 0 ? (8 * G) / 32 : 1;
            if (8 * G >= 32) {
#pragma unroll
                for (int e = 0; e < PER; e++) { const int idx = lane * PER + e; pw[(i0 + idx / G) * G + idx % G] = part[e]; }
            } else {
                constexpr int SH = G == 2 ? 1 : 2;      // 16 or 8 values: lanes with equal (lane >> SH) hold duplicates
                const int idx = lane >> SH;
                if ((lane & ((1 << SH) - 1)) == 0) pw[(i0 + idx / G) * G + idx % G] = part[0];
            }
        }
        __syncwarp();
#pragma unroll
        for (int g = 0; g < G; g++) if (pbase + lane < n) sc[g] = pw[lane * G + g];
        __syncwarp();
        // ---- online softmax over the tile (lane = position)
        float corr[G];
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float mt = pb_warp_max(sc[g]);
            const float mn = fmaxf(m_run[g], mt);
            corr[g] = m_run[g] == -INFINITY ? 0.f : expf(m_run[g] - mn);
            const float pr = sc[g] == -INFINITY ? 0.f : expf(sc[g] - mn);
            l_run[g] = l_run[g] * corr[g] + pb_warp_sum(pr);
            m_run[g] = mn;
            pw[lane * G + g] = pr;
#pragma unroll
            for (int j = 0; j < 8; j++) acc[g][j] *= corr[g];
        }
        __syncwarp();
        // ---- P.V for the tile
#pragma unroll 4
        for (int i = 0; i < AT_TILE; i++) {
            const int64_t pp = pbase + i;
            if (pp >= n) break;
            float vv[8];
            if (packed) {
                const uint32_t w = tvw[i * (hd / 8) + lane];
                const float s = tvs[i * (hd / 32) + (lane >> 2)];
#pragma unroll
                for (int j = 0; j < 8; j++) vv[j] = pb_kv4_dequant(w, j, s);
            } else {
                const float4* src = reinterpret_cast<const float4*>(vr + (size_t)(pp % p.ring_cap) * hd + 8 * lane);
                const float4 a = src[0], c = src[1];
                vv[0] = a.x; vv[1] = a.y; vv[2] = a.z; vv[3] = a.w; vv[4] = c.x; vv[5] = c.y; vv[6] = c.z; vv[7] = c.w;
            }
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float pr = pw[i * G + g];
#pragma unroll
                for (int j = 0; j < 8; j++) acc[g][j] = fmaf(pr, vv[j], acc[g][j]);
            }
        }
        __syncwarp();
    }

    // ---- merge the 8 warps of the CTA, then write the split's partial
    float* mw = mrg + (size_t)warp * G * (2 + hd);
#pragma unroll
    for (int g = 0; g < G; g++) {
        if (lane == 0) { mw[g * (2 + hd)] = m_run[g]; mw[g * (2 + hd) + 1] = l_run[g]; }
#pragma unroll
        for (int j = 0; j < 8; j++) mw[g * (2 + hd) + 2 + 8 * lane + j] = acc[g][j];
    }
    __syncthreads();
    for (int g = warp; g < G; g += AT_WARPS) {
        float M = -INFINITY;
        for (int w = 0; w < AT_WARPS; w++) M = fmaxf(M, mrg[((size_t)w * G + g) * (2 + hd)]);
        float L = 0.f, o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int w = 0; w < AT_WARPS; w++) {
            const float* src = mrg + ((size_t)w * G + g) * (2 + hd);
            const float f = src[0] == -INFINITY ? 0.f : expf(src[0] - M);
            L += src[1] * f;
#pragma unroll
            for (int j = 0; j < 8; j++) o[j] = fmaf(src[2 + 8 * lane + j], f, o[j]);
        }
        const size_t pi = (((size_t)b * p.n_kv + kvh) * gridDim.x + sp) * G + g;
        if (lane == 0) { p.part_ml[pi * 2] = M; p.part_ml[pi * 2 + 1] = L; }
#pragma unroll
        for (int j = 0; j < 8; j++) p.part_acc[pi * hd + 8 * lane + j] = o[j];
    }
}

// ------------------------------------------------------------------------------------ combine

// grid (n_head, batch), 4 * hd threads: merge splits, normalize, gate with sigmoid(gate)  (:1607-1610).
// Thread (q, d) sums the splits s = q, q+4, ... of dimension d; the four partial sums meet in shared memory.
__global__ void __launch_bounds__(1024) pb_attn_combine_kernel(const PbAttnParams p) {
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x % p.hd, q = threadIdx.x / p.hd;
    const int G = p.n_head / p.n_kv, kvh = h / G, g = h % G;
    pb_pdl_wait();
    pb_pdl_trigger();
    __shared__ float fs[128];     // per-split factor exp(m_s - M)
    __shared__ float ML[2];
    __shared__ float part[3][256];
    const size_t base = ((size_t)b * p.n_kv + kvh) * p.nsplit;
    if (threadIdx.x < 32) {
        const int l = threadIdx.x;
        float M = -INFINITY;
        for (int s = l; s < p.nsplit; s += 32) M = fmaxf(M, p.part_ml[((base + s) * G + g) * 2]);
        M = pb_warp_max(M);
        float L = 0.f;
        for (int s = l; s < p.nsplit; s += 32) {
            const float m = p.part_ml[((base + s) * G + g) * 2];
            const float f = m == -INFINITY ? 0.f : expf(m - M);
            fs[s] = f;
            L += p.part_ml[((base + s) * G + g) * 2 + 1] * f;
        }
        L = pb_warp_sum(L);
        if (l == 0) { ML[0] = M; ML[1] = L; }
    }
    __syncthreads();
    float o = 0.f;
#pragma unroll 4
    for (int s = q; s < p.nsplit; s += 4) o = fmaf(p.part_acc[((base + s) * G + g) * p.hd + d], fs[s], o);
    if (q > 0) part[q - 1][d] = o;
    __syncthreads();
    if (q == 0) {
        o = ((o + part[0][d]) + part[1][d]) + part[2][d];
        const float gate = p.proj[(size_t)b * p.ldp + (size_t)h * 2 * p.hd + p.hd + d];
        p.att[(size_t)b * p.lda + (size_t)h * p.hd + d] = (o * (1.0f / ML[1])) * pb_sigm(gate);
    }
}

// ------------------------------------------------------------------------------------ launchers

int pb_launch_kv_append(pb_ctx* ctx, const PbAttnParams& p) {
    if (p.hd % 32 || p.n_rot > p.hd || p.n_rot % 2 || p.n_kv > 8) PB_FAIL(ctx, PB_UNSUPPORTED, "attention: head dim %d / rotary dim %d not supported", p.hd, p.n_rot);
    pb_launch_k(ctx, pb_kv_append_kernel, dim3(p.batch), dim3(AT_THREADS), (size_t)(0), p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

int pb_launch_attn(pb_ctx* ctx, const PbAttnParams& p) {
    const int G = p.n_head / p.n_kv;
    if (p.hd != 256 || p.nsplit > 128 || p.n_head % p.n_kv || (G != 8 && G != 4 && G != 2 && G != 1))
        PB_FAIL(ctx, PB_UNSUPPORTED, "attention: head dim %d with %d query heads per KV head not supported", p.hd, G);
    const dim3 grid(p.nsplit, p.n_kv, p.batch);
    const size_t smem = ((size_t)G * p.hd + (size_t)AT_WARPS * AT_TILE * G + (size_t)AT_WARPS * G * (2 + p.hd) + (size_t)AT_WARPS * 2 * (AT_TILE * (p.hd / 8) + AT_TILE * (p.hd / 32))) * 4;
    if (smem > (size_t)ctx->max_smem_optin) PB_FAIL(ctx, PB_UNSUPPORTED, "attention needs %zu bytes of shared memory", smem);
#define GO(GG)                                                                                                                   \
    {                                                                                                                            \
        static bool cfgd = false;                                                                                                \
        if (!cfgd) { PB_CUDA(ctx, cudaFuncSetAttribute(pb_attn_partial_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, ctx->max_smem_optin)); cfgd = true; } \
        pb_launch_k(ctx, pb_attn_partial_kernel<GG>, dim3(grid), dim3(AT_THREADS), (size_t)(smem), p);                                                  \
    }
    if (G == 8) GO(8) else if (G == 4) GO(4) else if (G == 2) GO(2) else GO(1)
#undef GO
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    pb_launch_k(ctx, pb_attn_combine_kernel, dim3(p.n_head, p.batch), dim3(4 * p.hd), (size_t)(0), p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

int pb_launch_kv4_pack(pb_ctx* ctx, const float* x, int64_t n, uint32_t* w, float* sc) {
    const int64_t nblocks = n / 32;
    if (nblocks <= 0) return PB_OK;
    pb_launch_k(ctx, pb_kv4_pack_kernel, dim3((unsigned)((nblocks + 7) / 8)), dim3(256), (size_t)(0), x, nblocks, w, sc);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
int pb_launch_kv4_unpack(pb_ctx* ctx, const uint32_t* w, const float* sc, int64_t n, float* x) {
    if (n <= 0) return PB_OK;
    pb_launch_k(ctx, pb_kv4_unpack_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)(0), w, sc, n, x);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
