// Gated-attention decode with a 4-bit KV cache dequantized in the kernel.
//
// Restates attn_core (dense branch) and the KV layout rule of kv_push of the reference
// (src/model/qwen4exp_gguf.rs:1558-1615, 1517-1534), rope (:1436-1439, :529-533) and kv4
// pack/get (src/model/kv4.rs:12-42); replaces k_attn_prep / k_attn3 / k_attn3sc8 / k_attn3r8
// (src/model/qn_cube.rs:5419-5655, 7394-7500).
//
// Cache layout per attention layer (head-major, so the positions of one KV head are one
// contiguous stream): packed K words kw[b][kvh][pos][hd/8] (8 nibbles per u32, low nibble =
// element 0) with one f32 scale per 32 values ks[b][kvh][pos][hd/32]; packed V words are
// stored position-transposed, vw[b][kvh][pos/8][hd] with position pos%8 of one dimension in
// nibble pos%8 (same bytes per position, same quantization and scales vs[b][kvh][pos][hd/32]),
// which is the operand order of the P.V tensor-core product.  Positions older than the packed
// boundary q4n live there, the newest ones in an f32 ring kr[b][kvh][slot][hd], slot = pos mod
// ring capacity.  q4n = ((len - recent) / 64) * 64, the reference's rule.
//
//   pb_kv_append_kernel    RMSNorm(k) * kn, partial RoPE, append K and V at the position,
//                          move the packed boundary (packs whole multiples of 64 positions)
//   pb_attn_partial_kernel split-KV flash-decode: grid (split, KV head, sequence); the 8 query
//                          heads of a GQA group share every K/V byte that is read.  Splits below
//                          nsplit_packed walk the packed positions on the tensor cores
//                          (mma.sync m16n8k16 f16, f32 accumulate: nibbles are exact in f16,
//                          queries and probabilities go in as f16 high + low parts, block scales
//                          are applied in f32); the remaining splits walk the f32 ring with
//                          scalar FMAs
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

// nibble j of a cache word (offset binary)
__device__ __forceinline__ float pb_kv4_dequant8(uint32_t w, int j, float s) { return (float)((int)((w >> (4 * j)) & 0xF) - 8) * s; }

// one warp packs one 32-value block: lane = element.  kv4::pack, src/model/kv4.rs:12-32
// bias = 0: two's-complement nibbles (kv4.rs); bias = 8: offset-binary nibbles q + 8, the form the cache keeps
__device__ __forceinline__ void pb_kv4_pack_block(float v, int lane, uint32_t* words4, float* scale, int bias) {
    const float m = pb_warp_max(fabsf(v));
    const float s = (m > 0.f && isfinite(m)) ? m / 7.0f : 0.f;
    int q = 0;
    if (s > 0.f) { float r = roundf(v / s); r = fminf(fmaxf(r, -7.f), 7.f); q = (int)r; }
    uint32_t u = ((uint32_t)(q + bias) & 0xF) << (4 * (lane & 7));
    u |= __shfl_xor_sync(0xffffffffu, u, 1); u |= __shfl_xor_sync(0xffffffffu, u, 2); u |= __shfl_xor_sync(0xffffffffu, u, 4);
    if ((lane & 7) == 0) words4[lane >> 3] = u;
    if (lane == 0) *scale = s;
}

// one warp packs 32 dims of 8 consecutive positions into position-transposed words: lane = dim,
// v[i] = value of position i; same quantization as pb_kv4_pack_block, one scale per position
__device__ __forceinline__ uint32_t pb_kv4_pack_vt8(const float (&v)[8], int lane, float* scales, int scale_stride, int bias) {
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float m = pb_warp_max(fabsf(v[i]));
        const float s = (m > 0.f && isfinite(m)) ? m / 7.0f : 0.f;
        int q = 0;
        if (s > 0.f) { float r = roundf(v[i] / s); r = fminf(fmaxf(r, -7.f), 7.f); q = (int)r; }
        word |= ((uint32_t)(q + bias) & 0xF) << (4 * i);
        if (lane == 0) scales[(size_t)i * scale_stride] = s;
    }
    return word;
}
// x [npos][hd] f32 (npos a multiple of 8) -> w [npos/8][hd] words, sc [npos][hd/32]; one warp per (8 positions, 32 dims)
__global__ void __launch_bounds__(256) pb_kv4_pack_vt_kernel(const float* __restrict__ x, int64_t npos, int hd, uint32_t* __restrict__ w, float* __restrict__ sc, int bias) {
    const int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31, bpp = hd / 32;
    if (unit >= (npos / 8) * bpp) return;
    const int64_t pg = unit / bpp; const int blk = (int)(unit % bpp);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = x[(pg * 8 + i) * hd + blk * 32 + lane];
    w[pg * hd + blk * 32 + lane] = pb_kv4_pack_vt8(v, lane, sc + pg * 8 * bpp + blk, bpp, bias);
}

// generic packer: x [n] f32 -> words [n/8], scales [n/32]; one warp per block
__global__ void __launch_bounds__(256) pb_kv4_pack_kernel(const float* __restrict__ x, int64_t nblocks, uint32_t* __restrict__ w, float* __restrict__ sc, int bias) {
    const int64_t blk = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (blk >= nblocks) return;
    pb_kv4_pack_block(x[blk * 32 + (threadIdx.x & 31)], threadIdx.x & 31, w + blk * 4, sc + blk, bias);
}
__global__ void __launch_bounds__(256) pb_kv4_unpack_kernel(const uint32_t* __restrict__ w, const float* __restrict__ sc, int64_t n, float* __restrict__ x) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = pb_kv4_dequant(w[i / 8], (int)(i % 8), sc[i / 32]);
}

// Moves the packed boundary of sequence b to where `len` rows put it (kv_push :1520: whole multiples of 64 positions):
// the rows in between are read from the f32 ring and stored in 4-bit form.  All AT_THREADS threads of one CTA.
__device__ __forceinline__ void pb_kv_pack_upto(const PbAttnParams& p, int b, int64_t len, int tid, int warp, int lane) {
    const int hd = p.hd, nkv = p.n_kv;
    const int64_t have = p.q4n[b];
    const int64_t want = len > p.kv_recent ? ((len - p.kv_recent) / 64) * 64 : 0;
    if (want <= have) return;
    const int bpp = hd / 32;                                  // blocks per position per head
    const int64_t nblk = (want - have) * nkv * bpp;
    for (int64_t i = warp; i < nblk; i += AT_WARPS) {
        const int blk = (int)(i % bpp); const int h = (int)((i / bpp) % nkv); const int64_t pp = have + i / ((int64_t)bpp * nkv);
        const size_t src = (((size_t)b * nkv + h) * p.ring_cap + (pp % p.ring_cap)) * hd + blk * 32 + lane;
        const size_t row = ((size_t)b * nkv + h) * p.max_ctx + pp;
        pb_kv4_pack_block(p.kr[src], lane, p.kw + row * (hd / 8) + blk * 4, p.ks + row * bpp + blk, 8);
    }
    // V: groups of 8 positions (have and want are multiples of 64)
    const int64_t nvt = (want - have) / 8 * nkv * bpp;
    for (int64_t i = warp; i < nvt; i += AT_WARPS) {
        const int blk = (int)(i % bpp); const int h = (int)((i / bpp) % nkv); const int64_t pg = have / 8 + i / ((int64_t)bpp * nkv);
        const size_t head = (size_t)b * nkv + h;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = p.vr[(head * p.ring_cap + ((pg * 8 + j) % p.ring_cap)) * hd + blk * 32 + lane];
        p.vw[head * p.max_ctx * (hd / 8) + (size_t)pg * hd + blk * 32 + lane] = pb_kv4_pack_vt8(v, lane, p.vs + (head * p.max_ctx + pg * 8) * bpp + blk, bpp, 8);
    }
    __syncthreads();
    if (tid == 0) p.q4n[b] = want;
}

// ------------------------------------------------------------------------------------ append

// grid (batch), 256 threads
__global__ void __launch_bounds__(AT_THREADS) pb_kv_append_kernel(const PbAttnParams p) {
    const int b = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = p.hd, nkv = p.n_kv, half = p.n_rot / 2;
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t pos = p.pos[b];
    const int cb = p.window ? 0 : b;                          // cache of the sequence this token belongs to
    const float* proj = p.proj + (size_t)b * p.ldp;
    const float* kraw = proj + (size_t)p.n_head * 2 * hd;
    const float* vraw = kraw + (size_t)nkv * hd;
    const int64_t slot = pos % p.ring_cap;
    __shared__ float sc[8];
    if (hd == 256 && p.n_rot == 64) {
        // the model's head shape: a lane owns dims lane + 32 k of the head.  All of its loads are issued before anything is
        // computed (the loop below pays a trip to L2 per iteration), the rope partner of dim i < 32 is the same lane's
        // dim i + 32, and both use the same angle: one sincosf per lane.  Same arithmetic as the general loop.
        for (int h = warp; h < nkv; h += AT_WARPS) {
            float kv[8], wn[8], vv[8];
#pragma unroll
            for (int k = 0; k < 8; k++) { kv[k] = kraw[h * hd + lane + 32 * k]; wn[k] = p.kn[lane + 32 * k]; vv[k] = vraw[h * hd + lane + 32 * k]; }
            const float ang = (float)pos * p.rope_inv[lane], ms = p.rope_inv[half];
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < 8; k++) ss += kv[k] * kv[k];
            ss = pb_warp_sum(ss);
            const float s = 1.0f / sqrtf(ss / (float)hd + p.eps);
            float sn, co;
            sincosf(ang, &sn, &co);
            if (ms != 1.0f) { co *= ms; sn *= ms; }
            float* kd = p.kr + (((size_t)cb * nkv + h) * p.ring_cap + slot) * hd;
            float* vd = p.vr + (((size_t)cb * nkv + h) * p.ring_cap + slot) * hd;
            const float x0 = kv[0] * (s * wn[0]), x1 = kv[1] * (s * wn[1]);
            kd[lane] = x0 * co - x1 * sn;
            kd[lane + 32] = x1 * co + x0 * sn;
#pragma unroll
            for (int k = 2; k < 8; k++) kd[lane + 32 * k] = kv[k] * (s * wn[k]);
#pragma unroll
            for (int k = 0; k < 8; k++) vd[lane + 32 * k] = vv[k];
        }
    } else
    for (int h = warp; h < nkv; h += AT_WARPS) {
        float ss = 0.f;
        for (int i = lane; i < hd; i += 32) { const float v = kraw[h * hd + i]; ss += v * v; }
        ss = pb_warp_sum(ss);
        if (lane == 0) sc[h & 7] = 1.0f / sqrtf(ss / (float)hd + p.eps);
        __syncwarp();
        const float s = sc[h & 7];
        float* kd = p.kr + (((size_t)cb * nkv + h) * p.ring_cap + slot) * hd;
        float* vd = p.vr + (((size_t)cb * nkv + h) * p.ring_cap + slot) * hd;
        for (int i = lane; i < hd; i += 32) {
            // rms_inplace: x *= s * w  (:210); rope rotates dims i and i + n_rot/2 for i < n_rot/2 (:1436-1439)
            float x = kraw[h * hd + i] * (s * p.kn[i]);
            if (i < p.n_rot) {
                const int j = i < half ? i : i - half;
                const float other = kraw[h * hd + (i < half ? i + half : i - half)] * (s * p.kn[i < half ? i + half : i - half]);
                float sn, co;
                sincosf((float)pos * p.rope_inv[j], &sn, &co);
                const float ms = p.rope_inv[half];     // YaRN mscale behind the table, applied only when it is not 1 (:528-533)
                if (ms != 1.0f) { co *= ms; sn *= ms; }
                x = i < half ? x * co - other * sn : x * co + other * sn;
            }
            kd[i] = x;
            vd[i] = vraw[h * hd + i];
        }
    }
    if (p.kv_bits != 4 || p.window) return;
    __syncthreads();
    pb_kv_pack_upto(p, b, pos + 1, tid, warp, lane);
}

// window mode: one CTA moves the packed boundary of sequence 0 to where the window's last token puts it, and keeps the
// boundary from before the window in q4n[1]
__global__ void __launch_bounds__(AT_THREADS) pb_kv_pack_kernel(const PbAttnParams p) {
    const int tid = threadIdx.x;
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t have = p.q4n[0];
    __syncthreads();
    if (tid == 0) p.q4n[1] = have;
    pb_kv_pack_upto(p, 0, p.pos[p.batch - 1] + 1, tid, tid >> 5, tid & 31);
}

// ------------------------------------------------------------------------------------ partial

#define AT_BUF_WORDS 2688     // one tile buffer: K 32 x 36 words (padded rows), V 1024, K scales 256, V scales 256
#define AT_STAGE_WORDS (2 * AT_BUF_WORDS + 256)   // per warp: two tile buffers (the next tile loads while this one is used) + 256 scores
#define AT_KSTRIDE 36

__device__ __forceinline__ void pb_mma16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// f16 pair of (a, b) and the f16 pair of what the first rounding lost
__device__ __forceinline__ void pb_split_h2(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(a, b);
    const float2 r = __half22float2(h);
    const __half2 l = __floats2half2_rn(a - r.x, b - r.y);
    hi = *reinterpret_cast<const uint32_t*>(&h); lo = *reinterpret_cast<const uint32_t*>(&l);
}
// nibbles q and q + 4 of a cache word (offset-binary nibbles) -> f16 pair of the signed values
__device__ __forceinline__ uint32_t pb_nib2_h2(uint32_t x, int sh) {
    const uint32_t t = ((x >> sh) & 0x000F000Fu) | 0x64006400u;           // 1024 + n
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&t), __float2half2_rn(1032.0f));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ void pb_cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(pb_smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void pb_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void pb_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// shared-memory loads that the compiler may not hoist over the per-tile restaging of the buffers
__device__ __forceinline__ uint32_t pb_ldsv32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ uint4 pb_ldsv128(uint32_t a) { uint4 v; asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory"); return v; }
__device__ __forceinline__ float pb_exp2i(int k) { k = k < -126 ? -126 : (k > 127 ? 127 : k); return __int_as_float((k + 127) << 23); }

// Packed positions on the tensor cores.  Thread (g, q) = (lane >> 2, lane & 3).
//   S = Q K^T: A rows 0..7 = the query heads in f16 (rows >= G are zero), rows 8..15 = what the f16
//     rounding of the same heads lost; k = the 16 dims of two packed words, in the order (q, q+4)
//     per thread and word; B = K nibbles as f16; column c of an 8-position group is position
//     (c >> 1) + 4 (c & 1), so that a thread ends up with the scores of positions q and q + 4
//     (hi part in its row g, lo part in its row g + 8, added in f32).
//   O^T = V^T P^T: A rows = 16 dims, k = the 16 positions of two groups (nibbles q, q+4 of the
//     transposed V words); B = P times the V block scale (made per 32-dim block in f32, relative
//     to a running power-of-two 2^E so that f16 neither overflows nor flushes), as f16 in one mma
//     and the rounding remainder in a second one.
template <int G>
__device__ __forceinline__ void pb_attn_mma_tiles(const float* qs, uint32_t* stage, int warp, int lane, int sp, int nsp, const uint32_t* kw,
                                                  const uint32_t* vw, const float* ks, const float* vs, int64_t ntiles, float* mw, const uint32_t* mk) {
    constexpr int HD = 256;
    const int g = lane >> 2, q = lane & 3, sh = 4 * q;
    // A fragments of the scores: rows 0..7 = the f16 of the heads' queries, rows 8..15 = what that rounding lost;
    // the 16 k of fragment i are the dims of cache words 2i and 2i + 1 (dims 8w + q and 8w + q + 4 per word w).
    // Kept as register quads {hi w, lo w, hi w+1, lo w+1}: exactly the operand layout of the instruction.
    uint32_t qa[16][4];
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const float x0 = g < G ? qs[g * HD + 8 * i + q] : 0.f, x1 = g < G ? qs[g * HD + 8 * i + q + 4] : 0.f;
        pb_split_h2(x0, x1, qa[i >> 1][2 * (i & 1)], qa[i >> 1][2 * (i & 1) + 1]);
    }
    float m_run = -INFINITY, l_run = 0.f, acc[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    constexpr int E_NONE = -100000;
    int E = E_NONE;
    float2* sbuf = reinterpret_cast<float2*>(stage + 2 * AT_BUF_WORDS);   // [4 groups][32 lanes]: scores, then probabilities
    const int krow = (g >> 1) + 4 * (g & 1);
    // asynchronous copy of tile t into buffer `buf`: every lane moves 8 + 8 + 2 + 2 pieces of 16 bytes
    auto fetch = [&](int64_t t, int buf) {
        uint32_t* bk = stage + buf * AT_BUF_WORDS; uint32_t* bv = bk + 32 * AT_KSTRIDE; uint32_t* bs = bv + 1024;
        const int64_t pbase = t * AT_TILE;
        const uint4* gk = reinterpret_cast<const uint4*>(kw + pbase * (HD / 8));
        const uint4* gv = reinterpret_cast<const uint4*>(vw + pbase * (HD / 8));
        const uint4* gks = reinterpret_cast<const uint4*>(ks + pbase * (HD / 32));
        const uint4* gvs = reinterpret_cast<const uint4*>(vs + pbase * (HD / 32));
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int f = i * 32 + lane;
            pb_cp_async16(bk + (f >> 3) * AT_KSTRIDE + 4 * (f & 7), gk + f);
            pb_cp_async16(bv + 4 * f, gv + f);
        }
        pb_cp_async16(bs + 4 * lane, gks + lane); pb_cp_async16(bs + 128 + 4 * lane, gks + 32 + lane);
        pb_cp_async16(bs + 256 + 4 * lane, gvs + lane); pb_cp_async16(bs + 384 + 4 * lane, gvs + 32 + lane);
        pb_cp_async_commit();
    };
    // with a position mask (mk: one word per tile), tiles without a set bit are skipped before they are fetched
    const int64_t t_step = (int64_t)AT_WARPS * nsp;
    int64_t t_first = (int64_t)warp * nsp + sp;
    while (mk && t_first < ntiles && mk[t_first] == 0u) t_first += t_step;
    if (t_first < ntiles) fetch(t_first, 0);
    int buf = 0;
    for (int64_t t = t_first, t_next; t < ntiles; t = t_next, buf ^= 1) {
        {
            t_next = t + t_step;
            while (mk && t_next < ntiles && mk[t_next] == 0u) t_next += t_step;
            const uint32_t mword = mk ? mk[t] : 0xFFFFFFFFu;
            if (t_next < ntiles) { fetch(t_next, buf ^ 1); pb_cp_async_wait<1>(); } else pb_cp_async_wait<0>();
            __syncwarp();   // every lane's pieces of this tile have landed
            uint32_t* tk = stage + buf * AT_BUF_WORDS; uint32_t* tv = tk + 32 * AT_KSTRIDE;
            float* tks = reinterpret_cast<float*>(tv + 1024); float* tvs = tks + 256;
            const uint32_t tk_s = pb_smem_u32(tk), tv_s = pb_smem_u32(tv);
            // largest V scale of the tile -> running exponent
            const float4 sc0 = *reinterpret_cast<const float4*>(tvs + 4 * lane), sc1 = *reinterpret_cast<const float4*>(tvs + 128 + 4 * lane);
            float vm = fmaxf(fmaxf(fmaxf(sc0.x, sc0.y), fmaxf(sc0.z, sc0.w)), fmaxf(fmaxf(sc1.x, sc1.y), fmaxf(sc1.z, sc1.w)));
            vm = pb_warp_max(vm);
            float facc = 1.0f;
            if (vm > 0.f && vm <= 3.0e38f) {
                const int e = ilogbf(vm) + 1;
                if (e > E) { facc = E == E_NONE ? 0.f : pb_exp2i(E - e); E = e; }
            }
            const float vscl = E == E_NONE ? 0.f : pb_exp2i(-E);

            // ---- scores.  The loops over the four 8-position groups stay rolled (a fully unrolled tile is
            //      ~40 KB of straight-line code that no warp reuses: instruction fetch then bounds the
            //      kernel); their per-group values pass through this lane's slots of sbuf
#pragma unroll 1
            for (int nt = 0; nt < 4; nt++) {
                float s0 = 0.f, s1 = 0.f;
                const uint32_t ka = tk_s + (uint32_t)((8 * nt + krow) * AT_KSTRIDE) * 4;
                const float* sk = tks + (8 * nt + q) * 8;
#pragma unroll
                for (int blk = 0; blk < 8; blk++) {
                    const uint4 kk = pb_ldsv128(ka + blk * 16);
                    float c4[4] = {0.f, 0.f, 0.f, 0.f};
                    pb_mma16(c4, qa[2 * blk][0], qa[2 * blk][1], qa[2 * blk][2], qa[2 * blk][3], pb_nib2_h2(kk.x, sh), pb_nib2_h2(kk.y, sh));
                    pb_mma16(c4, qa[2 * blk + 1][0], qa[2 * blk + 1][1], qa[2 * blk + 1][2], qa[2 * blk + 1][3], pb_nib2_h2(kk.z, sh), pb_nib2_h2(kk.w, sh));
                    // rows g and g + 8 of the product: the hi and the lo part of the same score
                    s0 = fmaf(sk[blk], c4[0] + c4[2], s0);
                    s1 = fmaf(sk[32 + blk], c4[1] + c4[3], s1);
                }
                // positions q and q + 4 of group nt; unselected ones leave the softmax
                if (!((mword >> (8 * nt + q)) & 1u)) s0 = -INFINITY;
                if (!((mword >> (8 * nt + q + 4)) & 1u)) s1 = -INFINITY;
                sbuf[nt * 32 + lane] = make_float2(s0, s1);
            }
            // ---- online softmax: this thread holds 8 of the 32 scores of head g, its quad the rest
            float2 S0 = sbuf[lane], S1 = sbuf[32 + lane], S2 = sbuf[64 + lane], S3 = sbuf[96 + lane];
            float mt = fmaxf(fmaxf(fmaxf(S0.x, S0.y), fmaxf(S1.x, S1.y)), fmaxf(fmaxf(S2.x, S2.y), fmaxf(S3.x, S3.y)));
            mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1)); mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
            const float mn = fmaxf(m_run, mt);
            const float corr = m_run == -INFINITY ? 0.f : expf(m_run - mn);
            S0.x = expf(S0.x - mn); S0.y = expf(S0.y - mn); S1.x = expf(S1.x - mn); S1.y = expf(S1.y - mn);
            S2.x = expf(S2.x - mn); S2.y = expf(S2.y - mn); S3.x = expf(S3.x - mn); S3.y = expf(S3.y - mn);
            float psum = ((S0.x + S0.y) + (S1.x + S1.y)) + ((S2.x + S2.y) + (S3.x + S3.y));
            sbuf[lane] = S0; sbuf[32 + lane] = S1; sbuf[64 + lane] = S2; sbuf[96 + lane] = S3;
            psum += __shfl_xor_sync(0xffffffffu, psum, 1); psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            l_run = l_run * corr + psum; m_run = mn;
            // the output columns of this thread are heads 2q and 2q + 1
            const float cf = corr * facc;
            const float ca = __shfl_sync(0xffffffffu, cf, 8 * q), cb = __shfl_sync(0xffffffffu, cf, 8 * q + 4);
#pragma unroll
            for (int i = 0; i < 16; i++) { acc[i][0] *= ca; acc[i][1] *= cb; acc[i][2] *= ca; acc[i][3] *= cb; }
            // ---- O^T += V^T (P * scale)^T, two 8-position groups per mma (k = 16 positions), once with the f16 of
            //      the scaled probabilities and once with what that rounding lost
#pragma unroll 1
            for (int np = 0; np < 2; np++) {
                const float2 pr0 = sbuf[(2 * np) * 32 + lane], pr1 = sbuf[(2 * np + 1) * 32 + lane];
                const float* sv = tvs + (16 * np + q) * 8;
                const uint32_t va = tv_s + (uint32_t)(2 * np * HD + g) * 4;
#pragma unroll
                for (int blk = 0; blk < 8; blk++) {
                    uint32_t bh0, bl0, bh1, bl1;
                    pb_split_h2(pr0.x * (sv[blk] * vscl), pr0.y * (sv[32 + blk] * vscl), bh0, bl0);
                    pb_split_h2(pr1.x * (sv[64 + blk] * vscl), pr1.y * (sv[96 + blk] * vscl), bh1, bl1);
#pragma unroll
                    for (int h2 = 0; h2 < 2; h2++) {
                        const int mtile = 2 * blk + h2;
                        const uint32_t a0 = pb_nib2_h2(pb_ldsv32(va + (uint32_t)(16 * mtile) * 4), sh);
                        const uint32_t a1 = pb_nib2_h2(pb_ldsv32(va + (uint32_t)(16 * mtile + 8) * 4), sh);
                        const uint32_t a2 = pb_nib2_h2(pb_ldsv32(va + (uint32_t)(HD + 16 * mtile) * 4), sh);
                        const uint32_t a3 = pb_nib2_h2(pb_ldsv32(va + (uint32_t)(HD + 16 * mtile + 8) * 4), sh);
                        pb_mma16(acc[mtile], a0, a1, a2, a3, bh0, bh1);
                        pb_mma16(acc[mtile], a0, a1, a2, a3, bl0, bl1);
                    }
                }
            }
            __syncwarp();   // all lanes are done with this buffer before the next iteration refills it
        }
    }
    // ---- this warp's partial in the merge layout [G][2 + hd]; the merge buffer overlays the tile buffers,
    //      so every warp of the CTA (all of them run this function) must be done with its tiles first
    __syncthreads();
    const float oscale = E == E_NONE ? 0.f : pb_exp2i(E);
#ifdef PB_ATTN_DBG
    if (lane == 0) printf("E %d oscale %g acc0 %g %g %g %g m %g l %g\n", E, oscale, acc[0][0], acc[0][1], acc[0][2], acc[0][3], m_run, l_run);
#endif
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const int d0 = 16 * i + g;
        if (2 * q < G) { mw[(2 * q) * (2 + HD) + 2 + d0] = acc[i][0] * oscale; mw[(2 * q) * (2 + HD) + 2 + d0 + 8] = acc[i][2] * oscale; }
        if (2 * q + 1 < G) { mw[(2 * q + 1) * (2 + HD) + 2 + d0] = acc[i][1] * oscale; mw[(2 * q + 1) * (2 + HD) + 2 + d0 + 8] = acc[i][3] * oscale; }
    }
    if (q == 0 && g < G) { mw[g * (2 + HD)] = m_run; mw[g * (2 + HD) + 1] = l_run; }
}

// grid (nsplit, n_kv, batch), 256 threads; a warp walks tiles of 32 positions.  Splits
// [0, nsplit_packed) take the packed tiles through pb_attn_mma_tiles; the other splits take the
// tiles from the packed boundary on (all tiles when nsplit_packed == 0) with scalar FMAs, where
// lane l owns dims 8l..8l+7 of the head.
template <int G>
__global__ void __launch_bounds__(AT_THREADS, 1) pb_attn_partial_kernel(const PbAttnParams p) {
    const int sp = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = p.hd, half = p.n_rot / 2;
    pb_pdl_wait();
    pb_pdl_trigger();
    const int64_t pos = p.pos[b], n = pos + 1;
    // window mode: this token sees as packed what a token-by-token run would have packed when it was appended
    int64_t q4n = 0;
    if (p.kv_bits == 4) {
        if (p.window) { const int64_t rule = n > p.kv_recent ? ((n - p.kv_recent) / 64) * 64 : 0, prev = p.q4n[1]; q4n = rule > prev ? rule : prev; }
        else q4n = p.q4n[b];
    }
    const float* proj = p.proj + (size_t)b * p.ldp;
    const uint32_t* mk = p.qsa_on && p.qsa_on[b] ? p.qsa_mask + (size_t)b * p.qsa_ld : nullptr;   // block-sparse: the positions attended

    extern __shared__ float asm_[];
    float* qs = asm_;                         // [G][hd] normalized, roped, scaled queries
    float* prob = asm_ + G * hd;              // [AT_WARPS][AT_TILE][G] tile probabilities
    // per-warp tile buffers; the merge buffer [AT_WARPS][G][2 + hd] reuses their space once every warp is done with its tiles
    uint32_t* stage_base = reinterpret_cast<uint32_t*>(prob + AT_WARPS * AT_TILE * G);
    float* mrg = reinterpret_cast<float*>(stage_base);

    // queries of this GQA group: rms_inplace(q, qn), rope, times 1/sqrt(hd)  (:1603-1606)
    if (hd == 256 && p.n_rot == 64) {
        // as in pb_kv_append_kernel: the loads of a head up front, one sincosf per lane
        for (int g = warp; g < G; g += AT_WARPS) {
            const float* qraw = proj + (size_t)(kvh * G + g) * 2 * hd;
            float qv[8], wn[8];
#pragma unroll
            for (int k = 0; k < 8; k++) { qv[k] = qraw[lane + 32 * k]; wn[k] = p.qn[lane + 32 * k]; }
            const float ang = (float)pos * p.rope_inv[lane], ms = p.rope_inv[half];
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < 8; k++) ss += qv[k] * qv[k];
            ss = pb_warp_sum(ss);
            const float s = 1.0f / sqrtf(ss / (float)hd + p.eps);
            const float scale = 1.0f / sqrtf((float)hd);
            float sn, co;
            sincosf(ang, &sn, &co);
            if (ms != 1.0f) { co *= ms; sn *= ms; }
            const float x0 = qv[0] * (s * wn[0]), x1 = qv[1] * (s * wn[1]);
            qs[g * hd + lane] = (x0 * co - x1 * sn) * scale;
            qs[g * hd + lane + 32] = (x1 * co + x0 * sn) * scale;
#pragma unroll
            for (int k = 2; k < 8; k++) qs[g * hd + lane + 32 * k] = (qv[k] * (s * wn[k])) * scale;
        }
    } else
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
                const float ms = p.rope_inv[half];
                if (ms != 1.0f) { co *= ms; sn *= ms; }
                x = i < half ? x * co - other * sn : x * co + other * sn;
            }
            qs[g * hd + i] = x * scale;
        }
    }
    __syncthreads();

    const int64_t ntiles = (n + AT_TILE - 1) / AT_TILE;
    // tiles are dealt round-robin to (split, warp) so that the slower f32 tiles of the recent window
    // are spread over all CTAs instead of landing on the last splits
    const size_t hrow = (size_t)(p.window ? 0 : b) * p.n_kv + kvh;
    const uint32_t* kw = p.kw + hrow * p.max_ctx * (hd / 8);
    const uint32_t* vw = p.vw + hrow * p.max_ctx * (hd / 8);
    const float* ks = p.ks + hrow * p.max_ctx * (hd / 32);
    const float* vs = p.vs + hrow * p.max_ctx * (hd / 32);
    const float* kr = p.kr + hrow * p.ring_cap * hd;
    const float* vr = p.vr + hrow * p.ring_cap * hd;
    float* pw = prob + warp * AT_TILE * G;
    float* mw = mrg + (size_t)warp * G * (2 + hd);
    // per-warp staging of one packed tile
    uint32_t* tkw = stage_base + (size_t)warp * AT_STAGE_WORDS;
    // Share of the splits that walk the packed positions on the tensor cores (p.nsplit_packed > 0 enables that
    // path), by estimated work at the sequence's current length: an f32 tile of 8 positions costs about two
    // and a half packed tiles of 32 (p.ring_weight).  Computed here, from the position and the packed boundary the device holds, so that a
    // captured graph keeps the right share however far the context has grown since its capture.
    int nsp = 0;
    if (p.nsplit_packed > 0) {
        const int64_t q4 = q4n < n ? q4n : n;
        const float wp = (float)(q4 / 32), wr = p.ring_weight * (float)((n - q4 + 7) / 8);
        int nr = (int)((float)gridDim.x * wr / (wr + wp) + 0.5f);
        nr = nr < 1 ? 1 : (nr > (int)gridDim.x - 1 ? (int)gridDim.x - 1 : nr);
        nsp = (int)gridDim.x - nr;
    }
    const int nrs = (int)gridDim.x - nsp;
    // tiles that are packed and entirely below the current length go to the tensor-core splits
    const int64_t tpk = nsp > 0 ? (q4n < n ? q4n : n) / AT_TILE : 0;
    if (sp < nsp) {
        if (G <= 8) pb_attn_mma_tiles<(G <= 8 ? G : 8)>(qs, tkw, warp, lane, sp, nsp, kw, vw, ks, vs, tpk, mw, mk);
    } else {
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

    float* tks = reinterpret_cast<float*>(tkw + AT_TILE * (hd / 8));
    uint32_t* tvw = reinterpret_cast<uint32_t*>(tks + AT_TILE * (hd / 32));
    float* tvs = reinterpret_cast<float*>(tvw + AT_TILE * (hd / 8));

    // scalar tiles: 32 positions when this path also walks packed tiles (no tensor-core splits), else 8, so that
    // the f32 window spreads over many warps (a 32-position f32 tile is ten times a packed one and would
    // alone set the kernel's duration)
    const int stile = nsp > 0 ? 8 : AT_TILE;
    const int64_t ntiles_s = (n + stile - 1) / stile;
    for (int64_t t = tpk * (AT_TILE / stile) + (int64_t)warp * nrs + (sp - nsp); t < ntiles_s; t += (int64_t)AT_WARPS * nrs) {
        const int64_t pbase = t * stile;
        // block-sparse: the tile's bits of the position mask (tiles start at multiples of 8 and never straddle a word)
        const uint32_t mbits = mk ? (mk[pbase >> 5] >> (pbase & 31)) & (stile == 32 ? 0xFFFFFFFFu : 0xFFu) : 0xFFFFFFFFu;
        if (mbits == 0u) continue;
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
        for (int i0 = 0; i0 < stile; i0 += 8) {
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
                    for (int j = 0; j < 8; j++) kv[j] = pb_kv4_dequant8(w, j, s);
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
        for (int g = 0; g < G; g++) if (lane < stile && pbase + lane < n && ((mbits >> lane) & 1u)) sc[g] = pw[lane * G + g];
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
        for (int i = 0; i < stile; i++) {
            const int64_t pp = pbase + i;
            if (pp >= n) break;
            float vv[8];
            if (packed) {
                const float s = tvs[i * (hd / 32) + (lane >> 2)];
#pragma unroll
                for (int j = 0; j < 8; j++) vv[j] = pb_kv4_dequant8(tvw[(i >> 3) * hd + 8 * lane + j], i & 7, s);   // position-transposed words
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

    __syncthreads();   // the merge buffer overlays the tile buffers of all warps
#pragma unroll
    for (int g = 0; g < G; g++) {
        if (lane == 0) { mw[g * (2 + hd)] = m_run[g]; mw[g * (2 + hd) + 1] = l_run[g]; }
#pragma unroll
        for (int j = 0; j < 8; j++) mw[g * (2 + hd) + 2 + 8 * lane + j] = acc[g][j];
    }
    }
    // ---- merge the 8 warps of the CTA, then write the split's partial
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
        // a lane's (up to four: nsplit <= 128) splits, maximum and sum of each, fetched in one go
        float2 ml[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int s = l + 32 * k;
            ml[k] = s < p.nsplit ? *reinterpret_cast<const float2*>(p.part_ml + ((base + s) * G + g) * 2) : make_float2(-INFINITY, 0.f);
        }
        float M = fmaxf(fmaxf(ml[0].x, ml[1].x), fmaxf(ml[2].x, ml[3].x));
        M = pb_warp_max(M);
        float L = 0.f;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int s = l + 32 * k;
            if (s < p.nsplit) {
                const float f = ml[k].x == -INFINITY ? 0.f : expf(ml[k].x - M);
                fs[s] = f;
                L += ml[k].y * f;
            }
        }
        L = pb_warp_sum(L);
        if (l == 0) { ML[0] = M; ML[1] = L; }
    }
    // this thread's rows of the splits' accumulators (and its gate value) are requested before the factors are awaited
    const float gate_raw = q == 0 ? p.proj[(size_t)b * p.ldp + (size_t)h * 2 * p.hd + p.hd + d] : 0.f;
    float pa[32];
#pragma unroll
    for (int k = 0; k < 32; k++) { const int s = q + 4 * k; pa[k] = s < p.nsplit ? p.part_acc[((base + s) * G + g) * p.hd + d] : 0.f; }
    __syncthreads();
    float o = 0.f;
#pragma unroll
    for (int k = 0; k < 32; k++) { const int s = q + 4 * k; if (s < p.nsplit) o = fmaf(pa[k], fs[s], o); }
    if (q > 0) part[q - 1][d] = o;
    __syncthreads();
    if (q == 0) {
        o = ((o + part[0][d]) + part[1][d]) + part[2][d];
        p.att[(size_t)b * p.lda + (size_t)h * p.hd + d] = (o * (1.0f / ML[1])) * pb_sigm(gate_raw);
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

int pb_launch_kv_pack(pb_ctx* ctx, const PbAttnParams& p) {
    if (!p.window || p.kv_bits != 4) return PB_OK;
    pb_launch_k(ctx, pb_kv_pack_kernel, dim3(1), dim3(AT_THREADS), (size_t)(0), p);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}

int pb_launch_attn(pb_ctx* ctx, const PbAttnParams& p) {
    const int G = p.n_head / p.n_kv;
    if (p.nsplit_packed < 0 || p.nsplit_packed >= p.nsplit || (p.nsplit_packed > 0 && (G > 8 || p.kv_bits != 4))) PB_FAIL(ctx, PB_ERR_ARG, "attention: %d of %d splits on the packed path", p.nsplit_packed, p.nsplit);
    if (p.hd != 256 || p.nsplit > 128 || p.n_head % p.n_kv || (G != 8 && G != 4 && G != 2 && G != 1))
        PB_FAIL(ctx, PB_UNSUPPORTED, "attention: head dim %d with %d query heads per KV head not supported", p.hd, G);
    const dim3 grid(p.nsplit, p.n_kv, p.batch);
    const size_t smem = ((size_t)G * p.hd + (size_t)AT_WARPS * AT_TILE * G + (size_t)AT_WARPS * AT_STAGE_WORDS) * 4;   // the merge buffer (AT_WARPS * G * (2 + hd) floats) fits inside the tile buffers
    if (smem > (size_t)ctx->max_smem_optin) PB_FAIL(ctx, PB_UNSUPPORTED, "attention needs %zu bytes of shared memory", smem);
#define GO(GG)                                                                                                                   \
    {                                                                                                                            \
        PB_TRY(pb_ensure_smem(ctx, pb_attn_partial_kernel<GG>, (size_t)ctx->max_smem_optin));                                     \
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

int pb_launch_kv4_pack(pb_ctx* ctx, const float* x, int64_t n, uint32_t* w, float* sc, int bias) {
    const int64_t nblocks = n / 32;
    if (nblocks <= 0) return PB_OK;
    pb_launch_k(ctx, pb_kv4_pack_kernel, dim3((unsigned)((nblocks + 7) / 8)), dim3(256), (size_t)(0), x, nblocks, w, sc, bias);
    ctx->kernels_launched++;
    PB_CUDA(ctx, cudaGetLastError());
    return PB_OK;
}
int pb_launch_kv4_pack_vt(pb_ctx* ctx, const float* x, int64_t npos, int hd, uint32_t* w, float* sc, int bias) {
    if (npos <= 0) return PB_OK;
    if (npos % 8 || hd % 32) PB_FAIL(ctx, PB_ERR_ARG, "kv4 pack: %lld positions of %d dims (multiples of 8 and 32 needed)", (long long)npos, hd);
    const int64_t units = npos / 8 * (hd / 32);
    pb_launch_k(ctx, pb_kv4_pack_vt_kernel, dim3((unsigned)((units + 7) / 8)), dim3(256), (size_t)(0), x, npos, hd, w, sc, bias);
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
