// Building blocks shared by the streaming dequant kernels (GEMV modes, expert SwiGLU):
// the shared-memory stage ring fed by 1-D bulk copies, and the in-kernel preparation of
// activations (RMSNorm variants + split into two int8 levels).
#pragma once
#include "pb_qdot.cuh"

#define PB_CONSUMERS 16
#define PB_KTHREADS ((PB_CONSUMERS + 1) * 32)
#define PB_STAGES 4

struct PbRing {
    uint64_t* full;
    uint64_t* empty;
    uint8_t* stages;
    uint32_t stage_bytes;
};

__device__ __forceinline__ void pb_named_barrier(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }

// thread 0 initialises, every thread of the CTA must then pass a __syncthreads()
__device__ __forceinline__ void pb_ring_init(const PbRing& r, int tid) {
    if (tid == 0) {
        for (int s = 0; s < PB_STAGES; s++) { pb_mbar_init(&r.full[s], 1); pb_mbar_init(&r.empty[s], PB_CONSUMERS); }
        pb_fence_barrier_init();
    }
}
// producer (one thread): make stage k % S writable, announce `bytes`; the caller then issues the copies
__device__ __forceinline__ bool pb_ring_acquire(const PbRing& r, int k, uint32_t bytes, int* status) {
    const int s = k % PB_STAGES;
    if (k >= PB_STAGES && !pb_mbar_wait_relaxed(&r.empty[s], ((k / PB_STAGES) - 1) & 1, status, PB_DEV_WAIT_EMPTY_TIMEOUT)) return false;
    pb_mbar_expect_tx(&r.full[s], bytes);
    return true;
}
// the same in two steps, for a producer that writes a chunk header between them: wait until stage
// k % S is writable, (plain shared-memory stores of the header), then announce `bytes`.  The arrive of
// pb_ring_announce has release semantics and the consumers' wait acquires, so they see the header.
__device__ __forceinline__ bool pb_ring_acquire_wait(const PbRing& r, int k, int* status) {
    return k < PB_STAGES || pb_mbar_wait_relaxed(&r.empty[k % PB_STAGES], ((k / PB_STAGES) - 1) & 1, status, PB_DEV_WAIT_EMPTY_TIMEOUT);
}
__device__ __forceinline__ void pb_ring_announce(const PbRing& r, int k, uint32_t bytes) { pb_mbar_expect_tx(&r.full[k % PB_STAGES], bytes); }
__device__ __forceinline__ uint8_t* pb_ring_stage(const PbRing& r, int k) { return r.stages + (size_t)(k % PB_STAGES) * r.stage_bytes; }
__device__ __forceinline__ void pb_ring_copy(const PbRing& r, int k, uint32_t dst_off, const void* src, uint32_t bytes) {
    pb_bulk_g2s(pb_ring_stage(r, k) + dst_off, src, bytes, &r.full[k % PB_STAGES]);
}
// producer error path: give the copies of the last stages a bounded chance to land before the CTA may exit
__device__ __forceinline__ void pb_ring_drain(const PbRing& r, int issued) {
    for (int k = max(0, issued - PB_STAGES); k < issued; k++) pb_mbar_wait(&r.full[k % PB_STAGES], (k / PB_STAGES) & 1, nullptr, 0);
}
__device__ __forceinline__ bool pb_ring_wait(const PbRing& r, int k, int* status) {
    return pb_mbar_wait(&r.full[k % PB_STAGES], (k / PB_STAGES) & 1, status, PB_DEV_WAIT_FULL_TIMEOUT);
}
// consumer warp: done with stage k
__device__ __forceinline__ void pb_ring_release(const PbRing& r, int k, int lane) {
    __syncwarp();
    if (lane == 0) pb_mbar_arrive(&r.empty[k % PB_STAGES]);
}

// word offset of quad i (4 words) of quarter qi inside one level array of nq quarters
// (quad-major so that a warp's 128-bit loads of consecutive quarters never conflict)
__device__ __forceinline__ int pb_xq_off(int qi, int i, int nq) { return (i * nq + qi) * 4; }

// Quantized activations of one column: PB_XLEVELS arrays of cols/4 words, then PB_XLEVELS scale
// arrays and the group sums, cols/32 floats each, then PB_XLEVELS arrays of cols/32 integers: -15 times the
// sum of each level's int8 values over a group (the offset term of weight formats coded as 2 c - 15)
__host__ __device__ static inline int pb_xq_words(int cols) { return PB_XLEVELS * (cols / 4) + (2 * PB_XLEVELS + 1) * (cols / 32); }

// One warp splits FOUR consecutive 32-value groups of a column at once: lane l owns elements
// 4*(l&7) .. +3 of group g0 + (l>>3), so a reduction over a group is 3 shuffles and every lane
// packs its own word.  v = the lane's four values.  Output: PB_XLEVELS int8 levels in the
// quad-major layout at `col` (shared or global memory), their scales and the group sums.
// All sixteen warps of a CTA run this at the same moment, so it is written for instruction throughput: rounding to
// an integer is a float addition of 1.5 * 2^23 (round-to-nearest-even, as cvt.rni; conversions are quarter-rate),
// and the integer sums of the three levels share one pair of shuffle reductions.  WITH_SUM = false skips the f32
// group sums, which only formats with a minimum (Q4_K) read.
template <bool WITH_SUM = true>
__device__ __forceinline__ void pb_split_groups4(float4 v, int lane, int g0, int cols, uint32_t* col) {
    const int ng = cols / 32, nq = cols / 64;
    float* sc = reinterpret_cast<float*>(col + PB_XLEVELS * (cols / 4));
    const int g = g0 + (lane >> 3), k = lane & 7;   // word k of group g = word 8*(g&1)+k of quarter g/2
    const int off = pb_xq_off(g >> 1, 2 * (g & 1) + (k >> 2), nq) + (k & 3);
    float sum = 0.f;
    if (WITH_SUM) {
        sum = (v.x + v.y) + (v.z + v.w);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1); sum += __shfl_xor_sync(0xffffffffu, sum, 2); sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    }
    float r[4] = {v.x, v.y, v.z, v.w};
    const float kMagic = 12582912.0f;   // 1.5 * 2^23: adding it leaves round-to-nearest-even(t) in the low mantissa bits
    int asum[PB_XLEVELS];
    float sl[PB_XLEVELS];
#pragma unroll
    for (int l = 0; l < PB_XLEVELS; l++) {
        float m = fmaxf(fmaxf(fabsf(r[0]), fabsf(r[1])), fmaxf(fabsf(r[2]), fabsf(r[3])));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1)); m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2)); m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
        // scale = max / 127 and its reciprocal, by a multiplication and the fast reciprocal: any scale with |r| / s <= 127.5
        // serves (what a level does not represent is carried into the next one); groups below 1e-30 count as zero
        const float s = m > 1e-30f && isfinite(m) ? m * (1.0f / 127.f) : 0.f;
        const float inv = s > 0.f ? __fdividef(1.0f, s) : 0.f;
        uint32_t pa = 0;
        int as = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float t = s > 0.f ? fminf(fmaxf(r[j] * inv, -127.f), 127.f) : 0.f;
            const float tm = t + kMagic;
            const int a = __float_as_int(tm) - 0x4B400000;
            r[j] = s > 0.f ? fmaf(-s, tm - kMagic, r[j]) : 0.f;
            pa |= (uint32_t)(a & 0xFF) << (8 * j);
            as += a;
        }
        col[l * (cols / 4) + off] = pa;
        asum[l] = as; sl[l] = s;
    }
    // sums of the levels over the group: levels 0 and 1 biased into the two halves of one word (|sum over 8 lanes| <= 4064)
    static_assert(PB_XLEVELS == 3, "the packed reduction below is written for three levels");
    int p01 = (asum[0] + 512) | ((asum[1] + 512) << 16), p2 = asum[2];
    p01 += __shfl_xor_sync(0xffffffffu, p01, 1); p01 += __shfl_xor_sync(0xffffffffu, p01, 2); p01 += __shfl_xor_sync(0xffffffffu, p01, 4);
    p2 += __shfl_xor_sync(0xffffffffu, p2, 1); p2 += __shfl_xor_sync(0xffffffffu, p2, 2); p2 += __shfl_xor_sync(0xffffffffu, p2, 4);
    if (k == 0) {
        const int tot[3] = {(p01 & 0xFFFF) - 4096, (p01 >> 16) - 4096, p2};
#pragma unroll
        for (int l = 0; l < PB_XLEVELS; l++) { sc[l * ng + g] = sl[l]; reinterpret_cast<int*>(sc)[(PB_XLEVELS + 1 + l) * ng + g] = -15 * tot[l]; }   // stored ready for 2 A - 15 S
        if (WITH_SUM) sc[PB_XLEVELS * ng + g] = sum;
    }
}

template <bool ISUM = false>
__device__ __forceinline__ void pb_load_xquarter(const uint32_t* xcol, int cols, int qi, PbXQuarter& o) {
    const int nq = cols / 64, ng = cols / 32;
    const float* sc = reinterpret_cast<const float*>(xcol + PB_XLEVELS * (cols / 4));
#pragma unroll
    for (int l = 0; l < PB_XLEVELS; l++) {
        const uint32_t* q = xcol + l * (cols / 4);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint4 a = *reinterpret_cast<const uint4*>(q + pb_xq_off(qi, i, nq));
            o.q[l][4 * i] = (int)a.x; o.q[l][4 * i + 1] = (int)a.y; o.q[l][4 * i + 2] = (int)a.z; o.q[l][4 * i + 3] = (int)a.w;
        }
        // the two groups of a quarter are neighbours: one 64-bit load (ng is even, so the pair is 8-byte aligned)
        const float2 s2 = *reinterpret_cast<const float2*>(sc + l * ng + 2 * qi);
        o.s[l][0] = s2.x; o.s[l][1] = s2.y;
    }
    const float2 m2 = *reinterpret_cast<const float2*>(sc + PB_XLEVELS * ng + 2 * qi);
    o.sum[0] = m2.x; o.sum[1] = m2.y;
    if (ISUM) {
        const int* is = reinterpret_cast<const int*>(sc) + (PB_XLEVELS + 1) * ng;
#pragma unroll
        for (int l = 0; l < PB_XLEVELS; l++) { const int2 i2 = *reinterpret_cast<const int2*>(is + l * ng + 2 * qi); o.is[l][0] = i2.x; o.is[l][1] = i2.y; }
    }
}

// Fill the shared-memory tables a format needs at `tab` (16-byte aligned, pb_tab_bytes<FMT>(rep) long):
// the sign look-up table first, then the codebook with `rep` copies of every entry (rep = 1, or one
// copy per bank so that random look-ups of a warp never conflict).  The caller synchronises after.
template <int FMT> __host__ __device__ constexpr int pb_tab_entry_bytes() { return FMT == PB_T_IQ3_S || FMT == PB_T_IQ3_XXS ? 4 : (FMT == PB_T_IQ2_XS || FMT == PB_T_IQ2_S || FMT == PB_T_IQ2_XXS || FMT == PB_T_IQ1_M ? 8 : 0); }
template <int FMT> __host__ __device__ constexpr int pb_tab_entries() { return FMT == PB_T_IQ3_XXS || FMT == PB_T_IQ2_XXS ? 256 : (FMT == PB_T_IQ2_S ? 1024 : (FMT == PB_T_IQ1_M ? 4096 : 512)); }
template <int FMT> __host__ __device__ constexpr uint32_t pb_tab_bytes(int rep) { return pb_tab_entry_bytes<FMT>() ? PB_SIGN_LUT_BYTES + pb_tab_entries<FMT>() * pb_tab_entry_bytes<FMT>() * rep : 0; }
// copies of every entry when the codebook is replicated: one per shared-memory bank, but no more than 64 KB in all
template <int FMT> __host__ __device__ constexpr int pb_tab_rep_max() {
    constexpr int e = pb_tab_entry_bytes<FMT>();
    if (e == 0) return 1;
    int rep = 128 / e;
    while (rep > 1 && pb_tab_entries<FMT>() * e * rep > 65536) rep /= 2;
    return rep;
}

template <int FMT>
__device__ __forceinline__ PbQTabs pb_fill_qtabs(uint8_t* tab, int rep, int tid, int nthreads, int lane) {
    PbQTabs T;
    T.sign256 = pb_smem_u32(tab);
    constexpr int entry = pb_tab_entry_bytes<FMT>();
    T.stride = entry * rep;
    T.grid = pb_smem_u32(tab + PB_SIGN_LUT_BYTES) + (lane & (rep - 1)) * entry;
    if (entry) {
        uint4* sg = reinterpret_cast<uint4*>(tab);
        for (int i = tid; i < 256; i += nthreads) {
            uint32_t lo = 0, hi = 0;
            for (int j = 0; j < 4; j++) { if (i & (1 << j)) lo |= 0xFFu << (8 * j); if (i & (16 << j)) hi |= 0xFFu << (8 * j); }
            sg[i] = make_uint4(lo, lo & 0x01010101u, hi, hi & 0x01010101u);
        }
    }
    if (FMT == PB_T_IQ3_S) {
        uint32_t* g = reinterpret_cast<uint32_t*>(tab + PB_SIGN_LUT_BYTES);
        for (int i = tid; i < 512 * rep; i += nthreads) g[i] = PB_IQ3S_GRID[i / rep];
    }
    if (FMT == PB_T_IQ2_XS) {
        uint64_t* g = reinterpret_cast<uint64_t*>(tab + PB_SIGN_LUT_BYTES);
        for (int i = tid; i < 512 * rep; i += nthreads) g[i] = PB_IQ2XS_GRID[i / rep];
    }
    if (FMT == PB_T_IQ3_XXS) {
        uint32_t* g = reinterpret_cast<uint32_t*>(tab + PB_SIGN_LUT_BYTES);
        for (int i = tid; i < 256 * rep; i += nthreads) g[i] = PB_IQ3XXS_GRID[i / rep];
    }
    if (FMT == PB_T_IQ2_S) {
        uint64_t* g = reinterpret_cast<uint64_t*>(tab + PB_SIGN_LUT_BYTES);
        for (int i = tid; i < 1024 * rep; i += nthreads) g[i] = PB_IQ2S_GRID[i / rep];
    }
    if (FMT == PB_T_IQ1_M) {   // entry (sign << 11 | index) = 8 * grid value + (sign ? -1 : 1) per byte: the weights in eighths, as int8
        uint64_t* g = reinterpret_cast<uint64_t*>(tab + PB_SIGN_LUT_BYTES);
        for (int i = tid; i < 4096 * rep; i += nthreads) {
            const int e = i / rep;
            const uint64_t v = PB_IQ1S_GRID[e & 2047];
            const int dl = e >> 11 ? -1 : 1;
            uint64_t r = 0;
            for (int j = 0; j < 8; j++) r |= (uint64_t)(uint8_t)(8 * (int)(int8_t)(uint8_t)(v >> (8 * j)) + dl) << (8 * j);
            g[i] = r;
        }
    }
    if (FMT == PB_T_IQ2_XXS) {
        uint64_t* g = reinterpret_cast<uint64_t*>(tab + PB_SIGN_LUT_BYTES);
        for (int i = tid; i < 256 * rep; i += nthreads) g[i] = PB_IQ2XXS_GRID[i / rep];
    }
    return T;
}

// sum over all consumer threads (PB_CONSUMERS warps) of v; red = PB_CONSUMERS floats of shared memory
__device__ __forceinline__ float pb_consumer_sum(float v, float* red, int warp, int lane) {
    v = pb_warp_sum(v);
    pb_named_barrier(2, PB_CONSUMERS * 32);
    if (lane == 0) red[warp] = v;
    pb_named_barrier(2, PB_CONSUMERS * 32);
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < PB_CONSUMERS; i++) t += red[i];
    return t;
}

// ---- pieces of the activation prologues shared by pb_gemvq_kernel and the fused step kernel (same bits from both) ----
// sum of squares of x[tid], x[tid + n], x[tid + 2n], ... : the partition of the RMSNorm prologue
__device__ __forceinline__ float pb_strided_ss(const float* x, int cols, int tid, int nthreads) {
    float ss = 0.f;
    for (int c = tid; c < cols; c += nthreads) { const float v = x[c]; ss = fmaf(v, v, ss); }   // spelled out: see pb_row_rms_scale
    return ss;
}
// x * s * w per element (rms(): qwen4exp_gguf.rs:209)
__device__ __forceinline__ float4 pb_norm_vec(float4 v, float s, float4 w) { v.x = v.x * s * w.x; v.y = v.y * s * w.y; v.z = v.z * s * w.z; v.w = v.w * s * w.w; return v; }
// one head of 128 values held by a warp (lane l: elements 4l..4l+3): rms_inplace(o, norm, eps), then * sg (= sigmoid(z), or ones)
// (linear_core, qwen4exp_gguf.rs:1667)
__device__ __forceinline__ float4 pb_gnorm_vec(float4 v, float4 w, float4 sg, int head_dim, float eps) {
    const float ss = pb_warp_sum(fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, __fmul_rn(v.w, v.w)))));   // spelled out: see pb_row_rms_scale
    const float s = 1.0f / sqrtf(ss / (float)head_dim + eps);
    v.x *= s * w.x; v.y *= s * w.y; v.z *= s * w.z; v.w *= s * w.w;
    v.x *= sg.x; v.y *= sg.y; v.z *= sg.z; v.w *= sg.w;
    return v;
}
