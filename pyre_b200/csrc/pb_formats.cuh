// Decoders for the GGUF block formats of the decode path, written for one warp per
// 256-weight super-step: lane l decodes 8 weights ("a unit") of the super-step.
//
// Layouts and decode expressions restate the reference's dequantizer
// (src/model/gguf_q.rs:67-166: Q8_0 :79, Q4_K :103-107 with scale_min_k4 :62-64,
// IQ2_XS :126-129, IQ3_S :141-151; geometry QType::geom :33-41).  Every scale is formed
// with the same separate f32 roundings as the reference (__fmul_rn, never contracted), so
// the dequantized value  s * w - m  is bit-identical to the reference's.
#pragma once
#include "pb_common.cuh"

#define PB_TABLE_QUAL static __device__ const
#include "pb_iq_tables.h"

enum : int { PB_T_F32 = 0, PB_T_F16 = 1, PB_T_Q4_0 = 2, PB_T_Q5_0 = 6, PB_T_Q3_K = 11, PB_T_Q5_K = 13, PB_T_Q8_0 = 8, PB_T_Q4_K = 12, PB_T_Q6_K = 14, PB_T_IQ2_XXS = 16, PB_T_Q2_0 = 42, PB_T_IQ1_M = 29, PB_T_IQ2_XS = 17, PB_T_IQ3_XXS = 18, PB_T_IQ4_NL = 20, PB_T_IQ3_S = 21, PB_T_IQ2_S = 22,
             PB_T_IQ4_XS = 23, PB_T_BF16 = 30,
             // internal, never a ggml id: IQ3_S re-coded at upload into 4-bit codes (see pb_repack.cu).  Every IQ3_S
             // codebook value is odd (1..15), so a weight is one of the sixteen values -15, -13, .. 15 = 2 c - 15.
             // Block of 256 weights, 136 bytes: [d f16][2 pad][4 bytes of 4-bit sub-scales as in IQ3_S][32 words];
             // word m holds weights 8m..8m+3 in the low nibbles of its bytes and 8m+4..8m+7 in the high nibbles.
             PB_T_IQ3S_N4 = 121 };

// Codebooks staged in shared memory by the kernel that decodes (see pb_load_tables).
struct PbTables {
    const uint32_t* iq3s;   // 512 x 4 grid bytes
    const uint64_t* iq2xs;  // 512 x 8 grid bytes
    const uint8_t* ksigns;  // 128 sign bytes
    const uint32_t* iq3xxs; // 256 x 4 grid bytes
    const uint64_t* iq2s;   // 1024 x 8 grid bytes
    const int8_t* kvalues;  // 16 values of the IQ4 non-linear code
    const uint64_t* iq2xxs; // 256 x 8 grid bytes
    const uint64_t* iq1s;   // 2048 x 8 signed grid bytes (-1, 0, 1): read where it lies in global memory, never copied to shared memory
};
#define PB_TABLE_BYTES (512 * 8 + 512 * 4 + 128 + 256 * 4 + 1024 * 8 + 16 + 256 * 8)

// Copy the codebooks a format needs into shared memory at `dst` (16-byte aligned,
// PB_TABLE_BYTES long).  All threads of the CTA call it; the caller synchronises after.
template <int FMT>
__device__ __forceinline__ PbTables pb_load_tables(uint8_t* dst, int tid, int nthreads) {
    PbTables t;
    uint64_t* g2 = reinterpret_cast<uint64_t*>(dst);
    uint32_t* g3 = reinterpret_cast<uint32_t*>(dst + 512 * 8);
    uint8_t* ks = dst + 512 * 8 + 512 * 4;
    if (FMT == PB_T_IQ3_S)
        for (int i = tid; i < 512; i += nthreads) g3[i] = PB_IQ3S_GRID[i];
    if (FMT == PB_T_IQ2_XS) {
        for (int i = tid; i < 512; i += nthreads) g2[i] = PB_IQ2XS_GRID[i];
        for (int i = tid; i < 128; i += nthreads) ks[i] = PB_KSIGNS_IQ2XS[i];
    }
    uint32_t* g3x = reinterpret_cast<uint32_t*>(dst + 512 * 8 + 512 * 4 + 128);
    uint64_t* g2s = reinterpret_cast<uint64_t*>(dst + 512 * 8 + 512 * 4 + 128 + 256 * 4);
    int8_t* kv = reinterpret_cast<int8_t*>(dst + 512 * 8 + 512 * 4 + 128 + 256 * 4 + 1024 * 8);
    if (FMT == PB_T_IQ3_XXS) {
        for (int i = tid; i < 256; i += nthreads) g3x[i] = PB_IQ3XXS_GRID[i];
        for (int i = tid; i < 128; i += nthreads) ks[i] = PB_KSIGNS_IQ2XS[i];
    }
    if (FMT == PB_T_IQ2_S)
        for (int i = tid; i < 1024; i += nthreads) g2s[i] = PB_IQ2S_GRID[i];
    if (FMT == PB_T_IQ4_NL || FMT == PB_T_IQ4_XS)
        for (int i = tid; i < 16; i += nthreads) kv[i] = PB_KVALUES_IQ4NL[i];
    uint64_t* g2x = reinterpret_cast<uint64_t*>(dst + 512 * 8 + 512 * 4 + 128 + 256 * 4 + 1024 * 8 + 16);
    if (FMT == PB_T_IQ2_XXS) {
        for (int i = tid; i < 256; i += nthreads) g2x[i] = PB_IQ2XXS_GRID[i];
        for (int i = tid; i < 128; i += nthreads) ks[i] = PB_KSIGNS_IQ2XS[i];
    }
    t.iq2xs = g2; t.iq3s = g3; t.ksigns = ks; t.iq3xxs = g3x; t.iq2s = g2s; t.kvalues = kv; t.iq2xxs = g2x; t.iq1s = PB_IQ1S_GRID;
    return t;
}

// One unit: 8 integer-valued weights w (sign applied), the scale of the first and of the
// second four (sa, sb) and, for formats with a minimum, the offsets (ma, mb):
//   value[j] = (j < 4 ? sa : sb) * w[j] - (j < 4 ? ma : mb)
struct PbUnit { float w[8]; float sa, sb, ma, mb; };

template <int FMT> struct PbFmt;

// ---- contiguous-8 formats share the x / y index maps: lane l owns weights 8l..8l+7 ----
struct PbContig8 {
    // index (in float4 units, within the 256-wide step) of the two activation quads a lane needs
    __device__ static __forceinline__ int xa(int lane) { return 2 * lane; }
    __device__ static __forceinline__ int xb(int lane) { return 2 * lane + 1; }
    // where float4 number k of a step is stored in the lane-major shared-memory copy of x
    __device__ static __forceinline__ int perm(int k) { return (k & 1) * 32 + (k >> 1); }
    // position of weight j of the lane inside the 256-wide step
    __device__ static __forceinline__ int pos(int lane, int j) { return 8 * lane + j; }
};

template <> struct PbFmt<PB_T_IQ3_S> : PbContig8 {
    static constexpr int STEP_BYTES = 110;  // [d f16][qs 64][qh 8][signs 32][scales 4]
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables& T, PbUnit& o) {
        const float d = pb_h2f(*reinterpret_cast<const uint16_t*>(p));
        const uint32_t qs = *reinterpret_cast<const uint16_t*>(p + 2 + 2 * u);
        const uint32_t qh = p[66 + (u >> 2)] >> (2 * (u & 3));
        const uint32_t sg = p[74 + u];
        const uint32_t sc = p[106 + (u >> 3)];
        const uint32_t nib = (u & 4) ? (sc >> 4) : (sc & 0xF);
        o.sa = o.sb = __fmul_rn(d, (float)(1 + 2 * (int)nib));
        o.ma = o.mb = 0.0f;
        const uint32_t g1 = T.iq3s[(qs & 0xFF) | ((qh & 1) << 8)];
        const uint32_t g2 = T.iq3s[(qs >> 8) | ((qh & 2) << 7)];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float a = (float)((g1 >> (8 * j)) & 0xFF), b = (float)((g2 >> (8 * j)) & 0xFF);
            o.w[j] = (sg >> j) & 1 ? -a : a;
            o.w[4 + j] = (sg >> (4 + j)) & 1 ? -b : b;
        }
    }
};

template <> struct PbFmt<PB_T_IQ2_XS> : PbContig8 {
    static constexpr int STEP_BYTES = 74;  // [d f16][qs 32 x u16][scales 8]
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables& T, PbUnit& o) {
        const float d = pb_h2f(*reinterpret_cast<const uint16_t*>(p));
        const uint32_t q = *reinterpret_cast<const uint16_t*>(p + 2 + 2 * u);
        const uint32_t sc = p[66 + (u >> 2)];
        const uint32_t nib = (u & 2) ? (sc >> 4) : (sc & 0xF);
        o.sa = o.sb = __fmul_rn(__fmul_rn(d, 0.5f + (float)nib), 0.25f);
        o.ma = o.mb = 0.0f;
        const uint64_t g = T.iq2xs[q & 511];
        const uint32_t sg = T.ksigns[q >> 9];
        const uint32_t lo = (uint32_t)g, hi = (uint32_t)(g >> 32);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float a = (float)((lo >> (8 * j)) & 0xFF), b = (float)((hi >> (8 * j)) & 0xFF);
            o.w[j] = (sg >> j) & 1 ? -a : a;
            o.w[4 + j] = (sg >> (4 + j)) & 1 ? -b : b;
        }
    }
};

// IQ3_XXS (gguf_q.rs:136-140): per 32 weights eight grid indices (two entries of four magnitudes per unit) and one u32 with
// four 7-bit sign-pattern indices and a 4-bit scale
template <> struct PbFmt<PB_T_IQ3_XXS> : PbContig8 {
    static constexpr int STEP_BYTES = 98;   // [d f16][qs 64][scales and signs 8 x u32]
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables& T, PbUnit& o) {
        const float d = pb_h2f(*reinterpret_cast<const uint16_t*>(p));
        const int ib = u >> 2, l = u & 3;
        const uint8_t* ss = p + 66 + 4 * ib;
        const uint32_t a = (uint32_t)ss[0] | ((uint32_t)ss[1] << 8) | ((uint32_t)ss[2] << 16) | ((uint32_t)ss[3] << 24);
        o.sa = o.sb = __fmul_rn(__fmul_rn(d, 0.5f + (float)(a >> 28)), 0.5f);
        o.ma = o.mb = 0.0f;
        const uint32_t g1 = T.iq3xxs[p[2 + 8 * ib + 2 * l]], g2 = T.iq3xxs[p[2 + 8 * ib + 2 * l + 1]];
        const uint32_t sg = T.ksigns[(a >> (7 * l)) & 127];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float x = (float)((g1 >> (8 * j)) & 0xFF), y = (float)((g2 >> (8 * j)) & 0xFF);
            o.w[j] = (sg >> j) & 1 ? -x : x;
            o.w[4 + j] = (sg >> (4 + j)) & 1 ? -y : y;
        }
    }
};

// IQ2_S (gguf_q.rs:130-135): per unit one 10-bit grid index (8 bits in qs, 2 in qh) and one explicit sign byte
template <> struct PbFmt<PB_T_IQ2_S> : PbContig8 {
    static constexpr int STEP_BYTES = 82;   // [d f16][qs 32][signs 32][qh 8][scales 8]
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables& T, PbUnit& o) {
        const float d = pb_h2f(*reinterpret_cast<const uint16_t*>(p));
        const int ib = u >> 2, l = u & 3;
        const uint32_t sc = p[74 + ib];
        const uint32_t nib = (l & 2) ? (sc >> 4) : (sc & 0xF);
        o.sa = o.sb = __fmul_rn(__fmul_rn(d, 0.5f + (float)nib), 0.25f);
        o.ma = o.mb = 0.0f;
        const uint32_t idx = (uint32_t)p[2 + 4 * ib + l] | ((((uint32_t)p[66 + ib]) << (8 - 2 * l)) & 0x300);
        const uint64_t g = T.iq2s[idx];
        const uint32_t sg = p[34 + 4 * ib + l];
        const uint32_t lo = (uint32_t)g, hi = (uint32_t)(g >> 32);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float x = (float)((lo >> (8 * j)) & 0xFF), y = (float)((hi >> (8 * j)) & 0xFF);
            o.w[j] = (sg >> j) & 1 ? -x : x;
            o.w[4 + j] = (sg >> (4 + j)) & 1 ? -y : y;
        }
    }
};

// IQ4_NL (gguf_q.rs:82-83): blocks of 32 = [d f16][16 bytes]; weight j < 16 is the low nibble of byte j, weight 16 + j the high one
template <> struct PbFmt<PB_T_IQ4_NL> : PbContig8 {
    static constexpr int STEP_BYTES = 8 * 18;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables& T, PbUnit& o) {
        const uint8_t* b = p + 18 * (u >> 2);
        const int part = u & 3;                       // weights 8 part .. 8 part + 7 of the block
        o.sa = o.sb = pb_h2f((uint16_t)(b[0] | (b[1] << 8)));
        o.ma = o.mb = 0.0f;
        const uint8_t* q = b + 2 + 8 * (part & 1);
#pragma unroll
        for (int j = 0; j < 8; j++) o.w[j] = (float)T.kvalues[part < 2 ? (q[j] & 0xF) : (q[j] >> 4)];
    }
};

// IQ4_XS (gguf_q.rs:84-89): super-block [d f16][scales_h u16][scales_l 4][qs 128]; per 32 weights a 6-bit scale ls, value = kvalue * (d * (ls - 32))
template <> struct PbFmt<PB_T_IQ4_XS> : PbContig8 {
    static constexpr int STEP_BYTES = 136;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables& T, PbUnit& o) {
        const float d = pb_h2f(*reinterpret_cast<const uint16_t*>(p));
        const int ib = u >> 2, part = u & 3;
        const uint32_t sh = (uint32_t)p[2] | ((uint32_t)p[3] << 8);
        const int ls = (int)((p[4 + (ib >> 1)] >> (4 * (ib & 1))) & 0xF) | (int)(((sh >> (2 * ib)) & 3) << 4);
        o.sa = o.sb = __fmul_rn(d, (float)(ls - 32));
        o.ma = o.mb = 0.0f;
        const uint8_t* q = p + 8 + 16 * ib + 8 * (part & 1);
#pragma unroll
        for (int j = 0; j < 8; j++) o.w[j] = (float)T.kvalues[part < 2 ? (q[j] & 0xF) : (q[j] >> 4)];
    }
};

// Q2_0 (gguf_q.rs:80-81, ggml id 42): blocks of 64 = [d f16][16 bytes]; weight 4k + j is field j (two bits) of byte k, value (field - 1) * d
template <> struct PbFmt<PB_T_Q2_0> : PbContig8 {
    static constexpr int STEP_BYTES = 4 * 18;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const uint8_t* b = p + 18 * (u >> 3);
        o.sa = o.sb = pb_h2f((uint16_t)(b[0] | (b[1] << 8)));
        o.ma = o.mb = 0.0f;
        const uint32_t two = (uint32_t)b[2 + 2 * (u & 7)] | ((uint32_t)b[3 + 2 * (u & 7)] << 8);
#pragma unroll
        for (int j = 0; j < 8; j++) o.w[j] = (float)((int)((two >> (2 * j)) & 3) - 1);
    }
};

// IQ2_XXS (gguf_q.rs:122-125): per 32 weights four 8-bit grid indices (entries of eight magnitudes) and one u32 with four
// 7-bit sign patterns and a 4-bit scale
template <> struct PbFmt<PB_T_IQ2_XXS> : PbContig8 {
    static constexpr int STEP_BYTES = 66;   // [d f16][8 x (4 index bytes, u32 signs and scale)]
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables& T, PbUnit& o) {
        const float d = pb_h2f(*reinterpret_cast<const uint16_t*>(p));
        const int ib = u >> 2, l = u & 3;
        const uint8_t* q = p + 2 + 8 * ib;
        const uint32_t a = (uint32_t)q[4] | ((uint32_t)q[5] << 8) | ((uint32_t)q[6] << 16) | ((uint32_t)q[7] << 24);
        o.sa = o.sb = __fmul_rn(__fmul_rn(d, 0.5f + (float)(a >> 28)), 0.25f);
        o.ma = o.mb = 0.0f;
        const uint64_t g = T.iq2xxs[q[l]];
        const uint32_t sg = T.ksigns[(a >> (7 * l)) & 127];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float x = (float)((uint32_t)(g >> (8 * j)) & 0xFF);
            o.w[j] = (sg >> j) & 1 ? -x : x;
        }
    }
};

// Q4_0 (gguf_q.rs:74-75): blocks of 32 = [d f16][16 bytes]; weight j < 16 is the low nibble of byte j, weight 16 + j the high one, value nibble - 8
template <> struct PbFmt<PB_T_Q4_0> : PbContig8 {
    static constexpr int STEP_BYTES = 8 * 18;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const uint8_t* b = p + 18 * (u >> 2);
        const int part = u & 3;
        o.sa = o.sb = pb_h2f((uint16_t)(b[0] | (b[1] << 8)));
        o.ma = o.mb = 0.0f;
        const uint8_t* q = b + 2 + 8 * (part & 1);
#pragma unroll
        for (int j = 0; j < 8; j++) o.w[j] = (float)((int)(part < 2 ? (q[j] & 0xF) : (q[j] >> 4)) - 8);
    }
};

// Q5_0 (gguf_q.rs:76-78): blocks of 32 = [d f16][qh u32][16 bytes]; as Q4_0 with bit i of qh as the fifth bit of weight i, value - 16
template <> struct PbFmt<PB_T_Q5_0> : PbContig8 {
    static constexpr int STEP_BYTES = 8 * 22;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const uint8_t* b = p + 22 * (u >> 2);
        const int part = u & 3;
        o.sa = o.sb = pb_h2f((uint16_t)(b[0] | (b[1] << 8)));
        o.ma = o.mb = 0.0f;
        const uint32_t qh = ((uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24)) >> (8 * part);
        const uint8_t* q = b + 6 + 8 * (part & 1);
#pragma unroll
        for (int j = 0; j < 8; j++) o.w[j] = (float)((int)((part < 2 ? (q[j] & 0xF) : (q[j] >> 4)) | (((qh >> j) & 1) << 4)) - 16);
    }
};

// Q3_K (gguf_q.rs:90-102): [hmask 32][qs 64][scales 12][d f16]; weight 128 n + 32 j + o takes two bits (shift 2 j) of qs[32 n + o] and, as
// "not minus four", bit 4 n + j of hmask[o]; sixteen 6-bit scales (minus 32), one per 16 weights, spread over the twelve scale bytes
template <> struct PbFmt<PB_T_Q3_K> : PbContig8 {
    static constexpr int STEP_BYTES = 110;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const float d = pb_h2f((uint16_t)(p[108] | (p[109] << 8)));
        const int n = u >> 4, j = (u >> 2) & 3, o0 = 8 * (u & 3), is = 8 * n + 2 * j + (o0 >> 4);
        const uint8_t* sc = p + 96;
        const int lo = is < 8 ? (sc[is] & 0xF) : (sc[is - 8] >> 4), hi = (sc[8 + (is & 3)] >> (2 * (is >> 2))) & 3;
        o.sa = o.sb = __fmul_rn(d, (float)((lo | (hi << 4)) - 32));
        o.ma = o.mb = 0.0f;
        const uint8_t* q = p + 32 + 32 * n + o0;
        const uint8_t* hm = p + o0;
#pragma unroll
        for (int k = 0; k < 8; k++) o.w[k] = (float)((int)((q[k] >> (2 * j)) & 3) - ((hm[k] >> (4 * n + j)) & 1 ? 0 : 4));
    }
};

// Q5_K (gguf_q.rs:108-113): [d f16][dmin f16][scales 12][qh 32][ql 128]; as Q4_K (64 weights per group: low nibbles, then high nibbles of 32
// bytes) with bits 2 g and 2 g + 1 of qh[l] as the fifth bit
template <> struct PbFmt<PB_T_Q5_K> : PbContig8 {
    static constexpr int STEP_BYTES = 176;
    static constexpr bool HAS_MIN = true;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const float d = pb_h2f(*reinterpret_cast<const uint16_t*>(p));
        const float mn = pb_h2f(*reinterpret_cast<const uint16_t*>(p + 2));
        const int g = u >> 3, r = u & 7, hi = r >> 2, l0 = 8 * (r & 3);
        uint32_t s, m;
        { const uint8_t* q = p + 4; const int j = 2 * g + hi;      // scale_min_k4, gguf_q.rs:62-64
          if (j < 4) { s = q[j] & 63; m = q[j + 4] & 63; }
          else { s = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); } }
        o.sa = o.sb = __fmul_rn(d, (float)s); o.ma = o.mb = __fmul_rn(mn, (float)m);
        const uint8_t* ql = p + 48 + 32 * g + l0;
        const uint8_t* qh = p + 16 + l0;
#pragma unroll
        for (int k = 0; k < 8; k++) o.w[k] = (float)((hi ? (ql[k] >> 4) : (ql[k] & 0xF)) + (((qh[k] >> (2 * g + hi)) & 1) << 4));
    }
};

// IQ1_M (gguf_q.rs:152-164): [qs 32][qh 16][scales 4 x u16]; per 8 weights an 11-bit grid index (8 bits in qs, 3 in a nibble of qh) into
// entries of eight values -1 / 0 / 1, the nibble's top bit the sign of a shift of 1/8; two 3-bit scales per 32 weights in the low twelve
// bits of the scale words, the block's f16 scale in their top nibbles.
template <> struct PbFmt<PB_T_IQ1_M> : PbContig8 {
    static constexpr int STEP_BYTES = 56;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables& T, PbUnit& o) {
        const uint16_t* scw = reinterpret_cast<const uint16_t*>(p + 48);
        const uint32_t s0 = scw[0], s1 = scw[1], s2 = scw[2], s3 = scw[3];
        const float d = pb_h2f((uint16_t)((s0 >> 12) | ((s1 >> 8) & 0x00f0) | ((s2 >> 4) & 0x0f00) | (s3 & 0xf000)));
        const int ib = u >> 2, l = u & 3;
        const uint32_t sw = scw[ib >> 1];
        o.sa = o.sb = __fmul_rn(d, (float)(2 * ((sw >> (6 * (ib & 1) + 3 * (l >> 1))) & 7) + 1));
        const uint32_t h = (uint32_t)p[32 + 2 * ib + (l >> 1)] >> (4 * (l & 1));
        const uint64_t g = T.iq1s[p[4 * ib + l] | ((h << 8) & 0x700)];
        const float delta = h & 8 ? -0.125f : 0.125f;
        o.ma = o.mb = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; j++) o.w[j] = __fadd_rn((float)(int8_t)(uint8_t)(g >> (8 * j)), delta);
    }
};

// Q6_K (gguf_q.rs:114-121): [ql 128][qh 64][scales 16 x i8][d f16]; per half of 128 weights, weight l + 32 g (g = 0..3) takes its
// low four bits from ql[l + 32 (g & 1)] (low nibble for g < 2, high nibble else), bits 4-5 from field g of qh[l], scale 2 g + l / 16
template <> struct PbFmt<PB_T_Q6_K> : PbContig8 {
    static constexpr int STEP_BYTES = 210;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const float d = pb_h2f((uint16_t)(p[208] | (p[209] << 8)));
        const int n = u >> 4, g = (u >> 2) & 3, l0 = 8 * (u & 3);
        const float sc = (float)(int8_t)p[192 + 8 * n + 2 * g + (l0 >> 4)];
        o.sa = o.sb = __fmul_rn(d, sc);
        o.ma = o.mb = 0.0f;
        const uint8_t* ql = p + 64 * n + 32 * (g & 1) + l0;
        const uint8_t* qh = p + 128 + 32 * n + l0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int lo = g < 2 ? (ql[j] & 0xF) : (ql[j] >> 4);
            o.w[j] = (float)((lo | (((qh[j] >> (2 * g)) & 3) << 4)) - 32);
        }
    }
};

template <> struct PbFmt<PB_T_Q8_0> : PbContig8 {
    static constexpr int STEP_BYTES = 8 * 34;  // eight [d f16][32 x i8] blocks
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const uint8_t* b = p + 34 * (u >> 2);
        o.sa = o.sb = pb_h2f(*reinterpret_cast<const uint16_t*>(b));
        o.ma = o.mb = 0.0f;
        const uint16_t* q = reinterpret_cast<const uint16_t*>(b + 2 + 8 * (u & 3));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t v = q[j];
            o.w[2 * j] = (float)(int8_t)(v & 0xFF);
            o.w[2 * j + 1] = (float)(int8_t)(v >> 8);
        }
    }
};

template <> struct PbFmt<PB_T_Q4_K> {
    static constexpr int STEP_BYTES = 144;  // [d f16][dmin f16][scales 12][qs 128]
    static constexpr bool HAS_MIN = true;
    // lane l = (group g = l / 8, quad i = l % 8): low nibbles of qs[32g + 4i .. +3] are weights
    // 64g + 4i + {0..3}, high nibbles are weights 64g + 32 + 4i + {0..3}
    __device__ static __forceinline__ int xa(int lane) { return 16 * (lane >> 3) + (lane & 7); }
    __device__ static __forceinline__ int xb(int lane) { return 16 * (lane >> 3) + 8 + (lane & 7); }
    __device__ static __forceinline__ int perm(int k) { int g = k >> 4, r = k & 15; return r < 8 ? 8 * g + r : 32 + 8 * g + (r - 8); }
    __device__ static __forceinline__ int pos(int lane, int j) { return 64 * (lane >> 3) + 4 * (lane & 7) + (j < 4 ? j : 32 + (j - 4)); }
    __device__ static __forceinline__ void scale_min(int j, const uint8_t* q, uint32_t& sc, uint32_t& m) {
        if (j < 4) { sc = q[j] & 63; m = q[j + 4] & 63; }
        else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
    }
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const float d = pb_h2f(*reinterpret_cast<const uint16_t*>(p));
        const float mn = pb_h2f(*reinterpret_cast<const uint16_t*>(p + 2));
        const int g = u >> 3, i = u & 7;
        uint32_t s1, m1, s2, m2;
        scale_min(2 * g, p + 4, s1, m1);
        scale_min(2 * g + 1, p + 4, s2, m2);
        o.sa = __fmul_rn(d, (float)s1); o.ma = __fmul_rn(mn, (float)m1);
        o.sb = __fmul_rn(d, (float)s2); o.mb = __fmul_rn(mn, (float)m2);
        const uint32_t q = *reinterpret_cast<const uint32_t*>(p + 16 + 32 * g + 4 * i);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            o.w[j] = (float)((q >> (8 * j)) & 0xF);
            o.w[4 + j] = (float)((q >> (8 * j + 4)) & 0xF);
        }
    }
};

// Unquantized storage (router weights, hyper-connection matrices): same unit interface.
template <> struct PbFmt<PB_T_F32> : PbContig8 {
    static constexpr int STEP_BYTES = 1024;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const float4 a = *reinterpret_cast<const float4*>(p + 32 * u), b = *reinterpret_cast<const float4*>(p + 32 * u + 16);
        o.w[0] = a.x; o.w[1] = a.y; o.w[2] = a.z; o.w[3] = a.w; o.w[4] = b.x; o.w[5] = b.y; o.w[6] = b.z; o.w[7] = b.w;
        o.sa = o.sb = 1.0f; o.ma = o.mb = 0.0f;
    }
};
template <> struct PbFmt<PB_T_F16> : PbContig8 {
    static constexpr int STEP_BYTES = 512;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const uint4 a = *reinterpret_cast<const uint4*>(p + 16 * u);
        const uint32_t v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; j++) { o.w[2 * j] = pb_h2f((uint16_t)(v[j] & 0xFFFF)); o.w[2 * j + 1] = pb_h2f((uint16_t)(v[j] >> 16)); }
        o.sa = o.sb = 1.0f; o.ma = o.mb = 0.0f;
    }
};
template <> struct PbFmt<PB_T_BF16> : PbContig8 {
    static constexpr int STEP_BYTES = 512;
    static constexpr bool HAS_MIN = false;
    __device__ static __forceinline__ void unit(const uint8_t* p, int u, const PbTables&, PbUnit& o) {
        const uint4 a = *reinterpret_cast<const uint4*>(p + 16 * u);
        const uint32_t v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; j++) { o.w[2 * j] = __uint_as_float(v[j] << 16); o.w[2 * j + 1] = __uint_as_float(v[j] & 0xFFFF0000u); }
        o.sa = o.sb = 1.0f; o.ma = o.mb = 0.0f;
    }
};

// Host-side geometry (QType::geom, gguf_q.rs:33-41).
static inline int pb_geom(int type, int* elems, int* bytes) {
    int e, b;
    switch (type) {
        case PB_T_F32: e = 1; b = 4; break;
        case PB_T_F16: case PB_T_BF16: e = 1; b = 2; break;
        case PB_T_Q8_0: e = 32; b = 34; break;
        case PB_T_Q4_K: e = 256; b = 144; break;
        case PB_T_IQ2_XS: e = 256; b = 74; break;
        case PB_T_IQ3_S: e = 256; b = 110; break;
        case PB_T_IQ3_XXS: e = 256; b = 98; break;
        case PB_T_IQ2_S: e = 256; b = 82; break;
        case PB_T_IQ4_NL: e = 32; b = 18; break;
        case PB_T_IQ4_XS: e = 256; b = 136; break;
        case PB_T_Q2_0: e = 64; b = 18; break;
        case PB_T_IQ2_XXS: e = 256; b = 66; break;
        case PB_T_Q6_K: e = 256; b = 210; break;
        case PB_T_IQ1_M: e = 256; b = 56; break;
        case PB_T_Q4_0: e = 32; b = 18; break;
        case PB_T_Q5_0: e = 32; b = 22; break;
        case PB_T_Q3_K: e = 256; b = 110; break;
        case PB_T_Q5_K: e = 256; b = 176; break;
        case PB_T_IQ3S_N4: e = 256; b = 136; break;
        default: return -1;
    }
    if (elems) *elems = e;
    if (bytes) *bytes = b;
    return 0;
}

// Dispatch a templated callable on the runtime type id.
#define PB_DISPATCH_FMT(type, F, ...)                                  \
    switch (type) {                                                    \
        case PB_T_IQ3_S: { constexpr int FMT = PB_T_IQ3_S; F(__VA_ARGS__); } break;  \
        case PB_T_IQ2_XS: { constexpr int FMT = PB_T_IQ2_XS; F(__VA_ARGS__); } break; \
        case PB_T_IQ3_XXS: { constexpr int FMT = PB_T_IQ3_XXS; F(__VA_ARGS__); } break; \
        case PB_T_IQ2_S: { constexpr int FMT = PB_T_IQ2_S; F(__VA_ARGS__); } break; \
        case PB_T_IQ4_NL: { constexpr int FMT = PB_T_IQ4_NL; F(__VA_ARGS__); } break; \
        case PB_T_IQ4_XS: { constexpr int FMT = PB_T_IQ4_XS; F(__VA_ARGS__); } break; \
        case PB_T_Q2_0: { constexpr int FMT = PB_T_Q2_0; F(__VA_ARGS__); } break; \
        case PB_T_IQ2_XXS: { constexpr int FMT = PB_T_IQ2_XXS; F(__VA_ARGS__); } break; \
        case PB_T_Q6_K: { constexpr int FMT = PB_T_Q6_K; F(__VA_ARGS__); } break; \
        case PB_T_IQ1_M: { constexpr int FMT = PB_T_IQ1_M; F(__VA_ARGS__); } break; \
        case PB_T_Q4_0: { constexpr int FMT = PB_T_Q4_0; F(__VA_ARGS__); } break; \
        case PB_T_Q5_0: { constexpr int FMT = PB_T_Q5_0; F(__VA_ARGS__); } break; \
        case PB_T_Q3_K: { constexpr int FMT = PB_T_Q3_K; F(__VA_ARGS__); } break; \
        case PB_T_Q5_K: { constexpr int FMT = PB_T_Q5_K; F(__VA_ARGS__); } break; \
        case PB_T_Q4_K: { constexpr int FMT = PB_T_Q4_K; F(__VA_ARGS__); } break;    \
        case PB_T_Q8_0: { constexpr int FMT = PB_T_Q8_0; F(__VA_ARGS__); } break;    \
        case PB_T_F32: { constexpr int FMT = PB_T_F32; F(__VA_ARGS__); } break;      \
        case PB_T_F16: { constexpr int FMT = PB_T_F16; F(__VA_ARGS__); } break;      \
        case PB_T_BF16: { constexpr int FMT = PB_T_BF16; F(__VA_ARGS__); } break;    \
        default: break;                                                \
    }
