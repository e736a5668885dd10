// Integer dot-product core of the dequant-GEMV kernels.
//
// A lane owns a quarter of a 256-weight super-step (64 consecutive weights).  It decodes
// them to 16 words of packed signed int8 (grid values with their signs, raw int8 for
// Q8_0, nibbles for Q4_K) plus f32 scales per 16 weights, and dots them with dp4a against
// activations that were split, per 32-value group, into PB_XLEVELS int8 levels:
//     x = s1*q1 + s2*q2 + s3*q3 + e,   |e| <= max|x| / (2 * 254^3)
// Integer partial sums are exact; each group contributes one f32 FMA per level.  The split
// keeps the result within f32 rounding noise of an f32-accumulated dot (the parity
// tolerance is 1e-3), and turns byte->float conversion, sign handling and 8 FMAs per 8
// weights into SWAR sign operations and PB_XLEVELS dp4a per 4 weights.  IQ3_S, the format of the
// model, has its own index / sign arithmetic (pb_iq3s_index, pb_iq3s_sign) and a fused decode + dot
// for one column (pb_iq3s_quarter_dot).
//
// All block bytes and tables are read from shared memory through 32-bit shared-space
// addresses (ld.shared), never through generic pointers.
//
// Block layouts restate src/model/gguf_q.rs:67-166 of the reference (see pb_formats.cuh).
#pragma once
#include "pb_formats.cuh"

__device__ __forceinline__ uint32_t pb_lds8(uint32_t a) { uint32_t v; asm("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t pb_lds16(uint32_t a) { uint32_t v; asm("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t pb_lds32(uint32_t a) { uint32_t v; asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint2 pb_lds64(uint32_t a) { uint2 v; asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v; }
__device__ __forceinline__ uint4 pb_lds128(uint32_t a) { uint4 v; asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a)); return v; }

// Shared-memory tables used by the decoders (shared-space byte addresses).
struct PbQTabs {
    uint32_t grid;      // codebook, already offset to this lane's copy; entry i at grid + i * stride
    uint32_t stride;    // bytes between consecutive entries (entry size * replication)
    uint32_t sign256;   // 256 x 16 B: sign byte -> (mask_lo, mask_lo & 0x01010101, mask_hi, mask_hi & 0x01010101)
};
#define PB_SIGN_LUT_BYTES 4096

// load N32 consecutive u32 from a 2-byte-aligned shared-memory address
template <int N32>
__device__ __forceinline__ void pb_ld_u32x(uint32_t p, uint32_t (&out)[N32]) {
    const uint32_t sh = (p & 2u) * 8u;          // 0 or 16 bits
    const uint32_t a = p & ~3u;
    uint32_t w[N32 + 1];
#pragma unroll
    for (int i = 0; i <= N32; i++) w[i] = pb_lds32(a + 4 * i);
#pragma unroll
    for (int i = 0; i < N32; i++) out[i] = __funnelshift_r(w[i], w[i + 1], sh);
}

// (g ^ M) + C : negate the bytes of g selected by the byte mask M (all bytes of g are <= 127)
__device__ __forceinline__ int pb_apply_sign(uint32_t g, uint32_t m, uint32_t c) { return (int)((g ^ m) + c); }

__device__ __forceinline__ uint32_t pb_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d; asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel)); return d;
}
// bit k of the nibble n -> byte k (0 or 1)
__device__ __forceinline__ uint32_t pb_spread4(uint32_t n) { return (n * 0x00204081u) & 0x01010101u; }
// IQ3_S: index of entry J of a group of four = qs byte J | high bit << 8.  hbytes = pb_spread4 of the
// group's four high bits; prmt zero-fills the upper bytes through its sign-replication mode.
template <int J> __device__ __forceinline__ uint32_t pb_iq3s_index(uint32_t qs_word, uint32_t hbytes) {
    constexpr uint32_t sel = (uint32_t)(((12 + J) << 12) | ((12 + J) << 8) | ((4 + J) << 4) | J);
    return pb_prmt(qs_word, hbytes, sel);
}
// IQ3_S grid values are odd (1, 3, .. 15), so xor with 0xFE negates a byte: -g = g ^ 0xFE.
// c = pb_spread4 of the entry's four sign bits.
__device__ __forceinline__ int pb_iq3s_sign(uint32_t g, uint32_t c) { return (int)(g ^ (c * 254u)); }
// The same from the packed sign bits: entry J (0..7) of a 32-weight half takes bits 4J..4J+3 of `sg`.
// n * 0x10204080 puts bit k of the nibble n at bit 8k + 7 (no two partial products meet, so no carries);
// prmt in sign-replication mode turns those into bytes 0x00 / 0xFF; one logic op then flips bits 1..7
// of the selected bytes.  Odd entries keep their nibble in place (n << 4) and multiply by the constant
// shifted down by 4, which saves the shift.
template <int J> __device__ __forceinline__ int pb_iq3s_sign8(uint32_t g, uint32_t sg) {
    const uint32_t t = (J >> 1) ? sg >> (8 * (J >> 1)) : sg;
    const uint32_t m = (J & 1) ? (t & 0xF0u) * 0x01020408u : (t & 0xFu) * 0x10204080u;
    return (int)(g ^ (pb_prmt(m, 0u, 0xBA98u) & 0xFEFEFEFEu));
}

struct PbQuarter {
    int w[16];      // packed signed int8, weight 4k+j of the quarter in byte j of w[k]
    float sc[4];    // scale of weights 16h .. 16h+15
    float mn[2];    // Q4_K only: offset of weights 32g .. 32g+31
};

template <int FMT> struct PbQDec;

template <> struct PbQDec<PB_T_IQ3_S> {
    static constexpr int STEP_BYTES = 110;
    static constexpr bool HAS_MIN = false, SCALE16 = false, AFFINE = false;
    // p = shared address of the 110-byte block, qt = quarter 0..3
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs& T, PbQuarter& o) {
        const float d = pb_h2f((uint16_t)pb_lds16(p));
        uint32_t qs[4], sg[2];
        pb_ld_u32x<4>(p + 2 + 16 * qt, qs);
        pb_ld_u32x<2>(p + 74 + 8 * qt, sg);
        const uint32_t qh = pb_lds16(p + 66 + 2 * qt);
        const uint32_t sc = pb_lds8(p + 106 + qt);
        const float d0 = d * (float)(1 + 2 * (int)(sc & 0xF)), d1 = d * (float)(1 + 2 * (int)(sc >> 4));
        o.sc[0] = o.sc[1] = d0; o.sc[2] = o.sc[3] = d1;
#pragma unroll
        for (int k = 0; k < 4; k++) {          // four entries: one qs word, four high bits, two sign bytes
            const uint32_t hb = pb_spread4((qh >> (4 * k)) & 0xF);
            const uint32_t sw = sg[k >> 1];
            const uint32_t g0 = pb_lds32(T.grid + pb_iq3s_index<0>(qs[k], hb) * T.stride), g1 = pb_lds32(T.grid + pb_iq3s_index<1>(qs[k], hb) * T.stride);
            const uint32_t g2 = pb_lds32(T.grid + pb_iq3s_index<2>(qs[k], hb) * T.stride), g3 = pb_lds32(T.grid + pb_iq3s_index<3>(qs[k], hb) * T.stride);
            o.w[4 * k + 0] = (k & 1) ? pb_iq3s_sign8<4>(g0, sw) : pb_iq3s_sign8<0>(g0, sw);
            o.w[4 * k + 1] = (k & 1) ? pb_iq3s_sign8<5>(g1, sw) : pb_iq3s_sign8<1>(g1, sw);
            o.w[4 * k + 2] = (k & 1) ? pb_iq3s_sign8<6>(g2, sw) : pb_iq3s_sign8<2>(g2, sw);
            o.w[4 * k + 3] = (k & 1) ? pb_iq3s_sign8<7>(g3, sw) : pb_iq3s_sign8<3>(g3, sw);
        }
    }
};

template <> struct PbQDec<PB_T_IQ2_XS> {
    static constexpr int STEP_BYTES = 74;
    static constexpr bool HAS_MIN = false, SCALE16 = true, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs& T, PbQuarter& o) {
        const float d = pb_h2f((uint16_t)pb_lds16(p));
        uint32_t qs[4];
        pb_ld_u32x<4>(p + 2 + 16 * qt, qs);
        const uint32_t sc = pb_lds16(p + 66 + 2 * qt);
#pragma unroll
        for (int h = 0; h < 4; h++) o.sc[h] = d * (0.5f + (float)((sc >> (4 * h)) & 0xF)) * 0.25f;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const uint32_t q = (qs[u >> 1] >> (16 * (u & 1))) & 0xFFFF;
            const uint2 g = pb_lds64(T.grid + (q & 511) * T.stride);
            const uint32_t s7 = q >> 9;
            const uint32_t s8 = s7 | ((__popc(s7) & 1) << 7);   // KSIGNS_IQ2XS[i] = i | parity(i) << 7
            const uint4 m = pb_lds128(T.sign256 + s8 * 16);
            o.w[2 * u] = pb_apply_sign(g.x, m.x, m.y);
            o.w[2 * u + 1] = pb_apply_sign(g.y, m.z, m.w);
        }
    }
};

template <> struct PbQDec<PB_T_Q8_0> {
    static constexpr int STEP_BYTES = 8 * 34;
    static constexpr bool HAS_MIN = false, SCALE16 = false, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const uint32_t blk = p + 34 * (2 * qt + b);
            const float d = pb_h2f((uint16_t)pb_lds16(blk));
            o.sc[2 * b] = o.sc[2 * b + 1] = d;
            uint32_t q[8];
            pb_ld_u32x<8>(blk + 2, q);
#pragma unroll
            for (int k = 0; k < 8; k++) o.w[8 * b + k] = (int)q[k];
        }
    }
};

template <> struct PbQDec<PB_T_Q4_K> {
    static constexpr int STEP_BYTES = 144;
    static constexpr bool HAS_MIN = true, SCALE16 = false, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
        const uint4 hdr = pb_lds128(p);            // d, dmin, 12 scale bytes
        const float d = pb_h2f((uint16_t)(hdr.x & 0xFFFF)), mn = pb_h2f((uint16_t)(hdr.x >> 16));
        const uint32_t scw[3] = {hdr.y, hdr.z, hdr.w};
        auto sb = [&](int i) -> uint32_t { return (scw[i >> 2] >> (8 * (i & 3))) & 0xFF; };
        uint32_t s[2], m[2];
#pragma unroll
        for (int e = 0; e < 2; e++) {              // scale_min_k4, gguf_q.rs:62-64
            const int j = 2 * qt + e;
            if (j < 4) { s[e] = sb(j) & 63; m[e] = sb(j + 4) & 63; }
            else { s[e] = (sb(j + 4) & 0xF) | ((sb(j - 4) >> 6) << 4); m[e] = (sb(j + 4) >> 4) | ((sb(j) >> 6) << 4); }
        }
        o.sc[0] = o.sc[1] = d * (float)s[0]; o.sc[2] = o.sc[3] = d * (float)s[1];
        o.mn[0] = mn * (float)m[0]; o.mn[1] = mn * (float)m[1];
        const uint4 a = pb_lds128(p + 16 + 32 * qt), b = pb_lds128(p + 32 + 32 * qt);
        const uint32_t q[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 8; k++) { o.w[k] = (int)(q[k] & 0x0F0F0F0Fu); o.w[8 + k] = (int)((q[k] >> 4) & 0x0F0F0F0Fu); }
    }
};

// IQ3_S re-coded into 4-bit codes c (weight = 2 c - 15): the quarter holds the codes, unsigned, and
// pb_quarter_dot removes the offset with the integer sums of the activation levels:
// sum (2 c - 15) q = 2 sum c q - 15 sum q, exact in integers.
template <> struct PbQDec<PB_T_IQ3S_N4> {
    static constexpr int STEP_BYTES = 136;
    static constexpr bool HAS_MIN = false, SCALE16 = false, AFFINE = true;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
        const uint32_t hdr = pb_lds32(p);
        const float d = pb_h2f((uint16_t)(hdr & 0xFFFF));
        const uint32_t sc = pb_lds8(p + 4 + qt);
        const float d0 = d * (float)(1 + 2 * (int)(sc & 0xF)), d1 = d * (float)(1 + 2 * (int)(sc >> 4));
        o.sc[0] = o.sc[1] = d0; o.sc[2] = o.sc[3] = d1;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint2 c = pb_lds64(p + 8 + 32 * qt + 8 * i);
            o.w[4 * i + 0] = (int)(c.x & 0x0F0F0F0Fu); o.w[4 * i + 1] = (int)((c.x >> 4) & 0x0F0F0F0Fu);
            o.w[4 * i + 2] = (int)(c.y & 0x0F0F0F0Fu); o.w[4 * i + 3] = (int)((c.y >> 4) & 0x0F0F0F0Fu);
        }
    }
};

// ---- IQ3_XXS: per 32 weights eight 8-bit grid indices (entries of four magnitudes) and one u32 with four 7-bit sign
// patterns and a 4-bit scale (gguf_q.rs:136-140).  Grid entries from shared memory (256 x 4 bytes), signs through the
// 256-entry mask table after the parity bit is restored, as IQ2_XS.
template <> struct PbQDec<PB_T_IQ3_XXS> {
    static constexpr int STEP_BYTES = 98;
    static constexpr bool HAS_MIN = false, SCALE16 = false, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs& T, PbQuarter& o) {
        const float d = pb_h2f((uint16_t)pb_lds16(p));
        uint32_t qs[4], aux[2];
        pb_ld_u32x<4>(p + 2 + 16 * qt, qs);
        pb_ld_u32x<2>(p + 66 + 8 * qt, aux);
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const float db = d * (0.5f + (float)(aux[b] >> 28)) * 0.5f;
            o.sc[2 * b] = o.sc[2 * b + 1] = db;
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint32_t two = (qs[2 * b + (l >> 1)] >> (16 * (l & 1))) & 0xFFFF;
                const uint32_t g1 = pb_lds32(T.grid + (two & 0xFF) * T.stride), g2 = pb_lds32(T.grid + (two >> 8) * T.stride);
                const uint32_t s7 = (aux[b] >> (7 * l)) & 127;
                const uint32_t s8 = s7 | ((__popc(s7) & 1) << 7);
                const uint4 m = pb_lds128(T.sign256 + s8 * 16);
                o.w[8 * b + 2 * l] = pb_apply_sign(g1, m.x, m.y);
                o.w[8 * b + 2 * l + 1] = pb_apply_sign(g2, m.z, m.w);
            }
        }
    }
};

// ---- IQ2_S: per 8 weights a 10-bit grid index (8 bits in qs, 2 in qh) and an explicit sign byte; a 4-bit scale per 16
// weights (gguf_q.rs:130-135).  Grid entries from shared memory (1024 x 8 bytes).
template <> struct PbQDec<PB_T_IQ2_S> {
    static constexpr int STEP_BYTES = 82;
    static constexpr bool HAS_MIN = false, SCALE16 = true, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs& T, PbQuarter& o) {
        const float d = pb_h2f((uint16_t)pb_lds16(p));
        uint32_t qs[2], sg[2];
        pb_ld_u32x<2>(p + 2 + 8 * qt, qs);
        pb_ld_u32x<2>(p + 34 + 8 * qt, sg);
        const uint32_t qh = pb_lds16(p + 66 + 2 * qt), sc = pb_lds16(p + 74 + 2 * qt);
#pragma unroll
        for (int h = 0; h < 4; h++) o.sc[h] = d * (0.5f + (float)((sc >> (4 * h)) & 0xF)) * 0.25f;
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const uint32_t hb = (qh >> (8 * b)) & 0xFF;
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint32_t idx = ((qs[b] >> (8 * l)) & 0xFF) | ((hb << (8 - 2 * l)) & 0x300);
                const uint2 g = pb_lds64(T.grid + idx * T.stride);
                const uint4 m = pb_lds128(T.sign256 + ((sg[b] >> (8 * l)) & 0xFF) * 16);
                o.w[8 * b + 2 * l] = pb_apply_sign(g.x, m.x, m.y);
                o.w[8 * b + 2 * l + 1] = pb_apply_sign(g.y, m.z, m.w);
            }
        }
    }
};

// ---- IQ4_NL / IQ4_XS: 4-bit codes into a table of 16 signed values (kvalues_iq4nl).  Sixteen bytes hold 32 weights:
// weight j < 16 is the low nibble of byte j, weight 16 + j the high one.  The table lives in four registers; prmt looks four
// codes up at once: its selector takes one nibble per output byte, and a 16-bit piece of the data IS four nibbles (low and
// high nibble of two bytes), so  prmt(table 0..7, piece & 0x7777)  and  prmt(table 8..15, piece & 0x7777)  give the
// values for both halves of the table, bit 3 of every nibble picks between them, and two more prmt put the low-nibble
// and the high-nibble weights of four bytes into their words.
__device__ __forceinline__ uint32_t pb_iq4_lut4(uint32_t piece) {
    constexpr uint32_t K0 = 0xBFAD9881u, K1 = 0xF6EADDCFu, K2 = 0x26190D01u, K3 = 0x71594535u;   // -127 -104 -83 -65 | -49 -35 -22 -10 | 1 13 25 38 | 53 69 89 113
    const uint32_t sel = piece & 0x7777u;
    const uint32_t v0 = pb_prmt(K0, K1, sel), v1 = pb_prmt(K2, K3, sel);
    const uint32_t mask = pb_prmt(0x0000FF00u, 0u, (piece >> 3) & 0x1111u);
    return (v0 & ~mask) | (v1 & mask);
}
// 16 bytes of codes (four words) -> weights 0..15 in lo[0..3], weights 16..31 in hi[0..3]
__device__ __forceinline__ void pb_iq4_block(const uint32_t (&q)[4], int* lo, int* hi) {
#pragma unroll
    for (int m = 0; m < 4; m++) {
        const uint32_t ra = pb_iq4_lut4(q[m] & 0xFFFFu), rb = pb_iq4_lut4(q[m] >> 16);   // [w j, w j+16, w j+1, w j+17] for bytes (4m, 4m+1) and (4m+2, 4m+3)
        lo[m] = (int)pb_prmt(ra, rb, 0x6420u);
        hi[m] = (int)pb_prmt(ra, rb, 0x7531u);
    }
}
template <> struct PbQDec<PB_T_IQ4_NL> {
    static constexpr int STEP_BYTES = 8 * 18;
    static constexpr bool HAS_MIN = false, SCALE16 = false, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const uint32_t blk = p + 18 * (2 * qt + b);
            o.sc[2 * b] = o.sc[2 * b + 1] = pb_h2f((uint16_t)pb_lds16(blk));
            uint32_t q[4];
            pb_ld_u32x<4>(blk + 2, q);
            pb_iq4_block(q, o.w + 8 * b, o.w + 8 * b + 4);
        }
    }
};
template <> struct PbQDec<PB_T_IQ4_XS> {
    static constexpr int STEP_BYTES = 136;   // [d f16][scales_h u16][scales_l 4][qs 128] (gguf_q.rs:84-89)
    static constexpr bool HAS_MIN = false, SCALE16 = false, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
        const uint2 hdr = pb_lds64(p);
        const float d = pb_h2f((uint16_t)(hdr.x & 0xFFFF));
        const uint32_t sh = hdr.x >> 16, sl = hdr.y;
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const int ib = 2 * qt + b;
            const int ls = (int)((sl >> (4 * ib)) & 0xF) | (int)(((sh >> (2 * ib)) & 3) << 4);
            o.sc[2 * b] = o.sc[2 * b + 1] = d * (float)(ls - 32);
            // blocks are 136 bytes: the codes of a sub-block start on an 8-byte boundary, on a 16-byte one only in every other block
            const uint2 v0 = pb_lds64(p + 8 + 16 * ib), v1 = pb_lds64(p + 16 + 16 * ib);
            const uint32_t q[4] = {v0.x, v0.y, v1.x, v1.y};
            pb_iq4_block(q, o.w + 8 * b, o.w + 8 * b + 4);
        }
    }
};

// ---- IQ2_XXS: per 32 weights four 8-bit grid indices (entries of eight magnitudes) and one u32 with four 7-bit sign patterns and
// a 4-bit scale (gguf_q.rs:122-125).  Grid entries from shared memory (256 x 8 bytes), signs as IQ3_XXS.
template <> struct PbQDec<PB_T_IQ2_XXS> {
    static constexpr int STEP_BYTES = 66;
    static constexpr bool HAS_MIN = false, SCALE16 = false, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs& T, PbQuarter& o) {
        const float d = pb_h2f((uint16_t)pb_lds16(p));
        uint32_t q[4];                               // [indices, signs and scale] of the quarter's two sub-blocks
        pb_ld_u32x<4>(p + 2 + 16 * qt, q);
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const uint32_t idx = q[2 * b], aux = q[2 * b + 1];
            const float db = d * (0.5f + (float)(aux >> 28)) * 0.25f;
            o.sc[2 * b] = o.sc[2 * b + 1] = db;
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint2 g = pb_lds64(T.grid + ((idx >> (8 * l)) & 0xFF) * T.stride);
                const uint32_t s7 = (aux >> (7 * l)) & 127;
                const uint32_t s8 = s7 | ((__popc(s7) & 1) << 7);
                const uint4 m = pb_lds128(T.sign256 + s8 * 16);
                o.w[8 * b + 2 * l] = pb_apply_sign(g.x, m.x, m.y);
                o.w[8 * b + 2 * l + 1] = pb_apply_sign(g.y, m.z, m.w);
            }
        }
    }
};

// ---- Q4_0 / Q5_0: sixteen bytes hold 32 weights (low nibbles, then high nibbles), Q5_0 with a fifth bit per weight from a 32-bit word;
// the offset (8 or 16) is taken off per byte with bit 7 set so that no borrow crosses.
template <> struct PbQDec<PB_T_Q4_0> {
    static constexpr int STEP_BYTES = 8 * 18;
    static constexpr bool HAS_MIN = false, SCALE16 = false, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const uint32_t blk = p + 18 * (2 * qt + b);
            o.sc[2 * b] = o.sc[2 * b + 1] = pb_h2f((uint16_t)pb_lds16(blk));
            uint32_t q[4];
            pb_ld_u32x<4>(blk + 2, q);
#pragma unroll
            for (int m = 0; m < 4; m++) {
                o.w[8 * b + m] = (int)((((q[m] & 0x0F0F0F0Fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u);
                o.w[8 * b + 4 + m] = (int)(((((q[m] >> 4) & 0x0F0F0F0Fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u);
            }
        }
    }
};
template <> struct PbQDec<PB_T_Q5_0> {
    static constexpr int STEP_BYTES = 8 * 22;
    static constexpr bool HAS_MIN = false, SCALE16 = false, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const uint32_t blk = p + 22 * (2 * qt + b);
            o.sc[2 * b] = o.sc[2 * b + 1] = pb_h2f((uint16_t)pb_lds16(blk));
            uint32_t q[5];                              // [qh, 16 bytes of nibbles]
            pb_ld_u32x<5>(blk + 2, q);
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const uint32_t lo = (q[1 + m] & 0x0F0F0F0Fu) | (pb_spread4((q[0] >> (4 * m)) & 0xFu) << 4);
                const uint32_t hi = ((q[1 + m] >> 4) & 0x0F0F0F0Fu) | (pb_spread4((q[0] >> (16 + 4 * m)) & 0xFu) << 4);
                o.w[8 * b + m] = (int)(((lo | 0x80808080u) - 0x10101010u) ^ 0x80808080u);
                o.w[8 * b + 4 + m] = (int)(((hi | 0x80808080u) - 0x10101010u) ^ 0x80808080u);
            }
        }
    }
};

// ---- Q3_K: a quarter is the two-bit planes j = 2 (qt & 1) and the next of half n = qt / 2: both read the 32 qs bytes of the half and the
// 32 hmask bytes; value = two bits + 4 * mask bit - 4.  The four scales of the quarter are the bytes of one word of the unpacked scales.
template <> struct PbQDec<PB_T_Q3_K> {
    static constexpr int STEP_BYTES = 110;
    static constexpr bool HAS_MIN = false, SCALE16 = true, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
        const float d = pb_h2f((uint16_t)pb_lds16(p + 108));
        const int n = qt >> 1, side = qt & 1;
        uint32_t hm[8], qs[8], a[3];
        pb_ld_u32x<8>(p, hm);
        pb_ld_u32x<8>(p + 32 + 32 * n, qs);
        pb_ld_u32x<3>(p + 96, a);
        const uint32_t aux = (((side ? a[1] : a[0]) >> (4 * n)) & 0x0F0F0F0Fu) | (((a[2] >> (2 * qt)) & 0x03030303u) << 4);
#pragma unroll
        for (int h = 0; h < 4; h++) o.sc[h] = d * (float)((int)((aux >> (8 * h)) & 0xFF) - 32);
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const int j = 2 * side + b;
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const uint32_t v = ((qs[k] >> (2 * j)) & 0x03030303u) | (((hm[k] >> (4 * n + j)) & 0x01010101u) << 2);
                o.w[8 * b + k] = (int)(((v | 0x80808080u) - 0x04040404u) ^ 0x80808080u);
            }
        }
    }
};

// ---- Q5_K: Q4_K's nibbles (at byte 48) with bits 2 qt and 2 qt + 1 of the 32 qh bytes (at byte 16) as the fifth bit; blocks of 176 bytes
// keep every field 16-byte aligned.
template <> struct PbQDec<PB_T_Q5_K> {
    static constexpr int STEP_BYTES = 176;
    static constexpr bool HAS_MIN = true, SCALE16 = false, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
        const uint4 hdr = pb_lds128(p);            // d, dmin, 12 scale bytes
        const float d = pb_h2f((uint16_t)(hdr.x & 0xFFFF)), mn = pb_h2f((uint16_t)(hdr.x >> 16));
        const uint32_t scw[3] = {hdr.y, hdr.z, hdr.w};
        auto sb = [&](int i) -> uint32_t { return (scw[i >> 2] >> (8 * (i & 3))) & 0xFF; };
        uint32_t s[2], m[2];
#pragma unroll
        for (int e = 0; e < 2; e++) {              // scale_min_k4, gguf_q.rs:62-64
            const int j = 2 * qt + e;
            if (j < 4) { s[e] = sb(j) & 63; m[e] = sb(j + 4) & 63; }
            else { s[e] = (sb(j + 4) & 0xF) | ((sb(j - 4) >> 6) << 4); m[e] = (sb(j + 4) >> 4) | ((sb(j) >> 6) << 4); }
        }
        o.sc[0] = o.sc[1] = d * (float)s[0]; o.sc[2] = o.sc[3] = d * (float)s[1];
        o.mn[0] = mn * (float)m[0]; o.mn[1] = mn * (float)m[1];
        const uint4 a = pb_lds128(p + 48 + 32 * qt), b = pb_lds128(p + 64 + 32 * qt), ha = pb_lds128(p + 16), hb = pb_lds128(p + 32);
        const uint32_t q[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w}, h[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
#pragma unroll
        for (int k = 0; k < 8; k++) {
            o.w[k] = (int)((q[k] & 0x0F0F0F0Fu) | (((h[k] >> (2 * qt)) & 0x01010101u) << 4));
            o.w[8 + k] = (int)(((q[k] >> 4) & 0x0F0F0F0Fu) | (((h[k] >> (2 * qt + 1)) & 0x01010101u) << 4));
        }
    }
};

// ---- IQ1_M: weights are s * (g + delta) with g in -1 / 0 / 1 and delta = +-1/8, i.e. (s / 8) * (8 g +- 1) with an int8 in the bracket.
// The shared-memory table holds those eight int8 per (sign, 11-bit index), so a look-up is the whole decode; scales per 16 weights.
template <> struct PbQDec<PB_T_IQ1_M> {
    static constexpr int STEP_BYTES = 56;    // blocks of 56 bytes keep every field below 8-byte aligned
    static constexpr bool HAS_MIN = false, SCALE16 = true, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs& T, PbQuarter& o) {
        const uint2 scw = pb_lds64(p + 48);
        const uint32_t su = ((scw.x >> 12) & 0xF) | ((scw.x >> 24) & 0xF0) | ((scw.y >> 4) & 0xF00) | ((scw.y >> 16) & 0xF000);
        const float d8 = pb_h2f((uint16_t)su) * 0.125f;
        const uint32_t sw = (qt & 2 ? scw.y : scw.x) >> (16 * (qt & 1));      // scale word qt: sub-blocks 2 qt and 2 qt + 1
#pragma unroll
        for (int h = 0; h < 4; h++) o.sc[h] = d8 * (float)(2 * ((sw >> (3 * h)) & 7) + 1);
        const uint2 qs = pb_lds64(p + 8 * qt);
        const uint32_t qh = pb_lds32(p + 32 + 4 * qt);
#pragma unroll
        for (int l = 0; l < 8; l++) {
            const uint32_t b = ((l < 4 ? qs.x : qs.y) >> (8 * (l & 3))) & 0xFF;
            const uint32_t h = (qh >> (4 * l)) & 0xF;                          // three index bits and the sign, together the table's high bits
            const uint2 g = pb_lds64(T.grid + (b | (h << 8)) * T.stride);
            o.w[2 * l] = (int)g.x; o.w[2 * l + 1] = (int)g.y;
        }
    }
};

// ---- Q2_0: blocks of 64 weights = [d f16][16 bytes], weight 4k + j in field j (two bits) of byte k, value field - 1.  A quarter is
// one block.  x * 0x1001 puts fields 0 and 2 of a byte at bits 0 and 16, (x >> 2) * 0x100100 fields 1 and 3 at bits 8 and 24
// (the partial products of an 8-bit x do not meet); the subtraction of 1 per byte runs with bit 7 set so that no borrow crosses.
template <> struct PbQDec<PB_T_Q2_0> {
    static constexpr int STEP_BYTES = 4 * 18;
    static constexpr bool HAS_MIN = false, SCALE16 = false, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
        const uint32_t blk = p + 18 * qt;
        const float d = pb_h2f((uint16_t)pb_lds16(blk));
        o.sc[0] = o.sc[1] = o.sc[2] = o.sc[3] = d;
        uint32_t q[4];
        pb_ld_u32x<4>(blk + 2, q);
#pragma unroll
        for (int m = 0; m < 4; m++) {
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const uint32_t x = (q[m] >> (8 * b)) & 0xFF;
                const uint32_t f = ((x * 0x1001u) & 0x00030003u) | (((x >> 2) * 0x100100u) & 0x03000300u);
                o.w[4 * m + b] = (int)((((f | 0x80808080u) - 0x01010101u)) ^ 0x80808080u);
            }
        }
    }
};

// ---- Q6_K: [ql 128][qh 64][16 x i8 scales][d f16] (gguf_q.rs:114-121).  Per half of 128 weights, weight l + 32 g takes four bits
// from ql[l + 32 (g & 1)] (low nibbles for g < 2) and two from field g of qh[l]; a quarter is groups g = 2 (qt & 1) and the next of half
// qt / 2, so both groups read the same nibble side of 64 ql bytes and two fields of the same 32 qh bytes.  value = six bits - 32.
template <> struct PbQDec<PB_T_Q6_K> {
    static constexpr int STEP_BYTES = 210;
    static constexpr bool HAS_MIN = false, SCALE16 = true, AFFINE = false;
    __device__ static __forceinline__ void quarter(uint32_t p, int qt, const PbQTabs&, PbQuarter& o) {
        const float d = pb_h2f((uint16_t)pb_lds16(p + 208));
        const int n = qt >> 1, side = qt & 1;
        uint32_t ql[16], qh[8], sc[1];
        pb_ld_u32x<16>(p + 64 * n, ql);
        pb_ld_u32x<8>(p + 128 + 32 * n, qh);
        pb_ld_u32x<1>(p + 192 + 8 * n + 4 * side, sc);
#pragma unroll
        for (int h = 0; h < 4; h++) o.sc[h] = d * (float)(int)(int8_t)((sc[0] >> (8 * h)) & 0xFF);
#pragma unroll
        for (int b = 0; b < 2; b++) {
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const uint32_t lo = (side ? ql[8 * b + k] >> 4 : ql[8 * b + k]) & 0x0F0F0F0Fu;
                const uint32_t hi = ((qh[k] >> (4 * side + 2 * b)) & 0x03030303u) << 4;
                o.w[8 * b + k] = (int)((((lo | hi) | 0x80808080u) - 0x20202020u) ^ 0x80808080u);
            }
        }
    }
};

// unsigned bytes of a times signed bytes of b
__device__ __forceinline__ int pb_dp4a_us(int a, int b, int c) {
    int d; asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}

// Number of int8 levels the activations are split into.  Each level divides the residual
// error by ~254: two levels leave ~2e-5 of the largest value of a 32-group, three ~1e-7,
// i.e. the size of f32 summation-order noise.  Three keeps router top-k decisions and
// greedy tokens aligned with an f32-accumulated reference over long runs.
#define PB_XLEVELS 3

// Activations of one column for one quarter: PB_XLEVELS int8 levels, their scales, and the
// f32 sum of each 32-value group (used by formats with a minimum).
struct PbXQuarter {
    int q[PB_XLEVELS][16];
    float s[PB_XLEVELS][2], sum[2];
    int is[PB_XLEVELS][2];   // -15 * integer sum of each level over a 32-group (loaded only for offset-coded formats)
};

template <int FMT>
__device__ __forceinline__ float pb_quarter_dot(const PbQuarter& w, const PbXQuarter& x) {
    using D = PbQDec<FMT>;
    float acc = 0.f;
    constexpr int NH = D::SCALE16 ? 4 : 2;   // integer sums per 16 or per 32 weights
    constexpr int WPH = 16 / NH;
#pragma unroll
    for (int h = 0; h < NH; h++) {
        int isum[PB_XLEVELS];
#pragma unroll
        for (int l = 0; l < PB_XLEVELS; l++) isum[l] = 0;
#pragma unroll
        for (int k = 0; k < WPH; k++)
#pragma unroll
            for (int l = 0; l < PB_XLEVELS; l++) isum[l] = D::AFFINE ? pb_dp4a_us(w.w[h * WPH + k], x.q[l][h * WPH + k], isum[l]) : __dp4a(w.w[h * WPH + k], x.q[l][h * WPH + k], isum[l]);
        const int g = h * WPH / 8;
        if (D::AFFINE) {
#pragma unroll
            for (int l = 0; l < PB_XLEVELS; l++) isum[l] = 2 * isum[l] + x.is[l][g];   // x.is = -15 * (sum of the level over the group)
        }
        float t = x.s[PB_XLEVELS - 1][g] * (float)isum[PB_XLEVELS - 1];   // smallest level first
#pragma unroll
        for (int l = PB_XLEVELS - 2; l >= 0; l--) t = fmaf(x.s[l][g], (float)isum[l], t);
        acc = fmaf(w.sc[h * (4 / NH)], t, acc);
    }
    if (D::HAS_MIN) { acc = fmaf(-w.mn[0], x.sum[0], acc); acc = fmaf(-w.mn[1], x.sum[1], acc); }
    return acc;
}

// ---- fused decode + dot for IQ3_S (one column) --------------------------------------------------------
// Same arithmetic as PbQDec<IQ3_S>::quarter followed by pb_quarter_dot, written so that each codebook
// entry costs one byte-permute (index = qs byte | high bit << 8), one multiply-add (address) and one
// load: the eight high bits of a 32-weight half are first spread into bytes with a multiply
// (n * 0x00204081 & 0x01010101 puts bit k of n into byte k), then prmt picks (qs byte, high byte)
// and zero-fills the rest through its sign-replication mode.  Integer sums go straight into the
// per-group accumulators; no decoded quarter is kept.
__device__ __forceinline__ float pb_iq3s_quarter_dot(uint32_t p, int qt, const PbQTabs& T, const PbXQuarter& x) {
    const float d = pb_h2f((uint16_t)pb_lds16(p));
    uint32_t qs[4], sg[2];
    pb_ld_u32x<4>(p + 2 + 16 * qt, qs);
    pb_ld_u32x<2>(p + 74 + 8 * qt, sg);
    const uint32_t qh = pb_lds16(p + 66 + 2 * qt);
    const uint32_t sc = pb_lds8(p + 106 + qt);
    float acc = 0.f;
#pragma unroll
    for (int h = 0; h < 2; h++) {                 // 32 weights = 8 entries = 4 sign bytes
        int isum[PB_XLEVELS];
#pragma unroll
        for (int l = 0; l < PB_XLEVELS; l++) isum[l] = 0;
#pragma unroll
        for (int k = 0; k < 2; k++) {             // 4 entries share one qs word and one spread of high bits
            const uint32_t word = qs[2 * h + k];
            const uint32_t hb = pb_spread4((qh >> (8 * h + 4 * k)) & 0xF);
            const uint32_t i0 = pb_iq3s_index<0>(word, hb), i1 = pb_iq3s_index<1>(word, hb), i2 = pb_iq3s_index<2>(word, hb), i3 = pb_iq3s_index<3>(word, hb);
            const uint32_t g0 = pb_lds32(T.grid + i0 * T.stride), g1 = pb_lds32(T.grid + i1 * T.stride);
            const uint32_t g2 = pb_lds32(T.grid + i2 * T.stride), g3 = pb_lds32(T.grid + i3 * T.stride);
            // signs by arithmetic: shared-memory wavefronts, not issue slots, bound this loop when the
            // masks came from a table
            const int w0 = k ? pb_iq3s_sign8<4>(g0, sg[h]) : pb_iq3s_sign8<0>(g0, sg[h]), w1 = k ? pb_iq3s_sign8<5>(g1, sg[h]) : pb_iq3s_sign8<1>(g1, sg[h]);
            const int w2 = k ? pb_iq3s_sign8<6>(g2, sg[h]) : pb_iq3s_sign8<2>(g2, sg[h]), w3 = k ? pb_iq3s_sign8<7>(g3, sg[h]) : pb_iq3s_sign8<3>(g3, sg[h]);
            const int e = 8 * h + 4 * k;
#pragma unroll
            for (int l = 0; l < PB_XLEVELS; l++) {
                isum[l] = __dp4a(w0, x.q[l][e], isum[l]); isum[l] = __dp4a(w1, x.q[l][e + 1], isum[l]);
                isum[l] = __dp4a(w2, x.q[l][e + 2], isum[l]); isum[l] = __dp4a(w3, x.q[l][e + 3], isum[l]);
            }
        }
        float t = x.s[PB_XLEVELS - 1][h] * (float)isum[PB_XLEVELS - 1];   // smallest level first, as pb_quarter_dot
#pragma unroll
        for (int l = PB_XLEVELS - 2; l >= 0; l--) t = fmaf(x.s[l][h], (float)isum[l], t);
        const float db = d * (float)(1 + 2 * (int)((sc >> (4 * h)) & 0xF));
        acc = fmaf(db, t, acc);
    }
    return acc;
}

// decode one quarter and dot it with one column's activations
template <int FMT>
__device__ __forceinline__ float pb_decode_dot(uint32_t p, int qt, const PbQTabs& T, const PbXQuarter& x) {
    if (FMT == PB_T_IQ3_S) return pb_iq3s_quarter_dot(p, qt, T, x);
    PbQuarter w;
    PbQDec<FMT>::quarter(p, qt, T, w);
    return pb_quarter_dot<FMT>(w, x);
}
