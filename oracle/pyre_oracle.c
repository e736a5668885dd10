/* CPU oracle for the Qwen-Next decode path -- TEST INFRASTRUCTURE ONLY (see pyre_oracle.h).
 *
 * Build:  make -C oracle      (gcc -O2 -ffp-contract=off -fopenmp; no reference sources are copied)
 * File/line citations name files of the reference project (Lyamc/pyre) by their path in it.
 */
#include "pyre_oracle.h"
#include "iq_tables.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ scalars */

/* f16 -> f32, exact (the reference uses half::f16::to_f32, gguf_q.rs:60) */
static float h2f(uint16_t h) {
    uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, m = h & 1023, u;
    if (e == 0) {
        if (m == 0) u = s;
        else { int sh = 0; while (!(m & 1024)) { m <<= 1; sh++; } m &= 1023; u = s | ((uint32_t)(113 - sh) << 23) | (m << 13); }
    } else if (e == 31) u = s | 0x7F800000u | (m << 13);
    else u = s | ((e + 112) << 23) | (m << 13);
    float f; memcpy(&f, &u, 4); return f;
}
/* f32 -> f16 round-to-nearest-even (used only by the synthetic generator) */
static uint16_t f2h(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    uint32_t s = (u >> 16) & 0x8000u; int32_t e = (int32_t)((u >> 23) & 255) - 127 + 15; uint32_t m = u & 0x7FFFFFu;
    if (((u >> 23) & 255) == 255) return (uint16_t)(s | 0x7C00u | (m ? 0x200u : 0));
    if (e >= 31) return (uint16_t)(s | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)s;
        m |= 0x800000u; int sh = 14 - e; uint32_t r = m >> sh, rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
        if (rem > half || (rem == half && (r & 1))) r++;
        return (uint16_t)(s | r);
    }
    uint32_t r = ((uint32_t)e << 10) | (m >> 13), rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) r++;
    return (uint16_t)(s | r);
}
static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

static inline float sigm(float x) { return 1.0f / (1.0f + expf(-x)); }            /* qwen4exp_gguf.rs:457 */
static inline float silu(float x) { return x * sigm(x); }                          /* :458 */
static inline float softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }  /* :459 */

/* rms :209 -- y = x * s * w ; rms_inplace :210 -- x *= s * w */
static void rms(const float* x, const float* w, float eps, float* y, int n) {
    float ss = 0.0f; for (int i = 0; i < n; i++) ss += x[i] * x[i];
    float s = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = 0; i < n; i++) y[i] = x[i] * s * w[i];
}
static void rms_inplace(float* x, const float* w, float eps, int n) {
    float ss = 0.0f; for (int i = 0; i < n; i++) ss += x[i] * x[i];
    float s = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = 0; i < n; i++) x[i] *= s * w[i];
}

int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Thread count of the row-parallel loops (QMat::matmul splits rows over rayon's pool, gguf_q.rs:233-241;
 * the reference sizes that pool itself, main.rs:251).  A launcher may have exported OMP_NUM_THREADS=1
 * for its worker processes; a timed CPU run calls this with the number of cores it may use. */
void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------ block formats */

int orc_type_geom(int type, int* el, int* by) {  /* gguf_q.rs:33-41 */
    int e, b;
    switch (type) {
        case ORC_F32: e = 1; b = 4; break;
        case ORC_F16: case ORC_BF16: e = 1; b = 2; break;
        case ORC_Q8_0: e = 32; b = 34; break;
        case ORC_Q4_K: e = 256; b = 144; break;
        case ORC_IQ2_XS: e = 256; b = 74; break;
        case ORC_IQ3_S: e = 256; b = 110; break;
        case ORC_IQ3_XXS: e = 256; b = 98; break;
        case ORC_IQ2_S: e = 256; b = 82; break;
        case ORC_IQ4_NL: e = 32; b = 18; break;
        case ORC_IQ4_XS: e = 256; b = 136; break;
        case ORC_Q2_0: e = 64; b = 18; break;
        case ORC_IQ2_XXS: e = 256; b = 66; break;
        case ORC_Q6_K: e = 256; b = 210; break;
        case ORC_IQ1_M: e = 256; b = 56; break;
        case ORC_Q4_0: e = 32; b = 18; break;
        case ORC_Q5_0: e = 32; b = 22; break;
        case ORC_Q3_K: e = 256; b = 110; break;
        case ORC_Q5_K: e = 256; b = 176; break;
        default: return -1;
    }
    if (el) *el = e;
    if (by) *by = b;
    return 0;
}
int64_t orc_row_bytes(int type, int64_t cols) { int e, b; if (orc_type_geom(type, &e, &b)) return -1; return cols / e * b; }

static void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {  /* gguf_q.rs:62-64 */
    if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
    else { *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}

/* put8, gguf_q.rs:58: y[j] = d * g[j] * s[j], evaluated left to right */
static inline void put8(float* y, float d, const uint8_t* g, uint8_t signs) {
    for (int j = 0; j < 8; j++) { float s = (signs >> j) & 1 ? -1.0f : 1.0f; float t = d * (float)g[j]; y[j] = t * s; }
}

int orc_dequant(int type, const uint8_t* x, int64_t n, float* y) {  /* gguf_q.rs:67-166 */
    int qk, bs; if (orc_type_geom(type, &qk, &bs)) return -1;
    int64_t nb = n / qk;
    switch (type) {
    case ORC_F32: memcpy(y, x, (size_t)n * 4); break;                                         /* :71 */
    case ORC_F16: for (int64_t i = 0; i < n; i++) y[i] = h2f(rd16(x + 2 * i)); break;          /* :72 */
    case ORC_BF16: for (int64_t i = 0; i < n; i++) { uint32_t u = (uint32_t)rd16(x + 2 * i) << 16; memcpy(&y[i], &u, 4); } break;  /* :73 */
    case ORC_Q8_0:                                                                             /* :79 */
        for (int64_t i = 0; i < nb; i++) { const uint8_t* b = x + i * bs; float d = h2f(rd16(b));
            for (int j = 0; j < 32; j++) y[i * 32 + j] = (float)(int8_t)b[2 + j] * d; }
        break;
    case ORC_Q4_K:                                                                             /* :103-107 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)), mn = h2f(rd16(b + 2)); const uint8_t* sc = b + 4; const uint8_t* q = b + 16; float* yy = y + i * 256;
            for (int j = 0; j < 4; j++) {
                uint8_t s1, m1, s2, m2; scale_min_k4(2 * j, sc, &s1, &m1); scale_min_k4(2 * j + 1, sc, &s2, &m2);
                float d1 = d * (float)s1, mm1 = mn * (float)m1, d2 = d * (float)s2, mm2 = mn * (float)m2;
                for (int l = 0; l < 32; l++) { yy[l] = d1 * (float)(q[l] & 0xF) - mm1; yy[l + 32] = d2 * (float)(q[l] >> 4) - mm2; }
                yy += 64; q += 32;
            }
        }
        break;
    case ORC_IQ2_XS:                                                                           /* :126-129 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)); const uint8_t* qs = b + 2; const uint8_t* sc = b + 66; float* yy = y + i * 256;
            for (int ib = 0; ib < 8; ib++) {
                float db[2]; db[0] = d * (0.5f + (float)(sc[ib] & 0xF)) * 0.25f; db[1] = d * (0.5f + (float)(sc[ib] >> 4)) * 0.25f;
                for (int l = 0; l < 4; l++) {
                    uint16_t q = rd16(qs + 2 * (4 * ib + l));
                    uint64_t g = PB_IQ2XS_GRID[q & 511]; uint8_t gb[8]; for (int j = 0; j < 8; j++) gb[j] = (uint8_t)(g >> (8 * j));
                    put8(yy, db[l / 2], gb, PB_KSIGNS_IQ2XS[q >> 9]); yy += 8;
                }
            }
        }
        break;
    case ORC_IQ4_NL:                                                                           /* :82-83 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)); float* yy = y + i * 32;
            for (int j = 0; j < 16; j++) { yy[j] = d * (float)PB_KVALUES_IQ4NL[b[2 + j] & 0xF]; yy[16 + j] = d * (float)PB_KVALUES_IQ4NL[b[2 + j] >> 4]; }
        }
        break;
    case ORC_IQ4_XS:                                                                           /* :84-89 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)); uint16_t sh = rd16(b + 2); const uint8_t* sl = b + 4; const uint8_t* qs = b + 8; float* yy = y + i * 256;
            for (int ib = 0; ib < 8; ib++) {
                int ls = (int)((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (int)(((sh >> (2 * ib)) & 3) << 4); float dl = d * (float)(ls - 32);
                for (int j = 0; j < 16; j++) { yy[j] = (float)PB_KVALUES_IQ4NL[qs[j] & 0xF] * dl; yy[16 + j] = (float)PB_KVALUES_IQ4NL[qs[j] >> 4] * dl; }
                yy += 32; qs += 16;
            }
        }
        break;
    case ORC_Q2_0:                                                                             /* :80-81: 64 weights, two bits each, value (code - 1) * d */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)); float* yy = y + i * 64;
            for (int k = 0; k < 16; k++) for (int j = 0; j < 4; j++) yy[4 * k + j] = (float)((int)((b[2 + k] >> (2 * j)) & 3) - 1) * d;
        }
        break;
    case ORC_Q6_K:                                                                             /* :114-121 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; const uint8_t* ql = b; const uint8_t* qh = b + 128; const int8_t* sc = (const int8_t*)(b + 192); float d = h2f(rd16(b + 208)); float* yy = y + i * 256;
            for (int n = 0; n < 2; n++) {
                for (int l = 0; l < 32; l++) { int is = l / 16;
                    int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32, q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32, q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                    yy[l] = d * (float)sc[is] * (float)q1; yy[l + 32] = d * (float)sc[is + 2] * (float)q2;
                    yy[l + 64] = d * (float)sc[is + 4] * (float)q3; yy[l + 96] = d * (float)sc[is + 6] * (float)q4; }
                yy += 128; ql += 64; qh += 32; sc += 8;
            }
        }
        break;
    case ORC_Q4_0:                                                                             /* :74-75 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)); float* yy = y + i * 32;
            for (int j = 0; j < 16; j++) { yy[j] = (float)((int)(b[2 + j] & 0xF) - 8) * d; yy[j + 16] = (float)((int)(b[2 + j] >> 4) - 8) * d; }
        }
        break;
    case ORC_Q5_0:                                                                             /* :76-78 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)); uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24); const uint8_t* qs = b + 6; float* yy = y + i * 32;
            for (int j = 0; j < 16; j++) { uint32_t h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
                yy[j] = (float)((int)((qs[j] & 0xF) | h0) - 16) * d; yy[j + 16] = (float)((int)((qs[j] >> 4) | h1) - 16) * d; }
        }
        break;
    case ORC_Q3_K:                                                                             /* :90-102: [hmask 32][qs 64][scales 12][d f16] */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; const uint8_t* hm = b; const uint8_t* q = b + 32; const uint8_t* sc = b + 96; float d_all = h2f(rd16(b + 108)); float* yy = y + i * 256;
            uint32_t a[3]; for (int k = 0; k < 3; k++) a[k] = (uint32_t)sc[4 * k] | ((uint32_t)sc[4 * k + 1] << 8) | ((uint32_t)sc[4 * k + 2] << 16) | ((uint32_t)sc[4 * k + 3] << 24);
            const uint32_t k1 = 0x03030303u, k2 = 0x0f0f0f0fu;
            uint32_t aux[4] = { (a[0] & k2) | ((a[2] & k1) << 4), (a[1] & k2) | (((a[2] >> 2) & k1) << 4), ((a[0] >> 4) & k2) | (((a[2] >> 4) & k1) << 4), ((a[1] >> 4) & k2) | (((a[2] >> 6) & k1) << 4) };
            int is = 0; uint8_t m = 1;
            for (int n = 0; n < 2; n++) { int shift = 0;
                for (int j = 0; j < 4; j++) {
                    for (int half = 0; half < 2; half++) { float dl = d_all * (float)((int)(int8_t)(uint8_t)(aux[is / 4] >> (8 * (is % 4))) - 32); is++;
                        for (int l = 0; l < 16; l++) { int oo = l + 16 * half; yy[l] = dl * (float)((int)((q[oo] >> shift) & 3) - (hm[oo] & m ? 0 : 4)); }
                        yy += 16; }
                    shift += 2; m = (uint8_t)(m << 1); }
                q += 32; }
        }
        break;
    case ORC_Q5_K:                                                                             /* :108-113: [d][dmin][scales 12][qh 32][ql 128] */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)), mn = h2f(rd16(b + 2)); const uint8_t* sc = b + 4; const uint8_t* qh = b + 16; const uint8_t* ql = b + 48; float* yy = y + i * 256;
            uint8_t u1 = 1, u2 = 2;
            for (int j = 0; j < 4; j++) { uint8_t s1, m1, s2, m2; scale_min_k4(2 * j, sc, &s1, &m1); scale_min_k4(2 * j + 1, sc, &s2, &m2);
                float d1 = d * (float)s1, mm1 = mn * (float)m1, d2 = d * (float)s2, mm2 = mn * (float)m2;
                for (int l = 0; l < 32; l++) { yy[l] = d1 * (float)((ql[l] & 0xF) + (qh[l] & u1 ? 16 : 0)) - mm1; yy[l + 32] = d2 * (float)((ql[l] >> 4) + (qh[l] & u2 ? 16 : 0)) - mm2; }
                yy += 64; ql += 32; u1 = (uint8_t)(u1 << 2); u2 = (uint8_t)(u2 << 2); }
        }
        break;
    case ORC_IQ1_M:                                                                            /* :152-164: [qs 32][qh 16][scales 4 x u16]; the f16 scale sits in the top nibbles of the scale words */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; const uint8_t* qs = b; const uint8_t* qh = b + 32; float* yy = y + i * 256;
            uint16_t sc[4]; for (int k = 0; k < 4; k++) sc[k] = rd16(b + 48 + 2 * k);
            float d = h2f((uint16_t)((sc[0] >> 12) | ((sc[1] >> 8) & 0x00f0) | ((sc[2] >> 4) & 0x0f00) | (sc[3] & 0xf000)));
            for (int ib = 0; ib < 8; ib++) {
                float dl1 = d * (float)(2 * ((sc[ib / 2] >> (6 * (ib % 2))) & 7) + 1), dl2 = d * (float)(2 * ((sc[ib / 2] >> (6 * (ib % 2) + 3)) & 7) + 1);
                for (int l = 0; l < 4; l++) {
                    uint8_t h = qh[l / 2]; int sh = 4 * (l & 1);
                    uint64_t g = PB_IQ1S_GRID[(size_t)qs[l] | ((((size_t)h >> sh) << 8) & 0x700)];
                    float delta = (h >> sh) & 0x08 ? -0.125f : 0.125f, sl = l < 2 ? dl1 : dl2;
                    for (int j = 0; j < 8; j++) yy[j] = sl * ((float)(int8_t)(uint8_t)(g >> (8 * j)) + delta);
                    yy += 8;
                }
                qs += 4; qh += 2;
            }
        }
        break;
    case ORC_IQ2_XXS:                                                                          /* :122-125 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)); const uint8_t* qs = b + 2; float* yy = y + i * 256;
            for (int ib = 0; ib < 8; ib++) {
                const uint8_t* a0 = qs + 8 * ib; uint32_t a1 = (uint32_t)qs[8 * ib + 4] | ((uint32_t)qs[8 * ib + 5] << 8) | ((uint32_t)qs[8 * ib + 6] << 16) | ((uint32_t)qs[8 * ib + 7] << 24);
                float db = d * (0.5f + (float)(a1 >> 28)) * 0.25f;
                for (int l = 0; l < 4; l++) {
                    uint64_t g = PB_IQ2XXS_GRID[a0[l]]; uint8_t gb[8]; for (int j = 0; j < 8; j++) gb[j] = (uint8_t)(g >> (8 * j));
                    put8(yy, db, gb, PB_KSIGNS_IQ2XS[(a1 >> (7 * l)) & 127]); yy += 8;
                }
            }
        }
        break;
    case ORC_IQ2_S:                                                                            /* :130-135 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)); const uint8_t* qs = b + 2; const uint8_t* signs = b + 34; const uint8_t* qh = b + 66; const uint8_t* sc = b + 74; float* yy = y + i * 256;
            for (int ib = 0; ib < 8; ib++) {
                float db[2]; db[0] = d * (0.5f + (float)(sc[ib] & 0xF)) * 0.25f; db[1] = d * (0.5f + (float)(sc[ib] >> 4)) * 0.25f;
                for (int l = 0; l < 4; l++) {
                    uint32_t idx = (uint32_t)qs[l] | ((((uint32_t)qh[ib]) << (8 - 2 * l)) & 0x300);
                    uint64_t g = PB_IQ2S_GRID[idx]; uint8_t gb[8]; for (int j = 0; j < 8; j++) gb[j] = (uint8_t)(g >> (8 * j));
                    put8(yy, db[l / 2], gb, signs[l]); yy += 8;
                }
                qs += 4; signs += 4;
            }
        }
        break;
    case ORC_IQ3_XXS:                                                                          /* :136-140 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)); const uint8_t* qs = b + 2; const uint8_t* ss = b + 66; float* yy = y + i * 256;
            for (int ib = 0; ib < 8; ib++) {
                uint32_t a = (uint32_t)ss[4 * ib] | ((uint32_t)ss[4 * ib + 1] << 8) | ((uint32_t)ss[4 * ib + 2] << 16) | ((uint32_t)ss[4 * ib + 3] << 24);
                float db = d * (0.5f + (float)(a >> 28)) * 0.5f;
                for (int l = 0; l < 4; l++) {
                    uint32_t g1 = PB_IQ3XXS_GRID[qs[8 * ib + 2 * l]], g2 = PB_IQ3XXS_GRID[qs[8 * ib + 2 * l + 1]];
                    uint8_t gb[8]; for (int j = 0; j < 4; j++) { gb[j] = (uint8_t)(g1 >> (8 * j)); gb[4 + j] = (uint8_t)(g2 >> (8 * j)); }
                    put8(yy, db, gb, PB_KSIGNS_IQ2XS[(a >> (7 * l)) & 127]); yy += 8;
                }
            }
        }
        break;
    case ORC_IQ3_S:                                                                            /* :141-151 */
        for (int64_t i = 0; i < nb; i++) {
            const uint8_t* b = x + i * bs; float d = h2f(rd16(b)); const uint8_t* qs = b + 2; const uint8_t* qh = b + 66; const uint8_t* signs = b + 74; const uint8_t* sc = b + 106; float* yy = y + i * 256;
            for (int ib = 0; ib < 8; ib += 2) {
                for (int half = 0; half < 2; half++) {
                    uint8_t s = sc[ib / 2]; float db = d * (float)(1 + 2 * (half == 0 ? (s & 0xF) : (s >> 4)));
                    for (int l = 0; l < 4; l++) {
                        uint32_t g1 = PB_IQ3S_GRID[qs[2 * l] | (((uint32_t)qh[half] << (8 - 2 * l)) & 256)];
                        uint32_t g2 = PB_IQ3S_GRID[qs[2 * l + 1] | (((uint32_t)qh[half] << (7 - 2 * l)) & 256)];
                        uint8_t gb[8]; for (int j = 0; j < 4; j++) { gb[j] = (uint8_t)(g1 >> (8 * j)); gb[4 + j] = (uint8_t)(g2 >> (8 * j)); }
                        put8(yy, db, gb, signs[l]); yy += 8;
                    }
                    qs += 8; signs += 4;
                }
                qh += 2;
            }
        }
        break;
    default: return -1;
    }
    return 0;
}

/* dot_avx2, gguf_q.rs:176-197: four 8-lane FMA accumulators over 32-element strides, an
 * 8-element tail on accumulator 0, (s0+s1)+(s2+s3) per lane, lanes summed in order, scalar tail. */
float orc_dot(const float* a, const float* b, int64_t n) {
    float s[4][8]; memset(s, 0, sizeof s);
    int64_t i = 0;
    for (; i + 32 <= n; i += 32)
        for (int k = 0; k < 4; k++) for (int l = 0; l < 8; l++) s[k][l] = fmaf(a[i + 8 * k + l], b[i + 8 * k + l], s[k][l]);
    for (; i + 8 <= n; i += 8) for (int l = 0; l < 8; l++) s[0][l] = fmaf(a[i + l], b[i + l], s[0][l]);
    float r = 0.0f;
    for (int l = 0; l < 8; l++) r += (s[0][l] + s[1][l]) + (s[2][l] + s[3][l]);
    for (; i < n; i++) r += a[i] * b[i];
    return r;
}

/* ------------------------------------------------------------------ seeded synthetic tensors
 *
 * Specification (mirrored by the CUDA generator; both must produce identical bytes):
 *   sm64(x)      = splitmix64 finaliser of x + 0x9E3779B97F4A7C15
 *   tkey         = sm64(sm64(seed) ^ tid)
 *   bkey(b)      = sm64(tkey ^ (b * 0xD1342543DE82EF95))         b = global block (or element) index
 *   word(b, j)   = sm64(bkey(b) + j)
 *   normal(w0..w2) = (sum of the twelve 16-bit fields of three words - 393210) / 65536   (Irwin-Hall, ~N(0,1))
 *   scale        = f16_rne(|normal| * 0.02f)
 * Q8_0 : d = scale(words 0-2); q[j] = (byte j of words 3-6) % 255 - 127
 * Q4_K : d = scale(0-2), dmin = scale(3-5), 140 payload bytes = words 6..
 * IQ2_XS: d = scale(0-2), 72 payload bytes = words 3..   IQ3_S: d = scale(0-2), 108 payload bytes = words 3..
 * F32  : element i = normal(words 0-2 of bkey(i)) * sigma      (orc_synth_normal)
 * All payload fields of the k-/i-quants are uniform bit fields, so uniform bytes give uniform
 * sub-scales, grid indices and signs.
 */
static inline uint64_t sm64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull; x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull; x = (x ^ (x >> 27)) * 0x94D049BB133111EBull; return x ^ (x >> 31);
}
static inline uint64_t synth_tkey(uint64_t seed, uint64_t tid) { return sm64(sm64(seed) ^ tid); }
static inline uint64_t synth_bkey(uint64_t tkey, uint64_t b) { return sm64(tkey ^ (b * 0xD1342543DE82EF95ull)); }
static inline float synth_normal(uint64_t bkey, int j0) {
    int32_t s = 0;
    for (int j = 0; j < 3; j++) { uint64_t w = sm64(bkey + (uint64_t)(j0 + j)); s += (int32_t)(w & 0xFFFF) + (int32_t)((w >> 16) & 0xFFFF) + (int32_t)((w >> 32) & 0xFFFF) + (int32_t)(w >> 48); }
    return (float)(s - 393210) * (1.0f / 65536.0f);
}
static inline uint16_t synth_scale(uint64_t bkey, int j0) { return f2h(fabsf(synth_normal(bkey, j0)) * 0.02f); }
static void synth_payload(uint64_t bkey, int j0, uint8_t* out, int nbytes) {
    for (int o = 0; o < nbytes; o += 8) { uint64_t w = sm64(bkey + (uint64_t)(j0 + o / 8)); for (int k = 0; k < 8 && o + k < nbytes; k++) out[o + k] = (uint8_t)(w >> (8 * k)); }
}
static void synth_block(int type, uint64_t tkey, uint64_t b, uint8_t* out) {
    uint64_t k = synth_bkey(tkey, b);
    uint16_t d = synth_scale(k, 0); out[0] = (uint8_t)d; out[1] = (uint8_t)(d >> 8);
    switch (type) {
    case ORC_Q8_0: { uint8_t raw[32]; synth_payload(k, 3, raw, 32); for (int j = 0; j < 32; j++) out[2 + j] = (uint8_t)(int8_t)((int)(raw[j] % 255) - 127); } break;
    case ORC_Q4_K: { uint16_t m = synth_scale(k, 3); out[2] = (uint8_t)m; out[3] = (uint8_t)(m >> 8); synth_payload(k, 6, out + 4, 140); } break;
    case ORC_IQ2_XS: synth_payload(k, 3, out + 2, 72); break;
    case ORC_IQ3_S: synth_payload(k, 3, out + 2, 108); break;
    case ORC_IQ3_XXS: synth_payload(k, 3, out + 2, 96); break;
    case ORC_IQ2_S: synth_payload(k, 3, out + 2, 80); break;
    case ORC_IQ4_NL: synth_payload(k, 3, out + 2, 16); break;
    case ORC_IQ4_XS: synth_payload(k, 3, out + 2, 134); break;
    case ORC_Q2_0: synth_payload(k, 3, out + 2, 16); break;
    case ORC_Q6_K:   /* the f16 scale closes the block; sub-block scales kept to -8..7 so that weights stay in the range of the other generators */
        synth_payload(k, 3, out, 208);
        for (int i = 192; i < 208; i++) out[i] = (uint8_t)(int8_t)((int)(out[i] & 15) - 8);
        out[208] = (uint8_t)d; out[209] = (uint8_t)(d >> 8); break;
    case ORC_IQ2_XXS: synth_payload(k, 3, out + 2, 64); break;
    case ORC_Q4_0: synth_payload(k, 3, out + 2, 16); break;
    case ORC_Q5_0: synth_payload(k, 3, out + 2, 20); break;
    case ORC_Q3_K: synth_payload(k, 3, out, 108); out[108] = (uint8_t)d; out[109] = (uint8_t)(d >> 8); break;   /* the f16 scale closes the block */
    case ORC_Q5_K: { uint16_t dm = synth_scale(k, 3); out[2] = (uint8_t)dm; out[3] = (uint8_t)(dm >> 8); synth_payload(k, 6, out + 4, 172); } break;
    case ORC_IQ1_M:   /* the f16 scale goes, a nibble each, into the top of the four scale words */
        synth_payload(k, 3, out, 56);
        for (int i = 0; i < 4; i++) out[49 + 2 * i] = (uint8_t)((out[49 + 2 * i] & 0x0F) | (((d >> (4 * i)) & 0xF) << 4));
        break;
    }
}
void orc_synth_rows(int type, uint64_t seed, uint64_t tid, int64_t cols, int64_t r0, int64_t nrows, uint8_t* out) {
    int el, bs; if (orc_type_geom(type, &el, &bs)) return;
    uint64_t tkey = synth_tkey(seed, tid); int64_t bpr = cols / el;
    if (type == ORC_F32) { orc_synth_normal(seed, tid, r0 * cols, nrows * cols, 0.02f, (float*)out); return; }
    #pragma omp parallel for schedule(static) if (nrows * bpr > 4096)
    for (int64_t i = 0; i < nrows * bpr; i++) synth_block(type, tkey, (uint64_t)(r0 * bpr + i), out + i * bs);
}
void orc_synth_normal(uint64_t seed, uint64_t tid, int64_t i0, int64_t n, float sigma, float* out) {
    uint64_t tkey = synth_tkey(seed, tid);
    #pragma omp parallel for schedule(static) if (n > 65536)
    for (int64_t i = 0; i < n; i++) out[i] = synth_normal(synth_bkey(tkey, (uint64_t)(i0 + i)), 0) * sigma;
}

/* ------------------------------------------------------------------ QMat */

/* ---- the reference's int8 CPU fast path (src/model/qdot.rs): activations quantized to int8 per 32 values, the row's
 * block integers dotted with them in integers.  The GPU path does not use it (it keeps three int8 levels, 21 bits);
 * it is restated so that the oracle covers the approximation the reference's CPU decode really runs. ---- */
/* quantize_into, qdot.rs:20-30: per 32 values d = amax / 127, q = round(x / d) (round half away from zero) */
void orc_q8_quantize(const float* x, int64_t n, int8_t* q, float* d) {
    for (int64_t b = 0; b < n / 32; b++) {
        const float* xb = x + b * 32; float amax = 0.0f;
        for (int j = 0; j < 32; j++) { float a = fabsf(xb[j]); if (a > amax) amax = a; }
        float dd = amax / 127.0f, id = dd > 0.0f ? 1.0f / dd : 0.0f;
        d[b] = dd;
        for (int j = 0; j < 32; j++) q[b * 32 + j] = (int8_t)roundf(xb[j] * id);
    }
}
/* the expected value of the reference's own test (q8_dot, qdot.rs:1046-1052): dequantized row times the int8
 * activations, one f32 sum per 32 values scaled by the activation block scale; any block format */
float orc_q8_dot_dequant(int type, const uint8_t* row, int64_t n, const int8_t* q, const float* d) {
    float* y = (float*)malloc((size_t)n * 4); float acc = 0.0f;
    orc_dequant(type, row, n, y);
    for (int64_t b = 0; b < n / 32; b++) { float s = 0.0f; for (int j = 0; j < 32; j++) s += y[b * 32 + j] * (float)q[b * 32 + j]; acc += s * d[b]; }
    free(y);
    return acc;
}
/* row_dot for IQ3_S, scalar structure of qdot.rs:278-286 (the AVX2 kernel iq3s_avx2 :169 computes the same integers):
 * per 32 values an exact integer sum of sign * grid byte * q, scaled by d * (1 + 2 * nibble) and the activation scale */
float orc_row_dot_q8_iq3s(const uint8_t* row, int64_t n, const int8_t* q, const float* d) {
    float acc = 0.0f;
    for (int64_t i = 0; i < n / 256; i++) {
        const uint8_t* b = row + i * 110; uint16_t hb; memcpy(&hb, b, 2); float dblk = h2f(hb);
        const uint8_t* qs = b + 2; const uint8_t* qh = b + 66; const uint8_t* sg = b + 74; const uint8_t* scb = b + 106;
        for (int ib = 0; ib < 8; ib++) {
            int nib = (ib & 1) ? scb[ib / 2] >> 4 : scb[ib / 2] & 0xF;
            float db = dblk * (float)(1 + 2 * nib);
            int32_t isum = 0;
            for (int l = 0; l < 4; l++) {
                uint32_t g1 = PB_IQ3S_GRID[qs[8 * ib + 2 * l] | (((uint32_t)qh[ib] << (8 - 2 * l)) & 256)];
                uint32_t g2 = PB_IQ3S_GRID[qs[8 * ib + 2 * l + 1] | (((uint32_t)qh[ib] << (7 - 2 * l)) & 256)];
                uint8_t sb = sg[4 * ib + l];
                for (int j = 0; j < 4; j++) {
                    int w1 = (int)((g1 >> (8 * j)) & 0xFF), w2 = (int)((g2 >> (8 * j)) & 0xFF);
                    if (sb & (1 << j)) w1 = -w1;
                    if (sb & (1 << (4 + j))) w2 = -w2;
                    isum += w1 * (int)q[i * 256 + ib * 32 + 8 * l + j] + w2 * (int)q[i * 256 + ib * 32 + 8 * l + 4 + j];
                }
            }
            acc += (float)isum * db * d[i * 8 + ib];
        }
    }
    return acc;
}

void orc_mat_row_raw(const orc_mat* m, int64_t r, uint8_t* out) {
    int64_t rb = orc_row_bytes(m->type, m->cols);
    if (m->data) memcpy(out, m->data + r * rb, (size_t)rb);
    else orc_synth_rows(m->type, m->seed, m->tid, m->cols, r, 1, out);
}
void orc_mat_row(const orc_mat* m, int64_t r, float* y) {  /* QMat::row :210 */
    int64_t rb = orc_row_bytes(m->type, m->cols);
    if (m->data) { orc_dequant(m->type, m->data + r * rb, m->cols, y); return; }
    uint8_t stackbuf[4096]; uint8_t* raw = rb <= (int64_t)sizeof stackbuf ? stackbuf : (uint8_t*)malloc((size_t)rb);
    orc_synth_rows(m->type, m->seed, m->tid, m->cols, r, 1, raw);
    orc_dequant(m->type, raw, m->cols, y);
    if (raw != stackbuf) free(raw);
}
/* QMat::matmul :217-242, the t < 16 branch (row dequantized once, dotted against every token);
 * rows are split over threads like the rayon chunks; every output element is produced by one
 * thread so the result does not depend on the thread count.  The t >= 16 branch of the
 * reference uses a blocked SGEMM whose summation order is not reproduced here. */
void orc_matmul(const orc_mat* m, const float* x, int t, float* y) {
    int64_t rows = m->rows, cols = m->cols;
    #pragma omp parallel
    {
        float* buf = (float*)malloc((size_t)cols * 4);
        #pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; r++) { orc_mat_row(m, r, buf); for (int ti = 0; ti < t; ti++) y[(int64_t)ti * rows + r] = orc_dot(buf, x + (int64_t)ti * cols, cols); }
        free(buf);
    }
}
/* ------------------------------------------------------------------ router / sampler / kv4 / rope */

/* top_k qwen4exp_gguf.rs:3132-3139: the k largest raw logits, weights = softmax over them
 * (max-subtracted).  The reference selects with select_nth_unstable_by, whose order inside
 * the selection is unspecified; the canonical order here is descending logit, ties to the
 * lower index, and the softmax denominator is summed in that order.  NaN logits are treated
 * as -inf (nan_clean :3121-3125); if the best selected logit is not finite the weights are uniform
 * (soft_top :3128). */
void orc_top_k(const float* r, int n, int k, int32_t* idx, float* w) {
    char* used = (char*)calloc((size_t)n, 1);
    for (int j = 0; j < k; j++) {
        int best = -1; float bv = 0;
        for (int i = 0; i < n; i++) { if (used[i]) continue; float v = isnan(r[i]) ? -INFINITY : r[i]; if (best < 0 || v > bv) { best = i; bv = v; } }
        used[best] = 1; idx[j] = best; w[j] = bv;
    }
    free(used);
    float mx = -INFINITY; for (int j = 0; j < k; j++) mx = fmaxf(mx, w[j]);
    if (!isfinite(mx)) { for (int j = 0; j < k; j++) w[j] = 1.0f / (float)(k > 0 ? k : 1); return; }
    float sum = 0.0f; for (int j = 0; j < k; j++) { w[j] = expf(w[j] - mx); sum += w[j]; }
    for (int j = 0; j < k; j++) w[j] = w[j] / sum;
}

uint32_t orc_argmax(const float* v, int64_t n) {  /* sampler.rs:142-148 */
    int64_t best = 0; for (int64_t i = 1; i < n; i++) if (v[i] > v[best]) best = i; return (uint32_t)best;
}

void orc_kv4_pack(const float* x, int64_t n, uint32_t* w, float* sc) {  /* kv4.rs:12-32 */
    for (int64_t b = 0; b < n / 32; b++) {
        const float* p = x + b * 32; float m = 0.0f; for (int j = 0; j < 32; j++) m = fmaxf(m, fabsf(p[j]));
        float s = (m > 0.0f && isfinite(m)) ? m / 7.0f : 0.0f; sc[b] = s;
        for (int c = 0; c < 4; c++) { uint32_t u = 0;
            for (int j = 0; j < 8; j++) { int q = 0; if (s > 0.0f) { float v = roundf(p[c * 8 + j] / s); v = v < -7.0f ? -7.0f : (v > 7.0f ? 7.0f : v); q = (int)v; }
                u |= ((uint32_t)(uint8_t)(int8_t)q & 0xF) << (4 * j); }
            w[b * 4 + c] = u; }
    }
}
float orc_kv4_get(const uint32_t* w, const float* sc, int64_t i) {  /* kv4.rs:35-40 */
    uint32_t nib = (w[i / 8] >> (4 * (i % 8))) & 0xF; int q = (int)nib - (nib >= 8 ? 16 : 0); return (float)q * sc[i / 32];
}
void orc_rope_inv(int n_rot, float base, float* inv) {  /* qn_ctx.rs:168 */
    for (int i = 0; i < n_rot / 2; i++) inv[i] = powf(base, -(2.0f * (float)i) / (float)n_rot);
}
/* Inverse rope frequencies for a context of `ctx` positions of a model trained on `ctx_train` (qn_ctx.rs:160-186): plain
 * base^(-2i/n_rot) at or under the trained length (or ctx_train = 0); above it YaRN with the llama.cpp / transformers
 * defaults (beta_fast 32, beta_slow 1): low indices are interpolated (divided by scale = ctx / ctx_train), high indices
 * keep the trained frequency, a linear ramp between the two correction dimensions.  Returns mscale = 1 + 0.1 ln(scale),
 * which the caller applies to cos and sin (qwen4exp_gguf.rs:528-533). */
float orc_rope_inv_yarn(int n_rot, float base, int64_t ctx_train, int64_t ctx, float* inv) {
    int half = n_rot / 2;
    float scale = ctx_train > 0 && ctx > ctx_train ? (float)ctx / (float)ctx_train : 1.0f;
    if (scale <= 1.0f) { orc_rope_inv(n_rot, base, inv); return 1.0f; }
    float dim = (float)n_rot;
    float lo = floorf((dim * logf((float)ctx_train / (32.0f * 2.0f * 3.14159265358979323846f))) / (2.0f * logf(base)));
    float hi = ceilf((dim * logf((float)ctx_train / (1.0f * 2.0f * 3.14159265358979323846f))) / (2.0f * logf(base)));
    if (lo < 0.0f) lo = 0.0f;
    float top = (float)(half > 0 ? half - 1 : 0);
    if (hi > top) hi = top;
    for (int i = 0; i < half; i++) {
        float extrap = powf(base, -(2.0f * (float)i) / dim), interp = extrap / scale;
        float ramp = fabsf(hi - lo) < 1e-6f ? 1.0f : ((float)i - lo) / (hi - lo);
        ramp = ramp < 0.0f ? 0.0f : (ramp > 1.0f ? 1.0f : ramp);
        inv[i] = interp * (1.0f - ramp) + extrap * ramp;
    }
    return 1.0f + 0.1f * logf(scale);
}
/* rope :1436-1439 with rope_cs :529-533; inv[n_rot / 2] holds mscale, applied only when it is not 1 */
static void rope(float* v, int64_t pos, const float* inv, int n_rot) {
    int half = n_rot / 2;
    float ms = inv[half];
    for (int i = 0; i < half; i++) {
        float a = (float)pos * inv[i]; float s = sinf(a), co = cosf(a);
        if (ms != 1.0f) { co *= ms; s *= ms; }
        float x0 = v[i], x1 = v[i + half]; v[i] = x0 * co - x1 * s; v[i + half] = x1 * co + x0 * s;
    }
}

/* ------------------------------------------------------------------ MoE block */

/* expert e of a fused [n_exp*rows_per][cols] tensor: QMat::slice_rows(e*rows_per, rows_per) :1756,1786 */
static void expert_row(const orc_mat* m, int64_t e, int64_t rows_per, int64_t r, float* y) { orc_mat_row(m, e * rows_per + r, y); }

void orc_moe(const orc_cfg* c, const orc_mat* router, const orc_mat* gate_e, const orc_mat* up_e, const orc_mat* down_e,
             const orc_mat* sh_gate, const orc_mat* sh_up, const orc_mat* sh_down, const float* sh_gate_inp,
             const float* x, int t, float* y, int32_t* sel, float* selw) {
    int d = c->d, ff = c->ff_exp, sf = (int)sh_gate->rows, ne = c->n_exp, k = c->top_k;
    /* ffn :1675-1684 */
    float* lg = (float*)malloc((size_t)t * ne * 4); float* g = (float*)malloc((size_t)t * sf * 4); float* u = (float*)malloc((size_t)t * sf * 4);
    orc_matmul(router, x, t, lg); orc_matmul(sh_gate, x, t, g); orc_matmul(sh_up, x, t, u);
    for (int64_t i = 0; i < (int64_t)t * sf; i++) g[i] = silu(g[i]) * u[i];
    orc_matmul(sh_down, g, t, y);
    /* routed :1723 shared gate */
    for (int ti = 0; ti < t; ti++) { float sg = sigm(orc_dot(sh_gate_inp, x + (int64_t)ti * d, d)); for (int i = 0; i < d; i++) y[(int64_t)ti * d + i] *= sg; }
    /* routing :1725-1731 */
    int32_t* ids = (int32_t*)malloc((size_t)t * k * 4); float* ws = (float*)malloc((size_t)t * k * 4);
    for (int ti = 0; ti < t; ti++) orc_top_k(lg + (int64_t)ti * ne, ne, k, ids + ti * k, ws + ti * k);
    if (sel) memcpy(sel, ids, (size_t)t * k * 4);
    if (selw) memcpy(selw, ws, (size_t)t * k * 4);
    /* f32 branch :1769-1793: per (expert, token) hidden = silu(gate.x) * (up.x); the down projections
     * accumulate w * (down_row . hidden) into o over experts in ascending expert id, then y += o. */
    float* o = (float*)calloc((size_t)t * d, 4);
    float* hid = (float*)malloc((size_t)t * ff * 4);
    for (int e = 0; e < ne; e++) {
        int nt = 0; int toks[1024]; float tw[1024];
        for (int ti = 0; ti < t && nt < 1024; ti++) for (int j = 0; j < k; j++) if (ids[ti * k + j] == e) { toks[nt] = ti; tw[nt] = ws[ti * k + j]; nt++; }
        if (!nt) continue;
        #pragma omp parallel
        {
            float* buf = (float*)malloc((size_t)(d > ff ? d : ff) * 4); float* gv = (float*)malloc((size_t)nt * 4);
            #pragma omp for schedule(static)
            for (int r = 0; r < ff; r++) {
                expert_row(gate_e, e, ff, r, buf); for (int j = 0; j < nt; j++) gv[j] = orc_dot(buf, x + (int64_t)toks[j] * d, d);
                expert_row(up_e, e, ff, r, buf); for (int j = 0; j < nt; j++) hid[(int64_t)j * ff + r] = silu(gv[j]) * orc_dot(buf, x + (int64_t)toks[j] * d, d);
            }
            #pragma omp for schedule(static)
            for (int r = 0; r < d; r++) { expert_row(down_e, e, d, r, buf); for (int j = 0; j < nt; j++) o[(int64_t)toks[j] * d + r] += tw[j] * orc_dot(buf, hid + (int64_t)j * ff, ff); }
            free(buf); free(gv);
        }
    }
    for (int64_t i = 0; i < (int64_t)t * d; i++) y[i] += o[i];
    free(o); free(hid); free(ids); free(ws); free(lg); free(g); free(u);
}

/* ------------------------------------------------------------------ Gated DeltaNet */

void orc_linear_core(const orc_cfg* c, const float* m, const float* zz, const float* bb, const float* aa,
                     const float* a, const float* dt, const float* conv, const float* norm,
                     float* cs, float* s, int t, float* o_all) {  /* linear_core :1624-1673 */
    int nk = c->lin_nk, nv = c->lin_nv, dk = c->lin_dk, dv = c->lin_dv, kk = c->conv_k; int ch = 2 * nk * dk + nv * dv; int w = nv * dv;
    float* co_all = (float*)malloc((size_t)t * ch * 4);
    /* 1) causal depthwise conv + SiLU, state shifts (:1643-1647) */
    for (int ti = 0; ti < t; ti++) {
        const float* cur = m + (int64_t)ti * ch; float* co = co_all + (int64_t)ti * ch;
        for (int cc = 0; cc < ch; cc++) { float o = conv[cc * kk + kk - 1] * cur[cc]; for (int k = 0; k < kk - 1; k++) o += conv[cc * kk + k] * cs[k * ch + cc]; co[cc] = silu(o); }
        memmove(cs, cs + ch, (size_t)(kk - 2) * ch * 4); memcpy(cs + (kk - 2) * ch, cur, (size_t)ch * 4);
    }
    /* 2) L2-normalise q (scaled by 1/sqrt(dk)) and k per head (:1649-1651) */
    for (int ti = 0; ti < t; ti++) { float* co = co_all + (int64_t)ti * ch;
        for (int h = 0; h < nk; h++) for (int which = 0; which < 2; which++) {
            float* buf = co + which * nk * dk + h * dk; float sc = which == 0 ? 1.0f / sqrtf((float)dk) : 1.0f;
            float ss = 0.0f; for (int i = 0; i < dk; i++) ss += buf[i] * buf[i];
            float n = 1.0f / sqrtf(ss + 1e-6f) * sc; for (int i = 0; i < dk; i++) buf[i] *= n; } }
    /* 3) delta-rule recurrence per V head (:1654-1669) */
    #pragma omp parallel for schedule(static)
    for (int h = 0; h < nv; h++) {
        float* sh = s + (int64_t)h * dk * dv; int kh = h % nk; float mem[1024], delta[1024];
        for (int ti = 0; ti < t; ti++) {
            const float* co = co_all + (int64_t)ti * ch; const float* qv = co + kh * dk; const float* kv = co + nk * dk + kh * dk; const float* vv = co + 2 * nk * dk + h * dv;
            float g = expf(softplus(aa[ti * nv + h] + dt[h]) * a[h]); float b = sigm(bb[ti * nv + h]);
            for (int i = 0; i < dk * dv; i++) sh[i] *= g;
            for (int j = 0; j < dv; j++) mem[j] = 0.0f;
            for (int i = 0; i < dk; i++) { float ki = kv[i]; const float* row = sh + i * dv; for (int j = 0; j < dv; j++) mem[j] += row[j] * ki; }
            for (int j = 0; j < dv; j++) delta[j] = (vv[j] - mem[j]) * b;
            float* oh = o_all + (int64_t)ti * w + h * dv; for (int j = 0; j < dv; j++) oh[j] = 0.0f;
            for (int i = 0; i < dk; i++) { float ki = kv[i], qi = qv[i]; float* row = sh + i * dv; for (int j = 0; j < dv; j++) { row[j] += ki * delta[j]; oh[j] += row[j] * qi; } }
            rms_inplace(oh, norm, c->eps, dv); const float* zh = zz + (int64_t)ti * w + h * dv; for (int j = 0; j < dv; j++) oh[j] *= sigm(zh[j]);
        }
    }
    free(co_all);
}

/* ------------------------------------------------------------------ gated attention */

void orc_attn_core(const orc_cfg* c, const float* qf, const float* kf_in, const float* vf,
                   const float* qn, const float* kn, const float* inv,
                   float* kc, float* vc, int64_t pos,
                   const uint32_t* kw, const float* ks, const uint32_t* vw, const float* vs, int64_t q4n,
                   float* att) {  /* attn_core :1558-1615, dense branch, one token */
    orc_attn_core_sel(c, qf, kf_in, vf, qn, kn, inv, kc, vc, pos, kw, ks, vw, vs, q4n, NULL, 0, att);
}
/* The same with the key positions the query attends to (`ps`, ascending, `nps` of them; NULL = every position <= pos):
 * the softmax runs over the listed positions only (:1605-1609, `sel`). */
void orc_attn_core_sel(const orc_cfg* c, const float* qf, const float* kf_in, const float* vf,
                       const float* qn, const float* kn, const float* inv,
                       float* kc, float* vc, int64_t pos,
                       const uint32_t* kw, const float* ks, const uint32_t* vw, const float* vs, int64_t q4n,
                       const int64_t* ps, int64_t nps, float* att) {
    int nh = c->n_head, nkv = c->n_kv, hd = c->hd; int row = nkv * hd; int grp = nh / nkv;
    /* k: RMSNorm * kn, rope, append (:1563-1564) */
    float* kf = kc + pos * row; memcpy(kf, kf_in, (size_t)row * 4);
    for (int h = 0; h < nkv; h++) { rms_inplace(kf + h * hd, kn, c->eps, hd); rope(kf + h * hd, pos, inv, c->n_rot); }
    memcpy(vc + pos * row, vf, (size_t)row * 4);
    float scale = 1.0f / sqrtf((float)hd); int64_t n = ps ? nps : pos + 1;
    #pragma omp parallel for schedule(static)
    for (int h = 0; h < nh; h++) {
        float* out = att + h * hd; for (int i = 0; i < hd; i++) out[i] = 0.0f;
        int base = h * 2 * hd; float qh[1024]; memcpy(qh, qf + base, (size_t)hd * 4); rms_inplace(qh, qn, c->eps, hd); rope(qh, pos, inv, c->n_rot);  /* :1603-1604 */
        int kvh = h / grp; float* sc = (float*)malloc((size_t)n * 4); float krow[1024];
        for (int64_t j = 0; j < n; j++) {
            const int64_t p = ps ? ps[j] : j;
            const float* kp;
            if (kw && p < q4n) { for (int i = 0; i < hd; i++) krow[i] = orc_kv4_get(kw, ks, p * row + kvh * hd + i); kp = krow; } else kp = kc + p * row + kvh * hd;
            sc[j] = orc_dot(qh, kp, hd) * scale;
        }
        float mx = -INFINITY; for (int64_t j = 0; j < n; j++) mx = fmaxf(mx, sc[j]);
        float sum = 0.0f; for (int64_t j = 0; j < n; j++) { sc[j] = expf(sc[j] - mx); sum += sc[j]; }
        float invs = 1.0f / sum;
        for (int64_t j = 0; j < n; j++) { const int64_t p = ps ? ps[j] : j; float wgt = sc[j] * invs;
            if (vw && p < q4n) { for (int i = 0; i < hd; i++) out[i] += wgt * orc_kv4_get(vw, vs, p * row + kvh * hd + i); }
            else { const float* vv = vc + p * row + kvh * hd; for (int i = 0; i < hd; i++) out[i] += wgt * vv[i]; } }
        const float* gate = qf + base + hd; for (int i = 0; i < hd; i++) out[i] *= sigm(gate[i]);  /* :1610 */
        free(sc);
    }
}

/* ------------------------------------------------------------------ QSA block-sparse selection (attn_core :1565-1599)
 *
 * Blocks of `ratio` tokens.  Every complete block has a pooled key: the mean of its tokens' raw index keys, RMS-normed
 * with the index key norm, roped at the block's first position.  A query past the dense range (more than
 * budget + ratio - 1 visible tokens, dense_n :1555) scores every complete block with
 *     sum over index heads of relu(q_h . pooled_b) / sqrt(idx_hd),   q_h = rope(rms(raw q_h) * q_norm, pos)
 * and attends to the budget / ratio best blocks plus the incomplete tail.  The reference picks them with
 * select_nth_unstable_by, which leaves the order among equal scores open; here: higher score first, lower block first. */
void orc_qsa_pool(const orc_cfg* c, int ratio, int ihd, const float* ik, const float* ikn, const float* inv, int64_t b, float* out) {
    for (int i = 0; i < ihd; i++) out[i] = 0.0f;
    for (int64_t p = b * ratio; p < (b + 1) * ratio; p++) for (int i = 0; i < ihd; i++) out[i] += ik[p * ihd + i];
    for (int i = 0; i < ihd; i++) out[i] /= (float)ratio;
    rms_inplace(out, ikn, c->eps, ihd); rope(out, b * ratio, inv, c->n_rot);
}
/* blocks[0 .. budget/ratio) <- the selected blocks, ascending; returns their number (0 when the query is in the dense
 * range).  *margin (may be NULL) <- score of the last block taken minus score of the best block left out. */
int orc_qsa_select(const orc_cfg* c, int budget, int ratio, int inh, int ihd, const float* iq_raw, const float* iqn, const float* inv,
                   const float* ib, int64_t pos, int32_t* blocks, float* margin) {
    int64_t n = pos + 1; if (n <= (int64_t)budget + ratio - 1) return 0;
    int64_t nb = n / ratio; int kk = budget / ratio; float iscale = 1.0f / sqrtf((float)ihd);
    float* q = (float*)malloc((size_t)inh * ihd * 4); memcpy(q, iq_raw, (size_t)inh * ihd * 4);
    for (int h = 0; h < inh; h++) { rms_inplace(q + h * ihd, iqn, c->eps, ihd); rope(q + h * ihd, pos, inv, c->n_rot); }
    float* sc = (float*)malloc((size_t)nb * 4); uint8_t* taken = (uint8_t*)calloc((size_t)nb, 1);
    for (int64_t b = 0; b < nb; b++) { float s = 0.0f; for (int h = 0; h < inh; h++) { float d = orc_dot(q + h * ihd, ib + b * ihd, ihd); s += d > 0.0f ? d : 0.0f; } sc[b] = s * iscale; }
    float last = INFINITY;
    for (int j = 0; j < kk; j++) { int64_t best = -1; for (int64_t b = 0; b < nb; b++) if (!taken[b] && (best < 0 || sc[b] > sc[best])) best = b; taken[best] = 1; last = sc[best]; }
    float nxt = -INFINITY; int k = 0;
    for (int64_t b = 0; b < nb; b++) { if (taken[b]) blocks[k++] = (int32_t)b; else nxt = fmaxf(nxt, sc[b]); }
    if (margin) *margin = last - nxt;
    free(q); free(sc); free(taken);
    return k;
}

/* ------------------------------------------------------------------ model / token loop */

typedef struct { orc_mat mat; int has_mat; float* vec; int64_t nvec; } orc_slot;

struct orc_model {
    orc_cfg cfg;
    orc_slot* slots;   /* [(n_layers + 1)][ORC_R_COUNT], index 0 = global */
    float* rope_inv;
    int idx_budget, idx_ratio, idx_nh, idx_hd;   /* QSA indexer (Cfg :24-25); idx_nh = 0: none */    int ple_ngram, ple_per_gram, ple_conv_k, ple_dim; uint32_t ple_eos; uint64_t ple_mult[8], ple_off[32], ple_vocab[32];   /* Cfg :477-480; ple_ngram = 0: none */
};
struct orc_state {
    const orc_model* m;
    int64_t pos;
    float** conv; float** ssm;           /* per linear layer */
    float** k; float** v;                /* per attention layer, f32 [max_ctx][row] (rows < q4n are stale) */
    uint32_t** kw; float** ks; uint32_t** vw; float** vs; int64_t* q4n;
    int n_lin, n_attn;
    float** ik; float** ib;              /* per attention layer: raw index keys [max_ctx][idx_hd], pooled block keys [max_ctx/ratio][idx_hd] (State :194) */
    float logit_margin, router_margin, qsa_margin;
    float* last_x; int64_t last_x_n;      /* final residual rows of the last forward call */    /* n-gram embeddings: the ids fed so far by position (State.tokens), and per layer that has them the normalized rows by
     * position.  The reference keeps the last (conv_k - 1) * ngram rows in a ring (ple_hist :196, drained and extended per token
     * :1432); row (hl - back) of that ring is the row of position p - back (zeros before the sequence starts), which is what
     * the by-position array gives, and a position set back (spec_keep :2508) needs no checkpoint. */
    uint32_t* tokens; float** ple_nrm;
};

static orc_slot* slot(const orc_model* m, int layer, int role) { return &m->slots[(size_t)(layer + 1) * ORC_R_COUNT + role]; }
static const orc_mat* M(const orc_model* m, int layer, int role) { orc_slot* s = slot(m, layer, role); return s->has_mat ? &s->mat : NULL; }
static const float* V(const orc_model* m, int layer, int role) { return slot(m, layer, role)->vec; }
static int is_full(const orc_cfg* c, int il) { return c->full_every > 0 && (il + 1) % c->full_every == 0; }  /* :498 */

orc_model* orc_model_new(const orc_cfg* cfg) {
    orc_model* m = (orc_model*)calloc(1, sizeof *m); m->cfg = *cfg;
    m->slots = (orc_slot*)calloc((size_t)(cfg->n_layers + 1) * ORC_R_COUNT, sizeof(orc_slot));
    m->rope_inv = (float*)malloc((size_t)(cfg->n_rot / 2 + 1) * 4); orc_rope_inv(cfg->n_rot, cfg->rope_base, m->rope_inv);
    m->rope_inv[cfg->n_rot / 2] = 1.0f;
    return m;
}
void orc_model_free(orc_model* m) {
    if (!m) return;
    for (size_t i = 0; i < (size_t)(m->cfg.n_layers + 1) * ORC_R_COUNT; i++) free(m->slots[i].vec);
    free(m->slots); free(m->rope_inv); free(m);
}
/* QSA indexer geometry (Cfg :24-25, keys attention.indexer.* :481-485); layers that have ORC_R_IDX_Q use it */
void orc_model_set_indexer(orc_model* m, int budget, int ratio, int n_head, int head_dim) {
    m->idx_budget = budget; m->idx_ratio = ratio < 1 ? 1 : ratio; m->idx_nh = n_head; m->idx_hd = head_dim;
}
void orc_model_set_ple(orc_model* m, int ngram, int per_gram, int conv_k, uint32_t eos, int dim, const uint64_t* mult, const uint64_t* off, const uint64_t* vocab) {
    m->ple_ngram = ngram; m->ple_per_gram = per_gram; m->ple_conv_k = conv_k; m->ple_eos = eos; m->ple_dim = dim;
    for (int i = 0; i < ngram && i < 8; i++) m->ple_mult[i] = mult[i];
    for (int i = 0; i < (ngram - 1) * per_gram && i < 32; i++) { m->ple_off[i] = off[i]; m->ple_vocab[i] = vocab[i]; }
}
/* ple_rows :1394-1403: a context is cut at the first missing or end-of-sequence predecessor (everything older reads as eos); n-gram size n
 * mixes the first n context ids, each times its multiplier (wrapping), by xor; head h of that size takes the mix modulo its own vocabulary */
void orc_ple_hash(const orc_model* m, const int64_t* ctx_in, int64_t* rows) {
    uint64_t ctx[8]; int cut = 0; ctx[0] = (uint64_t)ctx_in[0];
    for (int s = 1; s < m->ple_ngram; s++) { int none = cut || ctx_in[s] < 0; cut = cut || none || (uint32_t)ctx_in[s] == m->ple_eos; ctx[s] = cut ? (uint64_t)m->ple_eos : (uint64_t)ctx_in[s]; }
    for (int n = 2; n <= m->ple_ngram; n++) {
        uint64_t mixed = ctx[0] * m->ple_mult[0];
        for (int j = 1; j < n; j++) mixed ^= ctx[j] * m->ple_mult[j];
        for (int gi = 0; gi < m->ple_per_gram; gi++) { int h = (n - 2) * m->ple_per_gram + gi; rows[h] = (int64_t)(mixed % m->ple_vocab[h] + m->ple_off[h]); }
    }
}
/* Model::load :490-517: a context (cfg.max_ctx) past the trained length is YaRN-scaled for the whole run */
void orc_model_set_ctx_train(orc_model* m, int64_t ctx_train) {
    m->rope_inv[m->cfg.n_rot / 2] = orc_rope_inv_yarn(m->cfg.n_rot, m->cfg.rope_base, ctx_train, m->cfg.max_ctx, m->rope_inv);
}
int orc_model_set_mat(orc_model* m, int layer, int role, const orc_mat* mat) {
    if (layer < -1 || layer >= m->cfg.n_layers || role < 0 || role >= ORC_R_COUNT) return -1;
    orc_slot* s = slot(m, layer, role); s->mat = *mat; s->has_mat = 1; return 0;
}
int orc_model_set_vec(orc_model* m, int layer, int role, const float* v, int64_t n) {
    if (layer < -1 || layer >= m->cfg.n_layers || role < 0 || role >= ORC_R_COUNT) return -1;
    orc_slot* s = slot(m, layer, role); free(s->vec); s->vec = (float*)malloc((size_t)n * 4); memcpy(s->vec, v, (size_t)n * 4); s->nvec = n; return 0;
}

orc_state* orc_state_new(const orc_model* m) {  /* new_state :1345-1353 */
    const orc_cfg* c = &m->cfg; orc_state* s = (orc_state*)calloc(1, sizeof *s); s->m = m;
    int ch = 2 * c->lin_nk * c->lin_dk + c->lin_nv * c->lin_dv; int row = c->n_kv * c->hd;
    for (int il = 0; il < c->n_layers; il++) { if (is_full(c, il)) s->n_attn++; else s->n_lin++; }
    s->conv = (float**)calloc((size_t)s->n_lin + 1, sizeof(float*)); s->ssm = (float**)calloc((size_t)s->n_lin + 1, sizeof(float*));
    for (int i = 0; i < s->n_lin; i++) { s->conv[i] = (float*)calloc((size_t)(c->conv_k - 1) * ch, 4); s->ssm[i] = (float*)calloc((size_t)c->lin_nv * c->lin_dk * c->lin_dv, 4); }
    int na = s->n_attn + 1;
    s->k = (float**)calloc((size_t)na, sizeof(float*)); s->v = (float**)calloc((size_t)na, sizeof(float*));
    s->kw = (uint32_t**)calloc((size_t)na, sizeof(void*)); s->vw = (uint32_t**)calloc((size_t)na, sizeof(void*));
    s->ks = (float**)calloc((size_t)na, sizeof(void*)); s->vs = (float**)calloc((size_t)na, sizeof(void*)); s->q4n = (int64_t*)calloc((size_t)na, 8);
    s->ik = (float**)calloc((size_t)na, sizeof(void*)); s->ib = (float**)calloc((size_t)na, sizeof(void*));
    if (m->ple_ngram > 0) {
        s->tokens = (uint32_t*)calloc((size_t)c->max_ctx, 4); s->ple_nrm = (float**)calloc((size_t)c->n_layers, sizeof(float*));
        for (int il = 0; il < c->n_layers; il++) if (M(m, il, ORC_R_PLE_KEY)) s->ple_nrm[il] = (float*)calloc((size_t)c->max_ctx * (c->hc > 0 ? c->hc : 1) * c->d, 4);
    }
    for (int i = 0; i < s->n_attn; i++) {
        if (m->idx_nh > 0) { s->ik[i] = (float*)calloc((size_t)c->max_ctx * m->idx_hd, 4); s->ib[i] = (float*)calloc((size_t)(c->max_ctx / m->idx_ratio + 1) * m->idx_hd, 4); }
        s->k[i] = (float*)calloc((size_t)c->max_ctx * row, 4); s->v[i] = (float*)calloc((size_t)c->max_ctx * row, 4);
        if (c->kv_bits == 4) { s->kw[i] = (uint32_t*)calloc((size_t)c->max_ctx * row / 8, 4); s->vw[i] = (uint32_t*)calloc((size_t)c->max_ctx * row / 8, 4);
            s->ks[i] = (float*)calloc((size_t)c->max_ctx * row / 32, 4); s->vs[i] = (float*)calloc((size_t)c->max_ctx * row / 32, 4); }
    }
    return s;
}
void orc_state_free(orc_state* s) {
    if (!s) return;
    for (int i = 0; i < s->n_lin; i++) { free(s->conv[i]); free(s->ssm[i]); }
    for (int i = 0; i < s->n_attn; i++) { free(s->k[i]); free(s->v[i]); free(s->kw[i]); free(s->vw[i]); free(s->ks[i]); free(s->vs[i]); free(s->ik[i]); free(s->ib[i]); }
    if (s->ple_nrm) { for (int il = 0; il < s->m->cfg.n_layers; il++) free(s->ple_nrm[il]); free(s->ple_nrm); } free(s->tokens);
    free(s->ik); free(s->ib); free(s->last_x); free(s->conv); free(s->ssm); free(s->k); free(s->v); free(s->kw); free(s->vw); free(s->ks); free(s->vs); free(s->q4n); free(s);
}
/* Layout rule of the packed region (kv_push :1517-1534): with len positions held, the first
 * q4n = ((len - recent) / 64) * 64 are 4-bit (whole multiples of 64 positions), the rest f32. */
static void kv_repack(orc_state* s, int ai, int64_t len) {
    const orc_cfg* c = &s->m->cfg; if (c->kv_bits != 4 || len <= c->kv_recent) return;
    int row = c->n_kv * c->hd; int64_t want = ((len - c->kv_recent) / 64) * 64;
    if (want <= s->q4n[ai]) return;
    int64_t a = s->q4n[ai], n = (want - a) * row;
    orc_kv4_pack(s->k[ai] + a * row, n, s->kw[ai] + a * row / 8, s->ks[ai] + a * row / 32);
    orc_kv4_pack(s->v[ai] + a * row, n, s->vw[ai] + a * row / 8, s->vs[ai] + a * row / 32);
    s->q4n[ai] = want;
}
int orc_state_fill_kv(orc_state* s, int ai, const float* k, const float* v, int64_t n) {
    const orc_cfg* c = &s->m->cfg; int row = c->n_kv * c->hd; if (ai < 0 || ai >= s->n_attn || n > c->max_ctx) return -1;
    memcpy(s->k[ai], k, (size_t)n * row * 4); memcpy(s->v[ai], v, (size_t)n * row * 4); s->q4n[ai] = 0; kv_repack(s, ai, n); return 0;
}
int orc_state_set_pos(orc_state* s, int64_t pos) { s->pos = pos; return 0; }
void orc_last_margins(const orc_state* s, float* a, float* b) { if (a) *a = s->logit_margin; if (b) *b = s->router_margin; }
float orc_last_qsa_margin(const orc_state* s) { return s->qsa_margin; }   /* smallest selection margin of the last forward call (INFINITY: no sparse query) */

/* hc_mix :1357-1382 (f32 branch).  x [t][hc*d] -> mixed [t][d], inj [t][hc] */
static void hc_mix(const orc_model* m, int layer, int r_norm, int r_down, int r_up, int r_inj, const float* x, int t, float* mixed, float* inj) {
    const orc_cfg* c = &m->cfg; int d = c->d, hc = c->hc, w = hc * d, lr = c->hc_lr;
    const float* norm = V(m, layer, r_norm); const orc_mat* down = M(m, layer, r_down); const orc_mat* up = M(m, layer, r_up); const orc_mat* injm = r_inj >= 0 ? M(m, layer, r_inj) : NULL;
    float* xn = (float*)malloc((size_t)t * w * 4); float* lo = (float*)malloc((size_t)t * lr * 4); float* gate = (float*)malloc((size_t)t * w * 4);
    for (int i = 0; i < t * hc; i++) { int s = i % hc; rms(x + (int64_t)i * d, norm + s * d, c->eps, xn + (int64_t)i * d, d); }
    orc_matmul(down, xn, t, lo); for (int i = 0; i < t * lr; i++) lo[i] = silu(lo[i] / (float)hc);
    if (injm) { orc_matmul(injm, xn, t, inj); for (int i = 0; i < t * hc; i++) inj[i] /= (float)hc; } else for (int i = 0; i < t * hc; i++) inj[i] = 0.0f;
    orc_matmul(up, lo, t, gate);
    for (int ti = 0; ti < t; ti++) { float* mr = mixed + (int64_t)ti * d; for (int i = 0; i < d; i++) mr[i] = 0.0f;
        for (int s = 0; s < hc; s++) for (int i = 0; i < d; i++) { int64_t k = (int64_t)ti * w + s * d + i; mr[i] += xn[k] * sigm(gate[k]); }
        for (int i = 0; i < d; i++) mr[i] /= (float)hc; }
    free(xn); free(lo); free(gate);
}
/* hc_combine :1384-1388 */
static void hc_combine(const orc_cfg* c, float* x, const float* out, const float* inj, int t) {
    int d = c->d, hc = c->hc;
    for (int ti = 0; ti < t; ti++) for (int s = 0; s < hc; s++) { float w = 2.0f * sigm(inj[ti * hc + s]); float* r = x + ((int64_t)ti * hc + s) * d; for (int i = 0; i < d; i++) r[i] += out[(int64_t)ti * d + i] * w; }
}

/* forward_inner :2087-2157 (pure-CPU branch :2134-2142).  hc == 0 selects the plain pre-norm
 * residual form (x += mixer(rms(x)*attn_norm); x += ffn(rms(x)*ffn_norm); head on rms(x)*out_norm),
 * which the reference does not have; hc >= 1 is the reference's hyper-connection plumbing. */
/* ple :1409-1434 for one token at position pos: the table rows `emb` projected to a key per stream and one value; per stream a
 * gate from the normalized key and the normalized stream, value times gate, normalized again; x += gated + silu(depthwise conv over
 * the normalized rows of this and of earlier positions, conv_k taps ngram positions apart) */
static void ple_token(const orc_model* m, int il, float* nrm_all, const float* key, const float* val, float* xt, int64_t pos) {
    const orc_cfg* c = &m->cfg; int d = c->d, hcn = c->hc > 0 ? c->hc : 1, w = hcn * d, kk = m->ple_conv_k, dil = m->ple_ngram;
    const float* nk = V(m, il, ORC_R_PLE_NORM_KEY); const float* nq = V(m, il, ORC_R_PLE_NORM_QUERY); const float* nc = V(m, il, ORC_R_PLE_NORM_CONV); const float* cv = V(m, il, ORC_R_PLE_CONV);
    float* gated = (float*)malloc((size_t)w * 4); float* kn = (float*)malloc((size_t)d * 4); float* q = (float*)malloc((size_t)d * 4);
    float* nrm = nrm_all + pos * w;
    for (int s = 0; s < hcn; s++) {
        memcpy(kn, key + (int64_t)s * d, (size_t)d * 4); rms_inplace(kn, nk + (int64_t)s * d, c->eps, d);
        rms(xt + (int64_t)s * d, nq + (int64_t)s * d, c->eps, q, d);
        float sc = orc_dot(kn, q, d) / sqrtf((float)d);
        float g = sigm((signbit(sc) ? -1.0f : 1.0f) * sqrtf(fmaxf(fabsf(sc), 1e-6f)));
        for (int i = 0; i < d; i++) gated[s * d + i] = val[i] * g;
    }
    memcpy(nrm, gated, (size_t)w * 4);
    for (int s = 0; s < hcn; s++) rms_inplace(nrm + (int64_t)s * d, nc + (int64_t)s * d, c->eps, d);
    for (int ch = 0; ch < w; ch++) {
        float o = cv[ch * kk + kk - 1] * nrm[ch];
        for (int k = 0; k < kk - 1; k++) { int64_t p = pos - (int64_t)(kk - 1 - k) * dil; o += cv[ch * kk + k] * (p >= 0 ? nrm_all[p * w + ch] : 0.0f); }
        xt[ch] += gated[ch] + silu(o);
    }
    free(gated); free(kn); free(q);
}

/* ple_token for callers outside the forward pass (tests): nrm_all = rows by position [max positions][streams * d] */
void orc_ple_token(const orc_model* m, int il, float* nrm_all, const float* key, const float* val, float* xt, int64_t pos) { ple_token(m, il, nrm_all, key, val, xt, pos); }

int orc_forward(const orc_model* m, orc_state* st, const uint32_t* ids, int t, float* logits) {
    const orc_cfg* c = &m->cfg; int d = c->d, hc = c->hc; int xw = (hc > 0 ? hc : 1) * d; int64_t start = st->pos;
    if (start + t > c->max_ctx) return -2;
    float* x = (float*)malloc((size_t)t * xw * 4); float* mx = (float*)malloc((size_t)t * d * 4); float* o = (float*)malloc((size_t)t * d * 4); float* inj = (float*)malloc((size_t)t * (hc > 0 ? hc : 1) * 4);
    const orc_mat* embd = M(m, -1, ORC_R_TOKEN_EMBD);
    for (int ti = 0; ti < t; ti++) { orc_mat_row(embd, ids[ti], o); for (int s = 0; s < (hc > 0 ? hc : 1); s++) memcpy(x + ((int64_t)ti * (hc > 0 ? hc : 1) + s) * d, o, (size_t)d * 4); }  /* :2092 */
    /* :2089, 2093: the ids join the history, then the table rows of every fed position (shared by all layers that use them) */
    float* pemb = NULL; const int pnh = m->ple_ngram > 0 ? (m->ple_ngram - 1) * m->ple_per_gram : 0; const orc_mat* ptab = M(m, -1, ORC_R_PLE_TAB);
    if (pnh > 0 && ptab) {
        pemb = (float*)malloc((size_t)t * pnh * m->ple_dim * 4);
        for (int ti = 0; ti < t; ti++) st->tokens[start + ti] = ids[ti];
        for (int ti = 0; ti < t; ti++) {
            int64_t ctx[8], rows[32]; int64_t p = start + ti;
            for (int s = 0; s < m->ple_ngram; s++) ctx[s] = p >= s ? (int64_t)st->tokens[p - s] : -1;
            orc_ple_hash(m, ctx, rows);
            for (int h = 0; h < pnh; h++) orc_mat_row(ptab, rows[h], pemb + ((int64_t)ti * pnh + h) * m->ple_dim);
        }
    }
    int li = 0, ai = 0; st->router_margin = INFINITY; st->qsa_margin = INFINITY;
    int nk = c->lin_nk, nv = c->lin_nv, dk = c->lin_dk, dv = c->lin_dv; int ch = 2 * nk * dk + nv * dv; int row = c->n_kv * c->hd;
    for (int il = 0; il < c->n_layers; il++) {
        if (pemb && M(m, il, ORC_R_PLE_KEY)) {   /* :2112 */
            float* key = (float*)malloc((size_t)t * xw * 4); float* val = (float*)malloc((size_t)t * d * 4);
            orc_matmul(M(m, il, ORC_R_PLE_KEY), pemb, t, key); orc_matmul(M(m, il, ORC_R_PLE_VALUE), pemb, t, val);
            for (int ti = 0; ti < t; ti++) ple_token(m, il, st->ple_nrm[il], key + (int64_t)ti * xw, val + (int64_t)ti * d, x + (int64_t)ti * xw, start + ti);
            free(key); free(val);
        }
        if (hc > 0) hc_mix(m, il, ORC_R_HCA_NORM, ORC_R_HCA_DOWN, ORC_R_HCA_UP, ORC_R_HCA_INJECT, x, t, mx, inj);
        else for (int ti = 0; ti < t; ti++) rms(x + (int64_t)ti * d, V(m, il, ORC_R_ATTN_NORM), c->eps, mx + (int64_t)ti * d, d);
        if (is_full(c, il)) {  /* attn :1441-1446 */
            int nq = c->n_head * 2 * c->hd; float* qf = (float*)malloc((size_t)t * nq * 4); float* kf = (float*)malloc((size_t)t * row * 4); float* vf = (float*)malloc((size_t)t * row * 4); float* att = (float*)malloc((size_t)t * c->n_head * c->hd * 4);
            orc_matmul(M(m, il, ORC_R_ATTN_Q), mx, t, qf); orc_matmul(M(m, il, ORC_R_ATTN_K), mx, t, kf); orc_matmul(M(m, il, ORC_R_ATTN_V), mx, t, vf);
            /* QSA indexer: two more projections of the same input (:1567-1569) */
            const int qsa = m->idx_nh > 0 && M(m, il, ORC_R_IDX_Q) != NULL; const int inh = m->idx_nh, ihd = m->idx_hd, ir = m->idx_ratio;
            float* iqf = NULL; float* ikf = NULL; int32_t* blk = NULL; int64_t* ps = NULL;
            if (qsa) { iqf = (float*)malloc((size_t)t * inh * ihd * 4); ikf = (float*)malloc((size_t)t * ihd * 4); blk = (int32_t*)malloc((size_t)(m->idx_budget / ir + 1) * 4); ps = (int64_t*)malloc((size_t)(m->idx_budget + 2 * ir) * 8);
                orc_matmul(M(m, il, ORC_R_IDX_Q), mx, t, iqf); orc_matmul(M(m, il, ORC_R_IDX_K), mx, t, ikf); }
            for (int ti = 0; ti < t; ti++) {
                int64_t pos = start + ti;
                /* the packed boundary follows the row count after the append (pos + 1 rows); the rows it
                 * covers are all older than the recent window, so they are already normed and roped */
                kv_repack(st, ai, pos + 1);
                int64_t nps = 0;
                if (qsa) {
                    memcpy(st->ik[ai] + pos * ihd, ikf + (int64_t)ti * ihd, (size_t)ihd * 4);
                    if ((pos + 1) % ir == 0) orc_qsa_pool(c, ir, ihd, st->ik[ai], V(m, il, ORC_R_IDX_K_NORM), m->rope_inv, pos / ir, st->ib[ai] + (pos / ir) * ihd);
                    float mg; int k = orc_qsa_select(c, m->idx_budget, ir, inh, ihd, iqf + (int64_t)ti * inh * ihd, V(m, il, ORC_R_IDX_Q_NORM), m->rope_inv, st->ib[ai], pos, blk, &mg);
                    if (k > 0) { for (int j = 0; j < k; j++) for (int e = 0; e < ir; e++) ps[nps++] = (int64_t)blk[j] * ir + e;
                        for (int64_t p = ((pos + 1) / ir) * ir; p <= pos; p++) ps[nps++] = p;
                        st->qsa_margin = fminf(st->qsa_margin, mg); }
                }
                orc_attn_core_sel(c, qf + (int64_t)ti * nq, kf + (int64_t)ti * row, vf + (int64_t)ti * row, V(m, il, ORC_R_ATTN_Q_NORM), V(m, il, ORC_R_ATTN_K_NORM), m->rope_inv,
                                  st->k[ai], st->v[ai], pos, st->kw[ai], st->ks[ai], st->vw[ai], st->vs[ai], st->q4n[ai], nps > 0 ? ps : NULL, nps, att + (int64_t)ti * c->n_head * c->hd);
            }
            free(iqf); free(ikf); free(blk); free(ps);
            orc_matmul(M(m, il, ORC_R_ATTN_O), att, t, o); free(qf); free(kf); free(vf); free(att); ai++;
        } else {  /* linear :1617-1621 */
            float* qkv = (float*)malloc((size_t)t * ch * 4); float* z = (float*)malloc((size_t)t * nv * dv * 4); float* be = (float*)malloc((size_t)t * nv * 4); float* al = (float*)malloc((size_t)t * nv * 4); float* oa = (float*)malloc((size_t)t * nv * dv * 4);
            orc_matmul(M(m, il, ORC_R_LIN_QKV), mx, t, qkv); orc_matmul(M(m, il, ORC_R_LIN_Z), mx, t, z); orc_matmul(M(m, il, ORC_R_LIN_BETA), mx, t, be); orc_matmul(M(m, il, ORC_R_LIN_ALPHA), mx, t, al);
            orc_linear_core(c, qkv, z, be, al, V(m, il, ORC_R_LIN_A), V(m, il, ORC_R_LIN_DT), V(m, il, ORC_R_LIN_CONV), V(m, il, ORC_R_LIN_NORM), st->conv[li], st->ssm[li], t, oa);
            orc_matmul(M(m, il, ORC_R_LIN_OUT), oa, t, o); free(qkv); free(z); free(be); free(al); free(oa); li++;
        }
        if (hc > 0) { hc_combine(c, x, o, inj, t); hc_mix(m, il, ORC_R_HCF_NORM, ORC_R_HCF_DOWN, ORC_R_HCF_UP, ORC_R_HCF_INJECT, x, t, mx, inj); }
        else { for (int64_t i = 0; i < (int64_t)t * d; i++) x[i] += o[i]; for (int ti = 0; ti < t; ti++) rms(x + (int64_t)ti * d, V(m, il, ORC_R_FFN_NORM), c->eps, mx + (int64_t)ti * d, d); }
        {
            int32_t* sel = (int32_t*)malloc((size_t)t * c->top_k * 4);
            orc_moe(c, M(m, il, ORC_R_ROUTER), M(m, il, ORC_R_EXP_GATE), M(m, il, ORC_R_EXP_UP), M(m, il, ORC_R_EXP_DOWN), M(m, il, ORC_R_SH_GATE), M(m, il, ORC_R_SH_UP), M(m, il, ORC_R_SH_DOWN), V(m, il, ORC_R_SH_GATE_INP), mx, t, o, sel, NULL);
            /* 10th/11th router margin of the last token, for near-tie classification */
            { float* lg = (float*)malloc((size_t)c->n_exp * 4); orc_mat rt = *M(m, il, ORC_R_ROUTER); orc_matmul(&rt, mx + (int64_t)(t - 1) * d, 1, lg);
              float kth = INFINITY; for (int j = 0; j < c->top_k; j++) kth = fminf(kth, lg[sel[(t - 1) * c->top_k + j]]);
              float nxt = -INFINITY; for (int e = 0; e < c->n_exp; e++) { int in = 0; for (int j = 0; j < c->top_k; j++) if (sel[(t - 1) * c->top_k + j] == e) in = 1; if (!in) nxt = fmaxf(nxt, lg[e]); }
              st->router_margin = fminf(st->router_margin, kth - nxt); free(lg); }
            free(sel);
        }
        if (hc > 0) hc_combine(c, x, o, inj, t); else for (int64_t i = 0; i < (int64_t)t * d; i++) x[i] += o[i];
    }
    st->last_x = (float*)realloc(st->last_x, (size_t)t * xw * 4); memcpy(st->last_x, x, (size_t)t * xw * 4); st->last_x_n = (int64_t)t * xw;   /* mtp_keep_r :2150 */
    const float* last = x + (int64_t)(t - 1) * xw;
    if (hc > 0) hc_mix(m, -1, ORC_R_OUT_HC_NORM, ORC_R_OUT_HC_DOWN, ORC_R_OUT_HC_UP, -1, last, 1, mx, inj);  /* :2152 */
    else rms(last, V(m, -1, ORC_R_OUT_NORM), c->eps, mx, d);
    const orc_mat* out = M(m, -1, ORC_R_OUTPUT); if (!out) out = embd;                                          /* :511 */
    orc_matmul(out, mx, 1, logits);                                                                              /* head_logits :2361-2364 */
    { uint32_t b = orc_argmax(logits, c->vocab); float second = -INFINITY; for (int i = 0; i < c->vocab; i++) if ((uint32_t)i != b) second = fmaxf(second, logits[i]); st->logit_margin = logits[b] - second; }
    st->pos = start + t;
    free(x); free(mx); free(o); free(inj); free(pemb);
    return 0;
}

int orc_last_residual(const orc_state* s, float* out, int64_t cap_floats) {
    if (!s->last_x || s->last_x_n > cap_floats) return -1;
    memcpy(out, s->last_x, (size_t)s->last_x_n * 4); return (int)s->last_x_n;
}

/* ------------------------------------------------------------------ MTP drafter (src/model/mtp.rs) */
void orc_mtp_cell(const orc_model* dm, orc_state* ds, const float* R, const float* emb, int64_t pos, int64_t c0, int window, int full, float* s_out, float* rr_out) {
    const orc_cfg* c = &dm->cfg; int d = c->d, hc = c->hc, w = hc * d; int row = c->n_kv * c->hd; int nq = c->n_head * 2 * c->hd;
    float* en = (float*)malloc((size_t)d * 4); float* e2 = (float*)malloc((size_t)d * 4); float* hn = (float*)malloc((size_t)w * 4); float* rr = (float*)malloc((size_t)w * 4);
    float* m = (float*)malloc((size_t)d * 4); float* inj = (float*)malloc((size_t)hc * 4); float* o = (float*)malloc((size_t)d * 4);
    /* input :186-195: e = fc_embedding(rms(embed) * pre_e), h = fc_hidden per stream of rms over all hc*d values * pre_h, R' = h + e */
    rms(emb, V(dm, -1, ORC_R_MTP_PRE_E), c->eps, en, d); orc_matmul(M(dm, -1, ORC_R_MTP_FC_E), en, 1, e2);
    rms(R, V(dm, -1, ORC_R_MTP_PRE_H), c->eps, hn, w); orc_matmul(M(dm, -1, ORC_R_MTP_FC_H), hn, hc, rr);
    for (int s = 0; s < hc; s++) for (int i = 0; i < d; i++) rr[s * d + i] += e2[i];
    /* kv_append :156-170 */
    hc_mix(dm, 0, ORC_R_HCA_NORM, ORC_R_HCA_DOWN, ORC_R_HCA_UP, ORC_R_HCA_INJECT, rr, 1, m, inj);
    float* kf = (float*)malloc((size_t)row * 4); float* vf = (float*)malloc((size_t)row * 4);
    orc_matmul(M(dm, 0, ORC_R_ATTN_K), m, 1, kf); orc_matmul(M(dm, 0, ORC_R_ATTN_V), m, 1, vf);
    if (!full) {
        float* kd = ds->k[0] + pos * row; memcpy(kd, kf, (size_t)row * 4);
        for (int h = 0; h < c->n_kv; h++) { rms_inplace(kd + h * c->hd, V(dm, 0, ORC_R_ATTN_K_NORM), c->eps, c->hd); rope(kd + h * c->hd, pos, dm->rope_inv, c->n_rot); }
        memcpy(ds->v[0] + pos * row, vf, (size_t)row * 4);
    } else {
        /* step :184-236: dense attention over the window of cells, MoE, final mixer */
        float* qf = (float*)malloc((size_t)nq * 4); float* att = (float*)malloc((size_t)c->n_head * c->hd * 4);
        orc_matmul(M(dm, 0, ORC_R_ATTN_Q), m, 1, qf);
        int64_t lo = pos - window + 1; if (lo < c0) lo = c0; int64_t nps = pos - lo + 1; int64_t* ps = (int64_t*)malloc((size_t)nps * 8);
        for (int64_t j = 0; j < nps; j++) ps[j] = lo + j;
        orc_attn_core_sel(c, qf, kf, vf, V(dm, 0, ORC_R_ATTN_Q_NORM), V(dm, 0, ORC_R_ATTN_K_NORM), dm->rope_inv, ds->k[0], ds->v[0], pos, NULL, NULL, NULL, NULL, 0, ps, nps, att);
        orc_matmul(M(dm, 0, ORC_R_ATTN_O), att, 1, o); hc_combine(c, rr, o, inj, 1);
        hc_mix(dm, 0, ORC_R_HCF_NORM, ORC_R_HCF_DOWN, ORC_R_HCF_UP, ORC_R_HCF_INJECT, rr, 1, m, inj);
        int32_t* sel = (int32_t*)malloc((size_t)c->top_k * 4);
        orc_moe(c, M(dm, 0, ORC_R_ROUTER), M(dm, 0, ORC_R_EXP_GATE), M(dm, 0, ORC_R_EXP_UP), M(dm, 0, ORC_R_EXP_DOWN), M(dm, 0, ORC_R_SH_GATE), M(dm, 0, ORC_R_SH_UP), M(dm, 0, ORC_R_SH_DOWN), V(dm, 0, ORC_R_SH_GATE_INP), m, 1, o, sel, NULL);
        hc_combine(c, rr, o, inj, 1);
        hc_mix(dm, -1, ORC_R_OUT_HC_NORM, ORC_R_OUT_HC_DOWN, ORC_R_OUT_HC_UP, -1, rr, 1, s_out, inj);
        memcpy(rr_out, rr, (size_t)w * 4);
        free(qf); free(att); free(ps); free(sel);
    }
    free(en); free(e2); free(hn); free(rr); free(m); free(inj); free(o); free(kf); free(vf);
}
