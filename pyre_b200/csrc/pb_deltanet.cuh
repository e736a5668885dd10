// Gated DeltaNet decode step for one (sequence, V head, slice of state columns): the arithmetic shared by the
// stand-alone kernel (pb_deltanet.cu) and the fused step kernel (pb_step.cu), so that both produce the same bits.
//
// Restates linear_core of the reference (src/model/qwen4exp_gguf.rs:1624-1673; GPU twins k_conv / k_delta,
// src/model/qn_cube.rs:2753-2839).  256 threads: a warp owns RPW = dk / 8 state rows i, a lane one column j, so every
// row access is a coalesced 128-byte line and the two reductions over i (S^T k and S^T q) are RPW FMAs per lane
// plus a sum across the 8 warps in shared memory.
//
// The caller supplies a policy P with
//   P::sync()            barrier over the 256 threads that run the unit
//   p.wait_inputs()      returns once this step's projections (p.proj) are complete and visible; everything read
//                        before it (recurrent state, conv history and weights, gate constants) was written by
//                        earlier steps
#pragma once
#include "pb_common.cuh"
#include "pb_internal.h"

#define DN_THREADS 256
#define DN_COLS 32   // state columns per unit

// sm: (2 * dk + DN_COLS * NS + 8 * DN_COLS) floats of shared memory, nrm: 2 floats of shared memory
template <int RPW, int NS, class P>
__device__ __forceinline__ void pb_deltanet_unit(const PbDeltaParams& p, int64_t pos, int h, int j0, int b, int tid, bool early, float* sm, float* nrm, P& pol,
                                                 unsigned long long* stamps, bool st_first) {
    const int nk = p.nk, nv = p.nv, dk = p.dk, dv = p.dv, K = p.conv_k;
    const int ch = 2 * nk * dk + nv * dv;
    const int kh = h % nk;                                  // V head h reads K head h % nk (:1655)
    const int warp = tid >> 5, lane = tid & 31;
    const float* proj = p.proj + (size_t)b * p.ldp;        // [qkv (ch) | z | beta | alpha]
    float* ring = p.conv + (size_t)b * K * ch;             // [K slots][ch]
    const int wslot = (int)(pos % K);                       // slot that receives the current input (pos = the sequence's position)
    // slot of history entry k (oldest first): (pos + 1 + k) mod K, in 32-bit arithmetic from here on

    // the state slice is requested first: rows i in [warp*rpw, (warp+1)*rpw), column j0 + lane; its DRAM
    // latency then overlaps the conv / norm / gate phases below, which do not depend on it
    constexpr int rpw = RPW;   // rows per warp = dk / 8 (16 for dk = 128)
    float* S = p.ssm + (((size_t)b * nv + h) * dk) * dv + j0 + lane;
    float s[RPW];
    if (early) {
#pragma unroll
        for (int r = 0; r < rpw; r++) s[r] = S[(size_t)(warp * rpw + r) * dv];
    }
    // conv weights and history of this thread's channels (at most two: 2 dk + DN_COLS NS <= 2 * 256 for the built shapes),
    // and the gate constants: none of them depends on this step's projections
    const int nel = 2 * dk + DN_COLS * NS;
    constexpr int KMAX = 4;    // the early loads are built for conv kernels of 4 taps (every model so far); others load late
    float cw[2][KMAX], hist[2][KMAX - 1];
    int cidx[2];
    const bool pre = nel <= 2 * DN_THREADS && K == KMAX;
    if (pre) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int i = tid + e * DN_THREADS;
            int c = 0;
            if (i < nel) {
                if (i < dk) c = kh * dk + i;
                else if (i < 2 * dk) c = nk * dk + kh * dk + (i - dk);
                else c = 2 * nk * dk + h * dv + j0 + (i - 2 * dk);
#pragma unroll
                for (int k = 0; k < KMAX; k++) cw[e][k] = p.conv_w[c * KMAX + k];
#pragma unroll
                for (int k = 0; k < KMAX - 1; k++) hist[e][k] = ring[(size_t)((wslot + 1 + k) % KMAX) * ch + c];
            }
            cidx[e] = c;
        }
    }
    const float dt_h = p.dt[h], a_h = p.a[h];

    pol.wait_inputs();
    pb_stamp(stamps, 2, st_first);

    float* qs = sm;              // [dk] normalized q
    float* ks = sm + dk;         // [dk] normalized k
    float* vs = sm + 2 * dk;     // [DN_COLS * NS]
    float* red = sm + 2 * dk + DN_COLS * NS;   // [8 warps][DN_COLS]

    // 1) conv + SiLU for the channels this unit needs: q and k of head kh, v columns j0..j0+31 of head h
    //    o = w[c*K + K-1] * cur + sum_{k < K-1} w[c*K + k] * hist[k]  (hist oldest first)   (:1645)
    if (pre) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int i = tid + e * DN_THREADS;
            if (i < nel) {
                const int c = cidx[e];
                const float cur = __ldcg(proj + c);
                float o = cw[e][KMAX - 1] * cur;
#pragma unroll
                for (int k = 0; k < KMAX - 1; k++) o = fmaf(cw[e][k], hist[e][k], o);
                const float co = pb_silu(o);
                if (i < dk) qs[i] = co; else if (i < 2 * dk) ks[i - dk] = co; else vs[i - 2 * dk] = co;
                // the history slot of this step: q/k channels are written by the first V head that maps
                // to K head kh (slice 0); v channels by their own unit
                const bool owner = i >= 2 * dk || (h == kh && j0 == 0);
                if (owner) ring[(size_t)wslot * ch + c] = cur;
            }
        }
    } else {
        for (int i = tid; i < nel; i += DN_THREADS) {
            int c;
            if (i < dk) c = kh * dk + i;
            else if (i < 2 * dk) c = nk * dk + kh * dk + (i - dk);
            else c = 2 * nk * dk + h * dv + j0 + (i - 2 * dk);
            const float cur = __ldcg(proj + c);
            float o = p.conv_w[c * K + K - 1] * cur;
            for (int k = 0; k < K - 1; k++) o = fmaf(p.conv_w[c * K + k], ring[(size_t)((wslot + 1 + k) % K) * ch + c], o);
            const float co = pb_silu(o);
            if (i < dk) qs[i] = co; else if (i < 2 * dk) ks[i - dk] = co; else vs[i - 2 * dk] = co;
            const bool owner = i >= 2 * dk || (h == kh && j0 == 0);
            if (owner) ring[(size_t)wslot * ch + c] = cur;
        }
    }
    // 3') gate inputs, requested before the norm phase
    const float alpha = __ldcg(proj + ch + nv * dv + nv + h), beta = __ldcg(proj + ch + nv * dv + h);
    P::sync();
    // 2) L2 norms: x * (1/sqrt(sum x^2 + 1e-6)) * scale, q scaled by 1/sqrt(dk)  (:1650-1651)
    if (warp < 2) {
        const float* src = warp == 0 ? qs : ks;
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) ss = fmaf(src[i], src[i], ss);
        ss = pb_warp_sum(ss);
        if (lane == 0) nrm[warp] = 1.0f / sqrtf(ss + 1e-6f) * (warp == 0 ? 1.0f / sqrtf((float)dk) : 1.0f);
    }
    P::sync();
    for (int i = tid; i < 2 * dk; i += DN_THREADS) sm[i] *= nrm[i < dk ? 0 : 1];
    P::sync();
    pb_stamp(stamps, 3, st_first);   // conv and norms done

    // 3) gates (:1660)
    const float g = expf(pb_softplus(alpha + dt_h) * a_h);
    const float bt = pb_sigm(beta);

    // 4) state slices (the first one was requested at the top when `early`)
#pragma unroll 1
    for (int sl = 0; sl < NS; sl++) {
        float* Ss = S + sl * DN_COLS;
        float mem = 0.f;
#pragma unroll
        for (int r = 0; r < rpw; r++) {
            const int i = warp * rpw + r;
            s[r] = ((early && sl == 0) ? s[r] : Ss[(size_t)i * dv]) * g;   // S *= g
            mem = fmaf(s[r], ks[i], mem);           // mem_j = sum_i S[i][j] k_i
        }
        if (sl > 0) P::sync();                      // the previous slice's readers of red are done
        red[warp * DN_COLS + lane] = mem;
        P::sync();
        mem = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) mem += red[w * DN_COLS + lane];
        const float delta = (vs[sl * DN_COLS + lane] - mem) * bt;  // (:1663)
        P::sync();
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < rpw; r++) {
            const int i = warp * rpw + r;
            s[r] = fmaf(ks[i], delta, s[r]);        // S[i][j] += k_i * delta_j
            o = fmaf(s[r], qs[i], o);                // o_j = sum_i S[i][j] q_i
            Ss[(size_t)i * dv] = s[r];
        }
        red[warp * DN_COLS + lane] = o;
        P::sync();
        if (warp == 0) {
            o = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) o += red[w * DN_COLS + lane];
            p.out[(size_t)b * p.ldo + h * dv + j0 + sl * DN_COLS + lane] = o;   // readout before the gated norm
        }
    }
}
