// Fused decode step for one sequence: ONE persistent kernel walks a list of operations (projection GEMVs, Gated
// DeltaNet update, router, expert gate/up, expert down + combine) for a run of layers.
//
// Why: at one token every operation of the step moves a few MB, which the GPU streams in microseconds, while a
// kernel launch, its set-up and the wait for its first bytes cost more than that.  Here
//   - one CTA per SM stays resident for the whole run of layers: 16 consumer warps, 1 producer warp, 1 sync warp;
//   - the producer warp streams the weights of ALL operations, in program order, through one shared-memory ring of
//     1-D bulk (TMA) copies.  Weights do not depend on activations, so it runs ahead of the consumers across
//     operation boundaries: when the consumers reach an operation its first stages have already landed.  Only
//     the routed experts' rows wait for the routing result (top-k + softmax of the router logits, computed by the
//     consumers of every CTA with two rank-counting passes over shared memory);
//   - operations hand activations to each other through global memory (L2) and a grid-wide barrier: a monotonic
//     arrival counter in global memory, release / acquire at GPU scope.  The sync warp runs it: the consumer warps
//     announce "this CTA is done with the previous operation" on a shared-memory mbarrier and go on with work that
//     does not depend on other CTAs (norm weights, DeltaNet state, conv history, the shared expert's rows), the sync
//     warp publishes the arrival, polls the counter and releases them through a second mbarrier.  A consumer's
//     loads in flight therefore never delay its CTA's arrival;
//   - every wait is bounded: a time-out sets the device status word and ends the kernel instead of hanging the GPU;
//   - each warp keeps its own shared-memory copy of the operation it works on and requests the next one early: fields
//     read again after a barrier cost a shared-memory access, not a trip to L2.
// The arithmetic of every operation is the same code as the stand-alone kernels (pb_gemvq.cu, pb_moe.cu,
// pb_deltanet.cu), so both paths give the same bits.
//
// Replaces, for batch 1, the per-layer launch sequence of layer_cube (src/model/qwen4exp_gguf.rs:728-895).
#include "pb_stream.cuh"
#include "pb_step.cuh"
#include "pb_topk.cuh"
#include "pb_router.cuh"
#include "pb_deltanet.cuh"

#include <stdio.h>

#define PS_CT (PB_CONSUMERS * 32)     // consumer threads
#define PS_WARPS (PB_CONSUMERS + 2)   // + producer warp + sync warp
#define PS_THREADS (PS_WARPS * 32)
#define PS_FMT PB_T_IQ3S_N4
#define PS_GRID_SPIN (1u << 22)
#define PS_SLICE_ROWS 16              // output rows per expert slice of the down operation
#define PS_MAX_SLOTS 16
#define PS_OPBUF_OFF 2048             // per-warp copies of the running operation: PS_WARPS x 256 bytes

enum : int { PB_DEV_GRID_TIMEOUT = 4 };   // a grid barrier of the fused step was not completed in time

// misc area at the start of dynamic shared memory
struct PsMisc {
    uint64_t full[PS_STAGES], empty[PS_STAGES];
    uint64_t req, done;            // grid barrier: consumers -> sync warp, sync warp -> consumers
    int route_seq;                 // number of tokens routed so far in this launch (consumers -> producer warp)
    float red[PB_CONSUMERS];
    int route_e[PS_MAX_SLOTS];
    float route_w[PS_MAX_SLOTS];
    float gu[2][2][32];
    float res[PS_MAX_SLOTS * PS_SLICE_ROWS];
    float nrm[2];
    int abort;
};
static_assert(sizeof(PsMisc) <= PS_OPBUF_OFF, "misc area");

struct PsCtx {
    PsMisc* m;
    uint8_t* stages; uint32_t stage_bytes;
    float* xf; float* nw; uint32_t* xq;
    unsigned nbar;    // grid barriers this thread has arrived at
    unsigned ngu;     // gate/up operations seen (phase of the `route` barrier)
    int k;            // chunks of this CTA consumed (consumers) / issued (producer) so far
    int* status;
    int tid, warp, lane;
    int64_t pos;
    unsigned long long* trace;   // per-CTA stamps of the running operation, or null
};

__device__ __forceinline__ unsigned long long ps_ld_acquire(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint8_t* ps_stage(const PsCtx& c, int k) { return c.stages + (size_t)(k % PS_STAGES) * c.stage_bytes; }
__device__ __forceinline__ bool ps_wait_full(PsCtx& c, int k) { return pb_mbar_wait(&c.m->full[k % PS_STAGES], (k / PS_STAGES) & 1, c.status, PB_DEV_WAIT_FULL_TIMEOUT); }
__device__ __forceinline__ void ps_release(PsCtx& c, int k) { __syncwarp(); if (c.lane == 0) pb_mbar_arrive(&c.m->empty[k % PS_STAGES]); }
// producer, one thread: make the stage of chunk k writable and announce `bytes`
__device__ __forceinline__ bool ps_acquire(PsCtx& c, int k, uint32_t bytes) {
    const int s = k % PS_STAGES;
    if (k >= PS_STAGES && !pb_mbar_wait_relaxed(&c.m->empty[s], ((k / PS_STAGES) - 1) & 1, c.status, PB_DEV_WAIT_EMPTY_TIMEOUT)) return false;
    pb_mbar_expect_tx(&c.m->full[s], bytes);
    return true;
}
__device__ __forceinline__ void ps_copy(PsCtx& c, int k, uint32_t off, const void* src, uint32_t bytes) { pb_bulk_g2s(ps_stage(c, k) + off, src, bytes, &c.m->full[k % PS_STAGES]); }

// tracing: fine-grained stamps of CTA 0's first thread inside an operation (32 words after the per-CTA stamps)
__device__ __forceinline__ void ps_fine(const PsCtx& c, int n) { if (c.trace && c.tid == 0 && blockIdx.x == 0) c.trace[4 * gridDim.x + n] = pb_globaltimer(); }

// The activation split is kept as ONE non-inlined copy (scalar arguments only, so nothing is forced into local memory): the
// kernel is larger than the instruction cache, and a shared copy stays resident because some operation calls it every few
// microseconds.
__device__ __noinline__ void ps_split(float4 v, int lane, int g0, int cols, uint32_t* col) { pb_split_groups4<false>(v, lane, g0, cols, col); }

// Grid barrier, consumer side.  arrive: this warp is done with everything the previous operation stores (every consumer
// warp calls it once per barrier).  wait: returns once every CTA has arrived and their stores are visible; false after a
// time-out (the status word is set, the caller leaves the kernel).
__device__ __forceinline__ void ps_bar_arrive(PsCtx& c) {
    c.nbar++;
    __syncwarp();
    if (c.lane == 0) pb_mbar_arrive(&c.m->req);
}
__device__ __forceinline__ bool ps_bar_wait(PsCtx& c) {
    int ok = 1;
    if (c.lane == 0) ok = pb_mbar_wait(&c.m->done, (c.nbar - 1) & 1, c.status, PB_DEV_GRID_TIMEOUT) ? 1 : 0;
    __syncwarp();
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (c.trace && c.tid == 0) c.trace[4 * blockIdx.x + 1] = pb_globaltimer();
    return ok && *reinterpret_cast<volatile int*>(&c.m->abort) == 0;
}

// The warp's copy of operation i: lanes 0..15 hold 16 bytes each of the next operation (requested one operation
// earlier), store them to the warp's slot and request the one after.
struct PsOpFetch {
    uint4 nxt;
    __device__ __forceinline__ void request(const PbStepOp* ops, int i, int end, int lane) {
        if (i < end && lane < (int)(sizeof(PbStepOp) / 16)) nxt = __ldg(reinterpret_cast<const uint4*>(ops + i) + lane);
    }
    __device__ __forceinline__ const PbStepOp& take(uint8_t* slot, int lane) {
        __syncwarp();   // the warp is done reading the previous operation from the slot
        if (lane < (int)(sizeof(PbStepOp) / 16)) reinterpret_cast<uint4*>(slot)[lane] = nxt;
        __syncwarp();
        return *reinterpret_cast<const PbStepOp*>(slot);
    }
};

// ------------------------------------------------------------------------------------------------ GEMV

template <int PASSES>
__device__ __forceinline__ bool ps_gemv(PsCtx& c, const PbStepOp& op) {
    using D = PbQDec<PS_FMT>;
    const PsGemvOp& g = op.g;
    const int cols = g.cols, mode = g.mode;
    const int tid = c.tid, warp = c.warp, lane = c.lane;
    const bool barrier = (op.flags & PS_F_BARRIER) != 0;
    const bool st_first = tid == 0 && blockIdx.x == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1;
    pb_stamp(op.stamps, 0, st_first); pb_stamp(op.stamps, 6, st_last);
    if (barrier) ps_bar_arrive(c);
    // ---- loads that do not depend on the previous operation: norm weights; for the gated norm also z (produced two
    //      operations earlier)
    float4 wv[PASSES], sg[PASSES];
#pragma unroll
    for (int ps = 0; ps < PASSES; ps++) {
        const int e = 4 * (tid + PS_CT * ps);
        wv[ps] = make_float4(1.f, 1.f, 1.f, 1.f); sg[ps] = make_float4(1.f, 1.f, 1.f, 1.f);
        if (e < cols) {
            if (mode == PB_ACT_NORM) wv[ps] = *reinterpret_cast<const float4*>(g.norm_w + e);
            if (mode == PB_ACT_GNORM) {
                wv[ps] = *reinterpret_cast<const float4*>(g.norm_w + 4 * lane);
                const float4 z = __ldcg(reinterpret_cast<const float4*>(g.z + e));
                sg[ps] = make_float4(pb_sigm(z.x), pb_sigm(z.y), pb_sigm(z.z), pb_sigm(z.w));
            }
        }
    }
    ps_fine(c, 0);
    if (barrier && !ps_bar_wait(c)) return false;
    ps_fine(c, 1);
    pb_stamp(op.stamps, 2, st_first);
    // ---- activations: thread t owns values 4t..4t+3 (and 2048 + 4t.. for the second pass), the partition of the
    //      splitting pass of pb_gemvq_kernel (warp w: groups 4w..4w+3)
    float4 xv[PASSES];
#pragma unroll
    for (int ps = 0; ps < PASSES; ps++) {
        const int e = 4 * (tid + PS_CT * ps);
        xv[ps] = e < cols ? __ldcg(reinterpret_cast<const float4*>(g.x + e)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float s = 1.0f;
    if (mode == PB_ACT_NORM) {   // rms(): x * s * w  (qwen4exp_gguf.rs:209); the sum of squares in the partition of pb_gemvq_kernel
#pragma unroll
        for (int ps = 0; ps < PASSES; ps++) { const int e = 4 * (tid + PS_CT * ps); if (e < cols) *reinterpret_cast<float4*>(c.xf + e) = xv[ps]; }
        ps_fine(c, 2);
        pb_named_barrier(1, PS_CT);
        ps_fine(c, 3);
        float ss = pb_strided_ss(c.xf, cols, tid, PS_CT);
        ss = pb_consumer_sum(ss, c.m->red, warp, lane);
        s = 1.0f / sqrtf(ss / (float)cols + g.eps);
        ps_fine(c, 4);
    }
#pragma unroll
    for (int ps = 0; ps < PASSES; ps++) {
        const int e = 4 * (tid + PS_CT * ps);
        if (e < cols) {
            float4 v = xv[ps];
            if (mode == PB_ACT_NORM) v = pb_norm_vec(v, s, wv[ps]);
            if (mode == PB_ACT_GNORM) v = pb_gnorm_vec(v, wv[ps], sg[ps], g.head_dim, g.eps);
            ps_split(v, lane, 4 * warp + (PS_CT / 8) * ps, cols, c.xq);
        }
    }
    ps_fine(c, 5);
    pb_named_barrier(1, PS_CT);
    ps_fine(c, 6);
    pb_stamp(op.stamps, 3, st_first);

    const int nquarters = cols / 64;
    const int lpr = nquarters < 32 ? nquarters : 32, rpw = 32 / lpr;
    const int sub = lane / lpr, ql = lane - sub * lpr;
    const PbQTabs T = {0u, 0u, 0u};
    PbXQuarter xr;
    if (PASSES == 1) pb_load_xquarter<true>(c.xq, cols, ql, xr);
    ps_fine(c, 7);
    const int row_bytes = g.row_bytes, rpc = g.rows_per_chunk, nseg = g.nseg, nchunks = g.nchunks, accumulate = g.accumulate;
    bool first = true;
    for (int chunk = (int)blockIdx.x; chunk < nchunks; chunk += (int)gridDim.x, c.k++) {
        if (!ps_wait_full(c, c.k)) return false;
        if (first) { pb_stamp(op.stamps, 4, st_first); first = false; ps_fine(c, 8); }
        int sgi = 0;
        while (sgi + 1 < nseg && chunk >= g.seg[sgi + 1].chunk0) sgi++;
        const int r0 = (chunk - g.seg[sgi].chunk0) * rpc;
        const int nr = min(rpc, g.seg[sgi].rows - r0);
        const uint32_t base = pb_smem_u32(ps_stage(c, c.k));
        float* ybase = g.y + g.seg[sgi].yoff + r0;
        if (PASSES == 1 && lpr == 32) {
            // full-width rows: two rows per iteration, so that the two independent decode chains overlap each
            // other's shared-memory latency (a row past nr decodes stale bytes of the stage and is not stored)
            for (int ra = warp; ra < nr; ra += 2 * PB_CONSUMERS) {
                const int rc = ra + PB_CONSUMERS;
                const bool two = rc < rpc;
                float v0 = pb_decode_dot<PS_FMT>(base + (uint32_t)ra * (uint32_t)row_bytes + (ql >> 2) * D::STEP_BYTES, ql & 3, T, xr);
                float v1 = pb_decode_dot<PS_FMT>(base + (uint32_t)(two ? rc : ra) * (uint32_t)row_bytes + (ql >> 2) * D::STEP_BYTES, ql & 3, T, xr);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) { v0 += __shfl_xor_sync(0xffffffffu, v0, o); v1 += __shfl_xor_sync(0xffffffffu, v1, o); }
                if (lane == 0) {
                    ybase[ra] = accumulate ? __ldcg(ybase + ra) + v0 : v0;
                    if (two && rc < nr) ybase[rc] = accumulate ? __ldcg(ybase + rc) + v1 : v1;
                }
            }
        } else {
            for (int rb = warp * rpw; rb < nr; rb += PB_CONSUMERS * rpw) {
                const int r = rb + sub;
                const bool valid = r < nr;
                float acc = 0.f;
                if (valid) {
                    const uint32_t rowp = base + (uint32_t)r * (uint32_t)row_bytes;
#pragma unroll
                    for (int ps = 0; ps < PASSES; ps++) {
                        const int qi = ps * 32 + ql;
                        if (qi < nquarters) {
                            PbQuarter wq;
                            D::quarter(rowp + (qi >> 2) * D::STEP_BYTES, qi & 3, T, wq);
                            if (PASSES == 1) acc += pb_quarter_dot<PS_FMT>(wq, xr);
                            else { PbXQuarter xq2; pb_load_xquarter<true>(c.xq, cols, qi, xq2); acc += pb_quarter_dot<PS_FMT>(wq, xq2); }
                        }
                    }
                }
                for (int o = lpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (ql == 0 && valid) ybase[r] = accumulate ? __ldcg(ybase + r) + acc : acc;
            }
        }
        ps_release(c, c.k);
        ps_fine(c, 9 + min(chunk / (int)gridDim.x, 6));
    }
    pb_stamp(op.stamps, 5, st_first); pb_stamp(op.stamps, 7, st_last);
    return true;
}

__device__ __forceinline__ bool ps_gemv_produce(PsCtx& c, const PbStepOp& op) {
    const PsGemvOp& g = op.g;
    for (int chunk = (int)blockIdx.x; chunk < g.nchunks; chunk += (int)gridDim.x, c.k++) {
        int sgi = 0;
        while (sgi + 1 < g.nseg && chunk >= g.seg[sgi + 1].chunk0) sgi++;
        const int r0 = (chunk - g.seg[sgi].chunk0) * g.rows_per_chunk;
        const int nr = min(g.rows_per_chunk, g.seg[sgi].rows - r0);
        const uint32_t bytes = ((uint32_t)nr * (uint32_t)g.row_bytes + 15u) & ~15u;
        if (!ps_acquire(c, c.k, bytes)) return false;
        ps_copy(c, c.k, 0, g.seg[sgi].w + (size_t)r0 * g.row_bytes, bytes);
    }
    return true;
}

// ------------------------------------------------------------------------------------------------ DeltaNet

struct PsDeltaPolicy {
    PsCtx& c; bool barrier; bool ok;
    __device__ static __forceinline__ void sync() { pb_named_barrier(3, DN_THREADS); }
    __device__ __forceinline__ void wait_inputs() { if (barrier) ok = ps_bar_wait(c); }
};

__device__ __forceinline__ bool ps_delta(PsCtx& c, const PbStepOp& op) {
    const PbDeltaParams& p = op.d;
    const int units = p.nv * (p.dv / DN_COLS);
    const bool barrier = (op.flags & PS_F_BARRIER) != 0;
    const bool st_first = c.tid == 0 && blockIdx.x == 0, st_last = c.tid == 0 && blockIdx.x == gridDim.x - 1;
    pb_stamp(op.stamps, 0, st_first); pb_stamp(op.stamps, 6, st_last);
    if (barrier) ps_bar_arrive(c);
    bool ok = true;
    // one unit (V head, 32 state columns) per CTA, run by warps 0..7 (units <= grid is checked on the host); the unit's
    // threads wait for the barrier inside it, after the loads that do not depend on this step's projections
    const int u = (int)blockIdx.x;
    if (u < units && c.warp < DN_THREADS / 32) {
        PsDeltaPolicy pol{c, barrier, true};
        const int splits = p.dv / DN_COLS;
        pb_deltanet_unit<16, 1>(p, c.pos, u / splits, (u % splits) * DN_COLS, 0, c.tid, true, c.xf, c.m->nrm, pol, op.stamps, st_first);
        ok = pol.ok;
    } else if (barrier) {
        ok = ps_bar_wait(c);
    }
    pb_stamp(op.stamps, 5, st_first); pb_stamp(op.stamps, 7, st_last);
    return ok;
}

// ------------------------------------------------------------------------------------------------ router

__device__ __forceinline__ bool ps_router(PsCtx& c, const PbStepOp& op) {
    const PsRouterOp& r = op.r;
    const int cols = r.cols, tid = c.tid, warp = c.warp, lane = c.lane;
    const bool barrier = (op.flags & PS_F_BARRIER) != 0;
    const bool st_first = tid == 0 && blockIdx.x == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1;
    pb_stamp(op.stamps, 0, st_first); pb_stamp(op.stamps, 6, st_last);
    if (barrier) ps_bar_arrive(c);
    // norm weights into shared memory before the barrier (they feed both the split and the row products)
    for (int e = 4 * tid; e < cols; e += 4 * PS_CT) *reinterpret_cast<float4*>(c.nw + e) = *reinterpret_cast<const float4*>(r.norm_w + e);
    if (barrier && !ps_bar_wait(c)) return false;
    pb_stamp(op.stamps, 2, st_first);
    for (int e = 4 * tid; e < cols; e += 4 * PS_CT) *reinterpret_cast<float4*>(c.xf + e) = __ldcg(reinterpret_cast<const float4*>(r.x + e));
    pb_named_barrier(1, PS_CT);
    const float s = pb_row_rms_scale(c.xf, cols, r.eps, lane);   // every warp: the arithmetic of pb_router_kernel's per-token scale
    for (int g0 = 4 * warp; g0 < cols / 32; g0 += 4 * PB_CONSUMERS) {
        const float4 v = pb_norm_vec(*reinterpret_cast<const float4*>(c.xf + 32 * g0 + 4 * lane), s, *reinterpret_cast<const float4*>(c.nw + 32 * g0 + 4 * lane));
        ps_split(v, lane, g0, cols, c.xq);
    }
    pb_stamp(op.stamps, 3, st_first);
    const int rpc = r.rows_per_chunk, nchunks = r.nchunks, n_exp = r.n_exp;
    bool first = true;
    for (int chunk = (int)blockIdx.x; chunk < nchunks; chunk += (int)gridDim.x, c.k++) {
        if (!ps_wait_full(c, c.k)) return false;
        if (first) { pb_stamp(op.stamps, 4, st_first); first = false; }
        const float* st = reinterpret_cast<const float*>(ps_stage(c, c.k));
        const bool gate_vec = chunk == nchunks - 1;
        const int r0 = gate_vec ? n_exp : chunk * rpc;
        const int nr = gate_vec ? 1 : min(rpc, n_exp - r0);
        for (int rr = warp; rr < nr; rr += PB_CONSUMERS) {
            const float* wrow = st + (size_t)rr * cols;
            float acc;
            if (cols == 2048) acc = pb_router_row2048_dot1(wrow, c.nw, c.xf, s, lane);
            else acc = pb_router_row_dot(wrow, c.nw, c.xf, s, cols, lane);
            if (lane == 0) r.logits[r0 + rr] = acc;
        }
        ps_release(c, c.k);
    }
    pb_stamp(op.stamps, 5, st_first); pb_stamp(op.stamps, 7, st_last);
    return true;
}

__device__ __forceinline__ bool ps_router_produce(PsCtx& c, const PbStepOp& op) {
    const PsRouterOp& r = op.r;
    for (int chunk = (int)blockIdx.x; chunk < r.nchunks; chunk += (int)gridDim.x, c.k++) {
        const bool gate_vec = chunk == r.nchunks - 1;
        const int r0 = chunk * r.rows_per_chunk;
        const int nr = gate_vec ? 1 : min(r.rows_per_chunk, r.n_exp - r0);
        const uint32_t bytes = (uint32_t)nr * (uint32_t)r.cols * 4u;
        if (!ps_acquire(c, c.k, bytes)) return false;
        ps_copy(c, c.k, 0, gate_vec ? r.sh_gate_inp : r.router + (size_t)r0 * r.cols, bytes);
    }
    return true;
}

// ------------------------------------------------------------------------------------------------ expert gate / up

// Routing of the token by all consumer threads of the CTA (top_k :3132-3139, soft_top :3126-3131): every logit becomes a
// 64-bit key (order-preserving value bits, then ~id: descending key = descending logit, ties to the lower id, NaN as
// -inf; slots past n_exp get distinct keys below every real one).  Pass 1: each warp ranks its own 32 (64) keys by
// counting the greater ones and passes on its top_k.  Pass 2: the 16 * top_k candidates are ranked the same way, the
// counting of each candidate cut over several threads (partial counts meet in shared memory); rank j < top_k is the
// j-th pick.  Warp 0 then finishes as pb_route_token does and releases the producer warp.
__device__ __forceinline__ void ps_route(PsCtx& c, const PsMoeOp& m) {
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(c.xf);          // [16 warps][32 * kpt]
    const int kpt = (m.n_exp + PS_CT - 1) / PS_CT, gsz = 32 * kpt, top_k = m.top_k;
    unsigned long long* cand = keys + PB_CONSUMERS * gsz;                               // [16][top_k]
    unsigned long long* pick = cand + PB_CONSUMERS * PS_MAX_SLOTS;                      // [top_k]
    int* crank = reinterpret_cast<int*>(pick + PS_MAX_SLOTS);                           // [16 * top_k] rank of every candidate
    const int tid = c.tid, warp = c.warp, lane = c.lane;
    if (tid < PB_CONSUMERS * PS_MAX_SLOTS) crank[tid] = 0;
    unsigned long long mine[2];
#pragma unroll
    for (int j = 0; j < 2; j++) {
        mine[j] = 0;
        if (j < kpt) {
            const int e = tid + PS_CT * j;
            mine[j] = e < m.n_exp ? pb_topk_key(__ldcg(m.logits + e), e) : (unsigned long long)(0xFFFFFFFFu - (unsigned)e);
            keys[warp * gsz + j * 32 + lane] = mine[j];
        }
    }
    ps_fine(c, 2);
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 2; j++) {
        if (j < kpt) {
            int rk = 0;
            for (int i = 0; i < gsz; i++) rk += keys[warp * gsz + i] > mine[j] ? 1 : 0;
            if (rk < top_k) cand[warp * top_k + rk] = mine[j];
        }
    }
    ps_fine(c, 3);
    pb_named_barrier(1, PS_CT);
    const int ncand = PB_CONSUMERS * top_k, parts = PS_CT / ncand;   // parts >= 2: ncand <= 256
    if (tid < ncand * parts) {
        const int ci = tid % ncand, part = tid / ncand;
        const int i0 = part * ncand / parts, i1 = (part + 1) * ncand / parts;
        const unsigned long long key = cand[ci];
        int rk = 0;
#pragma unroll 4
        for (int i = i0; i < i1; i++) rk += cand[i] > key ? 1 : 0;
        if (rk) atomicAdd(&crank[ci], rk);
    }
    ps_fine(c, 4);
    pb_named_barrier(1, PS_CT);
    ps_fine(c, 5);
    if (warp == 0) {
        for (int i = lane; i < ncand; i += 32) { const int rk = crank[i]; if (rk < top_k) pick[rk] = cand[i]; }
        __syncwarp();
        int my_e, rank; float w;
        pb_route_finish(lane < top_k ? pick[lane] : 0ull, top_k, lane, my_e, w, rank);
        if (lane < top_k) { c.m->route_e[rank] = my_e; c.m->route_w[rank] = w; }
        __syncwarp();
        if (lane == 0) { __threadfence_block(); atomicAdd(&c.m->route_seq, 1); }   // the producer warp may request the selected experts' rows
    }
}

__device__ __forceinline__ bool ps_gu_chunk(PsCtx& c, const PsMoeOp& m, int ci, const PbXQuarter& xr, int lpr, int ql, int half, int r) {
    using D = PbQDec<PS_FMT>;
    const PbQTabs T = {0u, 0u, 0u};
    const int rg = m.rg, cpe = m.ff / rg;
    if (!ps_wait_full(c, c.k)) return false;
    // the shared expert's chunks come first (their rows never wait for the routing)
    const int slot = ci < cpe ? m.top_k : ci / cpe - 1, r0 = (ci % cpe) * rg;
    const uint32_t base = pb_smem_u32(ps_stage(c, c.k)) + (uint32_t)half * (uint32_t)rg * (uint32_t)m.row_bytes_gu + (uint32_t)r * (uint32_t)m.row_bytes_gu;
    float v = pb_decode_dot<PS_FMT>(base + (ql >> 2) * D::STEP_BYTES, ql & 3, T, xr);
    for (int o = lpr >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int par = c.k & 1;
    if (ql == 0) c.m->gu[par][half][r] = v;
    pb_named_barrier(1, PS_CT);
    // hidden = silu(gate . x) * (up . x)   (routed :1781-1783, ffn :1680)
    if (c.tid < rg) m.h[(size_t)slot * m.ff + r0 + c.tid] = pb_silu(c.m->gu[par][0][c.tid]) * c.m->gu[par][1][c.tid];
    ps_release(c, c.k);
    c.k++;
    return true;
}

__device__ __forceinline__ bool ps_gu(PsCtx& c, const PbStepOp& op) {
    const PsMoeOp& m = op.m;
    const int cols = m.d, tid = c.tid, warp = c.warp, lane = c.lane;
    const bool barrier = (op.flags & PS_F_BARRIER) != 0;
    const bool st_first = tid == 0 && blockIdx.x == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1;
    pb_stamp(op.stamps, 0, st_first); pb_stamp(op.stamps, 6, st_last);
    c.ngu++;
    if (barrier) ps_bar_arrive(c);
    pb_named_barrier(1, PS_CT);   // the split of the activations (router operation) is complete in this CTA
    const int nquarters = cols / 64;
    const int lpr = nquarters < 32 ? nquarters : 32, rpw = 32 / lpr;
    const int sub = lane / lpr, ql = lane - sub * lpr;
    PbXQuarter xr;
    pb_load_xquarter<true>(c.xq, cols, ql, xr);
    const int rg = m.rg, cpe = m.ff / rg, total = (m.top_k + 1) * cpe;
    const int half = warp >> 3, r = (warp & 7) * rpw + sub;
    // the shared expert's rows need nothing from other CTAs: they are processed while the grid barrier completes
    bool routed = false;
#pragma unroll 1
    for (int ci = (int)blockIdx.x, n = 0;; ci += (int)gridDim.x, n++) {
        if (!routed && ci >= cpe) {   // the shared expert's chunks of this CTA are done (or it had none)
            ps_fine(c, 0);
            if (barrier && !ps_bar_wait(c)) return false;
            ps_fine(c, 1);
            pb_stamp(op.stamps, 2, st_first);
            ps_route(c, m);
            ps_fine(c, 6);
            pb_stamp(op.stamps, 3, st_first);
            routed = true;
        }
        if (ci >= total) break;
        if (!ps_gu_chunk(c, m, ci, xr, lpr, ql, half, r)) return false;
        ps_fine(c, 7 + min(n, 8));
    }
    pb_stamp(op.stamps, 5, st_first); pb_stamp(op.stamps, 7, st_last);
    return true;
}

// Producer warp: the shared expert's chunks at once; the selected experts' chunks once the consumers have routed.
__device__ __forceinline__ bool ps_gu_produce(PsCtx& c, const PbStepOp& op) {
    const PsMoeOp& m = op.m;
    const int rg = m.rg, cpe = m.ff / rg, total = (m.top_k + 1) * cpe;
    const uint32_t half_bytes = (uint32_t)rg * (uint32_t)m.row_bytes_gu;
    c.ngu++;
    int ci = (int)blockIdx.x;
    for (; ci < cpe; ci += (int)gridDim.x, c.k++) {
        const size_t off = (size_t)ci * rg * m.row_bytes_gu;
        if (!ps_acquire(c, c.k, 2 * half_bytes)) return false;
        ps_copy(c, c.k, 0, m.sh_gate + off, half_bytes);
        ps_copy(c, c.k, half_bytes, m.sh_up + off, half_bytes);
    }
    {   // the routing of this gate/up operation (the ngu-th of the launch) is in shared memory
        bool routed = false;
        for (uint32_t i = 0; i < PS_GRID_SPIN; i++) {
            if (*reinterpret_cast<volatile int*>(&c.m->route_seq) >= (int)c.ngu) { routed = true; break; }
            if (i > 64) __nanosleep(64);
        }
        if (!routed) { atomicExch(c.status, PB_DEV_GRID_TIMEOUT); return false; }
        __threadfence_block();
    }
    for (; ci < total; ci += (int)gridDim.x, c.k++) {
        const int slot = ci / cpe - 1, r0 = (ci % cpe) * rg;
        const int e = c.m->route_e[slot];
        if (e < m.e_base || e >= m.n_exp) { atomicExch(c.status, PB_DEV_BAD_INDEX); return false; }
        const size_t off = ((size_t)(e - m.e_base) * m.ff + r0) * m.row_bytes_gu;
        if (!ps_acquire(c, c.k, 2 * half_bytes)) return false;
        ps_copy(c, c.k, 0, m.gate + off, half_bytes);
        ps_copy(c, c.k, half_bytes, m.up + off, half_bytes);
    }
    return true;
}

// ------------------------------------------------------------------------------------------------ expert down + combine

// The work is cut by OUTPUT ROWS: CTA c owns rows [16 c, 16 c + 16) of every selected expert and of the shared expert,
// so the weighted sum over the experts (ascending expert id, then the shared expert as in pb_combine_one) is formed
// inside the CTA and added to the residual directly (the arithmetic of pb_expert_down_rows_kernel).
__device__ __forceinline__ bool ps_down(PsCtx& c, const PbStepOp& op) {
    using D = PbQDec<PS_FMT>;
    const PsMoeOp& m = op.m;
    const int cols = m.ff, xw = pb_xq_words(cols), tid = c.tid, warp = c.warp, lane = c.lane;
    const int top_k = m.top_k, nsl = top_k + 1, spc = m.spc, row_bytes = m.row_bytes_dn;
    const bool barrier = (op.flags & PS_F_BARRIER) != 0;
    const bool st_first = tid == 0 && blockIdx.x == 0, st_last = tid == 0 && blockIdx.x == gridDim.x - 1;
    pb_stamp(op.stamps, 0, st_first); pb_stamp(op.stamps, 6, st_last);
    ps_fine(c, 0);
    if (barrier) { ps_bar_arrive(c); if (!ps_bar_wait(c)) return false; }
    ps_fine(c, 1);
    pb_stamp(op.stamps, 2, st_first);
    const int units = m.d / PS_SLICE_ROWS;
    if ((int)blockIdx.x >= units) { pb_stamp(op.stamps, 7, st_last); return true; }
    // int8 levels of every slot's hidden vector, four groups per warp pass; the passes' values are requested together
    const int gpe = cols / 128;
    {
        auto hload = [&](int i) { return __ldcg(reinterpret_cast<const float4*>(m.h + (size_t)(i / gpe) * cols + 32 * ((i % gpe) * 4) + 4 * lane)); };
        float4 nxt = make_float4(0.f, 0.f, 0.f, 0.f);
        if (warp < nsl * gpe) nxt = hload(warp);
#pragma unroll 1
        for (int i = warp; i < nsl * gpe; i += PB_CONSUMERS) {
            const float4 cur = nxt;
            if (i + PB_CONSUMERS < nsl * gpe) nxt = hload(i + PB_CONSUMERS);
            ps_split(cur, lane, (i % gpe) * 4, cols, c.xq + (size_t)(i / gpe) * xw);
        }
    }
    ps_fine(c, 2);
    pb_named_barrier(1, PS_CT);
    ps_fine(c, 3);
    pb_stamp(op.stamps, 3, st_first);
    const PbQTabs T = {0u, 0u, 0u};
    const int nquarters = cols / 64;                    // <= 32 (checked on the host)
    const int rpw = 32 / nquarters, sub = lane / nquarters, ql = lane - sub * nquarters;
    const int ppe = PS_SLICE_ROWS / rpw;                // warp passes per slice
    const uint32_t slice = (uint32_t)PS_SLICE_ROWS * (uint32_t)row_bytes;
    const int nchunk = (nsl + spc - 1) / spc, kbase = c.k;
    int cur = -1;
    for (int i = warp; i < nsl * ppe; i += PB_CONSUMERS) {
        const int k = i / ppe, r = (i - k * ppe) * rpw + sub;
        while (cur < k / spc) {
            if (cur >= 0) ps_release(c, kbase + cur);
            cur++;
            if (!ps_wait_full(c, kbase + cur)) return false;
            if (cur == 0) pb_stamp(op.stamps, 4, st_first);
            ps_fine(c, 4 + cur);
        }
        PbQuarter wq; PbXQuarter xv;
        D::quarter(pb_smem_u32(ps_stage(c, kbase + cur)) + (uint32_t)(k % spc) * slice + (uint32_t)r * (uint32_t)row_bytes + (ql >> 2) * D::STEP_BYTES, ql & 3, T, wq);
        pb_load_xquarter<true>(c.xq + (size_t)k * xw, cols, ql, xv);
        float acc = pb_quarter_dot<PS_FMT>(wq, xv);
        for (int o = nquarters >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (ql == 0) c.m->res[k * PS_SLICE_ROWS + r] = acc;
    }
    while (cur < nchunk - 1) {
        if (cur >= 0) ps_release(c, kbase + cur);
        cur++;
        if (!ps_wait_full(c, kbase + cur)) return false;
    }
    ps_release(c, kbase + cur);
    c.k = kbase + nchunk;
    ps_fine(c, 7);
    pb_named_barrier(1, PS_CT);
    ps_fine(c, 8);
    if (tid < PS_SLICE_ROWS) {
        // pb_combine_one: sigmoid(gate) * shared + sum over slots in ascending expert id; products rounded, then added
        float y = __fmul_rn(c.m->res[top_k * PS_SLICE_ROWS + tid], pb_sigm(__ldcg(m.logits + m.n_exp)));   // routed :1723
        float o = 0.f;
        for (int k = 0; k < top_k; k++) o = __fadd_rn(o, __fmul_rn(c.m->route_w[k], c.m->res[k * PS_SLICE_ROWS + tid]));
        y = __fadd_rn(y, o);
        float* dst = m.y + (int)blockIdx.x * PS_SLICE_ROWS + tid;
        *dst = __ldcg(dst) + y;
    }
    pb_stamp(op.stamps, 5, st_first); pb_stamp(op.stamps, 7, st_last);
    return true;
}

__device__ __forceinline__ bool ps_down_produce(PsCtx& c, const PbStepOp& op) {
    const PsMoeOp& m = op.m;
    const int units = m.d / PS_SLICE_ROWS, nsl = m.top_k + 1;
    if ((int)blockIdx.x >= units) return true;
    const uint32_t slice = (uint32_t)PS_SLICE_ROWS * (uint32_t)m.row_bytes_dn;
    const int r0 = (int)blockIdx.x * PS_SLICE_ROWS;
    for (int s0 = 0; s0 < nsl; s0 += m.spc, c.k++) {
        const int n = min(m.spc, nsl - s0);
        if (!ps_acquire(c, c.k, (uint32_t)n * slice)) return false;
        for (int j = 0; j < n; j++) {
            const int slot = s0 + j;
            const uint8_t* src;
            if (slot < m.top_k) {
                const int e = c.m->route_e[slot];
                // the expert id was range-checked when the gate/up rows were requested
                src = m.down + ((size_t)(e - m.e_base) * m.d + r0) * m.row_bytes_dn;
            } else src = m.sh_down + (size_t)r0 * m.row_bytes_dn;
            ps_copy(c, c.k, (uint32_t)j * slice, src, slice);
        }
    }
    return true;
}

// ------------------------------------------------------------------------------------------------ kernel

__global__ void __launch_bounds__(PS_THREADS, 1) pb_step_kernel(const PsParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    PsCtx c;
    c.m = reinterpret_cast<PsMisc*>(smem);
    c.xf = reinterpret_cast<float*>(smem + P.lay.xf_off);
    c.nw = reinterpret_cast<float*>(smem + P.lay.nw_off);
    c.xq = reinterpret_cast<uint32_t*>(smem + P.lay.xq_off);
    c.stages = smem + P.lay.stage_off; c.stage_bytes = P.lay.stage_bytes;
    c.nbar = 0; c.ngu = 0; c.k = 0; c.status = P.status;
    c.tid = threadIdx.x; c.warp = c.tid >> 5; c.lane = c.tid & 31; c.trace = nullptr;
    if (c.tid == 0) {
        for (int s = 0; s < PS_STAGES; s++) { pb_mbar_init(&c.m->full[s], 1); pb_mbar_init(&c.m->empty[s], PB_CONSUMERS); }
        pb_mbar_init(&c.m->req, PB_CONSUMERS); pb_mbar_init(&c.m->done, 1);
        c.m->abort = 0; c.m->route_seq = 0;
        pb_fence_barrier_init();
    }
    pb_pdl_trigger();   // the kernel after this one may become resident; it waits for this grid to complete before it reads anything of it
    uint8_t* opslot = smem + PS_OPBUF_OFF + c.warp * 256;
    PsOpFetch fetch;
    fetch.request(P.ops, P.op_begin, P.op_end, c.lane);
    c.pos = P.pos[0];
    __syncthreads();

    if (c.warp == PB_CONSUMERS + 1) {
        // ---- sync warp: one thread runs the grid barriers
        if (c.lane != 0) return;
        const unsigned long long base = __ldcg(P.sync + 1);   // arrivals counted before this launch (written at the end of the previous one)
        // tracing: the n-th barrier belongs to the n-th operation with PS_F_BARRIER; CTA 0's sync thread stamps its steps into
        // words 16.. of that operation's fine-grained area
        int opi = P.op_begin - 1;
        for (int n = 1; n <= P.nbar; n++) {
            unsigned long long* tr = nullptr;
            do { opi++; } while (opi < P.op_end && !(P.ops[opi].flags & PS_F_BARRIER));
            if (opi < P.op_end && blockIdx.x == 0 && P.ops[opi].trace) tr = P.ops[opi].trace + 4 * gridDim.x + 16;
            if (!pb_mbar_wait(&c.m->req, (n - 1) & 1, c.status, PB_DEV_GRID_TIMEOUT)) { c.m->abort = 1; return; }
            if (tr) tr[0] = pb_globaltimer();
            __threadfence();                                   // the consumers' stores (ordered before their arrival) become visible GPU-wide
            if (tr) tr[1] = pb_globaltimer();
            atomicAdd(P.sync, 1ULL);
            const unsigned long long target = base + (unsigned long long)n * gridDim.x;
            bool ok = false;
            for (uint32_t i = 0; i < PS_GRID_SPIN; i++) {
                if (ps_ld_acquire(P.sync) >= target) { ok = true; break; }
                if (i > 1024) __nanosleep(64);
            }
            if (tr) tr[2] = pb_globaltimer();
            if (!ok) { atomicExch(c.status, PB_DEV_GRID_TIMEOUT); c.m->abort = 1; }
            // (the load above is an acquire at GPU scope; the consumers read other CTAs' results with L1-bypassing loads)
            if (tr) tr[3] = pb_globaltimer();
            pb_mbar_arrive(&c.m->done);
            if (!ok) return;
        }
        // the next launch reads its base from sync[1]: every CTA of this launch read it before the first barrier completed
        if (blockIdx.x == 0 && P.nbar > 0) P.sync[1] = base + (unsigned long long)P.nbar * gridDim.x;
        return;
    }

    if (c.warp == PB_CONSUMERS) {
        // ---- producer warp: the weights of every operation, in program order (one thread issues)
        bool ok = true;
        for (int i = P.op_begin; i < P.op_end && ok; i++) {
            const PbStepOp& op = fetch.take(opslot, c.lane);
            fetch.request(P.ops, i + 1, P.op_end, c.lane);
            if (c.lane == 0) {
                switch (op.kind) {
                    case PS_GEMV: ok = ps_gemv_produce(c, op); break;
                    case PS_ROUTER: ok = ps_router_produce(c, op); break;
                    case PS_GU: ok = ps_gu_produce(c, op); break;
                    case PS_DOWN: ok = ps_down_produce(c, op); break;
                    default: break;
                }
                if (op.trace) op.trace[4 * blockIdx.x + 3] = pb_globaltimer();
            }
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        }
        if (!ok && c.lane == 0)   // give the copies of the last stages a bounded chance to land before the CTA may exit
            for (int k = max(0, c.k - PS_STAGES); k < c.k; k++) pb_mbar_wait(&c.m->full[k % PS_STAGES], (k / PS_STAGES) & 1, nullptr, 0);
        return;
    }

    // ---- consumers
    pb_pdl_wait();   // the activations come from the kernel before this one (the weights, streamed by the producer warp, do not)
    bool ok = true;
    for (int i = P.op_begin; i < P.op_end && ok; i++) {
        const PbStepOp& op = fetch.take(opslot, c.lane);
        fetch.request(P.ops, i + 1, P.op_end, c.lane);
        c.trace = op.trace;
        if (op.trace && c.tid == 0) op.trace[4 * blockIdx.x] = pb_globaltimer();
        switch (op.kind) {
            case PS_GEMV: ok = op.g.cols > 2048 ? ps_gemv<2>(c, op) : ps_gemv<1>(c, op); break;
            case PS_DELTA: ok = ps_delta(c, op); break;
            case PS_ROUTER: ok = ps_router(c, op); break;
            case PS_GU: ok = ps_gu(c, op); break;
            case PS_DOWN: ok = ps_down(c, op); break;
            default: break;
        }
        if (op.trace && c.tid == 0) op.trace[4 * blockIdx.x + 2] = pb_globaltimer();
    }
}

int pb_launch_step(pb_ctx* ctx, const PsParams& p) {
    if (p.lay.total > (uint32_t)ctx->max_smem_optin) PB_FAIL(ctx, PB_UNSUPPORTED, "fused step: %u bytes of shared memory needed", p.lay.total);
    PB_TRY(pb_ensure_smem(ctx, pb_step_kernel, (size_t)p.lay.total));
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(ctx->sm_count); cfg.blockDim = dim3(PS_THREADS); cfg.dynamicSmemBytes = p.lay.total; cfg.stream = ctx->stream;
    // the CTAs wait on one another: a cooperative launch guarantees that all of them are resident
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    // With step_pdl the kernel joins the dependent-launch chain on both sides: its set-up and the first weight copies (model data)
    // overlap the tail of the kernel before it, and the kernel after it is resident by the time this one ends.  Without, a
    // cooperative launch waits for the stream to drain and the next kernel for this one.
    const bool chain = ctx->step_pdl && ctx->pdl_scope > 0;
    cfg.attrs = at; cfg.numAttrs = chain && ctx->pdl_chain ? 2 : 1;
    ctx->pdl_chain = chain;
    cudaError_t e = cudaLaunchKernelEx(&cfg, pb_step_kernel, p);
    if (e != cudaSuccess) PB_FAIL(ctx, PB_ERR_CUDA, "fused step launch: %s", cudaGetErrorString(e));
    ctx->kernels_launched++;
    return PB_OK;
}
