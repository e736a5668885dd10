// Operation list of the fused decode step (pb_step.cu), shared with the engine that builds it (pb_engine.cu).
#pragma once
#include "pb_internal.h"

enum { PS_GEMV = 1, PS_DELTA = 2, PS_ROUTER = 3, PS_GU = 4, PS_DOWN = 5 };
enum { PS_F_BARRIER = 1 };     // every CTA waits for all CTAs to have finished the previous operation

// y[yoff_s + r] (+)= sum_c W_s[r][c] act(x)[c] over up to four row-concatenated re-coded IQ3_S matrices
struct PsGemvOp {
    PbGemvQSeg seg[4];
    int nseg, cols, row_bytes, rows_per_chunk, nchunks, mode, accumulate, head_dim;
    const float *x, *norm_w, *z;
    float* y;
    float eps;
};
// logits[e] = router[e] . rms(x) w, logits[n_exp] = sh_gate_inp . rms(x) w; leaves the int8 levels of rms(x) w in shared memory
struct PsRouterOp {
    const float *x, *norm_w, *router, *sh_gate_inp;
    float* logits;
    int n_exp, cols, rows_per_chunk, nchunks;   // nchunks counts the router's row chunks plus one for the shared-gate vector
    float eps;
};
// PS_GU: h[slot] = silu(gate_e x) * (up_e x) for the top_k selected experts (slot = rank by expert id) and the shared
// expert (slot top_k); PS_DOWN: y += sigmoid(shared-gate logit) * down_sh h[top_k] + sum_slots w_slot * down_e h[slot]
struct PsMoeOp {
    const uint8_t *gate, *up, *down, *sh_gate, *sh_up, *sh_down;
    const float* logits;
    float *h, *y;
    int n_exp, top_k, ff, d;
    int e_base;                 // first expert held by the fused expert tensors
    int row_bytes_gu, row_bytes_dn;
    int rg;                     // gate rows per gate/up chunk (the same number of up rows ride along)
    int spc;                    // down: expert slices (16 output rows each) per chunk
};
struct PbStepOp {
    int kind, flags;
    unsigned long long* stamps;
    unsigned long long* trace;   // tracing: [grid][4] per-CTA stamps (operation start, barrier passed, end, producer done), or null
    union { PsGemvOp g; PbDeltaParams d; PsRouterOp r; PsMoeOp m; };
};

// shared-memory layout of the fused step kernel (byte offsets), fixed per model
struct PsLayout { uint32_t xf_off, nw_off, xq_off, stage_off, stage_bytes, total; };
#define PS_STAGES 5

static_assert(sizeof(PbStepOp) <= 256 && sizeof(PbStepOp) % 16 == 0, "a warp copies an operation as 16 x 16 bytes");
struct PsParams {
    const PbStepOp* ops;
    int op_begin, op_end;
    int nbar;                   // operations with PS_F_BARRIER in [op_begin, op_end)
    unsigned long long* sync;   // [0] arrivals at grid barriers (monotonic), [1] its value when the running launch began
    const int64_t* pos;         // the sequence's position
    PsLayout lay;
    int* status;
};
int pb_launch_step(pb_ctx* ctx, const PsParams& p);
