// Model, state and the device-resident token loop behind the C ABI (include/pyre_b200.h).
//
// One decode step = one CUDA graph replay: embedding row -> per layer [fused RMSNorm +
// projection GEMV, Gated DeltaNet step or 4-bit-KV gated attention, output projection with
// residual add, router, top-k routing, grouped expert SwiGLU, combine] -> lm-head GEMV ->
// argmax -> position advance.  Windows of up to 8 consecutive tokens of one sequence (verify, prompt
// feed) run as one pass that streams every weight once (run_window).  Nothing returns to the host
// inside a token; the reference's
// loop (forward_inner, src/model/qwen4exp_gguf.rs:2087-2157, layer_cube :728-895) reads
// router logits back to the host in every layer.
#include "pb_stream.cuh"
#include "pb_internal.h"
#include "pb_step.cuh"

#include <stdio.h>
#include <stdlib.h>
#include <new>
#include <vector>

#define PB_MAX_WINDOW 8   // draft windows of the reference are at most 8 tokens (src/spec.rs:185)
#define PB_PREFILL_CHUNK 256   // prompt tokens per batched pass; prompts are cut on the absolute grid of this size (src/engine_qn.rs:34-38, 92-139)
#define PB_WIN_SPLITS 4        // attention splits per (token, KV head) of a prefill chunk: three walk the packed positions, one the f32 ring
#define PB_WIN_KEYS (4 * (PB_MAX_WINDOW + 1) + 1)   // graphs per (t <= 8, ckpt, all_logits), plus one for a full prefill chunk
static size_t conv_elems(const pb_cfg& c, int B) { return (size_t)B * c.conv_k * (2 * c.lin_nk * c.lin_dk + c.lin_nv * c.lin_dv); }
static size_t ssm_elems(const pb_cfg& c, int B) { return (size_t)B * c.lin_nv * c.lin_dk * c.lin_dv; }

struct PbSlot { pb_qmat* mat = nullptr; float* vec = nullptr; int64_t nvec = 0; };

struct pb_model {
    pb_ctx* ctx = nullptr;
    pb_cfg cfg{};
    std::vector<PbSlot> slots;      // [(n_layers + 1)][PB_R_COUNT], index 0 = global
    std::vector<int> kind, idx;     // per layer: 1 = full attention, 0 = DeltaNet; index among its kind
    int n_lin = 0, n_attn = 0;
    bool finalized = false;
    int ep_rank = 0, ep_world = 1, e_lo = 0, e_hi = 0;
    float* rope_inv = nullptr;   // n_rot / 2 inverse frequencies, then mscale
    int ctx_train = 0;           // trained context (0: unknown, no scaling)
    int idx_budget = 0, idx_ratio = 1, idx_nh = 0, idx_hd = 0;   // QSA indexer geometry (Cfg :24-25); idx_nh = 0: none
    bool qsa = false;            // the attention layers hold indexer tensors
    int mtp_window = 0;          // > 0: this model is an MTP drafter layer (pb_model_set_mtp)
    PbPleHash ple{}; int ple_conv_k = 0, ple_dim = 0, n_ple = 0;   // n-gram embeddings (pb_model_set_ple); ple.ngram = 0: none
    std::vector<int> ple_idx;    // per layer: index among the layers that hold PLE tensors, or -1
    uint64_t weight_bytes_step = 0;
};

struct PbKv { uint32_t *kw = nullptr, *vw = nullptr; float *ks = nullptr, *vs = nullptr, *kr = nullptr, *vr = nullptr; int64_t* q4n = nullptr;
              float *ik = nullptr, *ib = nullptr; };   // QSA: raw index keys [batch][max_ctx][idx_hd], pooled block keys [batch][nb_cap][idx_hd]

// MTP drafter attached to a state of the main model (src/model/mtp.rs; bookkeeping of mtp_draft_in, qwen4exp_gguf.rs:2179-2278)
struct PbMtp {
    pb_model* dm = nullptr; pb_state* ds = nullptr;     // the drafter layer and its own state (one sequence, f32 K/V by cell)
    int window = 128;
    float* ring = nullptr; int ring_cap = 0;            // the main model's final residual rows by position % ring_cap
    std::vector<int64_t> ring_pos;                      // position held by each slot (-1: none)
    std::vector<uint32_t> tokens; int64_t tok_base = 0; // ids the main state has been fed, tokens[i] at position tok_base + i
    int64_t kv_c0 = 0, kv_end = 0;                      // the drafter holds cells [kv_c0, kv_end)
    std::vector<uint32_t> ids; int n_ids = 0;           // draft vocabulary
    std::vector<float> lg_host;                         // the drafter's logits on their way to the caller's sampler (pb_draft_sampled)
    float *e_raw = nullptr, *en = nullptr, *e2 = nullptr, *hn = nullptr, *h2 = nullptr, *lg = nullptr;
    uint32_t *tok_dev = nullptr, *best = nullptr, *mask = nullptr; int* mask_on = nullptr;
    uint32_t* pin = nullptr;                            // pinned: [1..2] (index, probability bits) of a draft step, read back
};

struct pb_state {
    pb_model* m = nullptr;
    int batch = 0;
    int64_t pos_host = 0;
    std::vector<void*> allocs;
    int64_t* pos = nullptr; uint32_t* ids = nullptr; uint32_t* next = nullptr; unsigned long long* amax = nullptr; unsigned int* ticket = nullptr;
    float *x = nullptr, *xin = nullptr, *proj = nullptr, *olin = nullptr, *att = nullptr, *rlogits = nullptr, *yout = nullptr;
    uint32_t* xq = nullptr;
    int *sel_e = nullptr, *n_used = nullptr, *used_e = nullptr, *used_off = nullptr, *ent_tok = nullptr, *ent_slot = nullptr;
    uint32_t* hq = nullptr;
    float *sel_w = nullptr, *ent_w = nullptr, *h = nullptr, *h_sh = nullptr, *part = nullptr, *part_sh = nullptr, *logits = nullptr;
    float *part_ml = nullptr, *part_acc = nullptr;
    int nsplit = 1, nsplit_packed = 0;
    // sharded tokens (pb_state_create_sharded): this rank's `batch` sequences are tokens [tok0, tok0 + batch) of
    // moe_t = batch * ep_world; xg = residual rows of all ranks, part_rs = this rank's reduced partial rows
    bool sharded = false; int moe_t = 0, tok0 = 0;
    // window mode (batch 1): win_t > 0 while a window of consecutive tokens of the one sequence runs through
    // the layers as columns; wpos[j] = position of column j; win_ckpt = keep DeltaNet checkpoints
    int win_t = 0; bool win_ckpt = false; int64_t* wpos = nullptr;
    int moe_cap = 0;   // rows of the MoE work buffers
    cudaGraphExec_t win_graph[PB_WIN_KEYS] = {}; unsigned char win_runs[PB_WIN_KEYS] = {};
    float *hxn = nullptr, *hgate = nullptr, *hlo = nullptr, *hinj = nullptr, *hmix = nullptr;   // hyper-connection work rows (hc >= 1)
    float *xg = nullptr, *xs = nullptr, *part_rs = nullptr;   // gathered / local rows [token][d + logits], reduced partial rows
    int64_t ldg = 0;                                          // row stride of xg / xs
    // peer exchange (pb_ep.cu): xg and part_rs live in a block mapped into every rank; the kernels store into the peers' blocks
    bool p2p = false; PbEpSymm symm; PbEpExch exch{}; PbEpExch* exch_dev = nullptr; float** part_tok = nullptr; unsigned long long* ep_seq = nullptr;
    int64_t ldproj = 0, ring_cap = 0;
    struct PbMtp* mtp = nullptr;   // drafter attached to this (main, batch-1) state
    uint32_t* ext_mask = nullptr; int* ext_on = nullptr; int64_t ext_ld = 0;   // a position mask set from outside (the drafter's window of cells)
    float *iproj = nullptr, *qsa_scores = nullptr; uint32_t* qsa_mask = nullptr; int* qsa_on = nullptr; int64_t ldi = 0, nb_cap = 0, mask_ld = 0;   // QSA work buffers
    // n-gram embeddings: ids by position [batch][max_ctx], first position with a history per sequence, table rows / gathered rows /
    // key and value / gated values of the rows in flight, per PLE layer the normalized rows by position % ple_R [batch][ple_R][streams * d]
    uint32_t *tok_hist = nullptr, *ple_rows = nullptr; int64_t* ple_base = nullptr; int64_t ple_base_host = 0;
    float *ple_emb = nullptr, *ple_key = nullptr, *ple_val = nullptr, *ple_gated = nullptr; int ple_R = 0;
    std::vector<float*> ple_ring;
    std::vector<float*> conv, ssm;
    std::vector<PbKv> kv;
    uint32_t* trace = nullptr; int64_t* trace_len = nullptr; int64_t trace_cap = 0;
    uint32_t* pin_u32 = nullptr;   // pinned staging for ids / next tokens
    float* pin_logits = nullptr; size_t pin_logits_n = 0;   // pinned staging for logits on their way to the caller's (pageable) buffer
    cudaGraphExec_t graph = nullptr;
    // speculative verify: DeltaNet (conv ring, ssm) after each of the first t-1 tokens of the last window
    std::vector<float*> ck_conv, ck_ssm;   // [n_lin * PB_MAX_WINDOW]
    float** ck_tab = nullptr; float** ck_live = nullptr;   // the same pointers and the live buffers as device tables (pb_launch_ck_restore)
    int64_t* q4n_all = nullptr;   // packed boundaries of all attention layers [n_attn][batch]; PbKv::q4n points into it
    int verify_t = 0; int64_t verify_pos0 = 0;
    uint64_t steps = 0, kernels_per_step = 0;
    // fused step (pb_step.cu), one sequence on one GPU: operation list on the device, launch segments (runs of operations
    // between attention cores, which keep their own kernels), hidden vectors of the selected experts
    int fused = -1;                                   // -1 not decided yet, 0 not eligible, 1 built
    PbStepOp* fops = nullptr; float* fh = nullptr; PsLayout flay{};
    unsigned long long* ftrace = nullptr; int ftrace_ops = 0;   // tracing: per-CTA stamps [op][grid][4]
    struct FSeg { int begin, end, attn_layer, nbar; };   // attn_layer >= 0: the attention core of that layer follows the segment; nbar: its grid barriers
    std::vector<FSeg> fsegs;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;   // GPU time of the token-loop calls (pb_stats.device_ns)
    bool ev_open = false; uint64_t device_ns = 0;
};
extern "C" {
static void mtp_moved(pb_state* s, int64_t pos);
static void mtp_forget(PbMtp* t, int64_t pos);
}

// Brackets the GPU work of one token-loop call with two events; the elapsed time is added up once the call has synchronised.
static void timing_begin(pb_state* s) {
    pb_ctx* ctx = s->m->ctx;
    if (!s->ev0 && (cudaEventCreate(&s->ev0) != cudaSuccess || cudaEventCreate(&s->ev1) != cudaSuccess)) { s->ev0 = s->ev1 = nullptr; return; }
    s->ev_open = cudaEventRecord(s->ev0, ctx->stream) == cudaSuccess;
}
static void timing_stop(pb_state* s) { if (s->ev_open && cudaEventRecord(s->ev1, s->m->ctx->stream) != cudaSuccess) s->ev_open = false; }
static void timing_collect(pb_state* s) {   // after the stream was synchronised
    if (!s->ev_open) return;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, s->ev0, s->ev1) == cudaSuccess) s->device_ns += (uint64_t)((double)ms * 1e6);
    s->ev_open = false;
}

static PbSlot& slot(pb_model* m, int layer, int role) { return m->slots[(size_t)(layer + 1) * PB_R_COUNT + role]; }
static pb_qmat* M(pb_model* m, int layer, int role) { return slot(m, layer, role).mat; }
static float* V(pb_model* m, int layer, int role) { return slot(m, layer, role).vec; }

template <typename T>
static int dalloc(pb_state* s, T** p, size_t n) {
    pb_ctx* ctx = s->m->ctx;
    void* q = nullptr;
    PB_CUDA(ctx, cudaMalloc(&q, (n ? n : 1) * sizeof(T) + 256));
    PB_CUDA(ctx, cudaMemsetAsync(q, 0, (n ? n : 1) * sizeof(T) + 256, ctx->stream));
    s->allocs.push_back(q);
    *p = (T*)q;
    return PB_OK;
}

extern "C" {

// ------------------------------------------------------------------------------------ model

int pb_model_create(pb_ctx* ctx, const pb_cfg* cfg, pb_model** out) {
    if (!ctx || !out) return PB_ERR_ARG;
    *out = nullptr;
    if (!cfg) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_create: null config");
    const pb_cfg& c = *cfg;
    if (c.n_layers <= 0 || c.d <= 0 || c.vocab <= 0 || c.max_ctx <= 0) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_create: non-positive size in config");
    if (c.hc < 0 || c.hc > 16 || (c.hc > 0 && c.hc_lr <= 0)) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_create: hc=%d streams with low rank %d", c.hc, c.hc_lr);
    if (c.top_k > PB_MAX_TOPK || c.top_k > c.n_exp) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_create: top_k=%d with %d experts", c.top_k, c.n_exp);
    if (c.kv_bits != 0 && c.kv_bits != 4) PB_FAIL(ctx, PB_UNSUPPORTED, "pb_model_create: kv_bits=%d (0 and 4 are built)", c.kv_bits);
    if (c.kv_bits == 4 && c.kv_recent < 64) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_create: kv_recent must be at least 64");
    pb_model* m = new (std::nothrow) pb_model();
    if (!m) PB_FAIL(ctx, PB_ERR_OOM, "host allocation failed");
    m->ctx = ctx; m->cfg = c;
    m->slots.resize((size_t)(c.n_layers + 1) * PB_R_COUNT);
    for (int il = 0; il < c.n_layers; il++) {
        const bool full = c.full_every > 0 && (il + 1) % c.full_every == 0;   // :498
        m->kind.push_back(full ? 1 : 0);
        m->idx.push_back(full ? m->n_attn++ : m->n_lin++);
    }
    *out = m;
    return PB_OK;
}

int pb_model_set_tensor(pb_model* m, int layer, int role, pb_qmat* mat) {
    if (!m || !mat) return PB_ERR_ARG;
    pb_ctx* ctx = m->ctx;
    PB_TRY(pb_enter(ctx));
    if (layer < -1 || layer >= m->cfg.n_layers || role < 0 || role >= PB_R_COUNT) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_set_tensor: layer %d role %d out of range", layer, role);
    if (m->finalized) PB_FAIL(ctx, PB_ERR_STATE, "pb_model_set_tensor: model already finalized");
    PbSlot& s = slot(m, layer, role);
    if (s.mat) pb_qmat_free(s.mat);
    s.mat = mat;
    return PB_OK;
}

int pb_model_set_mtp(pb_model* m, int window) {
    if (!m) return PB_ERR_ARG;
    pb_ctx* ctx = m->ctx;
    PB_TRY(pb_enter(ctx));
    if (m->finalized) PB_FAIL(ctx, PB_ERR_STATE, "pb_model_set_mtp: model already finalized");
    if (window < 1) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_set_mtp: window %d", window);
    m->mtp_window = window;
    return PB_OK;
}

int pb_model_set_indexer(pb_model* m, int budget, int ratio, int n_head, int head_dim) {
    if (!m) return PB_ERR_ARG;
    pb_ctx* ctx = m->ctx;
    PB_TRY(pb_enter(ctx));
    if (m->finalized) PB_FAIL(ctx, PB_ERR_STATE, "pb_model_set_indexer: model already finalized");
    if (n_head < 0 || (n_head > 0 && (ratio < 1 || budget < ratio || budget % ratio || head_dim < m->cfg.n_rot || head_dim % 32 || head_dim > 256)))
        PB_FAIL(ctx, PB_ERR_ARG, "pb_model_set_indexer: budget %d ratio %d heads %d head dim %d (budget a multiple of ratio; head dim a multiple of 32 in [n_rot, 256])", budget, ratio, n_head, head_dim);
    m->idx_budget = budget; m->idx_ratio = ratio; m->idx_nh = n_head; m->idx_hd = head_dim;
    return PB_OK;
}

int pb_model_set_ple(pb_model* m, int ngram, int per_gram, int conv_k, uint32_t eos, int dim, const uint64_t* mult, const uint64_t* off, const uint64_t* vocab) {
    if (!m) return PB_ERR_ARG;
    pb_ctx* ctx = m->ctx;
    PB_TRY(pb_enter(ctx));
    if (m->finalized) PB_FAIL(ctx, PB_ERR_STATE, "pb_model_set_ple: the model is finalized");
    if (!mult || !off || !vocab) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_set_ple: null array");
    const int nh = (ngram - 1) * per_gram;
    if (ngram < 2 || ngram > 8 || per_gram < 1 || nh > 32 || conv_k < 1 || conv_k > 16 || dim < 256 || dim % 256)
        PB_FAIL(ctx, PB_ERR_ARG, "pb_model_set_ple: ngram %d (2..8), %d heads per n-gram (at most 32 heads in all), %d conv taps (1..16), dim %d (a multiple of 256)", ngram, per_gram, conv_k, dim);
    PbPleHash& h = m->ple;
    memset(&h, 0, sizeof h);
    h.ngram = ngram; h.per_gram = per_gram; h.nh = nh; h.eos = eos;
    for (int i = 0; i < ngram; i++) h.mult[i] = mult[i];
    for (int i = 0; i < nh; i++) {
        if (vocab[i] == 0 || off[i] + vocab[i] > 0xFFFFFFFFull) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_set_ple: head %d has vocabulary %llu at offset %llu", i, (unsigned long long)vocab[i], (unsigned long long)off[i]);
        h.off[i] = off[i]; h.vocab[i] = vocab[i];
    }
    m->ple_conv_k = conv_k; m->ple_dim = dim;
    return PB_OK;
}
int pb_model_set_ctx_train(pb_model* m, int ctx_train) {
    if (!m) return PB_ERR_ARG;
    pb_ctx* ctx = m->ctx;
    PB_TRY(pb_enter(ctx));
    if (ctx_train < 0) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_set_ctx_train: %d", ctx_train);
    if (m->finalized) PB_FAIL(ctx, PB_ERR_STATE, "pb_model_set_ctx_train: model already finalized");
    m->ctx_train = ctx_train;
    return PB_OK;
}

int pb_model_set_vec(pb_model* m, int layer, int role, const float* v, int64_t n) {
    if (!m) return PB_ERR_ARG;
    pb_ctx* ctx = m->ctx;
    PB_TRY(pb_enter(ctx));
    if (layer < -1 || layer >= m->cfg.n_layers || role < 0 || role >= PB_R_COUNT || !v || n <= 0) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_set_vec: bad argument (layer %d role %d n %lld)", layer, role, (long long)n);
    if (m->finalized) PB_FAIL(ctx, PB_ERR_STATE, "pb_model_set_vec: model already finalized");
    PbSlot& s = slot(m, layer, role);
    if (s.vec) cudaFree(s.vec);
    s.vec = nullptr;
    PB_CUDA(ctx, cudaMalloc(&s.vec, (size_t)n * 4 + 256));
    PB_CUDA(ctx, cudaMemcpyAsync(s.vec, v, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    s.nvec = n;
    return PB_OK;
}

static int need_mat(pb_model* m, int il, int role, int64_t rows, int64_t cols, const char* name, bool quant_only) {
    pb_ctx* ctx = m->ctx;
    pb_qmat* q = M(m, il, role);
    if (!q) PB_FAIL(ctx, PB_ERR_STATE, "layer %d: tensor %s is missing", il, name);
    if ((rows > 0 && q->rows != rows) || q->cols != cols) PB_FAIL(ctx, PB_ERR_ARG, "layer %d: %s is %lld x %lld, expected %lld x %lld", il, name, (long long)q->rows, (long long)q->cols, (long long)rows, (long long)cols);
    if (quant_only && !pb_gemvq_supported(q->type, (int)q->cols)) PB_FAIL(ctx, PB_UNSUPPORTED, "layer %d: %s has ggml type %d / %lld columns, which the fused path does not cover", il, name, q->type, (long long)q->cols);
    return PB_OK;
}
static int need_vec(pb_model* m, int il, int role, int64_t n, const char* name);
// the tensors of one hyper-connection mix (Hc, src/model/qwen4exp_gguf.rs:28, 492): f32 matrices only
static int need_hc(pb_model* m, int il, int r_norm, int r_down, int r_up, int r_inj, const char* name) {
    pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg; const int64_t w = (int64_t)c.hc * c.d;
    PB_TRY(need_vec(m, il, r_norm, w, name));
    PB_TRY(need_mat(m, il, r_down, c.hc_lr, w, name, false));
    PB_TRY(need_mat(m, il, r_up, w, c.hc_lr, name, false));
    if (r_inj >= 0) PB_TRY(need_mat(m, il, r_inj, c.hc, w, name, false));
    const int roles[3] = {r_down, r_up, r_inj};
    for (int i = 0; i < 3; i++) if (roles[i] >= 0 && M(m, il, roles[i])->type != PB_T_F32) PB_FAIL(ctx, PB_UNSUPPORTED, "layer %d: %s matrices must be f32 (ggml type %d given)", il, name, M(m, il, roles[i])->type);
    return PB_OK;
}
static int need_vec(pb_model* m, int il, int role, int64_t n, const char* name) {
    pb_ctx* ctx = m->ctx;
    if (!V(m, il, role)) PB_FAIL(ctx, PB_ERR_STATE, "layer %d: vector %s is missing", il, name);
    if (slot(m, il, role).nvec != n) PB_FAIL(ctx, PB_ERR_ARG, "layer %d: %s has %lld values, expected %lld", il, name, (long long)slot(m, il, role).nvec, (long long)n);
    return PB_OK;
}

int pb_model_finalize(pb_model* m, int ep_rank, int ep_world) {
    if (!m) return PB_ERR_ARG;
    pb_ctx* ctx = m->ctx;
    PB_TRY(pb_enter(ctx));
    const pb_cfg& c = m->cfg;
    if (ep_world < 1 || ep_rank < 0 || ep_rank >= ep_world || c.n_exp % ep_world) PB_FAIL(ctx, PB_ERR_ARG, "pb_model_finalize: rank %d of %d with %d experts", ep_rank, ep_world, c.n_exp);
    if (ep_world > 1 && (!ctx->ep_comm || ctx->ep_world != ep_world || ctx->ep_rank != ep_rank)) PB_FAIL(ctx, PB_ERR_STATE, "pb_model_finalize: call pb_ep_init(rank %d, world %d) on this context first", ep_rank, ep_world);
    m->ep_rank = ep_rank; m->ep_world = ep_world;
    m->e_lo = ep_rank * (c.n_exp / ep_world); m->e_hi = m->e_lo + c.n_exp / ep_world;
    const int ch = 2 * c.lin_nk * c.lin_dk + c.lin_nv * c.lin_dv, row = c.n_kv * c.hd;
    uint64_t wb = 0;
    int n_attn_seen = 0;
    if (m->mtp_window > 0) {
        // an MTP drafter layer (src/model/mtp.rs:104-123): one attention layer with hyper-connections, the input stage's tensors,
        // its OUTPUT = the draft-vocabulary head; embeddings come from the main model
        if (c.n_layers != 1 || c.full_every != 1 || c.hc < 1 || c.kv_bits != 0) PB_FAIL(ctx, PB_UNSUPPORTED, "an MTP drafter is one attention layer with hyper-connections and an f32 cache");
        PB_TRY(need_mat(m, -1, PB_R_MTP_FC_E, c.d, c.d, "fc_embedding", false));
        PB_TRY(need_mat(m, -1, PB_R_MTP_FC_H, c.d, c.d, "fc_hidden", false));
        PB_TRY(need_vec(m, -1, PB_R_MTP_PRE_E, c.d, "pre_fc_norm_embedding"));
        PB_TRY(need_vec(m, -1, PB_R_MTP_PRE_H, (int64_t)c.hc * c.d, "pre_fc_norm_hidden"));
        if (!M(m, -1, PB_R_OUTPUT)) PB_FAIL(ctx, PB_ERR_STATE, "an MTP drafter needs its draft-vocabulary head (OUTPUT)");
    } else
    PB_TRY(need_mat(m, -1, PB_R_TOKEN_EMBD, c.vocab, c.d, "token_embd", false));
    if (!M(m, -1, PB_R_OUTPUT)) { /* falls back to token_embd (:511) */ }
    else PB_TRY(need_mat(m, -1, PB_R_OUTPUT, c.vocab, c.d, "output", true));
    if (!pb_gemvq_supported((M(m, -1, PB_R_OUTPUT) ? M(m, -1, PB_R_OUTPUT) : M(m, -1, PB_R_TOKEN_EMBD))->type, c.d)) PB_FAIL(ctx, PB_UNSUPPORTED, "lm-head type is not covered by the fused path");
    if (c.hc == 0) PB_TRY(need_vec(m, -1, PB_R_OUT_NORM, c.d, "output_norm"));
    else PB_TRY(need_hc(m, -1, PB_R_OUT_HC_NORM, PB_R_OUT_HC_DOWN, PB_R_OUT_HC_UP, -1, "output_hc"));
    wb += (M(m, -1, PB_R_OUTPUT) ? M(m, -1, PB_R_OUTPUT) : M(m, -1, PB_R_TOKEN_EMBD))->nbytes;
    m->ple_idx.assign((size_t)c.n_layers, -1); m->n_ple = 0;
    if (m->ple.ngram > 0) {
        if (m->mtp_window > 0) PB_FAIL(ctx, PB_UNSUPPORTED, "an MTP drafter has no n-gram embeddings");
        pb_qmat* tab = M(m, -1, PB_R_PLE_TAB);
        if (!tab || tab->cols != m->ple_dim) PB_FAIL(ctx, PB_ERR_STATE, "per_layer_token_embd: missing, or not %d columns wide", m->ple_dim);
        for (int i = 0; i < m->ple.nh; i++)
            if ((int64_t)(m->ple.off[i] + m->ple.vocab[i]) > tab->rows) PB_FAIL(ctx, PB_ERR_ARG, "n-gram head %d reaches row %llu of a table of %lld rows", i, (unsigned long long)(m->ple.off[i] + m->ple.vocab[i]), (long long)tab->rows);
    }
    for (int il = 0; il < c.n_layers; il++) {
        if (M(m, il, PB_R_PLE_KEY)) {
            if (m->ple.ngram == 0) PB_FAIL(ctx, PB_ERR_STATE, "layer %d holds n-gram embedding tensors, but pb_model_set_ple was not called", il);
            const int64_t w = (int64_t)(c.hc > 0 ? c.hc : 1) * c.d, ein = (int64_t)m->ple.nh * m->ple_dim;
            PB_TRY(need_mat(m, il, PB_R_PLE_KEY, w, ein, "ple_key", false));
            PB_TRY(need_mat(m, il, PB_R_PLE_VALUE, c.d, ein, "ple_value", false));
            PB_TRY(need_vec(m, il, PB_R_PLE_NORM_KEY, w, "ple_norm_key"));
            PB_TRY(need_vec(m, il, PB_R_PLE_NORM_QUERY, w, "ple_norm_query"));
            PB_TRY(need_vec(m, il, PB_R_PLE_NORM_CONV, w, "ple_norm_conv"));
            PB_TRY(need_vec(m, il, PB_R_PLE_CONV, w * m->ple_conv_k, "ple_conv1d"));
            m->ple_idx[il] = m->n_ple++;
        }
        if (c.hc == 0) {
            PB_TRY(need_vec(m, il, PB_R_ATTN_NORM, c.d, "attn_norm"));
            PB_TRY(need_vec(m, il, PB_R_FFN_NORM, c.d, "ffn_norm"));
        } else {
            PB_TRY(need_hc(m, il, PB_R_HCA_NORM, PB_R_HCA_DOWN, PB_R_HCA_UP, PB_R_HCA_INJECT, "hc_attn"));
            PB_TRY(need_hc(m, il, PB_R_HCF_NORM, PB_R_HCF_DOWN, PB_R_HCF_UP, PB_R_HCF_INJECT, "hc_ffn"));
        }
        if (m->kind[il]) {
            PB_TRY(need_mat(m, il, PB_R_ATTN_Q, (int64_t)c.n_head * 2 * c.hd, c.d, "attn_q", true));
            PB_TRY(need_mat(m, il, PB_R_ATTN_K, row, c.d, "attn_k", true));
            PB_TRY(need_mat(m, il, PB_R_ATTN_V, row, c.d, "attn_v", true));
            PB_TRY(need_mat(m, il, PB_R_ATTN_O, c.d, (int64_t)c.n_head * c.hd, "attn_output", true));
            PB_TRY(need_vec(m, il, PB_R_ATTN_Q_NORM, c.hd, "attn_q_norm"));
            PB_TRY(need_vec(m, il, PB_R_ATTN_K_NORM, c.hd, "attn_k_norm"));
            if (M(m, il, PB_R_ATTN_Q)->type != M(m, il, PB_R_ATTN_K)->type || M(m, il, PB_R_ATTN_Q)->type != M(m, il, PB_R_ATTN_V)->type)
                PB_FAIL(ctx, PB_UNSUPPORTED, "layer %d: attn_q/k/v must share one ggml type", il);
            wb += M(m, il, PB_R_ATTN_Q)->nbytes + M(m, il, PB_R_ATTN_K)->nbytes + M(m, il, PB_R_ATTN_V)->nbytes + M(m, il, PB_R_ATTN_O)->nbytes;
            // QSA indexer (Mixer::Attn idx, :501): all attention layers or none
            const bool has = m->idx_nh > 0 && M(m, il, PB_R_IDX_Q) != nullptr;
            if (n_attn_seen > 0 && has != m->qsa) PB_FAIL(ctx, PB_UNSUPPORTED, "layer %d: indexer tensors on some attention layers only", il);
            m->qsa = has; n_attn_seen++;
            if (has) {
                PB_TRY(need_mat(m, il, PB_R_IDX_Q, (int64_t)m->idx_nh * m->idx_hd, c.d, "indexer.q_proj", true));
                PB_TRY(need_mat(m, il, PB_R_IDX_K, m->idx_hd, c.d, "indexer.k_proj", true));
                PB_TRY(need_vec(m, il, PB_R_IDX_Q_NORM, m->idx_hd, "indexer.q_norm"));
                PB_TRY(need_vec(m, il, PB_R_IDX_K_NORM, m->idx_hd, "indexer.k_norm"));
                if (M(m, il, PB_R_IDX_Q)->type != M(m, il, PB_R_IDX_K)->type) PB_FAIL(ctx, PB_UNSUPPORTED, "layer %d: indexer q_proj / k_proj must share one ggml type", il);
                wb += M(m, il, PB_R_IDX_Q)->nbytes + M(m, il, PB_R_IDX_K)->nbytes;
            }
        } else {
            PB_TRY(need_mat(m, il, PB_R_LIN_QKV, ch, c.d, "attn_qkv", true));
            PB_TRY(need_mat(m, il, PB_R_LIN_Z, (int64_t)c.lin_nv * c.lin_dv, c.d, "attn_gate", true));
            PB_TRY(need_mat(m, il, PB_R_LIN_BETA, c.lin_nv, c.d, "ssm_beta", true));
            PB_TRY(need_mat(m, il, PB_R_LIN_ALPHA, c.lin_nv, c.d, "ssm_alpha", true));
            PB_TRY(need_mat(m, il, PB_R_LIN_OUT, c.d, (int64_t)c.lin_nv * c.lin_dv, "ssm_out", true));
            PB_TRY(need_vec(m, il, PB_R_LIN_A, c.lin_nv, "ssm_a"));
            PB_TRY(need_vec(m, il, PB_R_LIN_DT, c.lin_nv, "ssm_dt.bias"));
            PB_TRY(need_vec(m, il, PB_R_LIN_CONV, (int64_t)ch * c.conv_k, "ssm_conv1d"));
            PB_TRY(need_vec(m, il, PB_R_LIN_NORM, c.lin_dv, "ssm_norm"));
            const int t0 = M(m, il, PB_R_LIN_QKV)->type;
            if (M(m, il, PB_R_LIN_Z)->type != t0 || M(m, il, PB_R_LIN_BETA)->type != t0 || M(m, il, PB_R_LIN_ALPHA)->type != t0)
                PB_FAIL(ctx, PB_UNSUPPORTED, "layer %d: attn_qkv/attn_gate/ssm_beta/ssm_alpha must share one ggml type", il);
            wb += M(m, il, PB_R_LIN_QKV)->nbytes + M(m, il, PB_R_LIN_Z)->nbytes + M(m, il, PB_R_LIN_BETA)->nbytes + M(m, il, PB_R_LIN_ALPHA)->nbytes + M(m, il, PB_R_LIN_OUT)->nbytes;
        }
        // MoE: the router is f32; expert tensors hold all experts or this rank's contiguous shard
        PB_TRY(need_mat(m, il, PB_R_ROUTER, c.n_exp, c.d, "ffn_gate_inp", false));
        if (M(m, il, PB_R_ROUTER)->type != PB_T_F32) PB_FAIL(ctx, PB_UNSUPPORTED, "layer %d: the router must be f32", il);
        const int64_t nloc = c.n_exp / ep_world;
        const int roles[3] = {PB_R_EXP_GATE, PB_R_EXP_UP, PB_R_EXP_DOWN};
        for (int r = 0; r < 3; r++) {
            pb_qmat* q = M(m, il, roles[r]);
            const int64_t per = r < 2 ? c.ff_exp : c.d, cols = r < 2 ? c.d : c.ff_exp;
            if (!q) PB_FAIL(ctx, PB_ERR_STATE, "layer %d: expert tensor %d is missing", il, r);
            if (q->cols != cols || (q->rows != per * c.n_exp && q->rows != per * nloc)) PB_FAIL(ctx, PB_ERR_ARG, "layer %d: expert tensor %d is %lld x %lld", il, r, (long long)q->rows, (long long)q->cols);
            if (!pb_gemvq_supported(q->type, (int)cols)) PB_FAIL(ctx, PB_UNSUPPORTED, "layer %d: expert tensor type %d is not covered by the fused path", il, q->type);
            wb += (uint64_t)c.top_k * per * q->row_bytes;
        }
        if (M(m, il, PB_R_EXP_GATE)->type != M(m, il, PB_R_EXP_UP)->type || M(m, il, PB_R_EXP_GATE)->rows != M(m, il, PB_R_EXP_UP)->rows) PB_FAIL(ctx, PB_UNSUPPORTED, "layer %d: gate and up experts must share type and shape", il);
        if (c.ff_sh != c.ff_exp) PB_FAIL(ctx, PB_UNSUPPORTED, "shared expert width %d differs from the routed width %d", c.ff_sh, c.ff_exp);
        PB_TRY(need_mat(m, il, PB_R_SH_GATE, c.ff_sh, c.d, "ffn_gate_shexp", true));
        PB_TRY(need_mat(m, il, PB_R_SH_UP, c.ff_sh, c.d, "ffn_up_shexp", true));
        PB_TRY(need_mat(m, il, PB_R_SH_DOWN, c.d, c.ff_sh, "ffn_down_shexp", true));
        if (M(m, il, PB_R_SH_GATE)->type != M(m, il, PB_R_EXP_GATE)->type || M(m, il, PB_R_SH_UP)->type != M(m, il, PB_R_EXP_GATE)->type || M(m, il, PB_R_SH_DOWN)->type != M(m, il, PB_R_EXP_DOWN)->type)
            PB_FAIL(ctx, PB_UNSUPPORTED, "layer %d: shared-expert tensors must have the types of the routed experts", il);
        PB_TRY(need_vec(m, il, PB_R_SH_GATE_INP, c.d, "ffn_gate_inp_shexp"));
        wb += M(m, il, PB_R_ROUTER)->nbytes + M(m, il, PB_R_SH_GATE)->nbytes + M(m, il, PB_R_SH_UP)->nbytes + M(m, il, PB_R_SH_DOWN)->nbytes;
    }
    // rope_inv, qn_ctx.rs:160-186: base^(-2i/n_rot) at or under the trained context; above it YaRN (beta_fast 32, beta_slow 1:
    // low indices divided by scale = max_ctx / ctx_train, high indices unchanged, a linear ramp between the correction
    // dimensions).  The entry behind the table holds mscale = 1 + 0.1 ln(scale), which the kernels apply to cos and sin.
    const int half = c.n_rot / 2;
    std::vector<float> inv((size_t)half + 1);
    const float scale = m->ctx_train > 0 && c.max_ctx > m->ctx_train ? (float)c.max_ctx / (float)m->ctx_train : 1.0f;
    for (int i = 0; i < half; i++) inv[i] = powf(c.rope_base, -(2.0f * (float)i) / (float)c.n_rot);
    inv[half] = 1.0f;
    if (scale > 1.0f) {
        const float dim = (float)c.n_rot, two_pi = 2.0f * 3.14159265358979323846f;
        float lo = floorf((dim * logf((float)m->ctx_train / (32.0f * two_pi))) / (2.0f * logf(c.rope_base)));
        float hi = ceilf((dim * logf((float)m->ctx_train / (1.0f * two_pi))) / (2.0f * logf(c.rope_base)));
        if (lo < 0.0f) lo = 0.0f;
        const float top = (float)(half > 0 ? half - 1 : 0);
        if (hi > top) hi = top;
        for (int i = 0; i < half; i++) {
            const float extrap = inv[i], interp = extrap / scale;
            float ramp = fabsf(hi - lo) < 1e-6f ? 1.0f : ((float)i - lo) / (hi - lo);
            ramp = ramp < 0.0f ? 0.0f : (ramp > 1.0f ? 1.0f : ramp);
            inv[i] = interp * (1.0f - ramp) + extrap * ramp;
        }
        inv[half] = 1.0f + 0.1f * logf(scale);
    }
    PB_CUDA(ctx, cudaMalloc(&m->rope_inv, inv.size() * 4));
    PB_CUDA(ctx, cudaMemcpy(m->rope_inv, inv.data(), inv.size() * 4, cudaMemcpyHostToDevice));
    m->weight_bytes_step = wb;
    m->finalized = true;
    return PB_OK;
}

int pb_model_cfg(const pb_model* m, pb_cfg* out) { if (!m || !out) return PB_ERR_ARG; *out = m->cfg; return PB_OK; }
int pb_model_destroy(pb_model* m) {
    if (!m) return PB_OK;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    for (auto& s : m->slots) { if (s.mat) pb_qmat_free(s.mat); if (s.vec) cudaFree(s.vec); }
    if (m->rope_inv) cudaFree(m->rope_inv);
    delete m;
    return PB_OK;
}

int pb_caps_get(const pb_model* m, pb_caps* caps) {
    if (!m || !caps) return PB_ERR_ARG;
    caps->multi_ok = 1; caps->max_window = 8; caps->max_ctx = m->cfg.max_ctx; caps->max_batch = 1024; caps->ep_world = m->ep_world;
    return PB_OK;
}

// ------------------------------------------------------------------------------------ state

static int state_create(pb_model* m, int batch, bool sharded, pb_state** out) {
    if (!m || !out) return PB_ERR_ARG;
    pb_ctx* ctx = m->ctx;
    *out = nullptr;
    PB_TRY(pb_enter(ctx));
    if (!m->finalized) PB_FAIL(ctx, PB_ERR_STATE, "pb_state_create: call pb_model_finalize first");
    if (batch < 1 || batch > 1024) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_create: batch %d outside 1..1024", batch);
    const pb_cfg& c = m->cfg;
    pb_state* s = new (std::nothrow) pb_state();
    if (!s) PB_FAIL(ctx, PB_ERR_OOM, "host allocation failed");
    s->m = m; s->batch = batch;
    const int B = batch;
    s->sharded = sharded && m->ep_world > 1;
    s->moe_t = s->sharded ? batch * m->ep_world : batch; s->tok0 = s->sharded ? batch * m->ep_rank : 0;
    const bool solo = B == 1 && !s->sharded;
    const int Ba = solo ? PB_PREFILL_CHUNK : B;   // activation rows: a batch-1 state also runs verify windows (up to 8 tokens) and prefill chunks (up to 256)
    const int Bm = s->moe_t > Ba ? s->moe_t : Ba;                 // tokens a MoE block of this state may see
    s->moe_cap = Bm;
    const int ch = 2 * c.lin_nk * c.lin_dk + c.lin_nv * c.lin_dv;
    const int64_t lin_proj = (int64_t)ch + (int64_t)c.lin_nv * c.lin_dv + 2 * c.lin_nv;
    const int64_t att_proj = (int64_t)c.n_head * 2 * c.hd + 2 * (int64_t)c.n_kv * c.hd;
    s->ldproj = ((lin_proj > att_proj ? lin_proj : att_proj) + 3) & ~(int64_t)3;
    const int64_t wide = (int64_t)c.lin_nv * c.lin_dv > (int64_t)c.n_head * c.hd ? (int64_t)c.lin_nv * c.lin_dv : (int64_t)c.n_head * c.hd;
    int rc = PB_OK;
#define A(p, n) if (rc == PB_OK) rc = dalloc(s, &s->p, (size_t)(n))
    A(pos, B); A(ids, Ba); A(next, Ba); A(amax, Ba); A(wpos, PB_PREFILL_CHUNK);
    A(ticket, 8 + (size_t)(Bm + 7) / 8);   // whole-launch counters, then one per group of 8 tokens of the router
    A(x, (size_t)Ba * c.d * (c.hc > 0 ? c.hc : 1));
    if (m->n_ple > 0) {
        const size_t w = (size_t)c.d * (c.hc > 0 ? c.hc : 1);
        s->ple_R = (m->ple_conv_k - 1) * m->ple.ngram + (solo ? PB_PREFILL_CHUNK : 1);
        A(tok_hist, (size_t)B * c.max_ctx); A(ple_base, B); A(ple_rows, (size_t)Ba * m->ple.nh); A(ple_emb, (size_t)Ba * m->ple.nh * m->ple_dim);
        A(ple_key, (size_t)Ba * w); A(ple_val, (size_t)Ba * c.d); A(ple_gated, (size_t)Ba * w);
        s->ple_ring.assign((size_t)m->n_ple, nullptr);
        for (int i = 0; i < m->n_ple; i++) { if (rc == PB_OK) rc = dalloc(s, &s->ple_ring[(size_t)i], (size_t)B * s->ple_R * w); }
    }
    if (c.hc > 0) { A(hxn, (size_t)Ba * c.hc * c.d); A(hgate, (size_t)Ba * c.hc * c.d); A(hlo, (size_t)Ba * c.hc_lr); A(hinj, (size_t)Ba * c.hc); A(hmix, (size_t)Ba * c.d); }
    A(xin, (size_t)Ba * (wide > c.d ? wide : c.d)); A(yout, (size_t)Ba * c.d);
    A(proj, (size_t)Ba * s->ldproj); A(olin, (size_t)Ba * wide); A(att, (size_t)Ba * wide);
    A(rlogits, (size_t)Bm * (c.n_exp + 1));
    A(xq, (size_t)Bm * pb_xq_words(c.d));
    A(sel_e, (size_t)Bm * c.top_k); A(sel_w, (size_t)Bm * c.top_k); A(n_used, 4); A(used_e, c.n_exp + 1); A(used_off, c.n_exp + 2);
    A(ent_tok, (size_t)Bm * c.top_k); A(ent_slot, (size_t)Bm * c.top_k); A(ent_w, (size_t)Bm * c.top_k);
    A(h, (size_t)Bm * c.top_k * c.ff_exp); A(h_sh, (size_t)Bm * c.ff_sh);
    A(hq, (size_t)Bm * (c.top_k + 1) * pb_xq_words(c.ff_exp > c.ff_sh ? c.ff_exp : c.ff_sh));
    A(part, (size_t)Bm * c.top_k * c.d); A(part_sh, (size_t)Bm * c.d);
    s->ldg = c.d + ((c.n_exp + 1 + 3) & ~3);
    if (s->sharded) {
        A(xs, (size_t)B * s->ldg); A(ep_seq, 4);
        // PYRE_B200_EP_EXCHANGE=nccl keeps the two NCCL collectives per MoE block; the default is the in-kernel peer exchange
        const char* ex = getenv("PYRE_B200_EP_EXCHANGE");
        const bool want_p2p = !(ex && strcmp(ex, "nccl") == 0) && m->ep_world <= PB_EP_MAX_WORLD;
        if (want_p2p && rc == PB_OK) {
            const size_t xg_bytes = ((size_t)Bm * s->ldg * 4 + 255) & ~(size_t)255, part_bytes = ((size_t)B * c.top_k * c.d * 4 + 255) & ~(size_t)255;
            const size_t flag_bytes = ((size_t)2 * m->ep_world * 8 + 255) & ~(size_t)255;
            rc = pb_ep_symm_alloc(ctx, xg_bytes + part_bytes + flag_bytes, &s->symm);
            if (rc == PB_OK) {
                s->p2p = true;
                s->xg = reinterpret_cast<float*>(s->symm.local);
                s->part_rs = reinterpret_cast<float*>(reinterpret_cast<char*>(s->symm.local) + xg_bytes);
                PbEpExch& x = s->exch;
                x.rank = m->ep_rank; x.world = m->ep_world; x.seq_base = s->ep_seq; x.wait_ns = s->ep_seq + 1; x.status = ctx->dev_status;
                const char* lim = getenv("PYRE_B200_EP_SPIN");
                x.spin_limit = lim ? (unsigned)atoi(lim) : (5u << 20);   // about a second of polling
                std::vector<float*> pt((size_t)Bm);
                for (int p = 0; p < m->ep_world; p++) {
                    char* base = reinterpret_cast<char*>(s->symm.peer[p]);
                    x.peer_xg[p] = reinterpret_cast<float*>(base);
                    x.peer_flags[p] = reinterpret_cast<unsigned long long*>(base + xg_bytes + part_bytes);
                    for (int j = 0; j < B; j++) pt[(size_t)p * B + j] = reinterpret_cast<float*>(base + xg_bytes) + (size_t)j * c.top_k * c.d;
                }
                A(part_tok, (size_t)Bm); A(exch_dev, 1);
                if (rc == PB_OK && cudaMemcpyAsync(s->part_tok, pt.data(), pt.size() * sizeof(float*), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) rc = PB_ERR_CUDA;
                if (rc == PB_OK && cudaMemcpyAsync(s->exch_dev, &s->exch, sizeof(PbEpExch), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) rc = PB_ERR_CUDA;
                if (rc == PB_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = PB_ERR_CUDA;   // `pt` is a local
            }
        } else { A(xg, (size_t)Bm * s->ldg); A(part_rs, (size_t)B * c.top_k * c.d); }
    }
    A(logits, (size_t)(solo ? PB_MAX_WINDOW : B) * c.vocab);   // a prefill chunk keeps only its last token's logits
    if (B == 1 && !s->sharded) { A(fops, (size_t)c.n_layers * 8 + 8); A(fh, (size_t)(c.top_k + 1) * c.ff_exp); }
    s->trace_cap = 4096;
    A(trace, (size_t)s->trace_cap * B); A(trace_len, 2);
    // attention: one CTA per SM (split x KV head x sequence)
    const int G = c.n_kv > 0 ? c.n_head / c.n_kv : 1;
    int ns = ctx->sm_count / (c.n_kv * B > 0 ? c.n_kv * B : 1);
    if (ns < 1) ns = 1;
    if (ns > 128) ns = 128;
    // 4-bit cache: one split per (sequence, KV head) walks the f32 ring, the others the packed positions
    static const bool attn_mma = !(getenv("PYRE_B200_ATTN_MMA") && atoi(getenv("PYRE_B200_ATTN_MMA")) == 0);
    s->nsplit_packed = 0;
    if (c.kv_bits == 4 && G <= 8 && c.hd == 256 && attn_mma) {
        if (ns >= 8) s->nsplit_packed = ns - 1;
        else {
            // many (sequence, KV head) pairs: several CTAs per SM's worth of work, so that the tail wave stays short
            int fine = 8 * ctx->sm_count / (c.n_kv * B);
            static const int fine_cap = getenv("PYRE_B200_ATTN_FINE") ? atoi(getenv("PYRE_B200_ATTN_FINE")) : 16;
            if (fine > fine_cap) fine = fine_cap;
            s->nsplit_packed = fine > ns ? fine : ns;
            ns = s->nsplit_packed + 1;
        }
    }
    s->nsplit = ns;
    const size_t nparts = solo && (size_t)PB_PREFILL_CHUNK * PB_WIN_SPLITS > (size_t)ns ? (size_t)PB_PREFILL_CHUNK * PB_WIN_SPLITS : (size_t)B * ns;   // a prefill chunk: its tokens x PB_WIN_SPLITS
    A(part_ml, nparts * c.n_kv * G * 2); A(part_acc, nparts * c.n_kv * G * c.hd);
    s->conv.assign(m->n_lin, nullptr); s->ssm.assign(m->n_lin, nullptr); s->kv.assign(m->n_attn, PbKv());
    s->ldi = (((int64_t)m->idx_nh + 1) * m->idx_hd + 3) & ~(int64_t)3; s->nb_cap = c.max_ctx / (m->idx_ratio > 0 ? m->idx_ratio : 1) + 1; s->mask_ld = c.max_ctx / 32 + 1;
    for (int i = 0; i < m->n_lin && rc == PB_OK; i++) {
        rc = dalloc(s, &s->conv[i], (size_t)B * c.conv_k * ch);
        if (rc == PB_OK) rc = dalloc(s, &s->ssm[i], (size_t)B * c.lin_nv * c.lin_dk * c.lin_dv);
    }
    const int64_t rowh = c.hd;
    // 4-bit cache: the f32 ring holds the recent positions, the 64 that wait for the next packing step, and (batch-1 states)
    // a whole prefill chunk appended before its packing step
    s->ring_cap = c.kv_bits == 4 ? (int64_t)c.kv_recent + 64 + (solo ? PB_PREFILL_CHUNK : 0) : (int64_t)c.max_ctx;
    if (rc == PB_OK) rc = dalloc(s, &s->q4n_all, (size_t)(m->n_attn > 0 ? m->n_attn : 1) * B);
    for (int i = 0; i < m->n_attn && rc == PB_OK; i++) {
        PbKv& k = s->kv[i];
        const size_t heads = (size_t)B * c.n_kv;
        rc = dalloc(s, &k.kr, heads * s->ring_cap * rowh);
        if (rc == PB_OK) rc = dalloc(s, &k.vr, heads * s->ring_cap * rowh);
        if (rc == PB_OK) k.q4n = s->q4n_all + (size_t)i * B;
        const size_t packed_pos = c.kv_bits == 4 ? (size_t)c.max_ctx : 1;
        if (rc == PB_OK) rc = dalloc(s, &k.kw, heads * packed_pos * (rowh / 8));
        if (rc == PB_OK) rc = dalloc(s, &k.vw, heads * packed_pos * (rowh / 8));
        if (rc == PB_OK) rc = dalloc(s, &k.ks, heads * packed_pos * (rowh / 32));
        if (rc == PB_OK) rc = dalloc(s, &k.vs, heads * packed_pos * (rowh / 32));
        if (rc == PB_OK && m->qsa) rc = dalloc(s, &k.ik, (size_t)B * c.max_ctx * m->idx_hd);
        if (rc == PB_OK && m->qsa) rc = dalloc(s, &k.ib, (size_t)B * s->nb_cap * m->idx_hd);
    }
    if (m->qsa) {
        A(iproj, (size_t)Ba * s->ldi); A(qsa_scores, (size_t)B * s->nb_cap); A(qsa_mask, (size_t)B * s->mask_ld); A(qsa_on, (size_t)B);
    }
#undef A
    if (rc == PB_OK && cudaMallocHost(&s->pin_u32, (size_t)(s->trace_cap + 2) * B * 4 + PB_PREFILL_CHUNK * 4) != cudaSuccess) { ctx->err = "pinned allocation failed"; rc = PB_ERR_OOM; }
    if (rc == PB_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) { ctx->err = "stream sync failed"; rc = PB_ERR_CUDA; }
    if (rc != PB_OK) { pb_state_destroy(s); return rc; }
    *out = s;
    return PB_OK;
}

int pb_state_create(pb_model* m, int batch, pb_state** out) { return state_create(m, batch, false, out); }
// Sharded tokens: `batch` is this rank's share of a global batch of batch * ep_world sequences
// (a plain state when the model is not expert-parallel).
int pb_state_create_sharded(pb_model* m, int batch, pb_state** out) { return state_create(m, batch, true, out); }

int pb_state_destroy(pb_state* s) {
    if (!s) return PB_OK;
    cudaSetDevice(s->m->ctx->device);
    cudaStreamSynchronize(s->m->ctx->stream);
    if (s->graph) cudaGraphExecDestroy(s->graph);
    if (s->ev0) cudaEventDestroy(s->ev0);
    if (s->ev1) cudaEventDestroy(s->ev1);
    for (cudaGraphExec_t g : s->win_graph) if (g) cudaGraphExecDestroy(g);
    for (void* p : s->allocs) cudaFree(p);
    if (s->mtp) { if (s->mtp->ds) pb_state_destroy(s->mtp->ds); if (s->mtp->pin) cudaFreeHost(s->mtp->pin); delete s->mtp; }   // its device buffers are in s->allocs
    pb_ep_symm_free(s->m->ctx, &s->symm);
    if (s->pin_u32) cudaFreeHost(s->pin_u32);
    if (s->pin_logits) cudaFreeHost(s->pin_logits);
    delete s;
    return PB_OK;
}

int pb_state_set_pos(pb_state* s, int64_t pos) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx;
    PB_TRY(pb_enter(ctx));
    if (pos < 0 || pos > s->m->cfg.max_ctx) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_set_pos: %lld outside 0..%d", (long long)pos, s->m->cfg.max_ctx);
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    // The packed boundary of the 4-bit cache only ever advances on the device (pb_kv_append_kernel): positions
    // below it exist in packed form only.  Rewinding to 0 starts a fresh sequence (boundary back to 0); a
    // position below the boundary cannot be served (the reference's spec_keep drops packed rows in that
    // case, kv8_drop :2507; here the f32 rows are gone) and is refused.
    if (s->m->cfg.kv_bits == 4 && s->m->n_attn > 0) {
        const size_t nq = (size_t)s->m->n_attn * s->batch;
        if (pos == 0) PB_CUDA(ctx, cudaMemsetAsync(s->q4n_all, 0, nq * 8, ctx->stream));
        else {
            std::vector<int64_t> q(nq);
            PB_CUDA(ctx, cudaMemcpy(q.data(), s->q4n_all, nq * 8, cudaMemcpyDeviceToHost));
            for (size_t i = 0; i < nq; i++)
                if (pos < q[i]) PB_FAIL(ctx, PB_ERR_STATE, "pb_state_set_pos: position %lld is below the packed KV boundary %lld of sequence %d", (long long)pos, (long long)q[i], (int)(i % s->batch));
        }
    }
    std::vector<int64_t> v((size_t)s->batch, pos);
    PB_CUDA(ctx, cudaMemcpyAsync(s->pos, v.data(), v.size() * 8, cudaMemcpyHostToDevice, ctx->stream));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    // n-gram embeddings: a position set ahead of the sequence (or back to 0) starts a history there; a position set back keeps what is below it
    if (s->ple_base && (pos == 0 || pos > s->pos_host || pos < s->ple_base_host)) {
        std::vector<int64_t> b((size_t)s->batch, pos);
        PB_CUDA(ctx, cudaMemcpy(s->ple_base, b.data(), b.size() * 8, cudaMemcpyHostToDevice));
        s->ple_base_host = pos;
    }
    s->pos_host = pos;
    mtp_moved(s, pos);
    return PB_OK;
}
int pb_state_reset(pb_state* s) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx;
    PB_TRY(pb_state_set_pos(s, 0));
    const pb_cfg& c = s->m->cfg;
    for (int li = 0; li < s->m->n_lin; li++) {
        PB_CUDA(ctx, cudaMemsetAsync(s->conv[li], 0, conv_elems(c, s->batch) * 4, ctx->stream));
        PB_CUDA(ctx, cudaMemsetAsync(s->ssm[li], 0, ssm_elems(c, s->batch) * 4, ctx->stream));
    }
    s->verify_t = 0;
    return PB_OK;
}
int pb_state_pos(const pb_state* s, int64_t* pos) { if (!s || !pos) return PB_ERR_ARG; *pos = s->pos_host; return PB_OK; }

// ---- layer pieces -----------------------------------------------------------------------------

static void seg(PbGemvQArgs& a, int i, pb_qmat* q, int64_t yoff) { a.seg[i].w = q->data; a.seg[i].wr = q->rdata; a.seg[i].rows = q->rows; a.seg[i].yoff = yoff; }

// y (+)= W_segs . act(x) for all batch columns, in tiles of 16 columns
static int gemv_cols(pb_ctx* ctx, PbGemvQArgs a, int B, bool prefill = false) {
    const float* x = a.x; float* y = a.y; const float* z = a.z; const uint32_t* xq = a.xq_in;
    a.exact = prefill ? 0 : 1;   // decode steps and verify windows keep exact weights; prefill chunks may take the tcgen05 GEMM
    // the tensor-core path takes all columns at once (one staging pass for all its launches)
    static const bool use_mma = !(getenv("PYRE_B200_MMA") && atoi(getenv("PYRE_B200_MMA")) == 0);
    if (use_mma && a.mode != PB_ACT_PREQ && pb_gemmh_supported(a.type, a.cols, B) && (size_t)B * a.cols * 4 + 256 * (size_t)((B + 7) / 8) <= PB_XH_BYTES) { a.t = B; return pb_launch_gemvq(ctx, a); }
    for (int b0 = 0; b0 < B; b0 += 16) {
        a.t = B - b0 < 16 ? B - b0 : 16;
        a.x = x ? x + (int64_t)b0 * a.ldx : nullptr; a.y = y + (int64_t)b0 * a.ldy; a.z = z ? z + (int64_t)b0 * a.ldz : nullptr;
        a.xq_in = xq ? xq + (size_t)b0 * pb_xq_words(a.cols) : nullptr;
        PB_TRY(pb_launch_gemvq(ctx, a));
    }
    return PB_OK;
}

// Gated DeltaNet mixer: x_in (normalized when norm_w == null) -> y (stored or added)
static int run_lin(pb_state* s, int il, const float* x_in, const float* norm_w, float* y, int64_t ldy, int accumulate) {
    pb_model* m = s->m; pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg; const int B = s->batch, li = m->idx[il];
    const int ch = 2 * c.lin_nk * c.lin_dk + c.lin_nv * c.lin_dv, w = c.lin_nv * c.lin_dv;
    PbGemvQArgs a; memset(&a, 0, sizeof a);
    a.type = M(m, il, PB_R_LIN_QKV)->type; a.cols = c.d; a.nseg = 4;
    seg(a, 0, M(m, il, PB_R_LIN_QKV), 0); seg(a, 1, M(m, il, PB_R_LIN_Z), ch); seg(a, 2, M(m, il, PB_R_LIN_BETA), ch + w); seg(a, 3, M(m, il, PB_R_LIN_ALPHA), ch + w + c.lin_nv);
    a.x = x_in; a.ldx = c.d; a.y = s->proj; a.ldy = s->ldproj; a.mode = norm_w ? PB_ACT_NORM : PB_ACT_PLAIN; a.norm_w = norm_w; a.eps = c.eps;
    const int ncol = s->win_t > 0 ? s->win_t : B;   // window mode: the columns are consecutive tokens of sequence 0
    const bool prefill = s->win_t >= 16 && !s->win_ckpt;
    PB_TRY(gemv_cols(ctx, a, ncol, prefill));
    PbDeltaParams d; memset(&d, 0, sizeof d);
    d.proj = s->proj; d.ldp = s->ldproj; d.conv_w = V(m, il, PB_R_LIN_CONV); d.a = V(m, il, PB_R_LIN_A); d.dt = V(m, il, PB_R_LIN_DT);
    d.conv = s->conv[li]; d.ssm = s->ssm[li]; d.pos = s->pos; d.out = s->olin; d.ldo = w;
    d.nk = c.lin_nk; d.nv = c.lin_nv; d.dk = c.lin_dk; d.dv = c.lin_dv; d.conv_k = c.conv_k; d.batch = B;
    if (s->win_t > 0 && pb_deltanet_seq_supported(d) && (!s->win_ckpt || s->win_t <= 8)) {
        // all tokens in one launch, the state slice stays in registers; a verify window also gets its rollback checkpoints
        // (the state after each token but the last) written from there
        d.pos = s->wpos; d.batch = 1;
        PbDeltaCk ck; memset(&ck, 0, sizeof ck);
        if (s->win_ckpt) for (int j = 0; j + 1 < s->win_t; j++) { ck.conv[j] = s->ck_conv[(size_t)li * PB_MAX_WINDOW + j]; ck.ssm[j] = s->ck_ssm[(size_t)li * PB_MAX_WINDOW + j]; }
        PB_TRY(pb_launch_deltanet_seq(ctx, d, s->win_t, s->win_ckpt ? &ck : nullptr));
    } else if (s->win_t > 0) {
        // the recurrence is sequential: one launch per token, with a rollback checkpoint after each but the last
        for (int j = 0; j < s->win_t; j++) {
            d.proj = s->proj + (size_t)j * s->ldproj; d.out = s->olin + (size_t)j * w; d.pos = s->wpos + j; d.batch = 1;
            PB_TRY(pb_launch_deltanet(ctx, d));
            if (s->win_ckpt && j + 1 < s->win_t) {
                PB_CUDA(ctx, cudaMemcpyAsync(s->ck_conv[(size_t)li * PB_MAX_WINDOW + j], s->conv[li], conv_elems(c, 1) * 4, cudaMemcpyDeviceToDevice, ctx->stream));
                PB_CUDA(ctx, cudaMemcpyAsync(s->ck_ssm[(size_t)li * PB_MAX_WINDOW + j], s->ssm[li], ssm_elems(c, 1) * 4, cudaMemcpyDeviceToDevice, ctx->stream));
                ctx->pdl_chain = false;
            }
        }
    } else PB_TRY(pb_launch_deltanet(ctx, d));
    PbGemvQArgs o; memset(&o, 0, sizeof o);
    o.type = M(m, il, PB_R_LIN_OUT)->type; o.cols = w; o.nseg = 1; seg(o, 0, M(m, il, PB_R_LIN_OUT), 0);
    o.x = s->olin; o.ldx = w; o.y = y; o.ldy = ldy; o.mode = PB_ACT_GNORM; o.norm_w = V(m, il, PB_R_LIN_NORM); o.z = s->proj + ch; o.ldz = s->ldproj; o.head_dim = c.lin_dv; o.eps = c.eps; o.accumulate = accumulate;
    return gemv_cols(ctx, o, ncol, prefill);
}

static void attn_params(pb_state* s, int il, PbAttnParams& p) {
    pb_model* m = s->m; const pb_cfg& c = m->cfg; const PbKv& k = s->kv[m->idx[il]];
    memset(&p, 0, sizeof p);
    p.proj = s->proj; p.ldp = s->ldproj; p.qn = V(m, il, PB_R_ATTN_Q_NORM); p.kn = V(m, il, PB_R_ATTN_K_NORM); p.rope_inv = m->rope_inv;
    p.n_rot = c.n_rot; p.eps = c.eps; p.n_head = c.n_head; p.n_kv = c.n_kv; p.hd = c.hd;
    p.kw = k.kw; p.ks = k.ks; p.vw = k.vw; p.vs = k.vs; p.kr = k.kr; p.vr = k.vr;
    p.max_ctx = c.kv_bits == 4 ? c.max_ctx : 1; p.ring_cap = s->ring_cap; p.kv_bits = c.kv_bits; p.kv_recent = c.kv_recent;
    p.pos = s->pos; p.q4n = k.q4n; p.part_ml = s->part_ml; p.part_acc = s->part_acc; p.nsplit = s->nsplit; p.nsplit_packed = s->nsplit_packed;
    { static const float rw = getenv("PYRE_B200_ATTN_RINGW") ? (float)atof(getenv("PYRE_B200_ATTN_RINGW")) : 2.5f; p.ring_weight = rw > 0.f ? rw : 2.5f; }   // measured: 2.5 .. 3.5 give the shortest batch-1 step, 2 .. 2.5 the shortest batch-32 step
    p.att = s->att; p.lda = (int64_t)c.n_head * c.hd; p.batch = s->batch;
}

static void qsa_params(pb_state* s, int il, PbQsaParams& qp) {
    pb_model* m = s->m; const pb_cfg& c = m->cfg; const PbKv& k = s->kv[m->idx[il]];
    memset(&qp, 0, sizeof qp);
    qp.iproj = s->iproj; qp.ldi = s->ldi; qp.iqn = V(m, il, PB_R_IDX_Q_NORM); qp.ikn = V(m, il, PB_R_IDX_K_NORM); qp.rope_inv = m->rope_inv; qp.n_rot = c.n_rot; qp.eps = c.eps;
    qp.inh = m->idx_nh; qp.ihd = m->idx_hd; qp.ratio = m->idx_ratio; qp.budget = m->idx_budget;
    qp.ik = k.ik; qp.ib = k.ib; qp.max_ctx = c.max_ctx; qp.nb_cap = s->nb_cap; qp.pos = s->pos;
    qp.scores = s->qsa_scores; qp.mask = s->qsa_mask; qp.mask_ld = s->mask_ld; qp.sparse = s->qsa_on; qp.batch = s->batch;
}

static int run_attn(pb_state* s, int il, const float* x_in, const float* norm_w, float* y, int64_t ldy, int accumulate) {
    pb_model* m = s->m; pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg; const int B = s->batch;
    const int64_t nq = (int64_t)c.n_head * 2 * c.hd, row = (int64_t)c.n_kv * c.hd;
    PbGemvQArgs a; memset(&a, 0, sizeof a);
    a.type = M(m, il, PB_R_ATTN_Q)->type; a.cols = c.d; a.nseg = 3;
    seg(a, 0, M(m, il, PB_R_ATTN_Q), 0); seg(a, 1, M(m, il, PB_R_ATTN_K), nq); seg(a, 2, M(m, il, PB_R_ATTN_V), nq + row);
    a.x = x_in; a.ldx = c.d; a.y = s->proj; a.ldy = s->ldproj; a.mode = norm_w ? PB_ACT_NORM : PB_ACT_PLAIN; a.norm_w = norm_w; a.eps = c.eps;
    const int ncol = s->win_t > 0 ? s->win_t : B;
    const bool prefill = s->win_t >= 16 && !s->win_ckpt;
    PB_TRY(gemv_cols(ctx, a, ncol, prefill));
    PbAttnParams p; attn_params(s, il, p);
    // QSA block-sparse attention (attn_core :1565-1599): two more projections of the same input give the raw index query
    // heads and the raw index key; after the KV append the indexer stores the key, pools the block the token completes,
    // and past the dense range writes the mask of positions this query attends to
    PbQsaParams qp; memset(&qp, 0, sizeof qp);
    if (m->qsa) {
        PbGemvQArgs ia; memset(&ia, 0, sizeof ia);
        ia.type = M(m, il, PB_R_IDX_Q)->type; ia.cols = c.d; ia.nseg = 2;
        seg(ia, 0, M(m, il, PB_R_IDX_Q), 0); seg(ia, 1, M(m, il, PB_R_IDX_K), (int64_t)m->idx_nh * m->idx_hd);
        ia.x = x_in; ia.ldx = c.d; ia.y = s->iproj; ia.ldy = s->ldi; ia.mode = a.mode; ia.norm_w = norm_w; ia.eps = c.eps;
        PB_TRY(gemv_cols(ctx, ia, ncol, false));
        qsa_params(s, il, qp);
        p.qsa_mask = s->qsa_mask; p.qsa_ld = s->mask_ld; p.qsa_on = s->qsa_on;
    }
    if (s->ext_mask) { p.qsa_mask = s->ext_mask; p.qsa_ld = s->ext_ld; p.qsa_on = s->ext_on; }
    if (s->win_t > 0 && !m->qsa) {
        // a prefill chunk or a verify window: all tokens are appended, the packed boundary moves once, then every token attends
        // to the positions <= its own in one launch (token j treats as packed what it would have found packed token by
        // token).  A verify window that is cut short afterwards gets its boundary back in pb_keep.
        p.window = 1; p.pos = s->wpos; p.batch = s->win_t;
        const bool mma = s->nsplit_packed > 0;
        // splits per token: four for a chunk of hundreds of tokens, more for a window of a few, so that the grid fills the GPU
        int ws = ctx->sm_count / (c.n_kv * s->win_t);
        ws = ws < PB_WIN_SPLITS ? PB_WIN_SPLITS : (ws > 64 ? 64 : ws);
        if ((size_t)ws * s->win_t > (size_t)PB_PREFILL_CHUNK * PB_WIN_SPLITS) ws = PB_WIN_SPLITS;
        p.nsplit = mma ? ws : 1; p.nsplit_packed = mma ? ws - 1 : 0;
        PB_TRY(pb_launch_kv_append(ctx, p));
        PB_TRY(pb_launch_kv_pack(ctx, p));
        PB_TRY(pb_launch_attn(ctx, p));
    } else if (s->win_t > 0) {
        // causal inside the window: token j is appended, then attends to positions <= its own
        // (models with an indexer take this form for prefill chunks too: every token makes its own selection)
        for (int j = 0; j < s->win_t; j++) {
            p.proj = s->proj + (size_t)j * s->ldproj; p.pos = s->wpos + j; p.att = s->att + (size_t)j * p.lda; p.batch = 1;
            PB_TRY(pb_launch_kv_append(ctx, p));
            if (m->qsa) { qp.iproj = s->iproj + (size_t)j * s->ldi; qp.pos = s->wpos + j; qp.batch = 1; PB_TRY(pb_launch_qsa_append(ctx, qp)); PB_TRY(pb_launch_qsa_select(ctx, qp)); }
            PB_TRY(pb_launch_attn(ctx, p));
        }
    } else {
        PB_TRY(pb_launch_kv_append(ctx, p));
        if (m->qsa) { PB_TRY(pb_launch_qsa_append(ctx, qp)); PB_TRY(pb_launch_qsa_select(ctx, qp)); }
        PB_TRY(pb_launch_attn(ctx, p));
    }
    PbGemvQArgs o; memset(&o, 0, sizeof o);
    o.type = M(m, il, PB_R_ATTN_O)->type; o.cols = c.n_head * c.hd; o.nseg = 1; seg(o, 0, M(m, il, PB_R_ATTN_O), 0);
    o.x = s->att; o.ldx = (int64_t)c.n_head * c.hd; o.y = y; o.ldy = ldy; o.mode = PB_ACT_PLAIN; o.accumulate = accumulate;
    return gemv_cols(ctx, o, ncol, prefill);
}

// MoE block on t tokens: x_in [t][d] (normalized when norm_w == null) -> y (stored or added)
static int run_moe(pb_state* s, int il, const float* x_in, const float* norm_w, int t, float* y, int64_t ldy, int accumulate) {
    pb_model* m = s->m; pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg;
    // sharded tokens: the block sees the rows of all ranks (tt tokens), this rank owns [tok0, tok0 + t)
    const bool sh = s->sharded && t == s->batch;
    const int tt = sh ? s->moe_t : t, tok0 = sh ? s->tok0 : 0;
    if (s->sharded && !sh) PB_FAIL(ctx, PB_UNSUPPORTED, "a sharded state runs its MoE blocks on whole steps (%d tokens), not on %d", s->batch, t);
    PbRouterParams r; memset(&r, 0, sizeof r);
    r.cols = c.d; r.norm_w = norm_w; r.eps = c.eps;
    r.router = reinterpret_cast<const float*>(M(m, il, PB_R_ROUTER)->data); r.sh_gate_inp = V(m, il, PB_R_SH_GATE_INP); r.n_exp = c.n_exp;
    r.xq_out = s->xq;
    PbRouteParams q; memset(&q, 0, sizeof q);
    q.t = tt; q.n_exp = c.n_exp; q.top_k = c.top_k; q.e_lo = m->e_lo; q.e_hi = m->e_hi;
    q.sel_e = s->sel_e; q.sel_w = s->sel_w; q.n_used = s->n_used; q.used_e = s->used_e; q.used_off = s->used_off;
    q.ent_tok = s->ent_tok; q.ent_slot = s->ent_slot; q.ent_w = s->ent_w;
    const float* logits; int64_t ldl;
    if (sh) {
        // router logits of the local tokens, written next to a copy of their residual rows; one all-gather
        // moves both; then every rank splits and routes all tokens
        r.phase = 1; r.x = x_in; r.ldx = c.d; r.t = t; r.logits = s->xs + c.d; r.ldl = s->ldg; r.xcopy = s->xs;
        if (s->p2p) { r.exch = s->exch_dev; r.exch_idx = 2 * il; r.peer_off = (int64_t)tok0 * s->ldg; }   // the router stores into every rank's gathered buffer and hand-shakes
        PB_TRY(pb_launch_router(ctx, r, q, s->ticket));
        if (s->p2p) r.exch = nullptr;
        else { PB_TRY(pb_ep_allgather(ctx, s->xs, s->xg, (size_t)t * s->ldg)); ctx->pdl_chain = false; }
        r.phase = 2; r.x = s->xg; r.ldx = s->ldg; r.t = tt; r.logits = s->xg + c.d; r.xcopy = nullptr;
        logits = s->xg + c.d; ldl = s->ldg;
    } else {
        r.phase = 0; r.x = x_in; r.ldx = c.d; r.t = tt; r.logits = s->rlogits; r.ldl = c.n_exp + 1;
        logits = s->rlogits; ldl = c.n_exp + 1;
    }
    q.logits = logits; q.ldl = ldl;
    if (m->ep_world > 1 && !(sh && s->p2p)) { r.zero = s->part; r.zero_n = (int64_t)tt * c.top_k * c.d; }   // rows of other ranks' experts stay zero (summed exchanges)
    PB_TRY(pb_launch_router(ctx, r, q, s->ticket));
    PbExpertParams e; memset(&e, 0, sizeof e);
    e.n_used = s->n_used; e.used_e = s->used_e; e.used_off = s->used_off; e.ent_tok = s->ent_tok; e.ent_slot = s->ent_slot; e.ent_w = s->ent_w;
    e.xq = s->xq; e.h = s->h; e.h_sh = s->h_sh; e.part = s->part; e.part_sh = s->part_sh;
    e.has_shared = 1; e.t = tt; e.top_k = c.top_k; e.n_exp = c.n_exp;
    e.sh_tok0 = tok0; e.sh_ntok = t;   // the shared expert runs where the token lives
    pb_qmat* g = M(m, il, PB_R_EXP_GATE);
    e.e_base = g->rows == (int64_t)c.ff_exp * c.n_exp ? 0 : m->e_lo;
    pb_qmat *up = M(m, il, PB_R_EXP_UP), *shg = M(m, il, PB_R_SH_GATE), *shu = M(m, il, PB_R_SH_UP);
    e.w_a = g->data; e.w_b = up->data; e.sh_a = shg->data; e.sh_b = shu->data;
    int gu_type = g->type;
    if (g->rdata && up->rdata && shg->rdata && shu->rdata) { e.w_a = g->rdata; e.w_b = up->rdata; e.sh_a = shg->rdata; e.sh_b = shu->rdata; gu_type = PB_T_IQ3S_N4; }   // re-coded copies
    e.rows_e = c.ff_exp; e.rows_sh = c.ff_sh;
    PB_TRY(pb_launch_expert_gu(ctx, e, gu_type, c.d));
    pb_qmat* dn = M(m, il, PB_R_EXP_DOWN);
    e.e_base = dn->rows == (int64_t)c.d * c.n_exp ? 0 : m->e_lo;
    pb_qmat* shd = M(m, il, PB_R_SH_DOWN);
    e.w_a = dn->data; e.w_b = nullptr; e.sh_a = shd->data; e.sh_b = nullptr;
    int dn_type = dn->type;
    if (dn->rdata && shd->rdata) { e.w_a = dn->rdata; e.sh_a = shd->rdata; dn_type = PB_T_IQ3S_N4; }
    e.rows_e = c.d; e.rows_sh = c.d;
    if (tt > s->moe_cap) PB_FAIL(ctx, PB_ERR_ARG, "MoE block on %d tokens, buffers hold %d", tt, s->moe_cap);
    e.hq = tt > 1 && c.ff_exp == c.ff_sh ? s->hq : nullptr;   // several tokens: levels of the hidden vectors made once
    PbCombineParams k; memset(&k, 0, sizeof k);
    k.part = s->part; k.part_sh = s->part_sh + (size_t)tok0 * c.d; k.logits = logits + (size_t)tok0 * ldl; k.ldl = ldl; k.t = t; k.d = c.d; k.top_k = c.top_k; k.n_exp = c.n_exp;
    if (sh) { k.logits = s->xs + c.d; k.ldl = s->ldg; }   // this rank's own copy of its tokens' logits: the gathered buffer may already be receiving the next block's rows
    if (sh && s->p2p) e.part_tok = s->part_tok;            // finished rows go straight into the memory of the token's owner
    k.y = y; k.ldy = ldy; k.accumulate = accumulate;
    // few tokens on one GPU: the down kernel's last CTA also combines (one launch less per layer)
    if (m->ep_world == 1 && (int64_t)t * c.d <= 8192) return pb_launch_expert_down(ctx, e, dn_type, c.ff_exp, &k, s->ticket + 1);
    PB_TRY(pb_launch_expert_down(ctx, e, dn_type, c.ff_exp));
    // expert parallelism: every (token, slot) row was produced on exactly one rank and is zero elsewhere,
    // so the sum is an exact gather and the combine below sees the same bits for every GPU count
    if (sh && s->p2p) { k.exch = s->exch_dev; k.exch_idx = 2 * il + 1; k.part = s->part_rs; }   // the combine kernel announces and waits
    else if (sh) { PB_TRY(pb_ep_reduce_scatter(ctx, s->part, s->part_rs, (size_t)t * c.top_k * c.d)); k.part = s->part_rs; ctx->pdl_chain = false; }
    else if (m->ep_world > 1) { PB_TRY(pb_ep_allreduce(ctx, s->part, (size_t)t * c.top_k * c.d)); ctx->pdl_chain = false; }
    return pb_launch_moe_combine(ctx, k);
}


// ------------------------------------------------------------------------------------ fused step (pb_step.cu)

static int qsa_pool_all(pb_state* s, int ai, int64_t n);
static bool recoded(pb_qmat* q) { return q && q->type == PB_T_IQ3_S && q->rdata != nullptr; }

// Decides whether the state can run its steps through the fused kernel and, if so, builds the operation list.
// Conditions: one sequence, one GPU, pre-norm residual, every quantized matrix with a re-coded copy (IQ3_S), widths
// the kernel's lane mappings cover.  PYRE_B200_FUSED=0 keeps the per-operation kernels.
static int fused_build(pb_state* s) {
    pb_model* m = s->m; pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg;
    s->fused = 0;
    // PYRE_B200_FUSED=1 (read when a state takes its first step): one cooperative kernel per run of layers.  Off by default: since
    // the per-operation kernels fetch their model data ahead of the dependency wait, their chain of dependent launches is the
    // shorter step (3.29 against 3.46 ms on the 48-layer model); both give the same bits.
    const bool on = getenv("PYRE_B200_FUSED") && atoi(getenv("PYRE_B200_FUSED")) == 1;
    if (!on || s->batch != 1 || s->sharded || m->ep_world != 1 || c.hc != 0 || m->n_ple > 0) return PB_OK;
    const int d = c.d, ff = c.ff_exp, w_lin = c.lin_nv * c.lin_dv, w_att = c.n_head * c.hd;
    auto pow2 = [](int v) { return v > 0 && (v & (v - 1)) == 0; };
    if (d % 256 || d > 2048 || !pow2(d / 64) || ff % 512 || !pow2(ff / 64) || ff / 64 > 32 || c.ff_sh != ff) return PB_OK;
    if (c.top_k + 1 > 16 || c.n_exp > 1024 || d % 16 || d / 16 > ctx->sm_count) return PB_OK;
    pb_qmat* head = M(m, -1, PB_R_OUTPUT) ? M(m, -1, PB_R_OUTPUT) : M(m, -1, PB_R_TOKEN_EMBD);
    if (!recoded(head)) return PB_OK;
    int maxcols = d;
    for (int il = 0; il < c.n_layers; il++) {
        if (m->kind[il]) {
            if (!recoded(M(m, il, PB_R_ATTN_Q)) || !recoded(M(m, il, PB_R_ATTN_K)) || !recoded(M(m, il, PB_R_ATTN_V)) || !recoded(M(m, il, PB_R_ATTN_O))) return PB_OK;
            if (m->qsa && (!recoded(M(m, il, PB_R_IDX_Q)) || !recoded(M(m, il, PB_R_IDX_K)))) return PB_OK;
            if (w_att % 256 || w_att > 4096 || !pow2(w_att / 64)) return PB_OK;
            maxcols = w_att > maxcols ? w_att : maxcols;
        } else {
            if (!recoded(M(m, il, PB_R_LIN_QKV)) || !recoded(M(m, il, PB_R_LIN_Z)) || !recoded(M(m, il, PB_R_LIN_BETA)) || !recoded(M(m, il, PB_R_LIN_ALPHA)) || !recoded(M(m, il, PB_R_LIN_OUT))) return PB_OK;
            if (w_lin % 256 || w_lin > 4096 || !pow2(w_lin / 64) || c.lin_dk != 128 || c.lin_dv != 128 || c.conv_k > 8 || c.lin_nv * (c.lin_dv / 32) > ctx->sm_count) return PB_OK;
            maxcols = w_lin > maxcols ? w_lin : maxcols;
        }
        const int roles[6] = {PB_R_EXP_GATE, PB_R_EXP_UP, PB_R_EXP_DOWN, PB_R_SH_GATE, PB_R_SH_UP, PB_R_SH_DOWN};
        for (int r : roles) if (!recoded(M(m, il, r))) return PB_OK;
        if (M(m, il, PB_R_EXP_GATE)->rows != (int64_t)c.n_exp * ff) return PB_OK;   // all experts resident (no expert parallelism)
    }
    // ---- shared-memory layout
    PsLayout L;
    auto up128 = [](size_t v) { return (uint32_t)((v + 127) & ~(size_t)127); };
    L.xf_off = 8192;                                                            // after the misc area and the warps' operation copies
    const size_t xf_bytes = (size_t)maxcols * 4 > 12288 ? (size_t)maxcols * 4 : 12288;   // also the DeltaNet unit's scratch and the routing keys (10.5 KB)
    L.nw_off = up128(L.xf_off + xf_bytes);
    L.xq_off = up128(L.nw_off + (size_t)d * 4);
    const size_t xq_a = (size_t)pb_xq_words(maxcols) * 4, xq_b = (size_t)(c.top_k + 1) * pb_xq_words(ff) * 4;
    L.stage_off = up128(L.xq_off + (xq_a > xq_b ? xq_a : xq_b));
    const size_t avail = (size_t)ctx->max_smem_optin > L.stage_off ? (size_t)ctx->max_smem_optin - L.stage_off : 0;
    size_t stage = avail / PS_STAGES;
    if (stage > 34944) stage = 34944;
    stage &= ~(size_t)127;
    L.stage_bytes = (uint32_t)stage; L.total = L.stage_off + PS_STAGES * L.stage_bytes;
    auto n4_row = [](int cols) { return cols / 256 * 136; };
    auto rows_per_chunk = [&](int cols) {
        const int lpr = cols / 64 < 32 ? cols / 64 : 32, step_rows = PB_CONSUMERS * (32 / lpr);
        int rpc = (int)(stage / (size_t)n4_row(cols)) / step_rows * step_rows;
        if (rpc > 2 * step_rows) rpc = 2 * step_rows;
        return rpc;
    };
    const int rpw_d = 32 / (d / 64 < 32 ? d / 64 : 32), rg = 8 * rpw_d;
    if (rows_per_chunk(d) <= 0 || rows_per_chunk(maxcols) <= 0 || ff % rg || (size_t)2 * rg * n4_row(d) > stage || (size_t)d * 4 > stage || (size_t)16 * n4_row(ff) > stage) return PB_OK;
    // ---- operations
    std::vector<PbStepOp> ops;
    s->fsegs.clear();
    int seg_begin = 0;
    auto push = [&](PbStepOp& op, int kind) {
        op.kind = kind;
        op.flags = (int)ops.size() == seg_begin ? 0 : PS_F_BARRIER;
        op.stamps = pb_stamp_slot(ctx, 100 + kind);   // traced as operation kinds 101..105
        ops.push_back(op);
    };
    auto gemv = [&](int cols, int mode, const float* x, const float* norm_w, const float* z, float* y, int accumulate, std::initializer_list<std::pair<pb_qmat*, int>> segs) {
        PbStepOp op; memset(&op, 0, sizeof op);
        PsGemvOp& g = op.g;
        g.cols = cols; g.row_bytes = n4_row(cols); g.rows_per_chunk = rows_per_chunk(cols); g.mode = mode; g.accumulate = accumulate; g.head_dim = c.lin_dv;
        g.x = x; g.norm_w = norm_w; g.z = z; g.y = y; g.eps = c.eps;
        int nchunks = 0;
        for (auto& sg : segs) {
            PbGemvQSeg& q = g.seg[g.nseg++];
            q.w = sg.first->rdata; q.rows = (int)sg.first->rows; q.yoff = sg.second; q.chunk0 = nchunks;
            nchunks += (int)((sg.first->rows + g.rows_per_chunk - 1) / g.rows_per_chunk);
        }
        g.nchunks = nchunks;
        push(op, PS_GEMV);
    };
    const int ch = 2 * c.lin_nk * c.lin_dk + w_lin;
    for (int il = 0; il < c.n_layers; il++) {
        if (m->kind[il]) {
            const int nq = c.n_head * 2 * c.hd, row = c.n_kv * c.hd;
            gemv(d, PB_ACT_NORM, s->x, V(m, il, PB_R_ATTN_NORM), nullptr, s->proj, 0, {{M(m, il, PB_R_ATTN_Q), 0}, {M(m, il, PB_R_ATTN_K), nq}, {M(m, il, PB_R_ATTN_V), nq + row}});
            if (m->qsa)   // the indexer's raw query heads and raw key, from the same normalized input
                gemv(d, PB_ACT_NORM, s->x, V(m, il, PB_R_ATTN_NORM), nullptr, s->iproj, 0, {{M(m, il, PB_R_IDX_Q), 0}, {M(m, il, PB_R_IDX_K), m->idx_nh * m->idx_hd}});
            s->fsegs.push_back({seg_begin, (int)ops.size(), il, 0});
            seg_begin = (int)ops.size();
            gemv(w_att, PB_ACT_PLAIN, s->att, nullptr, nullptr, s->x, 1, {{M(m, il, PB_R_ATTN_O), 0}});
        } else {
            const int li = m->idx[il];
            gemv(d, PB_ACT_NORM, s->x, V(m, il, PB_R_ATTN_NORM), nullptr, s->proj, 0,
                 {{M(m, il, PB_R_LIN_QKV), 0}, {M(m, il, PB_R_LIN_Z), ch}, {M(m, il, PB_R_LIN_BETA), ch + w_lin}, {M(m, il, PB_R_LIN_ALPHA), ch + w_lin + c.lin_nv}});
            PbStepOp op; memset(&op, 0, sizeof op);
            PbDeltaParams& dp = op.d;
            dp.proj = s->proj; dp.ldp = s->ldproj; dp.conv_w = V(m, il, PB_R_LIN_CONV); dp.a = V(m, il, PB_R_LIN_A); dp.dt = V(m, il, PB_R_LIN_DT);
            dp.conv = s->conv[li]; dp.ssm = s->ssm[li]; dp.pos = s->pos; dp.out = s->olin; dp.ldo = w_lin;
            dp.nk = c.lin_nk; dp.nv = c.lin_nv; dp.dk = c.lin_dk; dp.dv = c.lin_dv; dp.conv_k = c.conv_k; dp.batch = 1;
            push(op, PS_DELTA);
            gemv(w_lin, PB_ACT_GNORM, s->olin, V(m, il, PB_R_LIN_NORM), s->proj + ch, s->x, 1, {{M(m, il, PB_R_LIN_OUT), 0}});
        }
        {
            PbStepOp op; memset(&op, 0, sizeof op);
            PsRouterOp& r = op.r;
            r.x = s->x; r.norm_w = V(m, il, PB_R_FFN_NORM); r.router = reinterpret_cast<const float*>(M(m, il, PB_R_ROUTER)->data); r.sh_gate_inp = V(m, il, PB_R_SH_GATE_INP);
            r.logits = s->rlogits; r.n_exp = c.n_exp; r.cols = d; r.eps = c.eps;
            r.rows_per_chunk = (int)(stage / ((size_t)d * 4)) < PB_CONSUMERS ? (int)(stage / ((size_t)d * 4)) : PB_CONSUMERS;
            r.nchunks = (c.n_exp + r.rows_per_chunk - 1) / r.rows_per_chunk + 1;
            push(op, PS_ROUTER);
        }
        {
            PbStepOp op; memset(&op, 0, sizeof op);
            PsMoeOp& e = op.m;
            e.gate = M(m, il, PB_R_EXP_GATE)->rdata; e.up = M(m, il, PB_R_EXP_UP)->rdata; e.down = M(m, il, PB_R_EXP_DOWN)->rdata;
            e.sh_gate = M(m, il, PB_R_SH_GATE)->rdata; e.sh_up = M(m, il, PB_R_SH_UP)->rdata; e.sh_down = M(m, il, PB_R_SH_DOWN)->rdata;
            e.logits = s->rlogits; e.h = s->fh; e.y = s->x; e.n_exp = c.n_exp; e.top_k = c.top_k; e.ff = ff; e.d = d; e.e_base = 0;
            e.row_bytes_gu = n4_row(d); e.row_bytes_dn = n4_row(ff); e.rg = rg;
            const int spc = (int)(stage / ((size_t)16 * n4_row(ff)));
            e.spc = spc < c.top_k + 1 ? spc : c.top_k + 1;
            PbStepOp op2 = op;
            push(op, PS_GU);
            push(op2, PS_DOWN);
        }
    }
    gemv(d, PB_ACT_NORM, s->x, V(m, -1, PB_R_OUT_NORM), nullptr, s->logits, 0, {{head, 0}});
    s->fsegs.push_back({seg_begin, (int)ops.size(), -1, 0});
    for (pb_state::FSeg& sg : s->fsegs) for (int i = sg.begin; i < sg.end; i++) sg.nbar += (ops[i].flags & PS_F_BARRIER) ? 1 : 0;
    if (ctx->stamps) {   // tracing on: every CTA stamps every operation
        const size_t per = (size_t)ctx->sm_count * 4 + 32;   // per-CTA stamps, then 32 fine-grained stamps of CTA 0
        PB_TRY(dalloc(s, &s->ftrace, ops.size() * per));
        for (size_t i = 0; i < ops.size(); i++) ops[i].trace = s->ftrace + i * per;
        s->ftrace_ops = (int)ops.size();
    }
    PB_CUDA(ctx, cudaMemcpyAsync(s->fops, ops.data(), ops.size() * sizeof(PbStepOp), cudaMemcpyHostToDevice, ctx->stream));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // `ops` is a local
    s->flay = L;
    s->fused = 1;
    return PB_OK;
}

// one decode step of a batch-1 state through the fused kernel: embedding, then for every run of operations between
// attention cores one launch of pb_step_kernel, the attention cores with their own kernels, argmax, position advance
static int run_step_fused(pb_state* s) {
    pb_model* m = s->m; pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg;
    struct Scope { pb_ctx* c; Scope(pb_ctx* x) : c(x) { c->pdl_scope++; c->pdl_chain = false; } ~Scope() { c->pdl_scope--; c->pdl_chain = false; } } scope(ctx);
    pb_qmat* embd = M(m, -1, PB_R_TOKEN_EMBD);
    PB_TRY(pb_launch_embed(ctx, embd->type, embd->data, embd->rows, c.d, s->ids, 1, s->x, c.d));
    for (const pb_state::FSeg& sg : s->fsegs) {
        PsParams P; memset(&P, 0, sizeof P);
        P.ops = s->fops; P.op_begin = sg.begin; P.op_end = sg.end; P.nbar = sg.nbar; P.sync = ctx->grid_sync; P.pos = s->pos; P.lay = s->flay; P.status = ctx->dev_status;
        PB_TRY(pb_launch_step(ctx, P));
        if (sg.attn_layer >= 0) {
            PbAttnParams p; attn_params(s, sg.attn_layer, p);
            PB_TRY(pb_launch_kv_append(ctx, p));
            if (m->qsa) {
                PbQsaParams qp; qsa_params(s, sg.attn_layer, qp);
                p.qsa_mask = s->qsa_mask; p.qsa_ld = s->mask_ld; p.qsa_on = s->qsa_on;
                PB_TRY(pb_launch_qsa_append(ctx, qp)); PB_TRY(pb_launch_qsa_select(ctx, qp));
            }
            PB_TRY(pb_launch_attn(ctx, p));
        }
    }
    PB_TRY(pb_launch_argmax(ctx, s->logits, c.vocab, c.vocab, 1, s->amax));
    return pb_launch_advance(ctx, s->pos, 1, s->amax, s->next, s->ids, s->trace, s->trace_len, s->trace_cap);
}

// ---- per-layer n-gram embeddings (ple_rows :1390-1407, ple :1409-1434) ----
// y[t][ldy] = W . x[t][ldx] for a matrix of any type, 16 columns a launch
static int gemv_any(pb_ctx* ctx, pb_qmat* q, const float* x, int64_t ldx, int t, float* y, int64_t ldy) {
    for (int t0 = 0; t0 < t; t0 += 16) {
        PbGemvArgs g; memset(&g, 0, sizeof g);
        g.w = q->data; g.wr = q->rdata; g.type = q->type; g.rows = q->rows; g.cols = (int)q->cols;
        g.x = x + (int64_t)t0 * ldx; g.ldx = ldx; g.t = t - t0 < 16 ? t - t0 : 16; g.y = y + (int64_t)t0 * ldy; g.ldy = ldy;
        PB_TRY(pb_launch_gemv(ctx, g));
    }
    return PB_OK;
}
// the table rows of the t rows in flight (ids in s->ids; positions s->wpos inside a window, else one sequence per row at s->pos)
static int ple_gather(pb_state* s, int t) {
    pb_model* m = s->m; pb_ctx* ctx = m->ctx;
    if (m->n_ple == 0) return PB_OK;
    const int window = s->win_t > 0;
    PB_TRY(pb_launch_ple_rows(ctx, m->ple, s->ids, window ? s->wpos : s->pos, t, window, s->tok_hist, m->cfg.max_ctx, s->ple_base, s->ple_rows));
    pb_qmat* tab = M(m, -1, PB_R_PLE_TAB);
    PB_TRY(pb_launch_embed(ctx, tab->type, tab->data, tab->rows, m->ple_dim, s->ple_rows, t * m->ple.nh, s->ple_emb, m->ple_dim));
    ctx->pdl_chain = false;
    return PB_OK;
}
// layer il's injection into the residual rows x [t][w]
static int run_ple(pb_state* s, int il, float* x, int t) {
    pb_model* m = s->m; pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg;
    const int pi = m->ple_idx[il];
    if (pi < 0) return PB_OK;
    const int streams = c.hc > 0 ? c.hc : 1, w = streams * c.d, window = s->win_t > 0;
    const int64_t ein = (int64_t)m->ple.nh * m->ple_dim;
    const int64_t* posv = window ? s->wpos : s->pos;
    PB_TRY(gemv_any(ctx, M(m, il, PB_R_PLE_KEY), s->ple_emb, ein, t, s->ple_key, w));
    PB_TRY(gemv_any(ctx, M(m, il, PB_R_PLE_VALUE), s->ple_emb, ein, t, s->ple_val, c.d));
    PB_TRY(pb_launch_ple_gate(ctx, s->ple_key, w, s->ple_val, c.d, x, w, V(m, il, PB_R_PLE_NORM_KEY), V(m, il, PB_R_PLE_NORM_QUERY), V(m, il, PB_R_PLE_NORM_CONV),
                              s->ple_gated, s->ple_ring[(size_t)pi], s->ple_R, posv, t, window, c.d, streams, c.eps));
    return pb_launch_ple_conv(ctx, s->ple_gated, s->ple_ring[(size_t)pi], s->ple_R, V(m, il, PB_R_PLE_CONV), m->ple_conv_k, m->ple.ngram, posv, t, window, s->ple_base, x, w, w);
}

// ---- hyper-connection residual (hc >= 1): forward_inner :2087-2157 with hc_mix / hc_combine around every block ----
static void hc_params(pb_state* s, int il, int r_norm, int r_down, int r_up, int r_inj, PbHcParams& h) {
    pb_model* m = s->m; const pb_cfg& c = m->cfg;
    memset(&h, 0, sizeof h);
    h.norm = V(m, il, r_norm); h.down = reinterpret_cast<const float*>(M(m, il, r_down)->data); h.up = reinterpret_cast<const float*>(M(m, il, r_up)->data);
    h.inject = r_inj >= 0 ? reinterpret_cast<const float*>(M(m, il, r_inj)->data) : nullptr;
    h.d = c.d; h.hc = c.hc; h.lr = c.hc_lr; h.eps = c.eps; h.xn = s->hxn; h.gate = s->hgate; h.lo = s->hlo; h.inj = s->hinj;
}
// all layers on t rows of the residual s->x [t][hc*d]; then the head's mix of rows [h0, h0 + hn) into s->hmix [hn][d]
static int run_layers_hc(pb_state* s, int t, int h0, int hn) {
    pb_model* m = s->m; pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg;
    pb_qmat* embd = M(m, -1, PB_R_TOKEN_EMBD);
    PB_TRY(pb_launch_embed(ctx, embd->type, embd->data, embd->rows, c.d, s->ids, t, s->yout, c.d));
    PB_TRY(pb_launch_hc_spread(ctx, s->yout, s->x, t, c.d, c.hc));
    PB_TRY(ple_gather(s, t));
    PbHcParams h;
    for (int il = 0; il < c.n_layers; il++) {
        PB_TRY(run_ple(s, il, s->x, t));
        hc_params(s, il, PB_R_HCA_NORM, PB_R_HCA_DOWN, PB_R_HCA_UP, PB_R_HCA_INJECT, h);
        PB_TRY(pb_launch_hc_mix(ctx, h, s->x, t, s->hmix));
        if (m->kind[il]) PB_TRY(run_attn(s, il, s->hmix, nullptr, s->yout, c.d, 0));
        else PB_TRY(run_lin(s, il, s->hmix, nullptr, s->yout, c.d, 0));
        PB_TRY(pb_launch_hc_combine(ctx, h, s->x, s->yout, t));
        hc_params(s, il, PB_R_HCF_NORM, PB_R_HCF_DOWN, PB_R_HCF_UP, PB_R_HCF_INJECT, h);
        PB_TRY(pb_launch_hc_mix(ctx, h, s->x, t, s->hmix));
        PB_TRY(run_moe(s, il, s->hmix, nullptr, t, s->yout, c.d, 0));
        PB_TRY(pb_launch_hc_combine(ctx, h, s->x, s->yout, t));
    }
    hc_params(s, -1, PB_R_OUT_HC_NORM, PB_R_OUT_HC_DOWN, PB_R_OUT_HC_UP, -1, h);   // :2152
    return pb_launch_hc_mix(ctx, h, s->x + (size_t)h0 * c.hc * c.d, hn, s->hmix);
}

// one decode step for every sequence of the batch, ids already in s->ids
static int run_step(pb_state* s) {
    pb_model* m = s->m; pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg; const int B = s->batch;
    if (s->fused < 0) PB_TRY(fused_build(s));
    if (s->fused == 1) return run_step_fused(s);
    struct Scope { pb_ctx* c; Scope(pb_ctx* x) : c(x) { c->pdl_scope++; c->pdl_chain = false; } ~Scope() { c->pdl_scope--; c->pdl_chain = false; } } scope(ctx);
    pb_qmat* embd = M(m, -1, PB_R_TOKEN_EMBD);
    if (c.hc > 0) { PB_TRY(run_layers_hc(s, B, 0, B)); if (s->mtp) PB_TRY(pb_launch_mtp_keep(ctx, s->x, (int64_t)c.hc * c.d, s->pos, 1, s->mtp->ring, s->mtp->ring_cap, c.hc * c.d)); }
    else {
        PB_TRY(pb_launch_embed(ctx, embd->type, embd->data, embd->rows, c.d, s->ids, B, s->x, c.d));
        PB_TRY(ple_gather(s, B));
        for (int il = 0; il < c.n_layers; il++) {
            PB_TRY(run_ple(s, il, s->x, B));
            if (m->kind[il]) PB_TRY(run_attn(s, il, s->x, V(m, il, PB_R_ATTN_NORM), s->x, c.d, 1));
            else PB_TRY(run_lin(s, il, s->x, V(m, il, PB_R_ATTN_NORM), s->x, c.d, 1));
            PB_TRY(run_moe(s, il, s->x, V(m, il, PB_R_FFN_NORM), B, s->x, c.d, 1));
        }
    }
    pb_qmat* out = M(m, -1, PB_R_OUTPUT) ? M(m, -1, PB_R_OUTPUT) : embd;
    PbGemvQArgs a; memset(&a, 0, sizeof a);
    a.type = out->type; a.cols = c.d; a.nseg = 1; seg(a, 0, out, 0);
    a.x = s->x; a.ldx = c.d; a.y = s->logits; a.ldy = c.vocab; a.mode = PB_ACT_NORM; a.norm_w = V(m, -1, PB_R_OUT_NORM); a.eps = c.eps;
    if (c.hc > 0) { a.x = s->hmix; a.mode = PB_ACT_PLAIN; a.norm_w = nullptr; }   // the head's mix already normalized the streams
    PB_TRY(gemv_cols(ctx, a, B));
    PB_TRY(pb_launch_argmax(ctx, s->logits, c.vocab, c.vocab, B, s->amax));
    return pb_launch_advance(ctx, s->pos, B, s->amax, s->next, s->ids, s->trace, s->trace_len, s->trace_cap, s->p2p ? s->ep_seq : nullptr, 2ull * c.n_layers);
}

// A window of t consecutive tokens of the one sequence of a batch-1 state (ids already in s->ids[0..t)):
// every weight matrix is streamed once for all t tokens (tensor-core GEMM from 3 tokens on); only the
// recurrences (DeltaNet state, KV append + attention) run token by token.  Logits of all positions go to
// s->logits [t][vocab] when all_logits, else only the last position's to row 0.  Model::forward_multi,
// src/model/qwen4exp_gguf.rs:2365-2480.
static int run_window(pb_state* s, int t, bool ckpt, bool all_logits) {
    pb_model* m = s->m; pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg;
    struct Scope { pb_ctx* c; pb_state* s; Scope(pb_ctx* x, pb_state* y, int t, bool k) : c(x), s(y) { c->pdl_scope++; c->pdl_chain = false; s->win_t = t; s->win_ckpt = k; }
                   ~Scope() { c->pdl_scope--; c->pdl_chain = false; s->win_t = 0; s->win_ckpt = false; } } scope(ctx, s, t, ckpt);
    PB_TRY(pb_launch_window_pos(ctx, s->pos, s->wpos, t, 0));
    pb_qmat* embd = M(m, -1, PB_R_TOKEN_EMBD);
    if (c.hc > 0) { PB_TRY(run_layers_hc(s, t, all_logits ? 0 : t - 1, all_logits ? t : 1)); if (s->mtp) PB_TRY(pb_launch_mtp_keep(ctx, s->x, (int64_t)c.hc * c.d, s->wpos, t, s->mtp->ring, s->mtp->ring_cap, c.hc * c.d)); }
    else {
        PB_TRY(pb_launch_embed(ctx, embd->type, embd->data, embd->rows, c.d, s->ids, t, s->x, c.d));
        PB_TRY(ple_gather(s, t));
        for (int il = 0; il < c.n_layers; il++) {
            PB_TRY(run_ple(s, il, s->x, t));
            if (m->kind[il]) PB_TRY(run_attn(s, il, s->x, V(m, il, PB_R_ATTN_NORM), s->x, c.d, 1));
            else PB_TRY(run_lin(s, il, s->x, V(m, il, PB_R_ATTN_NORM), s->x, c.d, 1));
            PB_TRY(run_moe(s, il, s->x, V(m, il, PB_R_FFN_NORM), t, s->x, c.d, 1));
        }
    }
    pb_qmat* out = M(m, -1, PB_R_OUTPUT) ? M(m, -1, PB_R_OUTPUT) : embd;
    PbGemvQArgs a; memset(&a, 0, sizeof a);
    a.type = out->type; a.cols = c.d; a.nseg = 1; seg(a, 0, out, 0);
    a.x = all_logits ? s->x : s->x + (size_t)(t - 1) * c.d; a.ldx = c.d; a.y = s->logits; a.ldy = c.vocab; a.mode = PB_ACT_NORM; a.norm_w = V(m, -1, PB_R_OUT_NORM); a.eps = c.eps;
    if (c.hc > 0) { a.x = s->hmix; a.mode = PB_ACT_PLAIN; a.norm_w = nullptr; }   // rows [0, hn) of the head's mix
    PB_TRY(gemv_cols(ctx, a, all_logits ? t : 1));
    return pb_launch_window_pos(ctx, s->pos, s->wpos, t, 1);   // position += t
}

// run_window as a CUDA graph per (t, ckpt, all_logits): eager the first time (kernel attributes), captured the
// second, replayed afterwards -- a window is ~1500 launches, whose host cost would otherwise dominate.
static int window_once(pb_state* s, int t, bool ckpt, bool all_logits) {
    pb_ctx* ctx = s->m->ctx;
    // graphs: windows of up to 8 tokens per (t, ckpt, all_logits), and the full prefill chunk; other lengths (the ragged
    // ends of a prompt) run eagerly
    const int key = t <= PB_MAX_WINDOW ? t * 4 + (ckpt ? 2 : 0) + (all_logits ? 1 : 0) : (t == PB_PREFILL_CHUNK && !ckpt && !all_logits ? PB_WIN_KEYS - 1 : -1);
    if (key < 0) {
        PB_TRY(run_window(s, t, ckpt, all_logits));
    } else if (s->win_graph[key]) {
        PB_CUDA(ctx, cudaGraphLaunch(s->win_graph[key], ctx->stream));
    } else if (s->win_runs[key] == 0) {
        PB_TRY(run_window(s, t, ckpt, all_logits));
        s->win_runs[key] = 1;
    } else {
        cudaGraph_t g = nullptr;
        PB_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        const uint64_t k0 = ctx->kernels_launched;
        const int rc = run_window(s, t, ckpt, all_logits);
        ctx->kernels_launched = k0;
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
        if (rc != PB_OK) { if (g) cudaGraphDestroy(g); return rc; }
        if (e != cudaSuccess) PB_FAIL(ctx, PB_ERR_CUDA, "window graph capture failed: %s", cudaGetErrorString(e));
        e = cudaGraphInstantiate(&s->win_graph[key], g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) { s->win_graph[key] = nullptr; PB_FAIL(ctx, PB_ERR_CUDA, "window graph instantiate failed: %s", cudaGetErrorString(e)); }
        PB_CUDA(ctx, cudaGraphLaunch(s->win_graph[key], ctx->stream));
    }
    s->pos_host += t;
    return PB_OK;
}

// Replays the step graph (captured on first use after one eager warm-up step would be wasteful:
// the first call runs eagerly and also serves as the configuration pass for kernel attributes).
static int step_once(pb_state* s) {
    pb_ctx* ctx = s->m->ctx;
    if (s->pos_host + 1 > s->m->cfg.max_ctx) PB_FAIL(ctx, PB_ERR_STATE, "context is full (%d positions)", s->m->cfg.max_ctx);
    if (s->graph) {
        PB_CUDA(ctx, cudaGraphLaunch(s->graph, ctx->stream));
        ctx->kernels_launched += s->kernels_per_step;
    } else if (s->steps == 0) {
        const uint64_t k0 = ctx->kernels_launched;
        PB_TRY(run_step(s));
        s->kernels_per_step = ctx->kernels_launched - k0;
    } else {
        cudaGraph_t g = nullptr;
        PB_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        const uint64_t k0 = ctx->kernels_launched;
        const int rc = run_step(s);
        ctx->kernels_launched = k0;
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
        if (rc != PB_OK) { if (g) cudaGraphDestroy(g); return rc; }
        if (e != cudaSuccess) PB_FAIL(ctx, PB_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        e = cudaGraphInstantiate(&s->graph, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) { s->graph = nullptr; PB_FAIL(ctx, PB_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e)); }
        PB_CUDA(ctx, cudaGraphLaunch(s->graph, ctx->stream));
        ctx->kernels_launched += s->kernels_per_step;
    }
    s->steps++; s->pos_host++;
    return PB_OK;
}

// Logits leave through a pinned buffer of the state: a device -> pageable-host copy is staged by the driver in small pieces
// (about 0.1 ms for one 608 KB row), a copy into pinned memory runs at link speed and the host copies it on.
// A destination in page-locked host memory (pb_host_alloc, or the caller's own registered buffer) takes the copy directly.
static bool host_pinned(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeHost;
}
static int logits_stage(pb_state* s, size_t n, float* dst = nullptr, bool* direct = nullptr) {
    pb_ctx* ctx = s->m->ctx;
    if (direct) *direct = false;
    if (dst && direct && host_pinned(dst)) {
        PB_CUDA(ctx, cudaMemcpyAsync(dst, s->logits, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        *direct = true;
        return PB_OK;
    }
    if (n > s->pin_logits_n) {
        if (s->pin_logits) cudaFreeHost(s->pin_logits);
        s->pin_logits = nullptr; s->pin_logits_n = 0;
        if (cudaMallocHost(&s->pin_logits, n * 4) != cudaSuccess) PB_FAIL(ctx, PB_ERR_OOM, "pinned allocation of %zu bytes failed", n * 4);
        s->pin_logits_n = n;
    }
    PB_CUDA(ctx, cudaMemcpyAsync(s->pin_logits, s->logits, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return PB_OK;
}

// ---- MTP drafter bookkeeping on the host: which tokens the main state was fed and which residual rows the ring holds ----
static void mtp_forget(PbMtp* t, int64_t pos) { t->tokens.clear(); t->tok_base = pos; std::fill(t->ring_pos.begin(), t->ring_pos.end(), (int64_t)-1); t->kv_c0 = t->kv_end = pos; }
// the state is about to process `n` tokens `ids` at positions [pos0, pos0 + n)
static void mtp_note(pb_state* s, int64_t pos0, const uint32_t* ids, int n) {
    PbMtp* t = s->mtp;
    if (!t) return;
    if (pos0 < t->tok_base || pos0 > t->tok_base + (int64_t)t->tokens.size()) mtp_forget(t, pos0);
    t->tokens.resize((size_t)(pos0 - t->tok_base));
    for (int j = 0; j < n; j++) { t->tokens.push_back(ids[j]); t->ring_pos[(size_t)((pos0 + j) % t->ring_cap)] = pos0 + j; }
}
// the position moved to `pos` by other means (rollback, restore, reset): keep what lies before it
static void mtp_moved(pb_state* s, int64_t pos) {
    PbMtp* t = s->mtp;
    if (!t) return;
    if (pos < t->tok_base || pos > t->tok_base + (int64_t)t->tokens.size()) { mtp_forget(t, pos); return; }
    t->tokens.resize((size_t)(pos - t->tok_base));
    for (int64_t& p : t->ring_pos) if (p >= pos) p = -1;
    if (t->kv_end > pos) t->kv_end = pos;
    if (t->kv_c0 > t->kv_end) t->kv_c0 = t->kv_end;
}

int pb_forward(pb_state* s, const uint32_t* ids_host, int t, float* logits_host) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx;
    PB_TRY(pb_enter(ctx));
    if (!ids_host || !logits_host || t < 1) PB_FAIL(ctx, PB_ERR_ARG, "pb_forward: bad argument");
    const int B = s->batch;
    if (B == 1 && !s->sharded && t >= 3) {
        // a prompt of one sequence: batched passes of up to PB_PREFILL_CHUNK tokens, each streaming the weights once, cut on
        // the absolute grid of that size -- the first piece runs up to the next multiple of the chunk, so a prompt resumed
        // from a snapshot taken on the grid is split exactly like a prefill from position 0 (src/engine_qn.rs:117-128)
        if (s->pos_host + t > s->m->cfg.max_ctx) PB_FAIL(ctx, PB_ERR_STATE, "context is full (%d positions)", s->m->cfg.max_ctx);
        mtp_note(s, s->pos_host, ids_host, t);
        timing_begin(s);
        for (int j0 = 0, n = 0; j0 < t; j0 += n) {
            const int64_t to_grid = PB_PREFILL_CHUNK - s->pos_host % PB_PREFILL_CHUNK;
            n = t - j0 < to_grid ? t - j0 : (int)to_grid;
            for (int j = 0; j < n; j++) s->pin_u32[j] = ids_host[j0 + j];
            PB_CUDA(ctx, cudaMemcpyAsync(s->ids, s->pin_u32, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
            PB_TRY(window_once(s, n, false, false));
            if (j0 + n < t) PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // the pinned id buffer is reused
        }
        s->verify_t = 0;
        timing_stop(s);
        bool direct = false;
        PB_TRY(logits_stage(s, (size_t)s->m->cfg.vocab, logits_host, &direct));
        const int rcw = pb_sync_check(ctx, "pb_forward");
        timing_collect(s);
        if (rcw == PB_OK && !direct) memcpy(logits_host, s->pin_logits, (size_t)s->m->cfg.vocab * 4);
        return rcw;
    }
    if (B == 1) mtp_note(s, s->pos_host, ids_host, t);
    timing_begin(s);
    for (int j = 0; j < t; j++) {
        for (int b = 0; b < B; b++) s->pin_u32[b] = ids_host[(size_t)b * t + j];
        PB_CUDA(ctx, cudaMemcpyAsync(s->ids, s->pin_u32, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
        PB_TRY(step_once(s));
        if (j + 1 < t) PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // the pinned id buffer is reused
    }
    timing_stop(s);
    bool direct = false;
    PB_TRY(logits_stage(s, (size_t)B * s->m->cfg.vocab, logits_host, &direct));
    const int rc = pb_sync_check(ctx, "pb_forward");
    timing_collect(s);
    if (rc == PB_OK && !direct) memcpy(logits_host, s->pin_logits, (size_t)B * s->m->cfg.vocab * 4);
    return rc;
}

int pb_step_greedy(pb_state* s, const uint32_t* tok_host, uint32_t* next_host) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx;
    PB_TRY(pb_enter(ctx));
    if (!tok_host || !next_host) PB_FAIL(ctx, PB_ERR_ARG, "pb_step_greedy: null buffer");
    const int B = s->batch;
    if (B == 1) mtp_note(s, s->pos_host, tok_host, 1);
    memcpy(s->pin_u32, tok_host, (size_t)B * 4);
    PB_CUDA(ctx, cudaMemcpyAsync(s->ids, s->pin_u32, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
    timing_begin(s);
    PB_TRY(step_once(s));
    timing_stop(s);
    PB_CUDA(ctx, cudaMemcpyAsync(s->pin_u32 + B, s->next, (size_t)B * 4, cudaMemcpyDeviceToHost, ctx->stream));
    PB_TRY(pb_sync_check(ctx, "pb_step_greedy"));
    timing_collect(s);
    memcpy(next_host, s->pin_u32 + B, (size_t)B * 4);
    return PB_OK;
}

int pb_decode_greedy(pb_state* s, const uint32_t* tok_host, int n, uint32_t* out_host) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx;
    PB_TRY(pb_enter(ctx));
    if (!tok_host || !out_host || n < 1) PB_FAIL(ctx, PB_ERR_ARG, "pb_decode_greedy: bad argument");
    if (n > s->trace_cap) PB_FAIL(ctx, PB_ERR_ARG, "pb_decode_greedy: at most %lld tokens per call", (long long)s->trace_cap);
    const int B = s->batch;
    memcpy(s->pin_u32, tok_host, (size_t)B * 4);
    PB_CUDA(ctx, cudaMemcpyAsync(s->ids, s->pin_u32, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
    PB_CUDA(ctx, cudaMemsetAsync(s->trace_len, 0, 8, ctx->stream));
    timing_begin(s);
    for (int j = 0; j < n; j++) PB_TRY(step_once(s));
    timing_stop(s);
    PB_CUDA(ctx, cudaMemcpyAsync(s->pin_u32 + 2 * B, s->trace, (size_t)n * B * 4, cudaMemcpyDeviceToHost, ctx->stream));
    PB_TRY(pb_sync_check(ctx, "pb_decode_greedy"));
    timing_collect(s);
    for (int j = 0; j < n; j++) for (int b = 0; b < B; b++) out_host[(size_t)b * n + j] = s->pin_u32[2 * B + (size_t)j * B + b];
    if (B == 1 && s->mtp) { mtp_note(s, s->pos_host - n, tok_host, 1); if (n > 1) mtp_note(s, s->pos_host - n + 1, out_host, n - 1); }   // fed: the first token, then each output but the last
    return PB_OK;
}



// Model::forward_multi, src/model/qwen4exp_gguf.rs:2365-2480: logits for every fed position and a
// rollback checkpoint of the recurrent state after each of the first t-1 tokens (:2386-2387).
// The window runs through run_window: weights are streamed once for all t tokens (tensor-core GEMM from
// three tokens on), the recurrences token by token; results agree with t calls of pb_forward to rounding
// (different summation order), not bit for bit.
int pb_verify(pb_state* s, const uint32_t* ids_host, int t, float* logits_host) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    if (!ids_host || !logits_host) PB_FAIL(ctx, PB_ERR_ARG, "pb_verify: null buffer");
    if (s->batch != 1) PB_FAIL(ctx, PB_ERR_STATE, "pb_verify: the state must have batch 1 (it has %d)", s->batch);
    if (s->sharded) PB_FAIL(ctx, PB_UNSUPPORTED, "pb_verify: a sharded state holds the rows of one token per sequence; windows run on a plain batch-1 state");
    if (t < 1 || t > PB_MAX_WINDOW) PB_FAIL(ctx, PB_ERR_ARG, "pb_verify: window of %d tokens (1..%d)", t, PB_MAX_WINDOW);
    if (s->pos_host + t > c.max_ctx) PB_FAIL(ctx, PB_ERR_STATE, "context is full (%d positions)", c.max_ctx);
    const int nl = s->m->n_lin;
    if (s->ck_conv.empty() && nl > 0) {
        s->ck_conv.assign((size_t)nl * PB_MAX_WINDOW, nullptr); s->ck_ssm.assign((size_t)nl * PB_MAX_WINDOW, nullptr);
        for (size_t i = 0; i < s->ck_conv.size(); i++) { PB_TRY(dalloc(s, &s->ck_conv[i], conv_elems(c, 1))); PB_TRY(dalloc(s, &s->ck_ssm[i], ssm_elems(c, 1))); }
        std::vector<float*> tab(s->ck_conv.size() * 2), live((size_t)nl * 2);
        for (size_t i = 0; i < s->ck_conv.size(); i++) { tab[2 * i] = s->ck_conv[i]; tab[2 * i + 1] = s->ck_ssm[i]; }
        for (int li = 0; li < nl; li++) { live[(size_t)li * 2] = s->conv[li]; live[(size_t)li * 2 + 1] = s->ssm[li]; }
        PB_TRY(dalloc(s, &s->ck_tab, tab.size())); PB_TRY(dalloc(s, &s->ck_live, live.size()));
        PB_CUDA(ctx, cudaMemcpy(s->ck_tab, tab.data(), tab.size() * sizeof(float*), cudaMemcpyHostToDevice));
        PB_CUDA(ctx, cudaMemcpy(s->ck_live, live.data(), live.size() * sizeof(float*), cudaMemcpyHostToDevice));
    }
    s->verify_pos0 = s->pos_host; s->verify_t = 0;
    mtp_note(s, s->pos_host, ids_host, t);
    for (int j = 0; j < t; j++) s->pin_u32[j] = ids_host[j];
    PB_CUDA(ctx, cudaMemcpyAsync(s->ids, s->pin_u32, (size_t)t * 4, cudaMemcpyHostToDevice, ctx->stream));
    timing_begin(s);
    PB_TRY(window_once(s, t, true, true));
    timing_stop(s);
    bool direct = false;
    PB_TRY(logits_stage(s, (size_t)t * c.vocab, logits_host, &direct));
    PB_TRY(pb_sync_check(ctx, "pb_verify"));
    timing_collect(s);
    if (!direct) memcpy(logits_host, s->pin_logits, (size_t)t * c.vocab * 4);
    s->verify_t = t;
    return PB_OK;
}

// Model::spec_keep :2495-2515: keep the first `keep` of the last t verified tokens: restore the
// DeltaNet state from checkpoint keep-1 and truncate the KV cache and position.  The packed KV
// boundary trails the newest position by at least kv_recent >= 64 > window, so truncation never
// reaches packed rows; ring rows of dropped positions are overwritten when new tokens arrive.
int pb_keep(pb_state* s, int t, int keep) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    if (s->verify_t == 0 || t != s->verify_t) PB_FAIL(ctx, PB_ERR_STATE, "pb_keep: t=%d does not match the last verify window (%d)", t, s->verify_t);
    if (keep < 1 || keep > t) PB_FAIL(ctx, PB_ERR_ARG, "pb_keep: keep=%d outside 1..%d", keep, t);
    if (keep < t) {
        if (s->m->n_lin > 0) PB_TRY(pb_launch_ck_restore(ctx, s->ck_tab, s->ck_live, s->m->n_lin, PB_MAX_WINDOW, keep - 1, (int64_t)conv_elems(c, 1), (int64_t)ssm_elems(c, 1)));
        PB_TRY(pb_state_set_pos(s, s->verify_pos0 + keep));
        // the window moved the packed boundary to where its last token put it; the kept prefix may not have reached that far.
        // Back to the rule for the kept length (kv_push :1520): the f32 rows of the positions in between are still in the
        // ring (it holds kv_recent + 64 + a prompt chunk), and they are packed again, to the same bits, when their turn comes.
        if (c.kv_bits == 4 && !s->m->qsa) {
            const int64_t nk = s->verify_pos0 + keep, rule = nk > c.kv_recent ? ((nk - c.kv_recent) / 64) * 64 : 0;
            std::vector<int64_t> rv((size_t)s->m->n_attn * s->batch, rule);
            if (!rv.empty()) PB_CUDA(ctx, cudaMemcpy(s->q4n_all, rv.data(), rv.size() * 8, cudaMemcpyHostToDevice));
        }
    }
    s->verify_t = 0;
    return PB_OK;
}

// ---------------------------------------------------------------- MTP drafter (src/model/mtp.rs, mtp_draft_in :2179-2278)
int pb_state_attach_drafter(pb_state* s, pb_model* dm, const uint32_t* vocab_ids_host, int n_ids) {
    if (!s || !dm) return PB_ERR_ARG;
    pb_model* m = s->m; pb_ctx* ctx = m->ctx; const pb_cfg& c = m->cfg; const pb_cfg& dc = dm->cfg;
    PB_TRY(pb_enter(ctx));
    if (s->mtp) PB_FAIL(ctx, PB_ERR_STATE, "pb_state_attach_drafter: the state already has a drafter");
    if (dm->ctx != ctx || !dm->finalized || dm->mtp_window < 1) PB_FAIL(ctx, PB_ERR_STATE, "pb_state_attach_drafter: not a finalized drafter model of this context (pb_model_set_mtp)");
    if (s->batch != 1 || s->sharded || c.hc < 1) PB_FAIL(ctx, PB_UNSUPPORTED, "pb_state_attach_drafter: the drafter follows one sequence of a model with hyper-connection streams");
    if (dc.d != c.d || dc.hc != c.hc || dc.max_ctx < c.max_ctx) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_attach_drafter: drafter of width %d x %d streams and %d positions for a model of %d x %d and %d", dc.d, dc.hc, dc.max_ctx, c.d, c.hc, c.max_ctx);
    if (!vocab_ids_host || n_ids != dc.vocab) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_attach_drafter: %d draft-vocabulary ids for a head of %d rows", n_ids, dc.vocab);
    for (int i = 0; i < n_ids; i++) if (vocab_ids_host[i] >= (uint32_t)c.vocab) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_attach_drafter: id %u outside the vocabulary", vocab_ids_host[i]);
    PbMtp* t = new PbMtp();
    s->mtp = t;
    t->dm = dm; t->window = dm->mtp_window; t->n_ids = n_ids; t->ids.assign(vocab_ids_host, vocab_ids_host + n_ids);
    PB_TRY(pb_state_create(dm, 1, &t->ds));
    const int w = c.hc * c.d;
    t->ring_cap = t->window + 16 + PB_PREFILL_CHUNK;   // the reference keeps window + 16 rows; a whole prompt chunk arrives at once here
    t->ring_pos.assign((size_t)t->ring_cap, (int64_t)-1);
    PB_TRY(dalloc(s, &t->ring, (size_t)t->ring_cap * w));
    PB_TRY(dalloc(s, &t->e_raw, (size_t)c.d)); PB_TRY(dalloc(s, &t->en, (size_t)c.d)); PB_TRY(dalloc(s, &t->e2, (size_t)c.d));
    PB_TRY(dalloc(s, &t->hn, (size_t)w)); PB_TRY(dalloc(s, &t->h2, (size_t)w)); PB_TRY(dalloc(s, &t->lg, (size_t)n_ids));
    PB_TRY(dalloc(s, &t->tok_dev, (size_t)4)); PB_TRY(dalloc(s, &t->best, (size_t)4));
    PB_TRY(dalloc(s, &t->mask, (size_t)dc.max_ctx / 32 + 2)); PB_TRY(dalloc(s, &t->mask_on, (size_t)1));
    if (cudaMallocHost(&t->pin, 64) != cudaSuccess) PB_FAIL(ctx, PB_ERR_OOM, "pinned allocation failed");
    t->ds->ext_mask = t->mask; t->ds->ext_on = t->mask_on; t->ds->ext_ld = 0;
    mtp_forget(t, s->pos_host);
    // the step graphs of this state were captured without the copy of the residual rows: drop them
    if (s->graph) { cudaGraphExecDestroy(s->graph); s->graph = nullptr; }
    for (cudaGraphExec_t& g : s->win_graph) if (g) { cudaGraphExecDestroy(g); g = nullptr; }
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PB_OK;
}

// One drafter cell at rope position `pos`: R = the residual row it pairs (device, hc*d), tok = the token at pos + 1.
// full = false: K/V only (catch_up, mtp.rs:172-175); full = true: the whole step (step, :184-236), leaving the final mixer's
// output in ds->hmix, the drafter's residual in ds->x and (index, probability) of the best draft-vocabulary token in t->best.
static int mtp_cell(pb_state* s, const float* R, uint32_t tok, int64_t pos, bool full) {
    PbMtp* t = s->mtp; pb_model* m = s->m; pb_ctx* ctx = m->ctx; pb_model* dm = t->dm; pb_state* ds = t->ds; const pb_cfg& c = dm->cfg;
    const int d = c.d, w = c.hc * c.d;
    // (pageable sources: the driver stages them at the call, so the next cell may reuse the variables at once)
    const uint32_t tk = tok; const int64_t p64 = pos;
    PB_CUDA(ctx, cudaMemcpyAsync(t->tok_dev, &tk, 4, cudaMemcpyHostToDevice, ctx->stream));
    PB_CUDA(ctx, cudaMemcpyAsync(ds->pos, &p64, 8, cudaMemcpyHostToDevice, ctx->stream));
    ds->pos_host = pos;
    pb_qmat* embd = M(m, -1, PB_R_TOKEN_EMBD);
    PB_TRY(pb_launch_embed(ctx, embd->type, embd->data, embd->rows, d, t->tok_dev, 1, t->e_raw, d));
    ctx->pdl_chain = false;
    // input (mtp.rs:186-195): e = fc_embedding(rms(embed) * pre_e); h = fc_hidden per stream of rms over all hc*d values * pre_h; R' = h + e
    PB_TRY(pb_launch_mtp_input(ctx, t->e_raw, V(dm, -1, PB_R_MTP_PRE_E), R, V(dm, -1, PB_R_MTP_PRE_H), t->en, t->hn, d, w, c.eps));
    PbGemvArgs g;
    pb_qmat* fe = M(dm, -1, PB_R_MTP_FC_E); pb_qmat* fh = M(dm, -1, PB_R_MTP_FC_H);
    g.w = fe->data; g.wr = fe->rdata; g.type = fe->type; g.rows = fe->rows; g.cols = d; g.x = t->en; g.ldx = d; g.t = 1; g.y = t->e2; g.ldy = d;
    PB_TRY(pb_launch_gemv(ctx, g));
    g.w = fh->data; g.wr = fh->rdata; g.type = fh->type; g.rows = fh->rows; g.x = t->hn; g.t = c.hc; g.y = t->h2;
    PB_TRY(pb_launch_gemv(ctx, g));
    PB_TRY(pb_launch_mtp_join(ctx, t->h2, t->e2, ds->x, d, w));
    PbHcParams h;
    hc_params(ds, 0, PB_R_HCA_NORM, PB_R_HCA_DOWN, PB_R_HCA_UP, PB_R_HCA_INJECT, h);
    PB_TRY(pb_launch_hc_mix(ctx, h, ds->x, 1, ds->hmix));
    if (!full) {
        // kv_append (:156-170): the cell's K and V
        const int64_t nq = (int64_t)c.n_head * 2 * c.hd, row = (int64_t)c.n_kv * c.hd;
        PbGemvQArgs a; memset(&a, 0, sizeof a);
        a.type = M(dm, 0, PB_R_ATTN_Q)->type; a.cols = d; a.nseg = 2;
        seg(a, 0, M(dm, 0, PB_R_ATTN_K), nq); seg(a, 1, M(dm, 0, PB_R_ATTN_V), nq + row);
        a.x = ds->hmix; a.ldx = d; a.y = ds->proj; a.ldy = ds->ldproj; a.mode = PB_ACT_PLAIN; a.eps = c.eps;
        PB_TRY(gemv_cols(ctx, a, 1, false));
        PbAttnParams p; attn_params(ds, 0, p);
        return pb_launch_kv_append(ctx, p);
    }
    int64_t lo = pos - t->window + 1;
    if (lo < t->kv_c0) lo = t->kv_c0;
    PB_TRY(pb_launch_mtp_mask(ctx, t->mask, t->mask_on, lo, pos));
    PB_TRY(run_attn(ds, 0, ds->hmix, nullptr, ds->yout, d, 0));
    PB_TRY(pb_launch_hc_combine(ctx, h, ds->x, ds->yout, 1));
    hc_params(ds, 0, PB_R_HCF_NORM, PB_R_HCF_DOWN, PB_R_HCF_UP, PB_R_HCF_INJECT, h);
    PB_TRY(pb_launch_hc_mix(ctx, h, ds->x, 1, ds->hmix));
    PB_TRY(run_moe(ds, 0, ds->hmix, nullptr, 1, ds->yout, d, 0));
    PB_TRY(pb_launch_hc_combine(ctx, h, ds->x, ds->yout, 1));
    hc_params(ds, -1, PB_R_OUT_HC_NORM, PB_R_OUT_HC_DOWN, PB_R_OUT_HC_UP, -1, h);   // the final mixer
    PB_TRY(pb_launch_hc_mix(ctx, h, ds->x, 1, ds->hmix));
    pb_qmat* head = M(dm, -1, PB_R_OUTPUT);
    g.w = head->data; g.wr = head->rdata; g.type = head->type; g.rows = head->rows; g.cols = d; g.x = ds->hmix; g.ldx = d; g.t = 1; g.y = t->lg; g.ldy = t->n_ids;
    PB_TRY(pb_launch_gemv(ctx, g));
    ctx->pdl_chain = false;
    return pb_launch_mtp_best(ctx, t->lg, t->n_ids, t->best);
}

// Model::mtp_draft :2177 (= Target::draft): up to max_draft tokens that follow the fed tokens and `pending` (the token chosen
// but not fed yet).  Token j > 0 is kept only while the drafter's probability of it is at least min_p (draft_gate, spec.rs:326).
// *n = 0 when nothing can be drafted (no drafter state for the last position); PB_UNSUPPORTED without a drafter.
int pb_draft(pb_state* s, uint32_t pending, int max_draft, float min_p, uint32_t* ids_host, float* probs_host, int* n) {
    return pb_draft_sampled(s, pending, max_draft, min_p, nullptr, nullptr, ids_host, probs_host, n);
}
int pb_draft_sampled(pb_state* s, uint32_t pending, int max_draft, float min_p, pb_draft_pick pick, void* user, uint32_t* ids_host, float* probs_host, int* n) {
    if (!s || !n) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx;
    PB_TRY(pb_enter(ctx));
    *n = 0;
    PbMtp* t = s->mtp;
    if (!t) PB_FAIL(ctx, PB_UNSUPPORTED, "no drafter attached: use the caller's n-gram drafter");
    if (max_draft < 0 || (max_draft > 0 && !ids_host)) PB_FAIL(ctx, PB_ERR_ARG, "pb_draft: bad argument");
    if (pending >= (uint32_t)s->m->cfg.vocab) PB_FAIL(ctx, PB_ERR_ARG, "pb_draft: token %u outside the vocabulary", pending);
    const int64_t np = s->pos_host;               // tokens fed so far: cells 0 .. np - 1 exist, cell i pairs R_i with token i + 1
    if (np == 0 || max_draft == 0) return PB_OK;
    const int w = s->m->cfg.hc * s->m->cfg.d;
    auto have_r = [&](int64_t p) { return p >= 0 && t->ring_pos[(size_t)(p % t->ring_cap)] == p; };
    auto r_of = [&](int64_t p) { return t->ring + (size_t)(p % t->ring_cap) * w; };
    auto tok_at = [&](int64_t p, uint32_t& out) { if (p < t->tok_base || p >= t->tok_base + (int64_t)t->tokens.size()) return false; out = t->tokens[(size_t)(p - t->tok_base)]; return true; };
    if (!have_r(np - 1)) return PB_OK;
    if (np + max_draft > t->dm->cfg.max_ctx) return PB_OK;
    if (t->kv_end > np - 1) t->kv_end = np - 1;   // kv.truncate(n - 1)
    if (t->kv_c0 > t->kv_end) t->kv_c0 = t->kv_end;
    // catch-up (:2191-2213): cells below np - 1 whose residual is known; a gap restarts the drafter's K/V
    int64_t first = np - 1;
    while (have_r(first - 1)) first--;
    const bool cont = t->kv_end > t->kv_c0 && t->kv_end >= first;
    int64_t lo = cont ? t->kv_end : (first > np - 1 - t->window ? first : np - 1 - t->window);
    if (lo < 0) lo = 0;
    bool ok = true;
    for (int64_t i = lo; i < np - 1 && ok; i++) { uint32_t tk; ok = have_r(i) && tok_at(i + 1, tk); }
    if (!ok) { lo = np - 1; t->kv_c0 = t->kv_end = lo; }
    else if (!cont) { t->kv_c0 = t->kv_end = lo; }
    for (int64_t i = lo; i < np - 1; i++) {
        uint32_t tk = 0; tok_at(i + 1, tk);
        PB_TRY(mtp_cell(s, r_of(i), tk, i, false));
        t->kv_end = i + 1;
    }
    // the draft loop (:2214-2272)
    const float* r = r_of(np - 1);
    uint32_t tok = pending;
    int made = 0;
    for (int j = 0; j < max_draft; j++) {
        PB_TRY(mtp_cell(s, r, tok, np - 1 + j, true));
        PB_CUDA(ctx, cudaMemcpyAsync(t->pin + 1, t->best, 8, cudaMemcpyDeviceToHost, ctx->stream));
        PB_TRY(pb_sync_check(ctx, "pb_draft"));
        if (j == 0) t->kv_end = np;               // the cell of the last fed position stays (its token is `pending`)
        const uint32_t bi = t->pin[1]; float p; memcpy(&p, t->pin + 2, 4);
        if (j > 0 && p < min_p) break;            // draft_gate
        uint32_t id = t->ids[bi < (uint32_t)t->n_ids ? bi : (uint32_t)t->n_ids - 1];
        if (pick) {   // :2246: the caller's sampler draws from the drafter's distribution
            if ((size_t)t->n_ids > t->lg_host.size()) t->lg_host.resize((size_t)t->n_ids);
            PB_CUDA(ctx, cudaMemcpyAsync(t->lg_host.data(), t->lg, (size_t)t->n_ids * 4, cudaMemcpyDeviceToHost, ctx->stream));
            PB_TRY(pb_sync_check(ctx, "pb_draft_sampled"));
            id = pick(user, t->lg_host.data(), t->ids.data(), t->n_ids);
            if (id >= (uint32_t)s->m->cfg.vocab) PB_FAIL(ctx, PB_ERR_ARG, "pb_draft_sampled: the sampler returned token %u, outside the vocabulary", id);
        }
        ids_host[made] = id; if (probs_host) probs_host[made] = p;
        made++;
        r = t->ds->x; tok = id;                   // the drafter's own residual feeds its next step
    }
    *n = made;
    return PB_OK;
}

// Model::snapshot / restore, Snap :3277-3298.  Layout: header, then per DeltaNet layer [conv ring][ssm],
// then per attention layer and (sequence, KV head): q4n, packed K words/scales, packed V words/scales for
// positions [0, q4n), f32 ring rows of K and V for positions [q4n, len).
struct PbSnapHeader { uint64_t magic; int32_t n_layers, d, batch, kv_bits; int64_t pos; uint64_t bytes; };
static const uint64_t kSnapMagic = 0x3150414e53425050ull;   // "PPBSNAP1"

// q4[ai * B + b] = packed boundary of sequence b in attention layer ai.  The boundary is what the device holds
// (after a rollback it is ahead of the value the current length alone would give), so a snapshot reads it back
// and stores it; a restore takes it from the snapshot.
// n-gram embeddings in a snapshot: the first position with a history, then per sequence the last ngram - 1 ids and per PLE layer the
// normalized rows of the last (conv_k - 1) * ngram positions (what a later token can still read), newest first
static size_t ple_snap_bytes(const pb_state* s) {
    const pb_model* m = s->m;
    if (m->n_ple == 0) return 0;
    const size_t w = (size_t)m->cfg.d * (m->cfg.hc > 0 ? m->cfg.hc : 1), hl = (size_t)(m->ple_conv_k - 1) * m->ple.ngram;
    return 8 + (size_t)s->batch * (m->ple.ngram - 1) * 4 + (size_t)m->n_ple * s->batch * hl * w * 4;
}
static size_t snap_size(const pb_state* s, const std::vector<int64_t>& q4) {
    const pb_cfg& c = s->m->cfg; const int B = s->batch;
    const int64_t len = s->pos_host;
    size_t n = sizeof(PbSnapHeader) + (size_t)s->m->n_lin * (conv_elems(c, B) + ssm_elems(c, B)) * 4;
    for (int ai = 0; ai < s->m->n_attn; ai++)
        for (int b = 0; b < B; b++) {
            const int64_t q4n = q4[(size_t)ai * B + b];
            n += (size_t)c.n_kv * (8 + 2 * ((size_t)q4n * (c.hd / 8) * 4 + (size_t)q4n * (c.hd / 32) * 4) + 2 * (size_t)(len - q4n) * c.hd * 4);
        }
    if (s->m->qsa) n += (size_t)s->m->n_attn * B * (size_t)len * s->m->idx_hd * 4;   // raw index keys; the pooled block keys are rebuilt
    return n + ple_snap_bytes(s);
}
static int snap_read_q4(pb_state* s, std::vector<int64_t>& q4) {
    pb_ctx* ctx = s->m->ctx; const int B = s->batch;
    q4.assign((size_t)s->m->n_attn * B, 0);
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (!q4.empty()) PB_CUDA(ctx, cudaMemcpy(q4.data(), s->q4n_all, q4.size() * 8, cudaMemcpyDeviceToHost));
    for (int64_t v : q4) if (v < 0 || v > s->pos_host || v % 64) PB_FAIL(ctx, PB_ERR_STATE, "packed KV boundary %lld does not fit the position %lld", (long long)v, (long long)s->pos_host);
    return PB_OK;
}

static int snap_io(pb_state* s, uint8_t* buf, bool save, const std::vector<int64_t>& q4) {
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg; const int B = s->batch;
    const cudaMemcpyKind kind = save ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice;
    const int64_t len = s->pos_host;
    uint8_t* p = buf + sizeof(PbSnapHeader);
    auto io = [&](void* dev, size_t bytes) -> int {
        if (bytes) { if (save) PB_CUDA(ctx, cudaMemcpy(p, dev, bytes, kind)); else PB_CUDA(ctx, cudaMemcpy(dev, p, bytes, kind)); }
        p += bytes; return PB_OK;
    };
    for (int li = 0; li < s->m->n_lin; li++) { PB_TRY(io(s->conv[li], conv_elems(c, B) * 4)); PB_TRY(io(s->ssm[li], ssm_elems(c, B) * 4)); }
    for (int ai = 0; ai < s->m->n_attn; ai++) {
        PbKv& k = s->kv[ai];
        for (int b = 0; b < B; b++)
            for (int h = 0; h < c.n_kv; h++) {
                const size_t head = (size_t)b * c.n_kv + h;
                const int64_t q4n = q4[(size_t)ai * B + b];
                int64_t q = q4n;
                if (save) memcpy(p, &q, 8); else PB_CUDA(ctx, cudaMemcpy(k.q4n + b, &q, 8, cudaMemcpyHostToDevice));
                p += 8;
                const size_t pm = c.kv_bits == 4 ? (size_t)c.max_ctx : 1;
                PB_TRY(io(k.kw + head * pm * (c.hd / 8), (size_t)q4n * (c.hd / 8) * 4)); PB_TRY(io(k.ks + head * pm * (c.hd / 32), (size_t)q4n * (c.hd / 32) * 4));
                PB_TRY(io(k.vw + head * pm * (c.hd / 8), (size_t)q4n * (c.hd / 8) * 4)); PB_TRY(io(k.vs + head * pm * (c.hd / 32), (size_t)q4n * (c.hd / 32) * 4));
                for (int which = 0; which < 2; which++) {
                    float* ring = (which ? k.vr : k.kr) + head * s->ring_cap * c.hd;
                    for (int64_t pp = q4n; pp < len;) {   // contiguous runs inside the ring
                        const int64_t slot = pp % s->ring_cap, run = (len - pp) < (s->ring_cap - slot) ? (len - pp) : (s->ring_cap - slot);
                        PB_TRY(io(ring + (size_t)slot * c.hd, (size_t)run * c.hd * 4));
                        pp += run;
                    }
                }
            }
    }
    if (s->m->qsa)
        for (int ai = 0; ai < s->m->n_attn; ai++)
            for (int b = 0; b < B; b++) PB_TRY(io(s->kv[ai].ik + (size_t)b * c.max_ctx * s->m->idx_hd, (size_t)len * s->m->idx_hd * 4));
    if (s->m->n_ple > 0) {
        const pb_model* m = s->m;
        const size_t w = (size_t)c.d * (c.hc > 0 ? c.hc : 1); const int hl = (m->ple_conv_k - 1) * m->ple.ngram;
        if (save) memcpy(p, &s->ple_base_host, 8);
        else {
            int64_t base; memcpy(&base, p, 8);
            if (base < 0 || base > len) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_restore: corrupt snapshot (history base %lld at position %lld)", (long long)base, (long long)len);
            std::vector<int64_t> bv((size_t)B, base);
            PB_CUDA(ctx, cudaMemcpy(s->ple_base, bv.data(), bv.size() * 8, cudaMemcpyHostToDevice));
            s->ple_base_host = base;
        }
        p += 8;
        auto io_or_skip = [&](void* dev, size_t bytes, bool have) -> int {
            if (have) return io(dev, bytes);
            if (save) memset(p, 0, bytes);
            p += bytes; return PB_OK;
        };
        for (int b = 0; b < B; b++)
            for (int j = 1; j < m->ple.ngram; j++) { const int64_t q = len - j; PB_TRY(io_or_skip(s->tok_hist + (size_t)b * c.max_ctx + (q >= 0 ? q : 0), 4, q >= 0)); }
        for (int pi = 0; pi < m->n_ple; pi++)
            for (int b = 0; b < B; b++)
                for (int j = 1; j <= hl; j++) { const int64_t q = len - j; PB_TRY(io_or_skip(s->ple_ring[(size_t)pi] + ((size_t)b * s->ple_R + (size_t)((q >= 0 ? q : 0) % s->ple_R)) * w, w * 4, q >= 0)); }
    }
    return PB_OK;
}

int pb_state_snapshot(pb_state* s, void* buf_host, size_t* nbytes) {
    if (!s || !nbytes) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx;
    PB_TRY(pb_enter(ctx));
    std::vector<int64_t> q4;
    PB_TRY(snap_read_q4(s, q4));
    const size_t need = snap_size(s, q4);
    if (!buf_host) { *nbytes = need; return PB_OK; }
    if (*nbytes < need) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_snapshot: buffer of %zu bytes, %zu needed", *nbytes, need);
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    PbSnapHeader h; memset(&h, 0, sizeof h);
    h.magic = kSnapMagic; h.n_layers = s->m->cfg.n_layers; h.d = s->m->cfg.d; h.batch = s->batch; h.kv_bits = s->m->cfg.kv_bits; h.pos = s->pos_host; h.bytes = need;
    memcpy(buf_host, &h, sizeof h);
    PB_TRY(snap_io(s, (uint8_t*)buf_host, true, q4));
    *nbytes = need;
    return PB_OK;
}

int pb_state_restore(pb_state* s, const void* buf_host, size_t nbytes) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx;
    PB_TRY(pb_enter(ctx));
    if (!buf_host || nbytes < sizeof(PbSnapHeader)) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_restore: truncated snapshot");
    PbSnapHeader h; memcpy(&h, buf_host, sizeof h);
    if (h.magic != kSnapMagic) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_restore: not a snapshot");
    if (h.n_layers != s->m->cfg.n_layers || h.d != s->m->cfg.d || h.batch != s->batch || h.kv_bits != s->m->cfg.kv_bits) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_restore: snapshot of a different model or batch");
    if (h.pos < 0 || h.pos > s->m->cfg.max_ctx || h.bytes != nbytes) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_restore: truncated or corrupt snapshot (%zu bytes, header says %llu)", nbytes, (unsigned long long)h.bytes);
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    // walk the snapshot once for the stored boundaries (first field of every (layer, sequence, KV head) section)
    const pb_cfg& c = s->m->cfg; const int B = s->batch;
    std::vector<int64_t> q4((size_t)s->m->n_attn * B, 0);
    {
        size_t off = sizeof(PbSnapHeader) + (size_t)s->m->n_lin * (conv_elems(c, B) + ssm_elems(c, B)) * 4;
        for (int ai = 0; ai < s->m->n_attn; ai++)
            for (int b = 0; b < B; b++)
                for (int hh = 0; hh < c.n_kv; hh++) {
                    if (off + 8 > nbytes) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_restore: truncated snapshot");
                    int64_t q; memcpy(&q, (const uint8_t*)buf_host + off, 8);
                    if (q < 0 || q > h.pos || q % 64 || (c.kv_bits != 4 && q != 0)) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_restore: corrupt snapshot (packed boundary %lld at position %lld)", (long long)q, (long long)h.pos);
                    q4[(size_t)ai * B + b] = q;
                    off += 8 + 2 * ((size_t)q * (c.hd / 8) * 4 + (size_t)q * (c.hd / 32) * 4) + 2 * (size_t)(h.pos - q) * c.hd * 4;
                }
        if (s->m->qsa) off += (size_t)s->m->n_attn * B * (size_t)h.pos * s->m->idx_hd * 4;
        off += ple_snap_bytes(s);
        if (off != nbytes) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_restore: size mismatch");
    }
    // position first (a fresh boundary of 0 so that any position is accepted), then the sections
    for (int ai = 0; ai < s->m->n_attn; ai++) PB_CUDA(ctx, cudaMemsetAsync(s->kv[ai].q4n, 0, (size_t)B * 8, ctx->stream));
    PB_TRY(pb_state_set_pos(s, h.pos));
    s->verify_t = 0;
    PB_TRY(snap_io(s, (uint8_t*)const_cast<void*>(buf_host), false, q4));
    if (s->mtp) mtp_forget(s->mtp, h.pos);   // the restored history is not the one the drafter followed
    if (s->m->qsa) for (int ai = 0; ai < s->m->n_attn; ai++) PB_TRY(qsa_pool_all(s, ai, h.pos));
    return PB_OK;
}

int pb_stats_get(const pb_state* s, pb_stats* out) {
    if (!s || !out) return PB_ERR_ARG;
    const pb_cfg& c = s->m->cfg;
    out->steps = s->steps; out->kernels_launched = s->kernels_per_step;
    out->weight_bytes_per_step = s->m->weight_bytes_step;
    const uint64_t len = (uint64_t)s->pos_host;
    const uint64_t packed = c.kv_bits == 4 && len > (uint64_t)c.kv_recent ? ((len - c.kv_recent) / 64) * 64 : 0;
    out->kv_bytes_per_step = (uint64_t)s->m->n_attn * s->batch * 2 * c.n_kv * (packed * (c.hd / 2 + c.hd / 8) + (len - packed) * c.hd * 4);
    out->state_bytes_per_step = (uint64_t)s->m->n_lin * s->batch * 2 * ((uint64_t)c.lin_nv * c.lin_dk * c.lin_dv * 4);
    out->device_ns = s->device_ns; out->exchange_ns = 0;
    if (s->p2p) {   // time inside the peer hand-shakes (store fence + flag + wait for the peer), averaged over the peers; synchronises the stream
        unsigned long long ns = 0;
        if (cudaStreamSynchronize(s->m->ctx->stream) == cudaSuccess && cudaMemcpy(&ns, s->ep_seq + 1, 8, cudaMemcpyDeviceToHost) == cudaSuccess) out->exchange_ns = ns / (uint64_t)s->m->ep_world;
    }
    return PB_OK;
}

// ------------------------------------------------------------------------------------ layer-level entry points

static int layer_ok(pb_state* s, int layer, int want_kind, const char* who) {
    pb_ctx* ctx = s->m->ctx;
    if (layer < 0 || layer >= s->m->cfg.n_layers) PB_FAIL(ctx, PB_ERR_ARG, "%s: layer %d out of range", who, layer);
    if (want_kind >= 0 && s->m->kind[layer] != want_kind) PB_FAIL(ctx, PB_ERR_ARG, "%s: layer %d is not a %s layer", who, layer, want_kind ? "full-attention" : "DeltaNet");
    return PB_OK;
}

int pb_moe_forward(pb_state* s, int layer, const float* x_host, int t, float* y_host, int32_t* sel_host) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    PB_TRY(layer_ok(s, layer, -1, "pb_moe_forward"));
    if (!x_host || !y_host || t < 0 || t > s->batch) PB_FAIL(ctx, PB_ERR_ARG, "pb_moe_forward: t=%d (state batch %d)", t, s->batch);
    if (t == 0) return PB_OK;
    PB_CUDA(ctx, cudaMemcpyAsync(s->xin, x_host, (size_t)t * c.d * 4, cudaMemcpyHostToDevice, ctx->stream));
    PB_TRY(run_moe(s, layer, s->xin, nullptr, t, s->yout, c.d, 0));
    PB_CUDA(ctx, cudaMemcpyAsync(y_host, s->yout, (size_t)t * c.d * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (sel_host) PB_CUDA(ctx, cudaMemcpyAsync(sel_host, s->sel_e, (size_t)t * c.top_k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return pb_sync_check(ctx, "pb_moe_forward");
}

int pb_deltanet_step(pb_state* s, int layer, const float* x_host, float* y_host) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    PB_TRY(layer_ok(s, layer, 0, "pb_deltanet_step"));
    if (!x_host || !y_host) PB_FAIL(ctx, PB_ERR_ARG, "pb_deltanet_step: null buffer");
    PB_CUDA(ctx, cudaMemcpyAsync(s->xin, x_host, (size_t)s->batch * c.d * 4, cudaMemcpyHostToDevice, ctx->stream));
    PB_TRY(run_lin(s, layer, s->xin, nullptr, s->yout, c.d, 0));
    PB_CUDA(ctx, cudaMemcpyAsync(y_host, s->yout, (size_t)s->batch * c.d * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return pb_sync_check(ctx, "pb_deltanet_step");
}

int pb_attn_step(pb_state* s, int layer, const float* x_host, float* y_host) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    PB_TRY(layer_ok(s, layer, 1, "pb_attn_step"));
    if (!x_host || !y_host) PB_FAIL(ctx, PB_ERR_ARG, "pb_attn_step: null buffer");
    if (s->pos_host + 1 > c.max_ctx) PB_FAIL(ctx, PB_ERR_STATE, "context is full (%d positions)", c.max_ctx);
    PB_CUDA(ctx, cudaMemcpyAsync(s->xin, x_host, (size_t)s->batch * c.d * 4, cudaMemcpyHostToDevice, ctx->stream));
    PB_TRY(run_attn(s, layer, s->xin, nullptr, s->yout, c.d, 0));
    PB_CUDA(ctx, cudaMemcpyAsync(y_host, s->yout, (size_t)s->batch * c.d * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return pb_sync_check(ctx, "pb_attn_step");
}

int pb_state_peek(pb_state* s, int what, float* out_host, int64_t n) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    const float* src = nullptr;
    switch (what) {
        case 0: src = s->x; break;
        case 1: src = s->proj; break;
        case 2: src = s->olin; break;
        case 3: src = s->att; break;
        case 4: src = s->rlogits; break;
        case 5: src = s->fused == 1 ? s->fh : s->h; break;
        case 6: src = s->fused == 1 ? s->fh + (size_t)c.top_k * c.ff_exp : s->h_sh; break;
        case 7: src = reinterpret_cast<const float*>(s->ftrace); break;   // per-CTA stamps of the fused step: [op][grid][4] uint64 (n counts floats)
        default: break;
    }
    if (!src || !out_host || n <= 0) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_peek: bad argument");
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    PB_CUDA(ctx, cudaMemcpy(out_host, src, (size_t)n * 4, cudaMemcpyDeviceToHost));
    return PB_OK;
}

// conv history oldest-first [batch][conv_k-1][ch] <-> ring slots (pos + 1 + k) mod conv_k
int pb_state_get_lin(pb_state* s, int layer, float* conv_host, float* ssm_host) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    PB_TRY(layer_ok(s, layer, 0, "pb_state_get_lin"));
    const int li = s->m->idx[layer], K = c.conv_k, ch = 2 * c.lin_nk * c.lin_dk + c.lin_nv * c.lin_dv;
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (conv_host)
        for (int b = 0; b < s->batch; b++) for (int k = 0; k < K - 1; k++)
            PB_CUDA(ctx, cudaMemcpy(conv_host + ((size_t)b * (K - 1) + k) * ch, s->conv[li] + ((size_t)b * K + (size_t)((s->pos_host + 1 + k) % K)) * ch, (size_t)ch * 4, cudaMemcpyDeviceToHost));
    if (ssm_host) PB_CUDA(ctx, cudaMemcpy(ssm_host, s->ssm[li], (size_t)s->batch * c.lin_nv * c.lin_dk * c.lin_dv * 4, cudaMemcpyDeviceToHost));
    return PB_OK;
}
int pb_state_set_lin(pb_state* s, int layer, const float* conv_host, const float* ssm_host) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    PB_TRY(layer_ok(s, layer, 0, "pb_state_set_lin"));
    const int li = s->m->idx[layer], K = c.conv_k, ch = 2 * c.lin_nk * c.lin_dk + c.lin_nv * c.lin_dv;
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (conv_host)
        for (int b = 0; b < s->batch; b++) for (int k = 0; k < K - 1; k++)
            PB_CUDA(ctx, cudaMemcpy(s->conv[li] + ((size_t)b * K + (size_t)((s->pos_host + 1 + k) % K)) * ch, conv_host + ((size_t)b * (K - 1) + k) * ch, (size_t)ch * 4, cudaMemcpyHostToDevice));
    if (ssm_host) PB_CUDA(ctx, cudaMemcpy(s->ssm[li], ssm_host, (size_t)s->batch * c.lin_nv * c.lin_dk * c.lin_dv * 4, cudaMemcpyHostToDevice));
    return PB_OK;
}

// Pre-fill one sequence's KV of one attention layer from host rows [n][n_kv*hd] (already normed and roped).
// pooled keys of the complete blocks among the first n positions of every sequence (after a fill or a restore)
static int qsa_pool_all(pb_state* s, int ai, int64_t n) {
    pb_model* m = s->m; const pb_cfg& c = m->cfg;
    int il = 0;
    for (int i = 0; i < c.n_layers; i++) if (m->kind[i] && m->idx[i] == ai) il = i;
    PbQsaParams qp; memset(&qp, 0, sizeof qp);
    qp.ikn = V(m, il, PB_R_IDX_K_NORM); qp.rope_inv = m->rope_inv; qp.n_rot = c.n_rot; qp.eps = c.eps;
    qp.inh = m->idx_nh; qp.ihd = m->idx_hd; qp.ratio = m->idx_ratio; qp.budget = m->idx_budget;
    qp.ik = s->kv[ai].ik; qp.ib = s->kv[ai].ib; qp.max_ctx = c.max_ctx; qp.nb_cap = s->nb_cap; qp.batch = s->batch;
    return pb_launch_qsa_pool_all(m->ctx, qp, n / m->idx_ratio);
}

// Raw index keys of the first n positions of sequence b of attention layer ai, [n][idx_hd] (f32, host): the companion of
// pb_state_fill_kv for models with an indexer.
int pb_state_fill_index_keys(pb_state* s, int b, int ai, const float* ik_host, int64_t n) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    if (!s->m->qsa) PB_FAIL(ctx, PB_ERR_STATE, "pb_state_fill_index_keys: the model has no indexer");
    if (b < 0 || b >= s->batch || ai < 0 || ai >= s->m->n_attn || !ik_host || n < 0 || n > c.max_ctx) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_fill_index_keys: bad argument");
    PB_CUDA(ctx, cudaMemcpyAsync(s->kv[ai].ik + (size_t)b * c.max_ctx * s->m->idx_hd, ik_host, (size_t)n * s->m->idx_hd * 4, cudaMemcpyHostToDevice, ctx->stream));
    PB_TRY(qsa_pool_all(s, ai, n));
    PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return PB_OK;
}

int pb_state_fill_kv(pb_state* s, int b, int ai, const float* k_host, const float* v_host, int64_t n) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    if (b < 0 || b >= s->batch || ai < 0 || ai >= s->m->n_attn || !k_host || !v_host || n < 0 || n > c.max_ctx) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_fill_kv: bad argument");
    PbKv& kv = s->kv[ai];
    const int hd = c.hd, nkv = c.n_kv;
    const int64_t q4n = c.kv_bits == 4 && n > c.kv_recent ? ((n - c.kv_recent) / 64) * 64 : 0;
    std::vector<float> tmp((size_t)(n > 0 ? n : 1) * hd);
    void* scr;
    PB_TRY(pb_scratch(ctx, (size_t)(q4n > 0 ? q4n : 1) * hd * 4 + 1024, &scr));
    for (int which = 0; which < 2; which++) {
        const float* src = which ? v_host : k_host;
        for (int h = 0; h < nkv; h++) {
            for (int64_t p = 0; p < n; p++) memcpy(&tmp[(size_t)p * hd], src + ((size_t)p * nkv + h) * hd, (size_t)hd * 4);
            const size_t head = (size_t)b * nkv + h;
            if (q4n > 0) {
                PB_CUDA(ctx, cudaMemcpyAsync(scr, tmp.data(), (size_t)q4n * hd * 4, cudaMemcpyHostToDevice, ctx->stream));
                if (which) PB_TRY(pb_launch_kv4_pack_vt(ctx, (const float*)scr, q4n, hd, kv.vw + head * c.max_ctx * (hd / 8), kv.vs + head * c.max_ctx * (hd / 32), 8));
                else PB_TRY(pb_launch_kv4_pack(ctx, (const float*)scr, q4n * hd, kv.kw + head * c.max_ctx * (hd / 8), kv.ks + head * c.max_ctx * (hd / 32), 8));
                PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            }
            float* ring = (which ? kv.vr : kv.kr) + head * s->ring_cap * hd;
            for (int64_t p = q4n; p < n; p++) PB_CUDA(ctx, cudaMemcpyAsync(ring + (size_t)(p % s->ring_cap) * hd, &tmp[(size_t)p * hd], (size_t)hd * 4, cudaMemcpyHostToDevice, ctx->stream));
            PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        }
    }
    PB_CUDA(ctx, cudaMemcpy(kv.q4n + b, &q4n, 8, cudaMemcpyHostToDevice));
    return PB_OK;
}

int pb_state_fill_kv_synth(pb_state* s, int ai, int64_t n, uint64_t seed) {
    if (!s) return PB_ERR_ARG;
    pb_ctx* ctx = s->m->ctx; const pb_cfg& c = s->m->cfg;
    PB_TRY(pb_enter(ctx));
    if (ai < 0 || ai >= s->m->n_attn || n < 0 || n > c.max_ctx) PB_FAIL(ctx, PB_ERR_ARG, "pb_state_fill_kv_synth: bad argument");
    PbKv& kv = s->kv[ai];
    const int hd = c.hd, nkv = c.n_kv;
    const int64_t q4n = c.kv_bits == 4 && n > c.kv_recent ? ((n - c.kv_recent) / 64) * 64 : 0;
    void* scr;
    PB_TRY(pb_scratch(ctx, (size_t)(n > 0 ? n : 1) * hd * 4 + 1024, &scr));
    float* f = (float*)scr;
    // element (which, b, h, p, i) of the synthetic cache = normal(seed, tensor id = (ai*2+which), index ((b*nkv+h)*max_ctx+p)*hd+i)
    for (int which = 0; which < 2; which++)
        for (int b = 0; b < s->batch; b++)
            for (int h = 0; h < nkv; h++) {
                const size_t head = (size_t)b * nkv + h;
                PB_TRY(pb_launch_synth_normal_at(ctx, f, n * hd, seed, (uint64_t)ai * 2 + which, (int64_t)(head * c.max_ctx) * hd, 1.0f));
                if (q4n > 0 && which) PB_TRY(pb_launch_kv4_pack_vt(ctx, f, q4n, hd, kv.vw + head * c.max_ctx * (hd / 8), kv.vs + head * c.max_ctx * (hd / 32), 8));
                if (q4n > 0 && !which) PB_TRY(pb_launch_kv4_pack(ctx, f, q4n * hd, kv.kw + head * c.max_ctx * (hd / 8), kv.ks + head * c.max_ctx * (hd / 32), 8));
                float* ring = (which ? kv.vr : kv.kr) + head * s->ring_cap * hd;
                for (int64_t p = q4n; p < n;) {   // contiguous runs inside the ring
                    const int64_t slot = p % s->ring_cap, run = (n - p) < (s->ring_cap - slot) ? (n - p) : (s->ring_cap - slot);
                    PB_CUDA(ctx, cudaMemcpyAsync(ring + (size_t)slot * hd, f + (size_t)p * hd, (size_t)run * hd * 4, cudaMemcpyDeviceToDevice, ctx->stream));
                    p += run;
                }
                PB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            }
    if (s->m->qsa) {
        // raw index keys of the n positions: normal(seed, tensor id 1000 + ai, index (b * max_ctx + p) * idx_hd + i); then every complete block is pooled
        PB_TRY(pb_launch_synth_normal_at(ctx, kv.ik, (int64_t)s->batch * c.max_ctx * s->m->idx_hd, seed, 1000 + (uint64_t)ai, 0, 1.0f));
        PB_TRY(qsa_pool_all(s, ai, n));
    }
    std::vector<int64_t> q((size_t)s->batch, q4n);
    PB_CUDA(ctx, cudaMemcpy(kv.q4n, q.data(), q.size() * 8, cudaMemcpyHostToDevice));
    return PB_OK;
}

int pb_kv4_pack(pb_ctx* ctx, const float* x_host, int64_t n, uint32_t* words_host, float* scales_host) {
    if (!ctx) return PB_ERR_ARG;
    if (!x_host || !words_host || !scales_host || n < 0 || n % 32) PB_FAIL(ctx, PB_ERR_ARG, "pb_kv4_pack: length %lld is not a multiple of 32", (long long)n);   // kv4.rs:13
    if (n == 0) return PB_OK;
    PB_TRY(pb_enter(ctx));
    void* scr;
    const size_t xb = (size_t)n * 4, wb = (size_t)n / 2, sb = (size_t)n / 8;
    PB_TRY(pb_scratch(ctx, xb + wb + sb + 1024, &scr));
    float* xd = (float*)scr; uint32_t* wd = (uint32_t*)((uint8_t*)scr + xb); float* sd = (float*)((uint8_t*)scr + xb + wb);
    PB_CUDA(ctx, cudaMemcpyAsync(xd, x_host, xb, cudaMemcpyHostToDevice, ctx->stream));
    PB_TRY(pb_launch_kv4_pack(ctx, xd, n, wd, sd, 0));
    PB_CUDA(ctx, cudaMemcpyAsync(words_host, wd, wb, cudaMemcpyDeviceToHost, ctx->stream));
    PB_CUDA(ctx, cudaMemcpyAsync(scales_host, sd, sb, cudaMemcpyDeviceToHost, ctx->stream));
    return pb_sync_check(ctx, "pb_kv4_pack");
}

int pb_kv4_unpack(pb_ctx* ctx, const uint32_t* words_host, const float* scales_host, int64_t n, float* x_host) {
    if (!ctx) return PB_ERR_ARG;
    if (!x_host || !words_host || !scales_host || n < 0 || n % 32) PB_FAIL(ctx, PB_ERR_ARG, "pb_kv4_unpack: length %lld is not a multiple of 32", (long long)n);
    if (n == 0) return PB_OK;
    PB_TRY(pb_enter(ctx));
    void* scr;
    const size_t xb = (size_t)n * 4, wb = (size_t)n / 2, sb = (size_t)n / 8;
    PB_TRY(pb_scratch(ctx, xb + wb + sb + 1024, &scr));
    float* xd = (float*)scr; uint32_t* wd = (uint32_t*)((uint8_t*)scr + xb); float* sd = (float*)((uint8_t*)scr + xb + wb);
    PB_CUDA(ctx, cudaMemcpyAsync(wd, words_host, wb, cudaMemcpyHostToDevice, ctx->stream));
    PB_CUDA(ctx, cudaMemcpyAsync(sd, scales_host, sb, cudaMemcpyHostToDevice, ctx->stream));
    PB_TRY(pb_launch_kv4_unpack(ctx, wd, sd, n, xd));
    PB_CUDA(ctx, cudaMemcpyAsync(x_host, xd, xb, cudaMemcpyDeviceToHost, ctx->stream));
    return pb_sync_check(ctx, "pb_kv4_unpack");
}

}  // extern "C"
