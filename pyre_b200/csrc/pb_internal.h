// Internal definitions shared by the .cu files of libpyre_b200.so (not part of the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <map>
#include <string>
#include <vector>

#include "../../include/pyre_b200.h"

struct pb_ctx {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;   // the stream every kernel of this context is launched on
    int* dev_status = nullptr;       // device status word (see PB_DEV_* in pb_common.cuh)
    uint8_t* xh_buf = nullptr;       // PB_XH_BYTES: activation fragments of the tensor-core GEMM (pb_gemmh.cu)
    int* host_status = nullptr;      // pinned host mirror, filled by an async copy before each sync
    int sm_count = 148;
    int max_smem_optin = 0;
    std::string err;
    // grow-only device scratch for host-buffer entry points
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    uint64_t kernels_launched = 0;
    // expert-parallel group (pb_ep.cu); ep_comm is an ncclComm_t
    // programmatic dependent launch is used only inside the token step, where every stream op is ours
    bool use_pdl = true;
    bool step_pdl = true;    // the fused step kernel takes part in the dependent-launch chain (PYRE_B200_STEP_PDL=0: it does not)
    int pdl_scope = 0;       // > 0 while run_step is issuing launches
    bool pdl_chain = false;  // the previous op on the stream was one of our kernels
    void* ep_comm = nullptr;
    int ep_rank = 0, ep_world = 1;
    // largest dynamic shared-memory size set so far per kernel function: the attribute belongs to the device's
    // copy of the function, so the cache lives in the context, not in the process
    std::map<const void*, size_t> smem_cfg;
    // tracing: stamp slots handed to the launches of the streaming kernels while enabled (pb_ctx_stamps_enable)
    unsigned long long* stamps = nullptr; int stamp_slots = 0, stamp_next = 0;
    std::vector<int> stamp_ids;   // kernel id (PB_K_*) per handed-out slot
    unsigned long long* grid_sync = nullptr;   // fused step kernel: [0] arrival counter of its grid barriers, [1] counter value at launch
    unsigned long owner_thread = 0;   // pthread id of the creating thread (checked when PYRE_B200_CHECK_THREAD=1)
    bool check_thread = false;
};
// Every extern "C" entry point that touches the device calls this first: makes the context's GPU current
// (a process may hold contexts on several GPUs) and, in the debug mode, verifies the calling thread.
int pb_enter(pb_ctx* ctx);
// In-kernel peer exchange of a sharded state (pb_ep.cu): every rank owns one block of device memory with the same layout,
// mapped into all ranks of the node (CUDA IPC); kernels store straight into the peers' blocks and hand over with
// sequence-numbered flags (bounded waits, a time-out sets the device status word).
#define PB_EP_MAX_WORLD 16
struct PbEpExch {
    int rank, world;
    float* peer_xg[PB_EP_MAX_WORLD];                  // each rank's gathered-row buffer [moe_t][ldg]
    unsigned long long* peer_flags[PB_EP_MAX_WORLD];  // each rank's flag array [2 kinds][world]: flags[kind][src] = last sequence number src finished
    const unsigned long long* seq_base;               // this rank's sequence base: advanced by 2 * n_layers per step
    unsigned int spin_limit;                          // polls (of about 0.2 us) before a wait gives up
    unsigned long long* wait_ns;                      // time spent in hand-shakes, summed over the world's CTAs (or null)
    int* status;
};
struct PbEpSymm {
    void* local = nullptr; size_t bytes = 0;
    void* peer[PB_EP_MAX_WORLD] = {};                 // peer[rank] == local
};
int pb_ep_symm_alloc(pb_ctx* ctx, size_t bytes, PbEpSymm* out);   // collective over the expert-parallel group
void pb_ep_symm_free(pb_ctx* ctx, PbEpSymm* m);
// rows[0 .. n) (floats) of this rank -> every rank's gathered-row buffer at float offset dst_off; then exchange `exch` of kind 0 is
// announced to every rank and awaited from every rank
int pb_launch_ep_push_rows(pb_ctx* ctx, const PbEpExch& x, const float* rows, int64_t n, int64_t dst_off, int exch);
// announce exchange `exch` of `kind` to every rank (this rank's stores into their memory are complete) and await theirs
int pb_launch_ep_signal_wait(pb_ctx* ctx, const PbEpExch& x, int kind, int exch);
int pb_ep_allreduce(pb_ctx* ctx, float* buf, size_t n);
int pb_ep_allgather(pb_ctx* ctx, const float* send, float* recv, size_t n);
int pb_ep_reduce_scatter(pb_ctx* ctx, const float* send, float* recv, size_t n);

struct pb_qmat {
    pb_ctx* ctx = nullptr;
    int type = 0;
    int64_t rows = 0, cols = 0;
    int64_t row_bytes = 0;
    uint8_t* data = nullptr;   // device, 256-byte aligned, padded by >= 256 bytes past the last row
    // IQ3_S only: the same weights re-coded as PB_T_IQ3S_N4 (4-bit codes, decoded with two logic operations per
    // eight weights instead of a codebook walk); the streaming kernels read this copy, `data` stays for
    // pb_qmat_read / dequant / embedding rows and the tensor-core GEMM
    uint8_t* rdata = nullptr;
    int64_t r_row_bytes = 0;
    size_t nbytes = 0;         // rows * row_bytes
    bool owns = true;          // false for row-range views into another matrix
};

#define PB_FAIL(ctx, code, ...)                                   \
    do {                                                          \
        char _b[512];                                             \
        snprintf(_b, sizeof _b, __VA_ARGS__);                     \
        if (ctx) (ctx)->err = _b;                                 \
        return (code);                                            \
    } while (0)

#define PB_CUDA(ctx, call)                                                                                   \
    do {                                                                                                     \
        cudaError_t _e = (call);                                                                             \
        if (_e != cudaSuccess) PB_FAIL(ctx, _e == cudaErrorMemoryAllocation ? PB_ERR_OOM : PB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(_e)); \
    } while (0)

#define PB_TRY(call)                 \
    do {                             \
        int _s = (call);             \
        if (_s != PB_OK) return _s;  \
    } while (0)

// Kernel launch on the context's stream; inside the token step consecutive kernels are chained with
// programmatic stream serialization (every such kernel calls pb_pdl_wait before touching dependent data).
template <typename K, typename... A>
static inline void pb_launch_k(pb_ctx* ctx, K kern, dim3 grid, dim3 block, size_t smem, A... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = (ctx->use_pdl && ctx->pdl_scope > 0 && ctx->pdl_chain) ? 1 : 0;
    ctx->pdl_chain = ctx->pdl_scope > 0;
    cudaLaunchKernelEx(&cfg, kern, args...);   // errors are picked up by cudaGetLastError at the call site
}

// Raise the kernel's dynamic shared-memory limit on this context's device when `smem` exceeds what was set before.
template <typename K>
static inline int pb_ensure_smem(pb_ctx* ctx, K kern, size_t smem) {
    const void* key = reinterpret_cast<const void*>(kern);
    auto it = ctx->smem_cfg.find(key);
    if (it != ctx->smem_cfg.end() && it->second >= smem) return PB_OK;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { char b[256]; snprintf(b, sizeof b, "cudaFuncSetAttribute(%zu bytes of shared memory): %s", smem, cudaGetErrorString(e)); ctx->err = b; return PB_ERR_CUDA; }
    ctx->smem_cfg[key] = smem;
    return PB_OK;
}

// next stamp slot (PB_STAMP_WORDS words), or null when tracing is off or the slots are used up; kernel_id is recorded on the host
unsigned long long* pb_stamp_slot(pb_ctx* ctx, int kernel_id);
enum { PB_K_GEMVQ = 1, PB_K_ROUTER = 2, PB_K_EXPERT_GU = 3, PB_K_EXPERT_DOWN = 4, PB_K_DELTANET = 5, PB_K_ATTN = 6, PB_K_STEP = 7 };

int pb_scratch(pb_ctx* ctx, size_t bytes, void** out);
int pb_sync_check(pb_ctx* ctx, const char* who);

// pb_dequant.cu
int pb_launch_dequant(pb_ctx* ctx, int type, const uint8_t* w, int64_t nsteps, float* out);
int pb_launch_synth(pb_ctx* ctx, int type, uint8_t* w, int64_t nblocks, uint64_t seed, uint64_t tid, int64_t block0 = 0);
int pb_launch_synth_normal(pb_ctx* ctx, float* out, int64_t n, uint64_t seed, uint64_t tid, float sigma);
int pb_launch_synth_normal_at(pb_ctx* ctx, float* out, int64_t n, uint64_t seed, uint64_t tid, int64_t i0, float sigma);

// pb_gemv.cu
// n-gram embedding hash (Cfg ple_*, src/model/qwen4exp_gguf.rs:477-480): nh = (ngram - 1) * per_gram heads
struct PbPleHash { int ngram, per_gram, nh; uint32_t eos; uint64_t mult[8], off[32], vocab[32]; };
int pb_launch_ple_rows(pb_ctx* ctx, const PbPleHash& hp, const uint32_t* ids, const int64_t* posv, int t, int window, uint32_t* tok_hist, int64_t max_ctx, const int64_t* base, uint32_t* rows_out);
int pb_launch_ple_gate(pb_ctx* ctx, const float* key, int64_t ldk, const float* val, int64_t ldv, const float* x, int64_t ldx, const float* nk, const float* nq, const float* nc,
                       float* gated, float* ring, int R, const int64_t* posv, int t, int window, int d, int streams, float eps);
int pb_launch_ple_conv(pb_ctx* ctx, const float* gated, const float* ring, int R, const float* conv, int K, int dil, const int64_t* posv, int t, int window, const int64_t* base, float* x, int64_t ldx, int w);

int pb_launch_ck_restore(pb_ctx* ctx, const float* const* tab, float* const* live, int n_lin, int stride, int idx, int64_t conv_n, int64_t ssm_n);
struct PbGemvArgs {
    const uint8_t* w;   // first row of the matrix (16-byte aligned)
    const uint8_t* wr = nullptr;   // the same rows in the re-coded form (pb_qmat::rdata), or null
    int type;
    int64_t rows;
    int cols;
    const float* x;     // [t][ldx]
    int64_t ldx;
    int t;              // 1..16 columns
    float* y;           // [t][ldy]
    int64_t ldy;
};
int pb_launch_gemv(pb_ctx* ctx, const PbGemvArgs& a);
int pb_launch_repack_iq3s(pb_ctx* ctx, const uint8_t* src, uint8_t* dst, int64_t nblocks);

// pb_gemvq.cu: integer-core GEMV over up to four same-shaped-row matrices with a fused
// activation prologue and an optional accumulate (residual) epilogue.
enum { PB_ACT_PLAIN = 0,   // x as given
       PB_ACT_NORM = 1,    // rms(x) * norm_w over the whole row
       PB_ACT_GNORM = 2,   // per head of head_dim: rms(x) * norm_w[head_dim], times sigmoid(z)
       PB_ACT_PREQ = 3 };  // activations already split into int8 levels (xq_in)
struct PbGemvSegArg { const uint8_t* w; int64_t rows; int64_t yoff; const uint8_t* wr; };   // wr: re-coded rows (pb_qmat::rdata) or null
#define PB_XH_BYTES (((size_t)16 << 20) + 8192)   // operand buffer of the tensor-core GEMMs: t * cols * 4 bytes + a header (e.g. 1024 tokens of 4096 columns)
struct PbGemvQArgs {
    int type, cols, nseg;
    PbGemvSegArg seg[4];
    const float* x; int64_t ldx; int t;
    float* y; int64_t ldy;
    int mode; const float* norm_w; const float* z; int64_t ldz; int head_dim; float eps;
    const uint32_t* xq_in;
    int accumulate;
    int exact;   // keep the kernels whose weights enter the products exactly (decode steps feed recurrent state); 0 lets 16+ tokens use the tcgen05 GEMM, whose f16 weights carry one rounding
};
struct PbGemvQSeg { const uint8_t* w; int rows; int chunk0; int yoff; };
struct PbGemvQParams {
    PbGemvQSeg seg[4];
    int nseg;
    int row_bytes, bpr, rows_per_chunk, nchunks;
    uint32_t stage_bytes, tab_bytes;
    int rep;
    const float* x; int64_t ldx; int t;
    float* y; int64_t ldy;
    int mode; const float* norm_w; const float* z; int64_t ldz; int head_dim; float eps;
    const uint32_t* xq_in;
    const uint8_t* xh_in; const float* xinv_in;   // pb_gemmh.cu: f16 fragments and prescale inverses made by its prep kernel
    int accumulate;
    int* status;
    unsigned long long* stamps;
};
bool pb_gemvq_supported(int type, int cols);
int pb_launch_gemvq(pb_ctx* ctx, const PbGemvQArgs& a);
// pb_gemmh.cu: tensor-core path for 3..16 columns of IQ3_S weights
bool pb_gemmh_supported(int type, int cols, int t);
int pb_launch_gemmh(pb_ctx* ctx, const PbGemvQArgs& a);
// pb_gemvi.cu: int8 tensor-core path for one and two columns of IQ3_S weights that have a re-coded copy
bool pb_gemvi_supported(int type, int cols, int t);
int pb_launch_gemvi(pb_ctx* ctx, const PbGemvQArgs& a);
// pb_gemmtc.cu: tcgen05 path for 16 and more columns of IQ3_S weights that have a re-coded copy
bool pb_gemmtc_supported(int type, int cols, int t);
int pb_launch_gemmtc(pb_ctx* ctx, const PbGemvQArgs& a);
int pb_gemmtc_min_tokens();            // tokens from which the dispatchers prefer this kernel (measured crossover)
int pb_gemmtc_max_tokens(int cols);   // tokens one launch accepts (operand buffer), a multiple of 128

// ---------------------------------------------------------------- pb_moe.cu
#define PB_MAX_TOPK 16
struct PbRouterParams {
    const float* x; int64_t ldx; int t; int cols;
    const float* norm_w; float eps;          // null: x is already normalized
    const float* router;                      // f32 [n_exp][cols]
    const float* sh_gate_inp;                 // f32 [cols] or null
    int n_exp;
    float* logits; int64_t ldl;               // [t][ldl >= n_exp + 1], entry n_exp = shared-gate logit
    uint32_t* xq_out;                         // [t][pb_xq_words(cols)] int8-split activations
    // phase 0: everything.  Sharded tokens split it around the all-gather: phase 1 = logits of the local
    // tokens plus a raw copy of their rows into xcopy (row stride ldl); phase 2 = split + routing of all
    // gathered tokens (no GEMV)
    int phase; float* xcopy;
    float* zero; int64_t zero_n;              // phases 0 and 2: zero_n floats (a multiple of 4) cleared for the expert kernels (expert parallelism)
    unsigned long long* stamps;
    // phase 1 with a peer exchange (device copy of the descriptor): rows and logits are also stored into every rank's
    // gathered buffer at float offset peer_off, and the last CTA hand-shakes exchange number exch_idx with all ranks
    const PbEpExch* exch; int exch_idx; int64_t peer_off;
};
struct PbRouteParams {
    const float* logits; int64_t ldl; int t, n_exp, top_k;
    int e_lo, e_hi;                           // experts held by this GPU
    int* sel_e; float* sel_w;                 // [t][top_k], ascending expert id
    int* n_used; int* used_e; int* used_off;  // distinct local experts, entry offsets [n_used + 1]
    int* ent_tok; int* ent_slot; float* ent_w;
};
struct PbExpertParams {
    const int* n_used; const int* used_e; const int* used_off;
    const int* ent_tok; const int* ent_slot; const float* ent_w;
    const uint32_t* xq;                       // gate/up: int8-split activations per token
    const uint8_t* w_a; const uint8_t* w_b;   // gate/up: gate_exps, up_exps; down: down_exps, unused
    const uint8_t* sh_a; const uint8_t* sh_b; // shared expert counterparts
    float* h; float* h_sh;                    // hidden [entry][ff], [t][ff_sh]
    uint32_t* hq;                             // down, several tokens: int8-split hidden vectors [t * top_k + t][pb_xq_words(ff)], else null
    float* part; float* part_sh;              // down: [t][top_k][d], [t][d]
    float* const* part_tok;                   // down, peer exchange: part_tok[token] = [top_k][d] block in the memory of the token's owner (else null)
    int rows_e, rows_sh, has_shared, t, top_k, n_exp, e_base;
    int sh_tok0, sh_ntok;                     // tokens [sh_tok0, sh_tok0 + sh_ntok) get the shared expert here
    int bpr, row_bytes, rows_per_chunk; uint32_t stage_bytes, tab_bytes; int rep;
    int nx;                                   // activation-level vectors of a chunk's first nx entries ride along with its weights
    int* status;
    unsigned long long* stamps;
};
struct PbCombineParams {
    const float* part; const float* part_sh; const float* logits; int64_t ldl;
    int t, d, top_k, n_exp;
    float* y; int64_t ldy; int accumulate;
    // peer exchange (device copy of the descriptor): before reading `part`, announce exchange exch_idx (kind 1: this
    // rank's expert rows are stored in their owners' memory) and wait for every rank's announcement
    const PbEpExch* exch; int exch_idx;
};
int pb_launch_router(pb_ctx* ctx, const PbRouterParams& p, const PbRouteParams& rp, unsigned int* ticket);
int pb_launch_expert_gu(pb_ctx* ctx, const PbExpertParams& p, int type, int cols);
int pb_launch_expert_down(pb_ctx* ctx, const PbExpertParams& p, int type, int cols, const PbCombineParams* cp = nullptr, unsigned int* ticket = nullptr);
int pb_launch_moe_combine(pb_ctx* ctx, const PbCombineParams& p);

// ---------------------------------------------------------------- pb_deltanet.cu
struct PbDeltaParams {
    const float* proj; int64_t ldp;           // [batch][qkv | z | beta | alpha]
    const float* conv_w; const float* a; const float* dt;
    float* conv;                              // [batch][conv_k slots][ch] ring
    float* ssm;                               // [batch][nv][dk][dv]
    const int64_t* pos;                       // [batch]
    float* out; int64_t ldo;                  // [batch][nv*dv] readout before the gated norm
    int nk, nv, dk, dv, conv_k, batch;
    unsigned long long* stamps;
};
int pb_launch_deltanet(pb_ctx* ctx, const PbDeltaParams& p);
bool pb_deltanet_seq_supported(const PbDeltaParams& p);
// rollback checkpoints of a window: the state as it is after token j (conv ring and ssm of one sequence), or null
struct PbDeltaCk { float* conv[8]; float* ssm[8]; };
int pb_launch_deltanet_seq(pb_ctx* ctx, const PbDeltaParams& p, int T, const PbDeltaCk* ck = nullptr);   // T consecutive tokens of sequence 0, state kept in registers

// ---------------------------------------------------------------- pb_attn.cu
struct PbAttnParams {
    const float* proj; int64_t ldp;           // [batch][q|gate per head (n_head*2*hd) | k | v]
    const float* qn; const float* kn; const float* rope_inv;
    int n_rot; float eps;
    int n_head, n_kv, hd;
    uint32_t* kw; float* ks; uint32_t* vw; float* vs;   // packed [batch][n_kv][max_ctx][hd/8], scales [..][hd/32]
    float* kr; float* vr;                                // f32 ring [batch][n_kv][ring_cap][hd]
    int64_t max_ctx; int64_t ring_cap; int kv_bits; int kv_recent;
    const int64_t* pos; int64_t* q4n;                    // [batch]
    float* part_ml; float* part_acc; int nsplit;
    int nsplit_packed;                                   // splits [0, nsplit_packed) walk the packed positions on the tensor cores
    float ring_weight;                                   // cost of a scalar tile of 8 f32 positions in packed tiles of 32 (split shares)
    float* att; int64_t lda;                             // [batch][n_head*hd]
    int batch;
    // window: the `batch` entries are consecutive tokens of sequence 0 (a prefill chunk): they share its cache; the append
    // kernel only writes the f32 ring, pb_launch_kv_pack then moves the packed boundary once for the whole window and
    // keeps the previous boundary in q4n[1]; token j treats as packed what a token-by-token run would have packed by then
    int window;
    // QSA block-sparse attention (pb_qsa.cu): when qsa_on[b] is set, sequence b attends only to the positions whose bit is
    // set in qsa_mask[b * qsa_ld + position / 32]; null = dense
    const uint32_t* qsa_mask; int64_t qsa_ld; const int* qsa_on;
};
// pb_qsa.cu: the indexer of QSA block-sparse attention
struct PbQsaParams {
    const float* iproj; int64_t ldi;        // [batch][idx_nh * idx_hd raw query heads | idx_hd raw key]
    const float* iqn; const float* ikn; const float* rope_inv; int n_rot; float eps;
    int inh, ihd, ratio, budget;
    float* ik; float* ib;                   // raw keys [batch][max_ctx][idx_hd], pooled block keys [batch][nb_cap][idx_hd]
    int64_t max_ctx, nb_cap;
    const int64_t* pos;                     // [batch]
    float* scores;                          // [batch][nb_cap]
    uint32_t* mask; int64_t mask_ld; int* sparse;   // out: see PbAttnParams
    int batch;
    int shared_seq;                         // the `batch` entries are tokens of sequence 0 (they share its keys)
};
int pb_launch_qsa_append(pb_ctx* ctx, const PbQsaParams& p);   // store the raw key, pool the block the token completes
int pb_launch_qsa_select(pb_ctx* ctx, const PbQsaParams& p);   // block scores and the position mask (sparse[b] = 0 in the dense range)
int pb_launch_qsa_pool_all(pb_ctx* ctx, const PbQsaParams& p, int64_t nblk);   // pooled keys of blocks [0, nblk) of every sequence
// pb_mtp.cu: pieces of the MTP drafter around its layer
int pb_launch_mtp_keep(pb_ctx* ctx, const float* x, int64_t ldx, const int64_t* pos, int t, float* ring, int cap, int w);
int pb_launch_mtp_input(pb_ctx* ctx, const float* e, const float* pre_e, const float* R, const float* pre_h, float* en, float* hn, int d, int w, float eps);
int pb_launch_mtp_join(pb_ctx* ctx, const float* h2, const float* e2, float* x, int d, int w);
int pb_launch_mtp_mask(pb_ctx* ctx, uint32_t* mask, int* on, int64_t lo, int64_t pos);
int pb_launch_mtp_best(pb_ctx* ctx, const float* lg, int n, uint32_t* out);
int pb_launch_kv_append(pb_ctx* ctx, const PbAttnParams& p);
int pb_launch_attn(pb_ctx* ctx, const PbAttnParams& p);
int pb_launch_kv_pack(pb_ctx* ctx, const PbAttnParams& p);   // window mode, after pb_launch_kv_append
int pb_launch_kv4_pack(pb_ctx* ctx, const float* x, int64_t n, uint32_t* w, float* sc, int bias);   // bias 0: kv4.rs nibbles; 8: cache form
int pb_launch_kv4_pack_vt(pb_ctx* ctx, const float* x, int64_t npos, int hd, uint32_t* w, float* sc, int bias);   // position-transposed V words
int pb_launch_kv4_unpack(pb_ctx* ctx, const uint32_t* w, const float* sc, int64_t n, float* x);

// ---------------------------------------------------------------- pb_hc.cu
struct PbHcParams {
    const float *norm, *down, *up, *inject;   // [hc*d], [lr][hc*d], [hc*d][lr], [hc][hc*d] or null
    int d, hc, lr; float eps;
    float *xn, *gate, *lo, *inj;               // work rows per token: [hc*d], [hc*d], [lr], [hc]
};
int pb_launch_hc_mix(pb_ctx* ctx, const PbHcParams& p, const float* x, int t, float* mixed);      // x [t][hc*d] -> mixed [t][d], p.inj [t][hc]
int pb_launch_hc_combine(pb_ctx* ctx, const PbHcParams& p, float* x, const float* out, int t);   // x [t][hc*d] += out [t][d] * 2 sigmoid(p.inj)
int pb_launch_hc_spread(pb_ctx* ctx, const float* e, float* x, int t, int d, int hc);

// ---------------------------------------------------------------- pb_misc.cu
int pb_launch_embed(pb_ctx* ctx, int type, const uint8_t* w, int64_t rows, int cols, const uint32_t* ids, int t, float* out, int64_t ldo);
int pb_launch_argmax(pb_ctx* ctx, const float* logits, int64_t ld, int n, int t, unsigned long long* keys);
int pb_launch_window_pos(pb_ctx* ctx, int64_t* pos, int64_t* wpos, int t, int advance);
int pb_launch_advance(pb_ctx* ctx, int64_t* pos, int t, unsigned long long* keys, uint32_t* next, uint32_t* ids, uint32_t* trace, int64_t* trace_len, int64_t trace_cap,
                      unsigned long long* ep_seq = nullptr, unsigned long long ep_seq_step = 0);
