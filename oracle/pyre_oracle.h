/* CPU oracle for the Qwen-Next decode path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU arithmetic (Lyamc/pyre):
 *   src/model/gguf_q.rs          block geometry, dequant, f32 dot, QMat::matmul
 *   src/model/qwen4exp_gguf.rs   router, MoE, Gated DeltaNet, gated attention, token loop
 *   src/model/kv4.rs             4-bit KV packing
 *   src/qn_ctx.rs                rope_inv
 *   src/sampler.rs               argmax
 * Every function cites the lines it follows.  Only tests, the smoke check and the
 * cpu_baseline / reference arm of the benchmark may link or call this library; the
 * CUDA product never does.
 *
 * Parity status: the reference cannot be compiled in this environment (Rust, no
 * toolchain) and its tree holds no golden vectors for dequant/GEMV/router/DeltaNet/
 * attention, so those parts are "parity unpinned" against the reference binary.  What
 * IS pinned: dequant of all four block formats bit-for-bit against gguf-py 0.19
 * (the tool the reference's authors checked against), and the kv4 round-trip
 * properties asserted by src/model/kv4.rs:52-104.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids, gguf_q.rs:23-29 */
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_Q4_0 = 2, ORC_Q5_0 = 6, ORC_Q3_K = 11, ORC_Q5_K = 13, ORC_Q8_0 = 8, ORC_Q4_K = 12, ORC_Q6_K = 14, ORC_IQ2_XXS = 16, ORC_Q2_0 = 42, ORC_IQ2_XS = 17, ORC_IQ3_XXS = 18, ORC_IQ4_NL = 20, ORC_IQ3_S = 21, ORC_IQ2_S = 22, ORC_IQ4_XS = 23, ORC_IQ1_M = 29, ORC_BF16 = 30 };

/* A quantized row-major matrix (QMat, gguf_q.rs:199-215).  data == NULL means the
 * matrix is synthetic: row bytes are generated on demand from (seed, tid). */
typedef struct {
    int32_t type;
    int64_t rows, cols;
    const uint8_t* data;
    uint64_t seed, tid;
} orc_mat;

int orc_type_geom(int type, int* elems, int* bytes);           /* QType::geom :33-41 */
int64_t orc_row_bytes(int type, int64_t cols);                 /* QType::row_bytes :42 */
int orc_dequant(int type, const uint8_t* x, int64_t n, float* y);  /* dequant :67-166 */
float orc_dot(const float* a, const float* b, int64_t n);      /* dot_avx2 :176-197 */
void orc_mat_row_raw(const orc_mat* m, int64_t r, uint8_t* out);
void orc_mat_row(const orc_mat* m, int64_t r, float* y);       /* QMat::row :210 */
void orc_matmul(const orc_mat* m, const float* x, int t, float* y);  /* QMat::matmul :217-242 (t<16 branch) */
/* the reference's int8 CPU fast path, qdot.rs:15-30 (quantize), :278-286 (IQ3_S row_dot), :1046-1052 (its test's expected value) */
void orc_q8_quantize(const float* x, int64_t n, int8_t* q, float* d);
float orc_q8_dot_dequant(int type, const uint8_t* row, int64_t n, const int8_t* q, const float* d);
float orc_row_dot_q8_iq3s(const uint8_t* row, int64_t n, const int8_t* q, const float* d);
int orc_threads(void);
void orc_set_threads(int n);   /* threads of the row-parallel loops from now on */

/* Seeded synthetic block fields (see the generator section of pyre_oracle.c). */
void orc_synth_rows(int type, uint64_t seed, uint64_t tid, int64_t cols, int64_t r0, int64_t nrows, uint8_t* out);
void orc_synth_normal(uint64_t seed, uint64_t tid, int64_t i0, int64_t n, float sigma, float* out);

/* router: top_k qwen4exp_gguf.rs:3132-3139 with a canonical order */
void orc_top_k(const float* r, int n, int k, int32_t* idx, float* w);

/* kv4.rs:12-42 */
void orc_kv4_pack(const float* x, int64_t n, uint32_t* w, float* sc);
float orc_kv4_get(const uint32_t* w, const float* sc, int64_t i);
void orc_rope_inv(int n_rot, float base, float* inv);          /* qn_ctx.rs:164-170, unscaled */
float orc_rope_inv_yarn(int n_rot, float base, int64_t ctx_train, int64_t ctx, float* inv);   /* qn_ctx.rs:160-186; returns mscale */
uint32_t orc_argmax(const float* v, int64_t n);                 /* sampler.rs:142-148 */

/* ---- model ---- */
typedef struct {
    int32_t n_layers, d, hc, hc_lr, n_head, n_kv, hd, n_rot;
    float rope_base, eps;
    int32_t n_exp, top_k, ff_exp, ff_sh;
    int32_t lin_nk, lin_nv, lin_dk, lin_dv, conv_k, full_every;
    int32_t vocab, max_ctx;
    int32_t kv_bits;      /* 0 = f32 KV, 4 = 4-bit for positions older than the recent window */
    int32_t kv_recent;    /* f32 window kept in front of the packed region (reference default 1024) */
} orc_cfg;

/* tensor roles; identical numbering to pb_role in include/pyre_b200.h */
enum {
    ORC_R_TOKEN_EMBD = 0, ORC_R_OUTPUT, ORC_R_OUT_NORM,
    ORC_R_ATTN_NORM, ORC_R_FFN_NORM,
    ORC_R_ATTN_Q, ORC_R_ATTN_K, ORC_R_ATTN_V, ORC_R_ATTN_O, ORC_R_ATTN_Q_NORM, ORC_R_ATTN_K_NORM,
    ORC_R_LIN_QKV, ORC_R_LIN_Z, ORC_R_LIN_BETA, ORC_R_LIN_ALPHA, ORC_R_LIN_OUT,
    ORC_R_LIN_A, ORC_R_LIN_DT, ORC_R_LIN_CONV, ORC_R_LIN_NORM,
    ORC_R_ROUTER, ORC_R_EXP_GATE, ORC_R_EXP_UP, ORC_R_EXP_DOWN,
    ORC_R_SH_GATE, ORC_R_SH_UP, ORC_R_SH_DOWN, ORC_R_SH_GATE_INP,
    ORC_R_HCA_NORM, ORC_R_HCA_DOWN, ORC_R_HCA_UP, ORC_R_HCA_INJECT,
    ORC_R_HCF_NORM, ORC_R_HCF_DOWN, ORC_R_HCF_UP, ORC_R_HCF_INJECT,
    ORC_R_OUT_HC_NORM, ORC_R_OUT_HC_DOWN, ORC_R_OUT_HC_UP,
    ORC_R_IDX_Q, ORC_R_IDX_K, ORC_R_IDX_Q_NORM, ORC_R_IDX_K_NORM,   /* QSA indexer of an attention layer (Mixer::Attn idx, :501) */
    ORC_R_MTP_FC_E, ORC_R_MTP_FC_H, ORC_R_MTP_PRE_E, ORC_R_MTP_PRE_H,   /* input stage of the MTP drafter (src/model/mtp.rs:186-195), global */
    /* per-layer n-gram embeddings (Ple :33, tensors :505, 512): the table (global), per layer key / value projections, three norm vectors, the conv taps */
    ORC_R_PLE_TAB, ORC_R_PLE_KEY, ORC_R_PLE_VALUE, ORC_R_PLE_NORM_KEY, ORC_R_PLE_NORM_QUERY, ORC_R_PLE_NORM_CONV, ORC_R_PLE_CONV,
    ORC_R_COUNT
};

typedef struct orc_model orc_model;
typedef struct orc_state orc_state;

orc_model* orc_model_new(const orc_cfg* cfg);
void orc_model_free(orc_model* m);
/* n-gram embedding geometry (Cfg ple_* :477-480): ngram, heads per n-gram size, conv taps, the end-of-sequence id that cuts a context,
 * the width of a table row; mult[ngram], off[nh], vocab[nh] with nh = (ngram - 1) * per_gram.  Layers that hold ORC_R_PLE_KEY use it. */
void orc_model_set_ple(orc_model* m, int ngram, int per_gram, int conv_k, uint32_t eos, int dim, const uint64_t* mult, const uint64_t* off, const uint64_t* vocab);
/* table rows of a token whose context (the token first, then its predecessors, -1 = none) is ctx[ngram]: rows[nh] (ple_rows :1390-1407) */
void orc_ple_hash(const orc_model* m, const int64_t* ctx, int64_t* rows);
/* ple :1409-1434 for one token at position pos, given its projected key [streams * d] and value [d]: updates xt [streams * d] and stores the
 * token's normalized row at nrm_all[pos] (rows of earlier positions are read from the same array) */
void orc_ple_token(const orc_model* m, int il, float* nrm_all, const float* key, const float* val, float* xt, int64_t pos);
void orc_model_set_indexer(orc_model* m, int budget, int ratio, int n_head, int head_dim);   /* QSA geometry, Cfg :24-25 */
void orc_model_set_ctx_train(orc_model* m, int64_t ctx_train);   /* YaRN when cfg.max_ctx > ctx_train (Model::load :490-517) */
int orc_model_set_mat(orc_model* m, int layer, int role, const orc_mat* mat);   /* layer -1 = global */
int orc_model_set_vec(orc_model* m, int layer, int role, const float* v, int64_t n);
orc_state* orc_state_new(const orc_model* m);
void orc_state_free(orc_state* s);
/* pre-fill attention layer ai's KV with n positions of f32 rows [n][n_kv*hd] (packed per kv_bits) */
int orc_state_fill_kv(orc_state* s, int ai, const float* k, const float* v, int64_t n);
int orc_state_set_pos(orc_state* s, int64_t pos);
/* forward_inner qwen4exp_gguf.rs:2087-2157: feed t tokens, logits of the last one */
int orc_forward(const orc_model* m, orc_state* s, const uint32_t* ids, int t, float* logits);
/* per-step margins for near-tie classification: top-2 logit margin, min 10th/11th router margin */
void orc_last_margins(const orc_state* s, float* logit_margin, float* router_margin);
float orc_last_qsa_margin(const orc_state* s);
/* final multi-stream residual rows [t][max(hc,1) * d] of the tokens of the last orc_forward call (what the MTP drafter pairs with the next token) */
int orc_last_residual(const orc_state* s, float* out, int64_t cap_floats);
/* MTP drafter (src/model/mtp.rs): `dm` is a model of ONE attention layer with hyper-connections and a MoE block, whose global slots
 * also hold ORC_R_MTP_*; its OUT_HC_* tensors are the final mixer and its OUTPUT the draft-vocabulary head.  One cell at rope position
 * `pos`: R = the main model's residual row of position pos [hc*d], emb = the embedding row of token pos + 1.  The cell's K/V go into
 * `ds` at row pos.  full = 0: K/V only (catch_up :172-175); full = 1: the whole step (step :184-236) attending to the cells
 * max(c0, pos - window + 1) .. pos, s_out [d] = the final mixer's output for the head, rr_out [hc*d] = the drafter's residual. */
void orc_mtp_cell(const orc_model* dm, orc_state* ds, const float* R, const float* emb, int64_t pos, int64_t c0, int window, int full, float* s_out, float* rr_out);

/* ---- layer-level entry points (same arithmetic as inside orc_forward) ---- */
/* MoE block: ffn :1675-1684 + routed (f32 branch) :1721-1793.  x [t][d] -> y [t][d].
 * sel (optional) receives the top_k expert ids per token, selw the weights. */
void orc_moe(const orc_cfg* c, const orc_mat* router, const orc_mat* gate_e, const orc_mat* up_e, const orc_mat* down_e,
             const orc_mat* sh_gate, const orc_mat* sh_up, const orc_mat* sh_down, const float* sh_gate_inp,
             const float* x, int t, float* y, int32_t* sel, float* selw);
/* linear_core :1624-1673 for one sequence: proj = qkv[t][ch], z[t][nv*dv], beta[t][nv], alpha[t][nv];
 * conv_state [(K-1)][ch] oldest first, ssm [nv][dk][dv]; out [t][nv*dv]. */
void orc_linear_core(const orc_cfg* c, const float* qkv, const float* z, const float* beta, const float* alpha,
                     const float* a, const float* dt, const float* conv_w, const float* norm_w,
                     float* conv_state, float* ssm, int t, float* out);
/* attn_core :1558-1615 (dense) for one new token at position pos against a cache that already
 * holds pos positions.  kc/vc: f32 rows [pos+1][n_kv*hd] (the new row is appended at index pos by
 * this call).  If kw != NULL the first q4n positions are read from the kv4-packed arrays instead. */
void orc_attn_core(const orc_cfg* c, const float* qf, const float* kf, const float* vf,
                   const float* qn, const float* kn, const float* rope_inv,
                   float* kc, float* vc, int64_t pos,
                   const uint32_t* kw, const float* ks, const uint32_t* vw, const float* vs, int64_t q4n,
                   float* att);
/* the same over a list of key positions (ascending; NULL = all positions <= pos): the QSA sparse branch, :1605-1609 */
void orc_attn_core_sel(const orc_cfg* c, const float* qf, const float* kf, const float* vf,
                       const float* qn, const float* kn, const float* rope_inv,
                       float* kc, float* vc, int64_t pos,
                       const uint32_t* kw, const float* ks, const uint32_t* vw, const float* vs, int64_t q4n,
                       const int64_t* ps, int64_t nps, float* att);
/* QSA indexer pieces (attn_core :1565-1599): pooled key of block b; the blocks a query at `pos` attends to */
void orc_qsa_pool(const orc_cfg* c, int ratio, int ihd, const float* ik, const float* ikn, const float* rope_inv, int64_t b, float* out);
int orc_qsa_select(const orc_cfg* c, int budget, int ratio, int inh, int ihd, const float* iq_raw, const float* iqn, const float* rope_inv,
                   const float* ib, int64_t pos, int32_t* blocks, float* margin);

#ifdef __cplusplus
}
#endif
