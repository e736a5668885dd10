/* pyre_b200 -- C ABI of the B200-native Qwen-Next decode engine.
 *
 * Drop-in boundary for the model surface that the reference's engine loop calls
 * (Lyamc/pyre: src/engine_qn.rs, src/spec.rs, src/qn_cli.rs).  The reference has no FFI
 * today; each entry point below names the Rust item it replaces (file:line inside the
 * reference project).  Plain pointers and sizes only; no C++ or torch types.
 *
 * Conventions
 *   - Every function returns a pb_status (0 = PB_OK).  Nothing aborts, traps or unwinds
 *     across this boundary; pb_last_error(ctx) gives the text of the last failure.
 *     (The reference panics on impossible states and its worker turns the panic into an
 *     error event, src/engine_qn.rs:56-59.)
 *   - A context is thread-affine: create it and make every call on one OS thread, as
 *     the reference's single "qn-worker" thread does (src/engine_qn.rs:13-17).
 *   - Pointers named *_host are caller-owned host memory; *_dev are device pointers on
 *     the context's GPU.  Weights are copied at upload; handles are freed by the caller.
 *   - Activations are token-major: x [t][cols], y [t][rows] (QMat::matmul, gguf_q.rs:217).
 *   - There is no CPU fallback: every compute entry point runs CUDA kernels or fails.
 */
#ifndef PYRE_B200_H
#define PYRE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pb_status {
    PB_OK = 0,
    PB_ERR_ARG = 1,        /* bad argument (shape, type id, null pointer, range) */
    PB_ERR_CUDA = 2,       /* a CUDA runtime call failed */
    PB_ERR_OOM = 3,        /* device allocation failed */
    PB_UNSUPPORTED = 4,    /* valid request that this build does not implement */
    PB_ERR_DEVICE = 5,     /* a kernel reported a failure in the device status word */
    PB_ERR_STATE = 6       /* call not valid in the handle's current state */
} pb_status;

typedef struct pb_ctx pb_ctx;
typedef struct pb_qmat pb_qmat;
typedef struct pb_model pb_model;
typedef struct pb_state pb_state;

/* ggml type ids accepted for matrices (QType::from_id, src/model/gguf_q.rs:23-29) */
enum { PB_TYPE_F32 = 0, PB_TYPE_F16 = 1, PB_TYPE_Q4_0 = 2, PB_TYPE_Q5_0 = 6, PB_TYPE_Q8_0 = 8, PB_TYPE_Q3_K = 11, PB_TYPE_Q4_K = 12, PB_TYPE_Q5_K = 13, PB_TYPE_Q6_K = 14, PB_TYPE_IQ2_XXS = 16, PB_TYPE_IQ2_XS = 17, PB_TYPE_IQ3_XXS = 18,
       PB_TYPE_IQ4_NL = 20, PB_TYPE_IQ3_S = 21, PB_TYPE_IQ2_S = 22, PB_TYPE_IQ4_XS = 23, PB_TYPE_IQ1_M = 29, PB_TYPE_BF16 = 30, PB_TYPE_Q2_0 = 42 };

/* ---------------------------------------------------------------- context */

/* One context per GPU and worker thread (replaces the reference's Cube / device handle,
 * src/model/qn_cube.rs:6237-6250). */
int pb_ctx_create(int device, pb_ctx** out);
int pb_ctx_destroy(pb_ctx* ctx);
const char* pb_last_error(const pb_ctx* ctx);
/* Launch on a caller-provided cudaStream_t (passed as void*; NULL is the legacy default stream).
 * pb_ctx_own_stream returns to the context's own non-blocking stream. */
int pb_ctx_set_stream(pb_ctx* ctx, void* cuda_stream);
int pb_ctx_own_stream(pb_ctx* ctx);
int pb_ctx_sync(pb_ctx* ctx);
/* Page-locked host memory for the caller's logits buffers: pb_forward / pb_verify copy straight into such a destination (one DMA),
 * where a pageable one costs a staging copy in the library and a second copy on the host (the reference reads logits into a fresh Vec
 * per step, Model::forward src/model/qwen4exp_gguf.rs:2050; a caller that reuses one buffer allocates it here).  Memory the caller
 * page-locked itself (cudaHostRegister) is recognised the same way. */
int pb_host_alloc(pb_ctx* ctx, size_t nbytes, void** out);
int pb_host_free(pb_ctx* ctx, void* p);   /* ctx may be NULL (the buffer outlived its context) */
/* Reads and clears the device status word (0 = no kernel reported a failure). */
int pb_ctx_device_status(pb_ctx* ctx, int* status);
/* Non-blocking check for the host's idle / step hooks (Model::idle_hook and step_hook,
 * src/model/qwen4exp_gguf.rs:2024-2034; the reference also resizes its expert cache there, which has no
 * counterpart: every expert is resident).  *busy = 1 while work of this context is still running on the GPU.
 * When the GPU is idle and a kernel has reported a failure the call returns PB_ERR_DEVICE and clears the word. */
int pb_poll(pb_ctx* ctx, int* busy);
/* Tracing (the reference stamps its expert chain with a device clock, src/model/xchain.rs:1-111).  While enabled,
 * every launch of a streaming kernel (GEMV, router, expert gate/up, expert down, DeltaNet, fused step) is handed
 * the next of `slots` stamp slots and records %globaltimer nanoseconds at fixed points: words 0-5 by its first CTA
 * (entry, set-up done, predecessor's data visible, activations ready, first weights landed, last store), words 6-7
 * by its last CTA (entry, last store); the fused step kernel records one word per phase instead.  A captured
 * graph keeps its slots, so a replay overwrites them: read after the step of interest.  slots = 0 turns tracing off.
 * pb_ctx_stamps_read copies min(max_slots, used) slots of 8 words and the kernel id of each (1 GEMV, 2 router,
 * 3 gate/up, 4 down, 5 DeltaNet; operations inside the fused step kernel: 101 GEMV, 102 DeltaNet, 103 router,
 * 104 gate/up, 105 down, stamped at operation start / grid barrier passed / activations ready / first weights
 * landed / end) and returns the number of slots used in *n_slots. */
int pb_ctx_stamps_enable(pb_ctx* ctx, int slots);
int pb_ctx_stamps_read(pb_ctx* ctx, uint64_t* stamps_host, int32_t* kernel_ids_host, int max_slots, int* n_slots);

/* Expert-parallel group over NCCL (NVLink / NVSwitch), one process per GPU.  It replaces the
 * reference's CPU/GPU expert split (XCache + CPU pool, src/model/qwen4exp_gguf.rs:66-72, 785-893):
 * rank r of `world` holds experts [r*n_exp/world, (r+1)*n_exp/world) of every layer.  Rank 0 calls
 * pb_ep_unique_id, the host distributes the 128 bytes (any transport), then every rank calls
 * pb_ep_init before pb_model_finalize(model, rank, world).  libnccl.so.2 is loaded on first use. */
int pb_ep_unique_id(pb_ctx* ctx, void* id128);
int pb_ep_init(pb_ctx* ctx, const void* id128, int rank, int world);
int pb_ep_destroy(pb_ctx* ctx);
/* Failure detection of the peer exchange, testable on one GPU: runs one bounded hand-shake (`spins` polls of about 0.2 us)
 * whose partner never answers.  Returns PB_ERR_DEVICE (the wait gave up and said so in the device status word); the context
 * stays usable.  The reference bounds its CPU/GPU hand-shakes the same way (pyre_wait_flag, src/model/qwen4exp_gguf.rs:229-238). */
int pb_ep_probe_wait_timeout(pb_ctx* ctx, unsigned int spins);

/* (elements per block, bytes per block) -- QType::geom, src/model/gguf_q.rs:33-41 */
int pb_type_geom(int ggml_type, int* elems, int* bytes);

/* ---------------------------------------------------------------- quantized matrices */

/* Copy a rows x cols matrix of GGUF blocks to the GPU, kept in its native block format.
 * Replaces QMat views over the mmapped file: Gguf::mat src/model/gguf_q.rs:326-331,
 * QMat::bytes/raw_rows :209-214. */
int pb_qmat_upload(pb_ctx* ctx, int ggml_type, int64_t rows, int64_t cols, const void* bytes_host, size_t nbytes, pb_qmat** out);
/* Seeded synthetic matrix generated on the GPU (benchmark weights; no counterpart in the
 * reference, whose tests patch LCG-random block bytes the same way, src/model/qdot.rs:1033-1047). */
int pb_qmat_synth(pb_ctx* ctx, int ggml_type, int64_t rows, int64_t cols, uint64_t seed, uint64_t tensor_id, pb_qmat** out);
/* Rows [row0, row0 + rows) of the synthetic tensor (seed, tensor_id): one GPU's shard of a fused expert tensor. */
int pb_qmat_synth_rows(pb_ctx* ctx, int ggml_type, int64_t rows, int64_t cols, uint64_t seed, uint64_t tensor_id, int64_t row0, pb_qmat** out);
int pb_qmat_free(pb_qmat* m);
int pb_qmat_info(const pb_qmat* m, int* ggml_type, int64_t* rows, int64_t* cols, size_t* nbytes);
/* Raw block bytes of rows [r0, r0+nrows) back to the host (QMat::raw_rows :214). */
int pb_qmat_read(pb_ctx* ctx, const pb_qmat* m, int64_t r0, int64_t nrows, void* bytes_host);
/* Dequantize rows [r0, r0+nrows) to f32, bit-identical to dequant(), src/model/gguf_q.rs:67-166
 * (QMat::row :210, QMat::to_f32 :211). */
int pb_qmat_dequant(pb_ctx* ctx, const pb_qmat* m, int64_t r0, int64_t nrows, float* out_host);
int pb_qmat_dequant_dev(pb_ctx* ctx, const pb_qmat* m, int64_t r0, int64_t nrows, float* out_dev);
/* y[ti*rows + r] = sum_c W[r,c] * x[ti*cols + c], f32 accumulate -- QMat::matmul,
 * src/model/gguf_q.rs:217-242.  Host-buffer form (what the reference's callers hold) and
 * device-buffer form. */
int pb_gemv(pb_ctx* ctx, const pb_qmat* m, const float* x_host, int t, float* y_host);
int pb_gemv_dev(pb_ctx* ctx, const pb_qmat* m, const float* x_dev, int t, float* y_dev);
/* pb_gemv for callers that must not allocate device memory.  No counterpart in the reference.
 * Some hosts of this library run with device allocation closed to them: a real-time worker that
 * may not take the driver's allocator lock in its serving loop, a process whose memory budget was
 * handed out in full at start-up, or a sandbox that filters cudaMalloc.  pb_gemv grows a
 * cudaMalloc'd staging buffer on demand; this variant stages x and y in a fixed array that is part
 * of the library image (PB_GEMV_STATIC_MAX_BYTES, resident on every GPU that loads the library until
 * the process exits) and calls no cudaMalloc / cudaFree or any allocating routine.  Same kernels and
 * same results as pb_gemv.  Limit: 256-rounded t*cols*4 plus t*rows*4 bytes must fit the array,
 * otherwise PB_ERR_ARG with a message naming both sizes.  The first call on a device looks up the
 * array's device address; make that call before starting any stream capture.  All calls share the one
 * array and it keeps the previous call's bytes (nothing in it needs to start at zero: x is
 * overwritten and every y element is stored); two calls that overlap on the GPU, from two contexts
 * or two streams, race on it. */
#define PB_GEMV_STATIC_MAX_BYTES (4u << 20)
int pb_gemv_static(pb_ctx* ctx, const pb_qmat* m, const float* x_host, int t, float* y_host);

/* ---------------------------------------------------------------- model */

/* Cfg, src/model/qwen4exp_gguf.rs:18-26 (fields of the decode path only). */
typedef struct pb_cfg {
    int32_t n_layers, d, hc, hc_lr, n_head, n_kv, hd, n_rot;
    float rope_base, eps;
    int32_t n_exp, top_k, ff_exp, ff_sh;
    int32_t lin_nk, lin_nv, lin_dk, lin_dv, conv_k, full_every;
    int32_t vocab, max_ctx;
    int32_t kv_bits;    /* 0: f32 KV; 4: positions older than the recent window are 4-bit (src/model/kv4.rs) */
    int32_t kv_recent;  /* f32 window in front of the packed region (reference default 1024, kv_push :1517-1534) */
} pb_cfg;

/* Tensor roles: the fields of Layer / Mixer / Hc, src/model/qwen4exp_gguf.rs:28-34, and the
 * GGUF names they are loaded from (:494-511). */
typedef enum pb_role {
    PB_R_TOKEN_EMBD = 0, PB_R_OUTPUT, PB_R_OUT_NORM,
    PB_R_ATTN_NORM, PB_R_FFN_NORM,
    PB_R_ATTN_Q, PB_R_ATTN_K, PB_R_ATTN_V, PB_R_ATTN_O, PB_R_ATTN_Q_NORM, PB_R_ATTN_K_NORM,
    PB_R_LIN_QKV, PB_R_LIN_Z, PB_R_LIN_BETA, PB_R_LIN_ALPHA, PB_R_LIN_OUT,
    PB_R_LIN_A, PB_R_LIN_DT, PB_R_LIN_CONV, PB_R_LIN_NORM,
    PB_R_ROUTER, PB_R_EXP_GATE, PB_R_EXP_UP, PB_R_EXP_DOWN,
    PB_R_SH_GATE, PB_R_SH_UP, PB_R_SH_DOWN, PB_R_SH_GATE_INP,
    PB_R_HCA_NORM, PB_R_HCA_DOWN, PB_R_HCA_UP, PB_R_HCA_INJECT,
    PB_R_HCF_NORM, PB_R_HCF_DOWN, PB_R_HCF_UP, PB_R_HCF_INJECT,
    PB_R_OUT_HC_NORM, PB_R_OUT_HC_DOWN, PB_R_OUT_HC_UP,
    /* QSA indexer of an attention layer (Mixer::Attn idx, :501): blk.N.indexer.q_proj / k_proj / q_norm / k_norm */
    PB_R_IDX_Q, PB_R_IDX_K, PB_R_IDX_Q_NORM, PB_R_IDX_K_NORM,
    /* input stage of an MTP drafter model (src/model/mtp.rs:104-123): fc_embedding, fc_hidden, pre_fc_norm_embedding, pre_fc_norm_hidden */
    PB_R_MTP_FC_E, PB_R_MTP_FC_H, PB_R_MTP_PRE_E, PB_R_MTP_PRE_H,
    /* per-layer n-gram embeddings (Ple, src/model/qwen4exp_gguf.rs:33, tensors :505, 512): per_layer_token_embd (global); per layer
     * ple_key [streams * d][heads * dim], ple_value [d][heads * dim], ple_norm_key / ple_norm_query / ple_norm_conv [streams * d],
     * ple_conv1d [streams * d][conv_kernel] */
    PB_R_PLE_TAB, PB_R_PLE_KEY, PB_R_PLE_VALUE, PB_R_PLE_NORM_KEY, PB_R_PLE_NORM_QUERY, PB_R_PLE_NORM_CONV, PB_R_PLE_CONV,
    PB_R_COUNT
} pb_role;

/* Model::load, src/model/qwen4exp_gguf.rs:462-524, split into create / set / finalize so the
 * Rust side keeps owning the GGUF mmap.  layer = -1 for global tensors. */
int pb_model_create(pb_ctx* ctx, const pb_cfg* cfg, pb_model** out);
int pb_model_set_tensor(pb_model* m, int layer, int role, pb_qmat* mat);   /* the model takes ownership */
int pb_model_set_vec(pb_model* m, int layer, int role, const float* v_host, int64_t n);
/* QSA block-sparse attention (attn_core, src/model/qwen4exp_gguf.rs:1565-1599; Cfg :24-25, keys attention.indexer.* :481-485).
 * `budget` tokens in blocks of `ratio`; the attention layers that hold PB_R_IDX_* tensors then attend, once a query sees
 * more than budget + ratio - 1 tokens, to the budget / ratio best-scoring blocks plus the incomplete tail.  n_head = 0
 * (the default) switches it off.  Before pb_model_finalize. */
int pb_model_set_indexer(pb_model* m, int budget, int ratio, int n_head, int head_dim);
/* Per-layer n-gram embeddings (ple_rows / ple, src/model/qwen4exp_gguf.rs:1390-1434; Cfg ple_* :477-480, metadata keys `ple.ngram_size`,
 * `ple.heads_per_ngram`, `ple.conv_kernel`, `ple.eos_token_id`, `embedding_length_per_layer_input`, `ple.layer_multipliers`,
 * `ple.head_offsets`, `ple.head_vocab_sizes`).  Every fed token is hashed, together with its ngram - 1 predecessors (cut at a missing or
 * end-of-sequence one), into heads = (ngram - 1) * heads_per_ngram rows of the PB_R_PLE_TAB table; the layers that hold PB_R_PLE_KEY add a
 * gated projection of those rows, and a causal depthwise convolution of its normalized form over earlier positions, to the residual
 * streams at their start.  multipliers[ngram], head_offsets[heads], head_vocab_sizes[heads]; 2 <= ngram <= 8, heads <= 32, dim a
 * multiple of 256.  Before pb_model_finalize. */
int pb_model_set_ple(pb_model* m, int ngram, int heads_per_ngram, int conv_kernel, uint32_t eos, int dim,
                     const uint64_t* multipliers, const uint64_t* head_offsets, const uint64_t* head_vocab_sizes);
/* Trained context of the checkpoint (`<arch>.context_length`).  When cfg.max_ctx exceeds it, the rope table is YaRN-scaled
 * for the whole run as the reference does at load (src/model/qwen4exp_gguf.rs:490-517, table src/qn_ctx.rs:160-186, mscale on
 * cos and sin :528-533); 0 (the default) or max_ctx <= ctx_train leave the plain table.  Before pb_model_finalize. */
int pb_model_set_ctx_train(pb_model* m, int ctx_train);
/* attach_gpu :555-657.  ep_rank/ep_world: this GPU holds routed experts
 * [ep_rank*n_exp/ep_world, (ep_rank+1)*n_exp/ep_world) of every layer; dense tensors are replicated. */
int pb_model_finalize(pb_model* m, int ep_rank, int ep_world);
int pb_model_cfg(const pb_model* m, pb_cfg* out);   /* the configuration the model was created with (Model.cfg) */
int pb_model_destroy(pb_model* m);

/* new_state :1345-1353; `batch` independent sequences decode together. */
int pb_state_create(pb_model* m, int batch, pb_state** out);
/* Expert-parallel models only (a plain state otherwise); no counterpart in the reference, which runs
 * one sequence on one GPU.  `batch` sequences are THIS rank's share of a global batch of
 * batch * ep_world: attention, DeltaNet, dense layers and the lm-head run on them alone, and every
 * MoE block all-gathers the residual rows of all ranks, applies the local experts to every token and
 * reduce-scatters the partial rows to the tokens' owners.  Every rank must step its state the same
 * number of times (the collectives pair up); tokens are identical to a single-GPU run. */
int pb_state_create_sharded(pb_model* m, int batch, pb_state** out);
int pb_state_destroy(pb_state* s);
/* Pre-fill attention layer `attn_index` of sequence `b` with n positions of already normed and
 * roped K and V rows [n][n_kv*hd] (f32, host); packs per cfg.kv_bits.  Benchmark set-up for a
 * long context without running a prefill. */
int pb_state_fill_kv(pb_state* s, int b, int attn_index, const float* k_host, const float* v_host, int64_t n);
/* Same with seeded synthetic N(0,1) rows generated on the GPU (and, for a model with an indexer, synthetic raw index keys). */
int pb_state_fill_kv_synth(pb_state* s, int attn_index, int64_t n, uint64_t seed);
/* Models with an indexer: the raw index keys [n][idx_hd] (f32, host) of the same n positions; the pooled block keys are derived. */
int pb_state_fill_index_keys(pb_state* s, int b, int attn_index, const float* ik_host, int64_t n);
int pb_state_set_pos(pb_state* s, int64_t pos);
/* A fresh conversation in an existing state: position 0, the DeltaNet conv history and recurrent state zeroed, the packed
 * boundary of the 4-bit KV cache back to 0 (Model::new_state, src/model/qwen4exp_gguf.rs:3199-3213, without its allocations). */
int pb_state_reset(pb_state* s);
int pb_state_pos(const pb_state* s, int64_t* pos);

/* Model::forward(ids, st) -> logits, src/model/qwen4exp_gguf.rs:2050-2157 (= spec::Target::step,
 * src/spec.rs:106-120, QnTarget::step src/engine_qn.rs:247).  ids_host [batch][t]; the logits of
 * the last fed token of each sequence go to logits_host [batch][vocab].  A prompt (t >= 3) of a
 * batch-1 state runs in windows of up to 8 tokens that stream every weight matrix once per window. */
int pb_forward(pb_state* s, const uint32_t* ids_host, int t, float* logits_host);
/* forward + sampler::argmax (src/sampler.rs:142-148) on the device: next_host [batch]. */
int pb_step_greedy(pb_state* s, const uint32_t* tok_host, uint32_t* next_host);
/* Decode n greedy tokens per sequence without leaving the device between steps;
 * out_host [batch][n].  Same arithmetic as n calls of pb_step_greedy. */
int pb_decode_greedy(pb_state* s, const uint32_t* tok_host, int n, uint32_t* out_host);

/* Model::forward_multi :2365-2480 (= Target::verify): logits for every fed position,
 * logits_host [t][vocab]; records per-position rollback checkpoints.  batch must be 1, t <= 8.
 * One batched pass: weights are streamed once for all t tokens (tensor cores from 3 tokens on), the
 * recurrences run token by token; agrees with t calls of pb_forward to rounding, not bit for bit. */
int pb_verify(pb_state* s, const uint32_t* ids_host, int t, float* logits_host);
/* Model::spec_keep :2495-2515 (= Target::keep): keep the first `keep` of the last t verified tokens. */
int pb_keep(pb_state* s, int t, int keep);
/* The model's own multi-token-prediction layer as a speculative drafter (src/model/mtp.rs; Mtp::load :104-123).
 * The drafter is a pb_model of its own: cfg with n_layers = 1, full_every = 1 (one attention layer), the main model's
 * d and hc, kv_bits = 0, max_ctx >= the main model's, vocab = the size of the draft vocabulary; tensors under the usual
 * roles of an attention layer with hyper-connections and a MoE block (layer 0), PB_R_OUT_HC_* = the final mixer,
 * PB_R_OUTPUT = the head rows of the draft vocabulary, PB_R_MTP_* = the input stage; norm vectors hold 1 + w as in
 * the main model.  pb_model_set_mtp marks it (window = cells a draft step attends to, reference default 128) before
 * pb_model_finalize. */
int pb_model_set_mtp(pb_model* drafter, int window);
/* Binds a finalized drafter to a batch-1 state of the main model (which must have hyper-connection streams: hc >= 1).
 * vocab_ids[i] = the token whose head row is row i of the drafter's PB_R_OUTPUT.  From here on the state keeps the final
 * residual row of every position it processes (mtp_keep_r :2279-2285) and the ids it is fed.  The drafter model must
 * outlive the state. */
int pb_state_attach_drafter(pb_state* s, pb_model* drafter, const uint32_t* vocab_ids_host, int n_ids);
/* Model::mtp_draft :2177-2278 (= Target::draft): up to max_draft tokens that follow the tokens fed so far and `pending`,
 * the token already chosen but not fed yet (the last element of spec.rs's history).  Cells of earlier positions the
 * drafter has not seen are caught up first (K/V only).  Token j > 0 is kept only while the drafter's probability of it
 * (softmax over the draft vocabulary) is at least min_p (draft_gate, src/spec.rs:326; reference default 0.9).
 * probs_host may be NULL.  *n = 0 when the residual of the last position is not held (e.g. right after a restore).
 * Every emitted token still comes from pb_verify, so greedy output is unchanged by drafting.
 * Without an attached drafter: PB_UNSUPPORTED, and the caller's n-gram drafter takes over (src/spec.rs:207). */
int pb_draft(pb_state* s, uint32_t pending, int max_draft, float min_p, uint32_t* ids_host, float* probs_host, int* n);
/* Drafts drawn from the drafter's distribution (the reference's sampled drafts, mtp_qsample :3321-3331, used when the request's
 * temperature is above 0, :2229-2246): after the min_p gate on the most probable token, `pick` -- the caller's sampler -- is handed the
 * drafter's logits over the draft vocabulary (host memory, valid during the call) with the token of every row, and returns the token to
 * draft; that token feeds the next step.  The caller keeps whatever it needs of the distribution for its acceptance test.  probs_host
 * holds the probability of the most probable token of each step, as with pb_draft.  pick = NULL is pb_draft. */
typedef uint32_t (*pb_draft_pick)(void* user, const float* logits, const uint32_t* vocab_ids, int n_ids);
int pb_draft_sampled(pb_state* s, uint32_t pending, int max_draft, float min_p, pb_draft_pick pick, void* user, uint32_t* ids_host, float* probs_host, int* n);

/* Model::snapshot / restore, Snap :3277-3298.  size query: pass buf_host = NULL. */
int pb_state_snapshot(pb_state* s, void* buf_host, size_t* nbytes);
int pb_state_restore(pb_state* s, const void* buf_host, size_t nbytes);

/* multi_ok :2352, spec_max_window :2486, max_ctx :526 */
typedef struct pb_caps { int32_t multi_ok, max_window, max_ctx, max_batch, ep_world; } pb_caps;
int pb_caps_get(const pb_model* m, pb_caps* caps);

/* Counters for the reference's metrics hooks (src/metrics.rs:6-7). */
typedef struct pb_stats {
    uint64_t steps, kernels_launched, weight_bytes_per_step, kv_bytes_per_step, state_bytes_per_step;
    uint64_t device_ns;     /* GPU time of this state's token-loop calls so far (CUDA events around each call; add_gpu_ns) */
    uint64_t exchange_ns;   /* of which: waiting for other GPUs in the expert exchange (0 on one GPU) */
} pb_stats;
int pb_stats_get(const pb_state* s, pb_stats* out);

/* ---------------------------------------------------------------- layer-level entry points
 * The blocks of the token loop, callable alone on device buffers (parity tests, benchmarks). */

/* MoE block: ffn :1675-1684 + routed :1721-1795.  x_host [t][d] -> y_host [t][d];
 * sel_host (optional) [t][top_k] expert ids in the order they are accumulated. */
int pb_moe_forward(pb_state* s, int layer, const float* x_host, int t, float* y_host, int32_t* sel_host);
/* Gated DeltaNet layer step: linear :1617-1621 + linear_core :1624-1673 for one token per
 * sequence.  x_host [batch][d] -> y_host [batch][d]; advances the layer's conv and ssm state. */
int pb_deltanet_step(pb_state* s, int layer, const float* x_host, float* y_host);
/* Gated attention layer step: attn :1441-1446 + attn_core :1558-1615 at the state's position. */
int pb_attn_step(pb_state* s, int layer, const float* x_host, float* y_host);
/* Copies of a DeltaNet layer's recurrent state for inspection / set-up: ssm [batch][nv][dk][dv],
 * conv [batch][conv_k-1][ch]. */
int pb_state_get_lin(pb_state* s, int layer, float* conv_host, float* ssm_host);
int pb_state_set_lin(pb_state* s, int layer, const float* conv_host, const float* ssm_host);
/* Inspection: the first n floats of one of the step's activation buffers as the last operation left them
 * (what: 0 residual x [batch][d], 1 projection outputs, 2 DeltaNet readout, 3 attention output, 4 router logits
 * [n_exp + 1], 5 routed experts' hidden vectors in accumulation order [top_k][ff], 6 shared expert's hidden vector,
 * 7 with tracing on before the state's first step: the fused step kernel's clock stamps, per operation uint64 [CTA][4]
 * (operation start, grid barrier passed, operation end, producer warp done) followed by 32 fine-grained stamps of CTA 0,
 * read as 2 floats per stamp). */
int pb_state_peek(pb_state* s, int what, float* out_host, int64_t n);

/* 4-bit KV packing on the device: kv4::pack / kv4::get, src/model/kv4.rs:12-42.
 * x_host [n] f32 (n a multiple of 32) -> words_host [n/8], scales_host [n/32]. */
int pb_kv4_pack(pb_ctx* ctx, const float* x_host, int64_t n, uint32_t* words_host, float* scales_host);
int pb_kv4_unpack(pb_ctx* ctx, const uint32_t* words_host, const float* scales_host, int64_t n, float* x_host);

#ifdef __cplusplus
}
#endif
#endif /* PYRE_B200_H */
