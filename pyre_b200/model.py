"""Model / State: the reference's Qwen-Next model surface over the C ABI.

Mirrors `Model` and `State` of src/model/qwen4exp_gguf.rs in the reference (load :462,
new_state :1345, forward :2050, forward_multi :2365, spec_keep :2495, snapshot/restore
:3280/:3294) and the `spec::Target` trait that the engine loop calls (src/spec.rs:106-120):
step -> forward, verify -> forward_multi, keep -> spec_keep.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import Caps, Cfg, Ctx, QMat, ROLE, Stats, _f32, _p, lib


class Model:
    def __init__(self, ctx: Ctx, cfg: Cfg):
        self.ctx, self.cfg = ctx, cfg
        self.h = C.c_void_p()
        ctx.check(lib().pb_model_create(ctx.h, C.byref(cfg), C.byref(self.h)))
        self.ep_rank, self.ep_world = 0, 1

    def set_tensor(self, layer: int, role: str, m: QMat):
        """The model takes ownership of the device matrix."""
        self.ctx.check(lib().pb_model_set_tensor(self.h, C.c_int(layer), C.c_int(ROLE[role]), m.h))
        m.owned = False

    def set_vec(self, layer: int, role: str, v: np.ndarray):
        v = _f32(v).reshape(-1)
        self.ctx.check(lib().pb_model_set_vec(self.h, C.c_int(layer), C.c_int(ROLE[role]), _p(v), C.c_int64(v.size)))

    def set_mtp(self, window: int = 128):
        """Marks this model (one attention layer with hyper-connections + the MTP_* tensors) as an MTP drafter (before finalize)."""
        self.ctx.check(lib().pb_model_set_mtp(self.h, C.c_int(window)))

    def set_indexer(self, budget: int, ratio: int, n_head: int, head_dim: int):
        """QSA block-sparse attention: attention layers that hold IDX_Q / IDX_K / IDX_Q_NORM / IDX_K_NORM attend to the
        budget / ratio best blocks of ratio tokens once a query sees more than budget + ratio - 1 tokens (before finalize)."""
        self.ctx.check(lib().pb_model_set_indexer(self.h, C.c_int(budget), C.c_int(ratio), C.c_int(n_head), C.c_int(head_dim)))
        self.indexer = (budget, ratio, n_head, head_dim)

    def set_ple(self, ngram: int, per_gram: int, conv_k: int, eos: int, dim: int, mult, off, vocab):
        """Per-layer n-gram embeddings (the metadata keys `ple.*` of a qwen4exp file): layers that hold PLE_KEY inject a gated
        projection of hashed table rows at their start (before finalize)."""
        a = lambda v: np.ascontiguousarray(v, dtype=np.uint64)
        mult, off, vocab = a(mult), a(off), a(vocab)
        if mult.size != ngram or off.size != (ngram - 1) * per_gram or vocab.size != off.size:
            raise ValueError("set_ple: multipliers[ngram], offsets / vocabulary sizes [(ngram - 1) * per_gram]")
        self.ctx.check(lib().pb_model_set_ple(self.h, C.c_int(ngram), C.c_int(per_gram), C.c_int(conv_k), C.c_uint32(eos), C.c_int(dim),
                                              mult.ctypes.data_as(C.c_void_p), off.ctypes.data_as(C.c_void_p), vocab.ctypes.data_as(C.c_void_p)))

    def set_ctx_train(self, ctx_train: int):
        """Trained context; a larger cfg.max_ctx is YaRN-scaled (before finalize)."""
        self.ctx.check(lib().pb_model_set_ctx_train(self.h, C.c_int(ctx_train)))

    def finalize(self, ep_rank: int = 0, ep_world: int = 1):
        self.ctx.check(lib().pb_model_finalize(self.h, C.c_int(ep_rank), C.c_int(ep_world)))
        self.ep_rank, self.ep_world = ep_rank, ep_world

    def new_state(self, batch: int = 1, sharded: bool = False) -> "State":
        """sharded=True (expert-parallel models): `batch` sequences are this rank's share of a global
        batch of batch * world; see pb_state_create_sharded."""
        return State(self, batch, sharded)

    def caps(self) -> Caps:
        c = Caps()
        self.ctx.check(lib().pb_caps_get(self.h, C.byref(c)))
        return c

    def destroy(self):
        if self.h:
            lib().pb_model_destroy(self.h)
            self.h = C.c_void_p()


class State:
    """One conversation per batch slot (State, src/model/qwen4exp_gguf.rs:184-207)."""

    def __init__(self, model: Model, batch: int = 1, sharded: bool = False):
        self.model, self.batch, self.ctx = model, batch, model.ctx
        self.h = C.c_void_p()
        create = lib().pb_state_create_sharded if sharded else lib().pb_state_create
        self.ctx.check(create(model.h, C.c_int(batch), C.byref(self.h)))

    # ---- token loop -------------------------------------------------------------------
    def forward(self, ids, out: np.ndarray = None) -> np.ndarray:
        """Feed ids [batch][t] (or [t] when batch == 1); logits of the last position, [batch][vocab].  out = a float32 array of
        that shape to reuse (Ctx.pinned_empty gives one the device writes into directly)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(self.batch, -1)
        if out is not None:
            if out.dtype != np.float32 or out.shape != (self.batch, self.model.cfg.vocab) or not out.flags.c_contiguous:
                raise ValueError("forward: out must be a C-contiguous float32 array [batch][vocab]")
            logits = out
        else:
            logits = np.empty((self.batch, self.model.cfg.vocab), dtype=np.float32)
        self.ctx.check(lib().pb_forward(self.h, _p(ids), C.c_int(ids.shape[1]), _p(logits)))
        return logits

    def step_greedy(self, tok) -> np.ndarray:
        tok = np.ascontiguousarray(tok, dtype=np.uint32).reshape(self.batch)
        nxt = np.empty(self.batch, dtype=np.uint32)
        self.ctx.check(lib().pb_step_greedy(self.h, _p(tok), _p(nxt)))
        return nxt

    def decode_greedy(self, tok, n: int) -> np.ndarray:
        """n greedy tokens per sequence without leaving the device between steps: [batch][n]."""
        tok = np.ascontiguousarray(tok, dtype=np.uint32).reshape(self.batch)
        out = np.empty((self.batch, n), dtype=np.uint32)
        self.ctx.check(lib().pb_decode_greedy(self.h, _p(tok), C.c_int(n), _p(out)))
        return out

    def forward_multi(self, ids) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
        logits = np.empty((ids.size, self.model.cfg.vocab), dtype=np.float32)
        self.ctx.check(lib().pb_verify(self.h, _p(ids), C.c_int(ids.size), _p(logits)))
        return logits

    def attach_drafter(self, drafter: "Model", vocab_ids):
        """Binds an MTP drafter model to this batch-1 state; vocab_ids[i] = token of row i of the drafter's head."""
        ids = np.ascontiguousarray(vocab_ids, dtype=np.uint32).reshape(-1)
        self.ctx.check(lib().pb_state_attach_drafter(self.h, drafter.h, _p(ids), C.c_int(ids.size)))
        self._drafter = drafter      # must outlive the state

    def draft(self, pending: int, max_draft: int, min_p: float = 0.9):
        """Target::draft: (token ids, their draft probabilities) that follow the fed tokens and `pending`."""
        ids = np.zeros(max(max_draft, 1), np.uint32); probs = np.zeros(max(max_draft, 1), np.float32); n = C.c_int(0)
        self.ctx.check(lib().pb_draft(self.h, C.c_uint32(pending), C.c_int(max_draft), C.c_float(min_p), _p(ids), _p(probs), C.byref(n)))
        return ids[:n.value].copy(), probs[:n.value].copy()

    def draft_sampled(self, pending: int, max_draft: int, min_p: float, pick):
        """As draft(), with every drafted token chosen by `pick(logits, vocab_ids) -> token id` from the drafter's logits over
        the draft vocabulary (the reference's sampled drafts, mtp_qsample, qwen4exp_gguf.rs:3321-3331)."""
        ids = np.zeros(max(max_draft, 1), np.uint32); probs = np.zeros(max(max_draft, 1), np.float32); n = C.c_int(0)
        PICK = C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.c_int)

        def tramp(_user, lg, vid, n_ids):
            return int(pick(np.ctypeslib.as_array(lg, shape=(n_ids,)).copy(), np.ctypeslib.as_array(vid, shape=(n_ids,)).copy()))

        cb = PICK(tramp)
        self.ctx.check(lib().pb_draft_sampled(self.h, C.c_uint32(pending), C.c_int(max_draft), C.c_float(min_p), cb, None, _p(ids), _p(probs), C.byref(n)))
        return ids[:n.value].copy(), probs[:n.value].copy()

    def spec_keep(self, t: int, keep: int):
        self.ctx.check(lib().pb_keep(self.h, C.c_int(t), C.c_int(keep)))

    def snapshot(self) -> bytes:
        n = C.c_size_t()
        self.ctx.check(lib().pb_state_snapshot(self.h, None, C.byref(n)))
        buf = np.empty(n.value, dtype=np.uint8)
        self.ctx.check(lib().pb_state_snapshot(self.h, _p(buf), C.byref(n)))
        return buf.tobytes()

    def restore(self, blob: bytes):
        buf = np.frombuffer(blob, dtype=np.uint8)
        self.ctx.check(lib().pb_state_restore(self.h, _p(buf), C.c_size_t(buf.size)))

    # ---- position / caches -----------------------------------------------------------
    def set_pos(self, pos: int):
        self.ctx.check(lib().pb_state_set_pos(self.h, C.c_int64(pos)))

    def reset(self):
        """A fresh conversation: position 0, recurrent state and conv history zeroed (pb_state_reset)."""
        self.ctx.check(lib().pb_state_reset(self.h))

    def pos(self) -> int:
        p = C.c_int64()
        self.ctx.check(lib().pb_state_pos(self.h, C.byref(p)))
        return p.value

    def fill_kv(self, b: int, attn_index: int, k: np.ndarray, v: np.ndarray):
        k, v = _f32(k), _f32(v)
        row = self.model.cfg.n_kv * self.model.cfg.hd
        self.ctx.check(lib().pb_state_fill_kv(self.h, C.c_int(b), C.c_int(attn_index), _p(k), _p(v), C.c_int64(k.size // row)))

    def fill_index_keys(self, b: int, attn_index: int, ik: np.ndarray):
        """Raw index keys [n][idx_hd] of the positions given to fill_kv (models with an indexer)."""
        ik = _f32(ik)
        self.ctx.check(lib().pb_state_fill_index_keys(self.h, C.c_int(b), C.c_int(attn_index), _p(ik), C.c_int64(ik.shape[0])))

    def fill_kv_synth(self, attn_index: int, n: int, seed: int):
        self.ctx.check(lib().pb_state_fill_kv_synth(self.h, C.c_int(attn_index), C.c_int64(n), C.c_uint64(seed)))

    def get_lin(self, layer: int):
        c = self.model.cfg
        ch = 2 * c.lin_nk * c.lin_dk + c.lin_nv * c.lin_dv
        conv = np.empty((self.batch, c.conv_k - 1, ch), dtype=np.float32)
        ssm = np.empty((self.batch, c.lin_nv, c.lin_dk, c.lin_dv), dtype=np.float32)
        self.ctx.check(lib().pb_state_get_lin(self.h, C.c_int(layer), _p(conv), _p(ssm)))
        return conv, ssm

    def set_lin(self, layer: int, conv: np.ndarray | None, ssm: np.ndarray | None):
        conv = None if conv is None else _f32(conv)
        ssm = None if ssm is None else _f32(ssm)
        self.ctx.check(lib().pb_state_set_lin(self.h, C.c_int(layer), _p(conv), _p(ssm)))

    def peek(self, what: int, n: int) -> np.ndarray:
        """First n floats of an activation buffer after the last step (pb_state_peek): 0 residual, 1 projections,
        2 DeltaNet readout, 3 attention output, 4 router logits, 5 routed hidden vectors, 6 shared hidden vector."""
        out = np.empty(n, dtype=np.float32)
        self.ctx.check(lib().pb_state_peek(self.h, C.c_int(what), _p(out), C.c_int64(n)))
        return out

    def stats(self) -> Stats:
        st = Stats()
        self.ctx.check(lib().pb_stats_get(self.h, C.byref(st)))
        return st

    # ---- layer-level entry points ------------------------------------------------------
    def moe_forward(self, layer: int, x: np.ndarray):
        x = _f32(x).reshape(-1, self.model.cfg.d)
        t = x.shape[0]
        y = np.empty_like(x)
        sel = np.empty((t, self.model.cfg.top_k), dtype=np.int32)
        self.ctx.check(lib().pb_moe_forward(self.h, C.c_int(layer), _p(x), C.c_int(t), _p(y), _p(sel)))
        return y, sel

    def deltanet_step(self, layer: int, x: np.ndarray) -> np.ndarray:
        x = _f32(x).reshape(self.batch, self.model.cfg.d)
        y = np.empty_like(x)
        self.ctx.check(lib().pb_deltanet_step(self.h, C.c_int(layer), _p(x), _p(y)))
        return y

    def attn_step(self, layer: int, x: np.ndarray) -> np.ndarray:
        x = _f32(x).reshape(self.batch, self.model.cfg.d)
        y = np.empty_like(x)
        self.ctx.check(lib().pb_attn_step(self.h, C.c_int(layer), _p(x), _p(y)))
        return y

    def destroy(self):
        if self.h:
            lib().pb_state_destroy(self.h)
            self.h = C.c_void_p()
