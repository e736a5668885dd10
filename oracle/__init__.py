"""ctypes front end of the CPU oracle (oracle/pyre_oracle.c) -- TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline / reference arm of the benchmark import
this module.  The product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_ref" / "libpyre_oracle.so"

F32, F16, Q8_0, Q4_K, IQ2_XS, IQ3_S, BF16 = 0, 1, 8, 12, 17, 21, 30
IQ3_XXS, IQ4_NL, IQ2_S, IQ4_XS = 18, 20, 22, 23
Q6_K, IQ2_XXS, Q2_0, IQ1_M = 14, 16, 42, 29
Q4_0, Q5_0, Q3_K, Q5_K = 2, 6, 11, 13
QUANT_TYPES = {"Q8_0": Q8_0, "Q4_K": Q4_K, "IQ2_XS": IQ2_XS, "IQ3_S": IQ3_S}
# formats of the GGUF loader beyond the four of the hot path: dequantization only (no synthetic generator)
EXTRA_TYPES = {"IQ3_XXS": IQ3_XXS, "IQ2_S": IQ2_S, "IQ4_NL": IQ4_NL, "IQ4_XS": IQ4_XS, "Q2_0": Q2_0, "IQ2_XXS": IQ2_XXS, "Q6_K": Q6_K, "IQ1_M": IQ1_M, "Q4_0": Q4_0, "Q5_0": Q5_0, "Q3_K": Q3_K, "Q5_K": Q5_K}

ROLES = [
    "TOKEN_EMBD", "OUTPUT", "OUT_NORM", "ATTN_NORM", "FFN_NORM",
    "ATTN_Q", "ATTN_K", "ATTN_V", "ATTN_O", "ATTN_Q_NORM", "ATTN_K_NORM",
    "LIN_QKV", "LIN_Z", "LIN_BETA", "LIN_ALPHA", "LIN_OUT", "LIN_A", "LIN_DT", "LIN_CONV", "LIN_NORM",
    "ROUTER", "EXP_GATE", "EXP_UP", "EXP_DOWN", "SH_GATE", "SH_UP", "SH_DOWN", "SH_GATE_INP",
    "HCA_NORM", "HCA_DOWN", "HCA_UP", "HCA_INJECT", "HCF_NORM", "HCF_DOWN", "HCF_UP", "HCF_INJECT",
    "OUT_HC_NORM", "OUT_HC_DOWN", "OUT_HC_UP",
    "IDX_Q", "IDX_K", "IDX_Q_NORM", "IDX_K_NORM",
    "MTP_FC_E", "MTP_FC_H", "MTP_PRE_E", "MTP_PRE_H",
    "PLE_TAB", "PLE_KEY", "PLE_VALUE", "PLE_NORM_KEY", "PLE_NORM_QUERY", "PLE_NORM_CONV", "PLE_CONV",
]
ROLE = {n: i for i, n in enumerate(ROLES)}


def build(force: bool = False) -> Path:
    """Compile the oracle with the Makefile beside it (gcc, a second or two)."""
    src = [_HERE / "pyre_oracle.c", _HERE / "pyre_oracle.h", _HERE / "iq_tables.h"]
    if force or not _SO.exists() or any(s.stat().st_mtime > _SO.stat().st_mtime for s in src):
        subprocess.run(["make", "-C", str(_HERE)] + (["-B"] if force else []), check=True, capture_output=True)
    return _SO


class Mat(C.Structure):
    _fields_ = [("type", C.c_int32), ("rows", C.c_int64), ("cols", C.c_int64), ("data", C.c_void_p),
                ("seed", C.c_uint64), ("tid", C.c_uint64)]


class Cfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "d", "hc", "hc_lr", "n_head", "n_kv", "hd", "n_rot")] + \
               [("rope_base", C.c_float), ("eps", C.c_float)] + \
               [(n, C.c_int32) for n in ("n_exp", "top_k", "ff_exp", "ff_sh", "lin_nk", "lin_nv", "lin_dk", "lin_dv",
                                         "conv_k", "full_every", "vocab", "max_ctx", "kv_bits", "kv_recent")]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_SO))
        L.orc_row_bytes.restype = C.c_int64
        L.orc_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.orc_dot.restype = C.c_float
        L.orc_kv4_get.restype = C.c_float
        L.orc_argmax.restype = C.c_uint32
        L.orc_model_new.restype = C.c_void_p
        L.orc_state_new.restype = C.c_void_p
        L.orc_threads.restype = C.c_int
        L.orc_last_qsa_margin.restype = C.c_float
        L.orc_rope_inv_yarn.restype = C.c_float
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_set_threads.restype = None
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def threads() -> int:
    return lib().orc_threads()


def set_threads(n: int) -> None:
    """Use n threads in the row-parallel loops (overrides an inherited OMP_NUM_THREADS)."""
    lib().orc_set_threads(int(n))


def geom(t: int):
    e, b = C.c_int(), C.c_int()
    if lib().orc_type_geom(t, C.byref(e), C.byref(b)):
        raise ValueError(f"unsupported ggml type {t}")
    return e.value, b.value


def row_bytes(t: int, cols: int) -> int:
    return lib().orc_row_bytes(t, cols)


def dequant(t: int, raw: np.ndarray, n: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    y = np.empty(n, dtype=np.float32)
    if lib().orc_dequant(t, _p(raw), C.c_int64(n), _p(y)):
        raise ValueError(f"unsupported ggml type {t}")
    return y


def synth_rows(t: int, seed: int, tid: int, cols: int, r0: int, nrows: int) -> np.ndarray:
    out = np.empty(nrows * row_bytes(t, cols), dtype=np.uint8)
    lib().orc_synth_rows(t, C.c_uint64(seed), C.c_uint64(tid), C.c_int64(cols), C.c_int64(r0), C.c_int64(nrows), _p(out))
    return out


def synth_normal(seed: int, tid: int, i0: int, n: int, sigma: float) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_synth_normal(C.c_uint64(seed), C.c_uint64(tid), C.c_int64(i0), C.c_int64(n), C.c_float(sigma), _p(out))
    return out


class QMat:
    """Quantized matrix view: explicit bytes (kept alive here) or a synthetic (seed, tid) tensor."""

    def __init__(self, t: int, rows: int, cols: int, data: np.ndarray | None = None, seed: int = 0, tid: int = 0):
        self.type, self.rows, self.cols, self.seed, self.tid = t, rows, cols, seed, tid
        self.data = None if data is None else np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        if self.data is not None:
            assert self.data.size == rows * row_bytes(t, cols), (self.data.size, rows, cols, t)
        self.c = Mat(t, rows, cols, None if self.data is None else self.data.ctypes.data, seed, tid)

    @classmethod
    def synth(cls, t, rows, cols, seed, tid):
        return cls(t, rows, cols, None, seed, tid)

    def raw(self) -> np.ndarray:
        if self.data is not None:
            return self.data
        return synth_rows(self.type, self.seed, self.tid, self.cols, 0, self.rows)

    def to_f32(self) -> np.ndarray:
        return dequant(self.type, self.raw(), self.rows * self.cols).reshape(self.rows, self.cols)

    def matmul(self, x: np.ndarray) -> np.ndarray:
        """x [t][cols] -> y [t][rows] (QMat::matmul, token-major)."""
        x = _f32(x).reshape(-1, self.cols)
        y = np.empty((x.shape[0], self.rows), dtype=np.float32)
        lib().orc_matmul(C.byref(self.c), _p(x), C.c_int(x.shape[0]), _p(y))
        return y


def q8_quantize(x: np.ndarray):
    """quantize, src/model/qdot.rs:15-30: int8 values and one f32 scale per 32 values."""
    x = _f32(x).reshape(-1)
    q = np.empty(x.size, dtype=np.int8)
    d = np.empty(x.size // 32, dtype=np.float32)
    lib().orc_q8_quantize(_p(x), C.c_int64(x.size), _p(q), _p(d))
    return q, d


def q8_dot_dequant(t: int, row: np.ndarray, q: np.ndarray, d: np.ndarray) -> float:
    row = np.ascontiguousarray(row, dtype=np.uint8)
    f = lib().orc_q8_dot_dequant
    f.restype = C.c_float
    return float(f(C.c_int(t), _p(row), C.c_int64(q.size), _p(q), _p(d)))


def row_dot_q8_iq3s(row: np.ndarray, q: np.ndarray, d: np.ndarray) -> float:
    row = np.ascontiguousarray(row, dtype=np.uint8)
    f = lib().orc_row_dot_q8_iq3s
    f.restype = C.c_float
    return float(f(_p(row), C.c_int64(q.size), _p(q), _p(d)))


def top_k(r: np.ndarray, k: int):
    r = _f32(r)
    idx = np.empty(k, dtype=np.int32)
    w = np.empty(k, dtype=np.float32)
    lib().orc_top_k(_p(r), C.c_int(r.size), C.c_int(k), _p(idx), _p(w))
    return idx, w


def argmax(v: np.ndarray) -> int:
    v = _f32(v)
    return lib().orc_argmax(_p(v), C.c_int64(v.size))


def kv4_pack(x: np.ndarray):
    x = _f32(x).reshape(-1)
    w = np.empty(x.size // 8, dtype=np.uint32)
    sc = np.empty(x.size // 32, dtype=np.float32)
    lib().orc_kv4_pack(_p(x), C.c_int64(x.size), _p(w), _p(sc))
    return w, sc


def kv4_unpack(w: np.ndarray, sc: np.ndarray, n: int) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint32)
    sc = _f32(sc)
    L = lib()
    return np.array([L.orc_kv4_get(_p(w), _p(sc), C.c_int64(i)) for i in range(n)], dtype=np.float32)


def rope_inv(n_rot: int, base: float) -> np.ndarray:
    inv = np.empty(n_rot // 2, dtype=np.float32)
    lib().orc_rope_inv(C.c_int(n_rot), C.c_float(base), _p(inv))
    return inv


def rope_inv_yarn(n_rot: int, base: float, ctx_train: int, ctx: int):
    """(inverse frequencies, mscale) for a context of ctx positions of a model trained on ctx_train."""
    inv = np.empty(n_rot // 2, dtype=np.float32)
    f = lib().orc_rope_inv_yarn
    f.restype = C.c_float
    ms = f(C.c_int(n_rot), C.c_float(base), C.c_int64(ctx_train), C.c_int64(ctx), _p(inv))
    return inv, float(ms)


def make_cfg(**kw) -> Cfg:
    c = Cfg()
    defaults = dict(n_layers=4, d=2048, hc=0, hc_lr=0, n_head=16, n_kv=2, hd=256, n_rot=64, rope_base=1e7, eps=1e-6,
                    n_exp=512, top_k=10, ff_exp=512, ff_sh=512, lin_nk=16, lin_nv=32, lin_dk=128, lin_dv=128,
                    conv_k=4, full_every=4, vocab=151936, max_ctx=4096, kv_bits=0, kv_recent=1024)
    defaults.update(kw)
    for k, v in defaults.items():
        setattr(c, k, v)
    return c


def moe(cfg: Cfg, router: QMat, gate_e: QMat, up_e: QMat, down_e: QMat, sh_gate: QMat, sh_up: QMat, sh_down: QMat,
        sh_gate_inp: np.ndarray, x: np.ndarray):
    x = _f32(x).reshape(-1, cfg.d)
    t = x.shape[0]
    y = np.empty((t, cfg.d), dtype=np.float32)
    sel = np.empty((t, cfg.top_k), dtype=np.int32)
    selw = np.empty((t, cfg.top_k), dtype=np.float32)
    sgi = _f32(sh_gate_inp)
    lib().orc_moe(C.byref(cfg), C.byref(router.c), C.byref(gate_e.c), C.byref(up_e.c), C.byref(down_e.c),
                  C.byref(sh_gate.c), C.byref(sh_up.c), C.byref(sh_down.c), _p(sgi), _p(x), C.c_int(t), _p(y), _p(sel), _p(selw))
    return y, sel, selw


def linear_core(cfg: Cfg, qkv, z, beta, alpha, a, dt, conv_w, norm_w, conv_state, ssm):
    """One sequence, t tokens.  conv_state and ssm are updated in place (float32, C-contiguous)."""
    qkv, z, beta, alpha = _f32(qkv), _f32(z), _f32(beta), _f32(alpha)
    a, dt, conv_w, norm_w = _f32(a), _f32(dt), _f32(conv_w), _f32(norm_w)
    assert conv_state.dtype == np.float32 and ssm.dtype == np.float32 and conv_state.flags.c_contiguous and ssm.flags.c_contiguous
    ch = 2 * cfg.lin_nk * cfg.lin_dk + cfg.lin_nv * cfg.lin_dv
    t = qkv.size // ch
    out = np.empty((t, cfg.lin_nv * cfg.lin_dv), dtype=np.float32)
    lib().orc_linear_core(C.byref(cfg), _p(qkv), _p(z), _p(beta), _p(alpha), _p(a), _p(dt), _p(conv_w), _p(norm_w),
                          _p(conv_state), _p(ssm), C.c_int(t), _p(out))
    return out


def qsa_pool(cfg: Cfg, ratio: int, ik, ikn, inv, b: int, mscale=1.0) -> np.ndarray:
    """Pooled, normed and roped key of block b from the raw index keys ik [>= (b+1)*ratio][idx_hd]."""
    ik, ikn = _f32(ik), _f32(ikn)
    ihd = ik.shape[1]
    inv = np.concatenate([_f32(inv)[:cfg.n_rot // 2], np.array([mscale], np.float32)])
    out = np.empty(ihd, np.float32)
    lib().orc_qsa_pool(C.byref(cfg), C.c_int(ratio), C.c_int(ihd), _p(ik), _p(ikn), _p(inv), C.c_int64(b), _p(out))
    return out


def qsa_select(cfg: Cfg, budget: int, ratio: int, iq_raw, iqn, inv, ib, pos: int, mscale=1.0):
    """(selected blocks ascending, margin) for the query at pos; ([], inf) in the dense range.  iq_raw [idx_nh][idx_hd]."""
    iq_raw, iqn, ib = _f32(iq_raw), _f32(iqn), _f32(ib)
    inh, ihd = iq_raw.shape
    inv = np.concatenate([_f32(inv)[:cfg.n_rot // 2], np.array([mscale], np.float32)])
    blocks = np.zeros(budget // ratio + 1, np.int32)
    mg = C.c_float(float("inf"))
    k = lib().orc_qsa_select(C.byref(cfg), C.c_int(budget), C.c_int(ratio), C.c_int(inh), C.c_int(ihd), _p(iq_raw), _p(iqn), _p(inv), _p(ib),
                             C.c_int64(pos), _p(blocks), C.byref(mg))
    return blocks[:k].copy(), float(mg.value)


def attn_core(cfg: Cfg, qf, kf, vf, qn, kn, inv, kc, vc, pos, packed=None, q4n=0, mscale=1.0, ps=None):
    """One new token at position pos.  kc/vc [>=pos+1][n_kv*hd] f32, updated in place at row pos."""
    qf, kf, vf, qn, kn = _f32(qf), _f32(kf), _f32(vf), _f32(qn), _f32(kn)
    inv = np.concatenate([_f32(inv)[:cfg.n_rot // 2], np.array([mscale], np.float32)])   # the C side reads mscale behind the table
    att = np.empty(cfg.n_head * cfg.hd, dtype=np.float32)
    if packed is None:
        kw = ks = vw = vs = None
    else:
        kw, ks, vw, vs = (_p(a) for a in packed)
    if ps is not None:
        ps = np.ascontiguousarray(ps, dtype=np.int64)
    lib().orc_attn_core_sel(C.byref(cfg), _p(qf), _p(kf), _p(vf), _p(qn), _p(kn), _p(inv), _p(kc), _p(vc), C.c_int64(pos),
                            kw, ks, vw, vs, C.c_int64(q4n), _p(ps) if ps is not None else None, C.c_int64(0 if ps is None else ps.size), _p(att))
    return att


class Model:
    def __init__(self, cfg: Cfg):
        self.cfg = cfg
        self._keep = []
        self.h = C.c_void_p(lib().orc_model_new(C.byref(cfg)))

    def set_mat(self, layer: int, role: str, m: QMat):
        self._keep.append(m)
        assert lib().orc_model_set_mat(self.h, C.c_int(layer), C.c_int(ROLE[role]), C.byref(m.c)) == 0

    def set_vec(self, layer: int, role: str, v: np.ndarray):
        v = _f32(v).reshape(-1)
        assert lib().orc_model_set_vec(self.h, C.c_int(layer), C.c_int(ROLE[role]), _p(v), C.c_int64(v.size)) == 0

    def set_ctx_train(self, ctx_train: int):
        """YaRN rope scaling when cfg.max_ctx exceeds the trained context."""
        lib().orc_model_set_ctx_train(self.h, C.c_int64(ctx_train))

    def set_indexer(self, budget: int, ratio: int, n_head: int, head_dim: int):
        """QSA block-sparse attention: layers that hold IDX_Q / IDX_K attend to budget / ratio blocks of ratio tokens."""
        lib().orc_model_set_indexer(self.h, C.c_int(budget), C.c_int(ratio), C.c_int(n_head), C.c_int(head_dim))

    def set_ple(self, ngram: int, per_gram: int, conv_k: int, eos: int, dim: int, mult, off, vocab):
        """Per-layer n-gram embeddings: layers that hold PLE_KEY add them at their start (ple, qwen4exp_gguf.rs:1409-1434)."""
        a = lambda v: np.ascontiguousarray(v, dtype=np.uint64)
        mult, off, vocab = a(mult), a(off), a(vocab)
        assert mult.size == ngram and off.size == vocab.size == (ngram - 1) * per_gram
        self.ple = (ngram, per_gram)
        lib().orc_model_set_ple(self.h, C.c_int(ngram), C.c_int(per_gram), C.c_int(conv_k), C.c_uint32(eos), C.c_int(dim),
                                mult.ctypes.data_as(C.c_void_p), off.ctypes.data_as(C.c_void_p), vocab.ctypes.data_as(C.c_void_p))

    def ple_token(self, layer: int, nrm_all: np.ndarray, key: np.ndarray, val: np.ndarray, x: np.ndarray, pos: int):
        """One token's injection (ple, qwen4exp_gguf.rs:1409-1434): x and nrm_all[pos] are updated in place."""
        assert nrm_all.dtype == np.float32 and x.dtype == np.float32 and nrm_all.flags.c_contiguous and x.flags.c_contiguous
        k = np.ascontiguousarray(key, dtype=np.float32); v = np.ascontiguousarray(val, dtype=np.float32)
        lib().orc_ple_token(self.h, C.c_int(layer), nrm_all.ctypes.data_as(C.c_void_p), k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p),
                            x.ctypes.data_as(C.c_void_p), C.c_int64(pos))

    def ple_hash(self, ctx):
        """Table rows of a token with context `ctx` (the token, then its predecessors; -1 = none)."""
        ngram, per = self.ple
        c = np.ascontiguousarray(ctx, dtype=np.int64); assert c.size == ngram
        rows = np.zeros((ngram - 1) * per, dtype=np.int64)
        lib().orc_ple_hash(self.h, c.ctypes.data_as(C.c_void_p), rows.ctypes.data_as(C.c_void_p))
        return rows

    def new_state(self) -> "State":
        return State(self)

    def __del__(self):
        try:
            lib().orc_model_free(self.h)
        except Exception:
            pass


class State:
    def __init__(self, model: Model):
        self.model = model
        self.h = C.c_void_p(lib().orc_state_new(model.h))

    def fill_kv(self, ai: int, k: np.ndarray, v: np.ndarray):
        k, v = _f32(k), _f32(v)
        row = self.model.cfg.n_kv * self.model.cfg.hd
        assert lib().orc_state_fill_kv(self.h, C.c_int(ai), _p(k), _p(v), C.c_int64(k.size // row)) == 0

    def set_pos(self, pos: int):
        lib().orc_state_set_pos(self.h, C.c_int64(pos))

    def forward(self, ids) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
        logits = np.empty(self.model.cfg.vocab, dtype=np.float32)
        rc = lib().orc_forward(self.model.h, self.h, _p(ids), C.c_int(ids.size), _p(logits))
        if rc:
            raise RuntimeError(f"orc_forward failed: {rc}")
        return logits

    def last_residual(self) -> np.ndarray:
        """Final residual rows [t][max(hc, 1) * d] of the tokens of the last forward call."""
        c = self.model.cfg
        buf = np.empty(4096 * max(c.hc, 1) * c.d, np.float32)
        n = lib().orc_last_residual(self.h, _p(buf), C.c_int64(buf.size))
        assert n >= 0
        return buf[:n].reshape(-1, max(c.hc, 1) * c.d).copy()

    def mtp_cell(self, R, emb, pos: int, c0: int, window: int, full: bool):
        """This state belongs to a drafter model (one attention layer + MTP tensors): one drafter cell.  Returns (s, rr) when full."""
        c = self.model.cfg
        R, emb = _f32(R).reshape(-1), _f32(emb).reshape(-1)
        s = np.empty(c.d, np.float32); rr = np.empty(c.hc * c.d, np.float32)
        lib().orc_mtp_cell(self.model.h, self.h, _p(R), _p(emb), C.c_int64(pos), C.c_int64(c0), C.c_int(window), C.c_int(1 if full else 0), _p(s), _p(rr))
        return (s, rr) if full else None

    def margins(self):
        a, b = C.c_float(), C.c_float()
        lib().orc_last_margins(self.h, C.byref(a), C.byref(b))
        return a.value, b.value

    def qsa_margin(self) -> float:
        """Smallest gap between the last block taken and the best block left out over the sparse queries of the last
        forward call (inf when none was sparse): a tiny value marks a selection that rounding may turn."""
        return float(lib().orc_last_qsa_margin(self.h))

    def __del__(self):
        try:
            lib().orc_state_free(self.h)
        except Exception:
            pass
