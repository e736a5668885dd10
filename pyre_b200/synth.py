"""Seeded synthetic Qwen-Next-style models (random-init weights of the benchmark shapes).

`model_spec` only *describes* the tensors: quantized matrices by (ggml type, rows, cols,
tensor id) for the counter-based block generator, f32 vectors as numpy arrays.  The same
description can therefore be realised on the GPU (`build_model`, device-side generation) and
by any independent checker that implements the documented generator.

Block fields follow the benchmark's config 0: fp16 super-block scale d ~ |N(0, 0.02)|,
uniform sub-scales, grid indices and sign bits (see the generator notes in csrc/pb_dequant.cu).
"""
from __future__ import annotations

import numpy as np

from . import Cfg, Ctx, F32, IQ3_S, QMat, ROLE
from . import parallel
from .model import Model


def tensor_id(layer: int, role: str) -> int:
    return (layer + 1) * 64 + ROLE[role]


def is_full(cfg: Cfg, il: int) -> bool:
    return cfg.full_every > 0 and (il + 1) % cfg.full_every == 0


def ple_geometry(layers, ngram: int = 3, per_gram: int = 2, conv_k: int = 4, eos: int = 2, dim: int = 256, head_vocab: int = 997):
    """Geometry of per-layer n-gram embeddings for a synthetic model (the reference's metadata keys `ple.*`,
    src/model/qwen4exp_gguf.rs:468-480): odd 64-bit multipliers, heads of slightly different vocabulary sizes laid end to end."""
    nh = (ngram - 1) * per_gram
    vocab = [head_vocab + 2 * i for i in range(nh)]
    off = [int(sum(vocab[:i])) for i in range(nh)]
    mult = [(0x9E3779B97F4A7C15 * (2 * i + 1) + 0x632BE59BD9B4E019 * i) % (1 << 64) | 1 for i in range(ngram)]
    return dict(layers=list(layers), ngram=ngram, per_gram=per_gram, conv_k=conv_k, eos=eos, dim=dim, mult=mult, off=off, vocab=vocab)


def model_spec(cfg: Cfg, seed: int = 0, qtype: int = IQ3_S, indexer=None, ple=None):
    """List of ('mat', layer, role, type, rows, cols, tid) and ('vec', layer, role, array).  indexer = (budget, ratio, heads,
    head dim) adds the QSA indexer tensors to every attention layer; ple = ple_geometry(...) adds the n-gram embedding table and
    the tensors of the layers it names."""
    rng = np.random.default_rng(seed)
    d, hd = cfg.d, cfg.hd
    ch = 2 * cfg.lin_nk * cfg.lin_dk + cfg.lin_nv * cfg.lin_dv
    spec = []

    def mat(layer, role, rows, cols, t=qtype):
        spec.append(("mat", layer, role, t, rows, cols, tensor_id(layer, role)))

    def vec(layer, role, arr):
        spec.append(("vec", layer, role, np.ascontiguousarray(arr, dtype=np.float32)))

    def gamma(n):  # norm weights, stored pre-folded as (1 + w) like the reference's GGUF
        return 1.0 + 0.1 * rng.standard_normal(n)

    hc, lr = cfg.hc, cfg.hc_lr

    def hyper(layer, prefix, inject=True):
        # one hyper-connection mix (Hc, src/model/qwen4exp_gguf.rs:28, 492): per-stream norm weights and small f32 matrices
        vec(layer, f"{prefix}_NORM", gamma(hc * d))
        mat(layer, f"{prefix}_DOWN", lr, hc * d, F32)
        mat(layer, f"{prefix}_UP", hc * d, lr, F32)
        if inject:
            mat(layer, f"{prefix}_INJECT", hc, hc * d, F32)

    mat(-1, "TOKEN_EMBD", cfg.vocab, d)
    mat(-1, "OUTPUT", cfg.vocab, d)
    if hc > 0:
        hyper(-1, "OUT_HC", inject=False)
    else:
        vec(-1, "OUT_NORM", gamma(d))
    if ple:
        mat(-1, "PLE_TAB", int(sum(ple["vocab"])), ple["dim"])
    for il in range(cfg.n_layers):
        if ple and il in ple["layers"]:
            w, ein = max(hc, 1) * d, (ple["ngram"] - 1) * ple["per_gram"] * ple["dim"]
            mat(il, "PLE_KEY", w, ein)
            mat(il, "PLE_VALUE", d, ein)
            vec(il, "PLE_NORM_KEY", gamma(w))
            vec(il, "PLE_NORM_QUERY", gamma(w))
            vec(il, "PLE_NORM_CONV", gamma(w))
            vec(il, "PLE_CONV", 0.5 * rng.standard_normal((w, ple["conv_k"])))
        if hc > 0:
            hyper(il, "HCA")
            hyper(il, "HCF")
        else:
            vec(il, "ATTN_NORM", gamma(d))
            vec(il, "FFN_NORM", gamma(d))
        if is_full(cfg, il):
            mat(il, "ATTN_Q", cfg.n_head * 2 * hd, d)
            mat(il, "ATTN_K", cfg.n_kv * hd, d)
            mat(il, "ATTN_V", cfg.n_kv * hd, d)
            mat(il, "ATTN_O", d, cfg.n_head * hd)
            vec(il, "ATTN_Q_NORM", gamma(hd))
            vec(il, "ATTN_K_NORM", gamma(hd))
            if indexer:
                _, _, inh, ihd = indexer
                mat(il, "IDX_Q", inh * ihd, d)
                mat(il, "IDX_K", ihd, d)
                vec(il, "IDX_Q_NORM", gamma(ihd))
                vec(il, "IDX_K_NORM", gamma(ihd))
        else:
            mat(il, "LIN_QKV", ch, d)
            mat(il, "LIN_Z", cfg.lin_nv * cfg.lin_dv, d)
            mat(il, "LIN_BETA", cfg.lin_nv, d)
            mat(il, "LIN_ALPHA", cfg.lin_nv, d)
            mat(il, "LIN_OUT", d, cfg.lin_nv * cfg.lin_dv)
            vec(il, "LIN_A", -np.exp(0.5 * rng.standard_normal(cfg.lin_nv)))      # ssm_a = -exp(A_log)
            vec(il, "LIN_DT", rng.standard_normal(cfg.lin_nv))
            vec(il, "LIN_CONV", 0.5 * rng.standard_normal((ch, cfg.conv_k)))
            vec(il, "LIN_NORM", gamma(cfg.lin_dv))
        mat(il, "ROUTER", cfg.n_exp, d, F32)                                        # f32 ~ N(0, 0.02)
        mat(il, "EXP_GATE", cfg.n_exp * cfg.ff_exp, d)
        mat(il, "EXP_UP", cfg.n_exp * cfg.ff_exp, d)
        mat(il, "EXP_DOWN", cfg.n_exp * d, cfg.ff_exp)
        mat(il, "SH_GATE", cfg.ff_sh, d)
        mat(il, "SH_UP", cfg.ff_sh, d)
        mat(il, "SH_DOWN", d, cfg.ff_sh)
        vec(il, "SH_GATE_INP", 0.02 * rng.standard_normal(d))
    return spec


def build_model(ctx: Ctx, cfg: Cfg, spec, seed: int = 0, ep_rank: int = 0, ep_world: int = 1, ctx_train: int = 0, indexer=None, ple=None) -> Model:
    m = Model(ctx, cfg)
    if ple:
        m.set_ple(ple["ngram"], ple["per_gram"], ple["conv_k"], ple["eos"], ple["dim"], ple["mult"], ple["off"], ple["vocab"])
    if ctx_train:
        m.set_ctx_train(ctx_train)
    if indexer:
        m.set_indexer(*indexer)
    for item in spec:
        if item[0] == "mat":
            _, layer, role, t, rows, cols, tid = item
            if ep_world > 1 and role in ("EXP_GATE", "EXP_UP", "EXP_DOWN"):
                # this rank's contiguous shard of the fused expert tensor
                per = rows // cfg.n_exp
                lo, hi = parallel.ep_range(cfg.n_exp, ep_rank, ep_world)
                m.set_tensor(layer, role, QMat.synth_rows(ctx, t, (hi - lo) * per, cols, seed, tid, lo * per))
            else:
                m.set_tensor(layer, role, QMat.synth(ctx, t, rows, cols, seed, tid))
        else:
            _, layer, role, arr = item
            m.set_vec(layer, role, arr)
    m.finalize(ep_rank, ep_world)
    return m
