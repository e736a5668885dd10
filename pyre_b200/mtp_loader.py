"""Loader for the MTP drafter's tensor file: the host side of Mtp::load (src/model/mtp.rs:104-123 of the reference).

The reference keeps the drafter layer in a safetensors file of BF16 tensors (8-byte little-endian header length, a JSON
header with dtype / shape / data_offsets per tensor, then the data; names carry an `mtp.` and a `layers.0.` prefix that
St::open strips, mtp.rs:27-44) and builds int8 matrices from it at load.  Here the matrices become GGUF Q8_0 blocks
(one f16 scale per 32 values, rounded as ggml's quantize_row_q8_0 does), the small hyper-connection and router matrices stay f32, the norm
vectors get the 1 the reference adds (`norm`, :47), the fused gate_up_proj is split into the gate and the up tensor,
and the head is the rows of the main model's output matrix for the draft vocabulary, in their own block bytes.

    spec = drafter_spec(read_safetensors(path), main_cfg)          # list of ('mat', role, type, rows, cols, bytes) / ('vec', role, array)
    drafter = load_drafter(ctx, path, main_model_cfg, head_qmat, vocab_ids, window=128)
    state.attach_drafter(drafter, vocab_ids)
"""
from __future__ import annotations

import json
import struct

import numpy as np

from . import Ctx, F32, Q8_0, QMat, make_cfg
from .model import Model


class MtpFileError(ValueError):
    pass


def read_safetensors(path) -> dict:
    """name (prefixes `mtp.` and `layers.0.` stripped) -> f32 array, from a file of BF16 tensors."""
    raw = np.fromfile(path, dtype=np.uint8)
    if raw.size < 8:
        raise MtpFileError(f"{path}: truncated")
    (n,) = struct.unpack("<Q", raw[:8].tobytes())
    if 8 + n > raw.size:
        raise MtpFileError(f"{path}: header of {n} bytes in a file of {raw.size}")
    header = json.loads(raw[8:8 + n].tobytes())
    base, out = 8 + n, {}
    for name, v in header.items():
        if name == "__metadata__":
            continue
        if v["dtype"] != "BF16":
            raise MtpFileError(f"{name}: dtype {v['dtype']} (BF16 expected)")
        a, b = v["data_offsets"]
        shape = tuple(int(x) for x in v["shape"])
        if base + b > raw.size or (b - a) != 2 * int(np.prod(shape, dtype=np.int64)):
            raise MtpFileError(f"{name}: data range {a}..{b} does not fit shape {shape}")
        bits = raw[base + a:base + b].view("<u2").astype(np.uint32) << 16
        key = name
        for pre in ("mtp.", "layers.0."):
            if key.startswith(pre):
                key = key[len(pre):]
        out[key] = bits.view(np.float32).reshape(shape)
    return out


def write_safetensors(path, tensors: dict):
    """The inverse, for tests: f32 arrays stored as BF16 (truncation of the low mantissa half, as a checkpoint converter does)."""
    header, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        a = np.ascontiguousarray(arr, dtype=np.float32)
        b = (a.view(np.uint32) >> 16).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b); off += len(b)
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h))); f.write(h)
        for b in blobs:
            f.write(b)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """Rows of f32 -> GGUF Q8_0 bytes ([f16 d][32 x i8] per 32 values; d = max|x| / 127, q = roundf(x * (1 / d))): ggml's
    quantize_row_q8_0, byte for byte what gguf-py writes."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    if cols % 32:
        raise MtpFileError(f"{cols} columns are not a multiple of 32")
    b = x.reshape(rows, cols // 32, 32)
    df = np.abs(b).max(axis=2) / np.float32(127.0)                 # the inverse comes from the f32 scale; the f16 rounding is only stored
    d = df.astype(np.float16)
    inv = np.where(df > 0, np.float32(1.0) / np.where(df > 0, df, np.float32(1.0)), np.float32(0.0)).astype(np.float32)
    v = b * inv[:, :, None]
    q = np.clip(np.sign(v) * np.floor(np.abs(v) + 0.5), -127, 127).astype(np.int8)     # roundf: halves away from zero, as ggml
    out = np.empty((rows, cols // 32, 34), dtype=np.uint8)
    out[:, :, :2] = d.view(np.uint8).reshape(rows, cols // 32, 2)
    out[:, :, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def drafter_spec(t: dict, main_cfg):
    """The file's tensors under the library's roles: (cfg keywords of the drafter model, list of items)."""
    d, hc = main_cfg.d, main_cfg.hc
    need = lambda n: t[n] if n in t else (_ for _ in ()).throw(MtpFileError(f"mtp tensor {n}"))
    items = []

    def q8(role, arr, layer=0):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        items.append(("mat", layer, role, Q8_0, arr.shape[0], arr.shape[1], quantize_q8_0(arr)))

    def f32(role, arr, layer=0):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        items.append(("mat", layer, role, F32, arr.shape[0], arr.shape[1], arr.view(np.uint8).reshape(-1)))

    def vec(role, arr, layer=0, plus_one=False):
        a = np.ascontiguousarray(arr, dtype=np.float32).reshape(-1)
        items.append(("vec", layer, role, a + 1.0 if plus_one else a))

    def hyper(prefix, role, layer, inject):
        vec(f"{role}_NORM", need(f"{prefix}.hc_norm.weight"), layer, plus_one=True)
        f32(f"{role}_DOWN", need(f"{prefix}.input_mix_weight_down.weight"), layer)
        f32(f"{role}_UP", need(f"{prefix}.input_mix_weight_up.weight"), layer)
        if inject:
            f32(f"{role}_INJECT", need(f"{prefix}.block_inject_weight.weight"), layer)

    vec("MTP_PRE_E", need("pre_fc_norm_embedding.weight"), -1, plus_one=True)
    vec("MTP_PRE_H", need("pre_fc_norm_hidden.weight"), -1, plus_one=True)
    q8("MTP_FC_E", need("fc_embedding.weight"), -1)
    q8("MTP_FC_H", need("fc_hidden.weight"), -1)
    hyper("attn_hyper_connection", "HCA", 0, True)
    hyper("mlp_hyper_connection", "HCF", 0, True)
    hyper("hyper_connection_mixer", "OUT_HC", -1, False)
    for role, n in (("ATTN_Q", "q_proj"), ("ATTN_K", "k_proj"), ("ATTN_V", "v_proj"), ("ATTN_O", "o_proj")):
        q8(role, need(f"self_attn.{n}.weight"))
    vec("ATTN_Q_NORM", need("self_attn.q_norm.weight"), plus_one=True)
    vec("ATTN_K_NORM", need("self_attn.k_norm.weight"), plus_one=True)
    f32("ROUTER", need("mlp.gate.weight"))
    gu, dn = need("mlp.experts.gate_up_proj"), need("mlp.experts.down_proj")       # [ne][2 ff][d], [ne][d][ff]
    ne, ff = dn.shape[0], dn.shape[2]
    if gu.shape != (ne, 2 * ff, d) or dn.shape != (ne, d, ff):
        raise MtpFileError(f"expert tensors {gu.shape} / {dn.shape} for width {d}")
    q8("EXP_GATE", gu[:, :ff, :].reshape(ne * ff, d))
    q8("EXP_UP", gu[:, ff:, :].reshape(ne * ff, d))
    q8("EXP_DOWN", dn.reshape(ne * d, ff))
    sg = need("mlp.shared_expert.gate_proj.weight")
    q8("SH_GATE", sg); q8("SH_UP", need("mlp.shared_expert.up_proj.weight")); q8("SH_DOWN", need("mlp.shared_expert.down_proj.weight"))
    vec("SH_GATE_INP", need("mlp.shared_expert_gate.weight"))
    lr = need("attn_hyper_connection.input_mix_weight_down.weight").shape[0]
    cfgkw = dict(n_layers=1, full_every=1, d=d, hc=hc, hc_lr=lr, n_head=main_cfg.n_head, n_kv=main_cfg.n_kv, hd=main_cfg.hd, n_rot=main_cfg.n_rot,
                 rope_base=main_cfg.rope_base, eps=main_cfg.eps, n_exp=ne, top_k=min(main_cfg.top_k, ne), ff_exp=ff, ff_sh=sg.shape[0],
                 max_ctx=main_cfg.max_ctx, kv_bits=0, kv_recent=main_cfg.kv_recent)
    return cfgkw, items


def load_drafter(ctx: Ctx, path, main_cfg, head: QMat, vocab_ids, window: int = 128) -> Model:
    """The drafter model of the file at `path` for a main model of `main_cfg`; `head` = the main model's output matrix (its
    rows of `vocab_ids`, in their block bytes, become the draft-vocabulary head)."""
    ids = np.ascontiguousarray(vocab_ids, dtype=np.uint32).reshape(-1)
    cfgkw, items = drafter_spec(read_safetensors(path), main_cfg)
    cfg = make_cfg(vocab=int(ids.size), **cfgkw)
    m = Model(ctx, cfg)
    for it in items:
        if it[0] == "mat":
            _, layer, role, ty, rows, cols, raw = it
            m.set_tensor(layer, role, QMat.upload(ctx, ty, rows, cols, raw))
        else:
            _, layer, role, arr = it
            m.set_vec(layer, role, arr)
    rows = np.concatenate([head.raw_rows(int(i), 1) for i in ids])
    m.set_tensor(-1, "OUTPUT", QMat.upload(ctx, head.ty, int(ids.size), head.cols, rows))
    m.set_mtp(window)
    m.finalize()
    return m
