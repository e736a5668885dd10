"""GGUF reader and qwen4exp model loader: the host side of `Model::load`.

`Gguf.open` restates the reference's reader (Gguf::open, src/model/gguf_q.rs:250-336): magic, version, tensor and
key/value counts, the typed metadata values (integers, floats, bools, strings, arrays), the tensor infos (name, shape
innermost dimension first, ggml type id, offset) and the data section aligned to `general.alignment` (32 by default);
a file named `<stem>-00001-of-0000N.gguf` brings in all N shards, later shards only add tensors and missing keys.
Tensor bytes are memory-mapped, never copied on the host.

`load_model` restates the reference's loader (Model::load, src/model/qwen4exp_gguf.rs:462-512): the config from the
`qwen4exp.*` metadata keys and the tensors by their `blk.N.*` names, uploaded in their GGUF block bytes
(pb_qmat_upload) and bound to the library's roles.  Expert-parallel ranks upload only their rows of the three fused
expert tensors.  The sparse-attention indexer (`attention.indexer.*` keys, `blk.N.indexer.*` tensors) and the trained context
are handed to the library when the file has them.  Per-layer-input embeddings (PLE) are not part of the built path and make
the loader refuse the file instead of ignoring them.
"""
from __future__ import annotations

import mmap
import re
import struct
from pathlib import Path

import numpy as np

from . import Ctx, QMat, make_cfg, type_geom
from . import parallel
from .model import Model

_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class GgufError(ValueError):
    pass


class _Rd:
    def __init__(self, buf):
        self.b, self.p = buf, 0

    def take(self, n: int):
        if self.p + n > len(self.b):
            raise GgufError("truncated GGUF")
        s = self.b[self.p:self.p + n]
        self.p += n
        return s

    def fmt(self, f: str):
        return struct.unpack(f, self.take(struct.calcsize(f)))[0]

    def string(self) -> str:
        n = self.fmt("<Q")
        return bytes(self.take(n)).decode("utf-8", "replace")

    def value(self, t: int):
        if t in _SCALARS:
            return self.fmt(_SCALARS[t])
        if t == 8:
            return self.string()
        if t == 9:
            et, n = self.fmt("<I"), self.fmt("<Q")
            return [self.value(et) for _ in range(n)]
        raise GgufError(f"bad GGUF value type {t}")


def shard_paths(p: Path):
    """All shards of a split GGUF given any one of them (`-NNNNN-of-MMMMM.gguf`), or the single file."""
    m = re.match(r"^(.*)-(\d{5})-of-(\d{5})\.gguf$", p.name)
    if not m:
        return [p]
    total = int(m.group(3))
    out = [p.with_name(f"{m.group(1)}-{k:05d}-of-{total:05d}.gguf") for k in range(1, total + 1)]
    for s in out:
        if not s.exists():
            raise GgufError(f"missing shard {s}")
    return out


class Gguf:
    def __init__(self):
        self.paths, self.maps, self.meta, self.tensors = [], [], {}, {}

    @classmethod
    def open(cls, first) -> "Gguf":
        g = cls()
        g.paths = shard_paths(Path(first))
        for si, p in enumerate(g.paths):
            f = open(p, "rb")
            mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            f.close()
            r = _Rd(memoryview(mm))
            if bytes(r.take(4)) != b"GGUF":
                raise GgufError(f"{p} is not GGUF")
            _ver, nt, nkv = r.fmt("<I"), r.fmt("<Q"), r.fmt("<Q")
            align = 32
            for _ in range(nkv):
                k = r.string()
                v = r.value(r.fmt("<I"))
                if k == "general.alignment":
                    align = int(v)
                if si == 0 or k not in g.meta:
                    g.meta[k] = v
            infos = []
            for _ in range(nt):
                name = r.string()
                nd = r.fmt("<I")
                shape = [r.fmt("<Q") for _ in range(nd)]
                infos.append((name, shape, r.fmt("<I"), r.fmt("<Q")))
            data = -(-r.p // align) * align
            for name, shape, ty, off in infos:
                g.tensors[name] = (shape, ty, si, data + off)
            g.maps.append(mm)
        return g

    def arch(self) -> str:
        return str(self.meta.get("general.architecture", ""))

    def has(self, name: str) -> bool:
        return name in self.tensors

    def shape(self, name: str):
        return self.tensors[name][0]

    def mat(self, name: str):
        """(ggml type, rows, cols, bytes) of a tensor viewed as a matrix [prod(shape[1:]), shape[0]] (gguf_q.rs:319-325)."""
        if name not in self.tensors:
            raise GgufError(f"missing tensor {name}")
        shape, ty, si, off = self.tensors[name]
        cols = int(shape[0])
        rows = max(1, int(np.prod(shape[1:], dtype=np.int64))) if len(shape) > 1 else 1
        el, bs = type_geom(ty)
        if cols % el:
            raise GgufError(f"{name}: row of {cols} is not a multiple of the block of {el}")
        nbytes = rows * (cols // el) * bs
        if off + nbytes > len(self.maps[si]):
            raise GgufError(f"{name}: data runs past the end of the file")
        return ty, rows, cols, np.frombuffer(self.maps[si], dtype=np.uint8, count=nbytes, offset=off)

    def file_bytes(self) -> int:
        return sum(len(m) for m in self.maps)

    def close(self):
        for m in self.maps:
            try:
                m.close()
            except BufferError:      # numpy views still alive: the map goes with them
                pass
        self.maps = []


_HC = (("norm", "NORM"), ("down", "DOWN"), ("up", "UP"), ("inject", "INJECT"))


def load_model(ctx: Ctx, path, max_ctx: int = 4096, kv_bits: int = 4, kv_recent: int = 1024, ep_rank: int = 0, ep_world: int = 1) -> Model:
    """Open a qwen4exp GGUF and build the device model (Model::load + the uploads of attach_gpu)."""
    g = Gguf.open(path)
    a = g.arch()
    if a != "qwen4exp":
        raise GgufError(f"{path}: arch '{a}' is not qwen4exp")

    def k(s, default=None):
        v = g.meta.get(f"{a}.{s}", default)
        if v is None:
            raise GgufError(f"gguf key {a}.{s}")
        return v

    cfg = make_cfg(n_layers=int(k("block_count")), d=int(k("embedding_length")), hc=int(k("hyper_connection.count")), hc_lr=int(k("hyper_connection.low_rank")),
                   n_head=int(k("attention.head_count")), n_kv=int(k("attention.head_count_kv")), hd=int(k("attention.key_length")), n_rot=int(k("rope.dimension_count")),
                   rope_base=float(k("rope.freq_base")), eps=float(k("attention.layer_norm_rms_epsilon")), n_exp=int(k("expert_count")), top_k=int(k("expert_used_count")),
                   ff_exp=int(k("expert_feed_forward_length")), ff_sh=int(g.shape("blk.0.ffn_gate_shexp.weight")[1]), lin_nk=int(k("ssm.group_count")), lin_nv=int(k("ssm.time_step_rank")),
                   lin_dk=int(k("ssm.state_size")), lin_dv=int(k("ssm.state_size")), conv_k=int(k("ssm.conv_kernel")), full_every=int(k("full_attention_interval", 4)),
                   vocab=int(g.shape("token_embd.weight")[1]), max_ctx=max_ctx, kv_bits=kv_bits, kv_recent=kv_recent)
    m = Model(ctx, cfg)
    # QSA indexer (Cfg :24-25, :481-489): budget = indexer.top_k, block size = the largest compress ratio
    first_attn = cfg.full_every - 1
    idx_nh = int(k("attention.indexer.head_count", 0))
    has_idx = idx_nh > 0 and first_attn >= 0 and g.has(f"blk.{first_attn}.indexer.q_proj.weight")
    if has_idx:
        ratios = g.meta.get(f"{a}.attention.compress_ratios") or [4]
        m.set_indexer(int(k("attention.indexer.top_k", 2048)), max(1, max(int(r) for r in ratios)), idx_nh, int(k("attention.indexer.key_length", 128)))
    m.set_ctx_train(int(g.meta.get(f"{a}.context_length", 0)))   # a longer max_ctx is YaRN-scaled (Model::load :490-517)
    # per-layer n-gram embeddings (Cfg ple_* :468, 477-480): the layers named by ple.layers hold the tensors
    ple_layers = [int(v) for v in (g.meta.get(f"{a}.ple.layers") or [])]
    if ple_layers:
        u64 = lambda key: [int(v) for v in (g.meta.get(f"{a}.{key}") or [])]
        m.set_ple(int(k("ple.ngram_size")), int(k("ple.heads_per_ngram")), int(k("ple.conv_kernel")), int(k("ple.eos_token_id", 0)), int(k("embedding_length_per_layer_input")),
                  u64("ple.layer_multipliers"), u64("ple.head_offsets"), u64("ple.head_vocab_sizes"))

    def mat(layer, role, name, expert_rows=False):
        ty, rows, cols, raw = g.mat(name)
        if expert_rows and ep_world > 1:          # this rank's contiguous shard of the fused expert tensor
            per = rows // cfg.n_exp
            lo, hi = parallel.ep_range(cfg.n_exp, ep_rank, ep_world)
            rb = raw.size // rows
            raw, rows = raw[lo * per * rb:hi * per * rb], (hi - lo) * per
        m.set_tensor(layer, role, QMat.upload(ctx, ty, rows, cols, raw))

    def vec(layer, role, name):
        ty, rows, cols, raw = g.mat(name)
        if ty == 0:
            arr = raw.view(np.float32)
        elif ty == 1:
            arr = raw.view(np.float16).astype(np.float32)
        else:                                      # a small quantized vector: dequantized on the device
            q = QMat.upload(ctx, ty, rows, cols, raw)
            arr = q.to_f32().reshape(-1)
            q.free()
        m.set_vec(layer, role, np.ascontiguousarray(arr, dtype=np.float32))

    def hyper(layer, prefix, role, inject):
        for suffix, r in _HC:
            if suffix == "inject" and not inject:
                continue
            name = f"{prefix}_{suffix}.weight"
            (vec if suffix == "norm" else mat)(layer, f"{role}_{r}", name)

    mat(-1, "TOKEN_EMBD", "token_embd.weight")
    if ple_layers:
        mat(-1, "PLE_TAB", "per_layer_token_embd.weight")
    if g.has("output.weight"):
        mat(-1, "OUTPUT", "output.weight")
    if cfg.hc > 0:
        hyper(-1, "output_hc", "OUT_HC", False)
    else:
        vec(-1, "OUT_NORM", "output_norm.weight")
    for il in range(cfg.n_layers):
        p = f"blk.{il}"
        if il in ple_layers:                       # Ple :505
            mat(il, "PLE_KEY", f"{p}.ple_key.weight")
            mat(il, "PLE_VALUE", f"{p}.ple_value.weight")
            for role, n in (("PLE_NORM_KEY", "ple_norm_key"), ("PLE_NORM_QUERY", "ple_norm_query"), ("PLE_NORM_CONV", "ple_norm_conv"), ("PLE_CONV", "ple_conv1d")):
                vec(il, role, f"{p}.{n}.weight")
        if cfg.hc > 0:
            hyper(il, f"{p}.hc_attn", "HCA", True)
            hyper(il, f"{p}.hc_ffn", "HCF", True)
        else:
            vec(il, "ATTN_NORM", f"{p}.attn_norm.weight")
            vec(il, "FFN_NORM", f"{p}.ffn_norm.weight")
        if cfg.full_every > 0 and (il + 1) % cfg.full_every == 0:
            for role, n in (("ATTN_Q", "attn_q"), ("ATTN_K", "attn_k"), ("ATTN_V", "attn_v"), ("ATTN_O", "attn_output")):
                mat(il, role, f"{p}.{n}.weight")
            vec(il, "ATTN_Q_NORM", f"{p}.attn_q_norm.weight")
            vec(il, "ATTN_K_NORM", f"{p}.attn_k_norm.weight")
            if has_idx:
                mat(il, "IDX_Q", f"{p}.indexer.q_proj.weight")
                mat(il, "IDX_K", f"{p}.indexer.k_proj.weight")
                vec(il, "IDX_Q_NORM", f"{p}.indexer.q_norm.weight")
                vec(il, "IDX_K_NORM", f"{p}.indexer.k_norm.weight")
        else:
            for role, n in (("LIN_QKV", "attn_qkv"), ("LIN_Z", "attn_gate"), ("LIN_BETA", "ssm_beta"), ("LIN_ALPHA", "ssm_alpha"), ("LIN_OUT", "ssm_out")):
                mat(il, role, f"{p}.{n}.weight")
            vec(il, "LIN_A", f"{p}.ssm_a")
            vec(il, "LIN_DT", f"{p}.ssm_dt.bias")
            vec(il, "LIN_CONV", f"{p}.ssm_conv1d.weight")
            vec(il, "LIN_NORM", f"{p}.ssm_norm.weight")
        mat(il, "ROUTER", f"{p}.ffn_gate_inp.weight")
        mat(il, "EXP_GATE", f"{p}.ffn_gate_exps.weight", True)
        mat(il, "EXP_UP", f"{p}.ffn_up_exps.weight", True)
        mat(il, "EXP_DOWN", f"{p}.ffn_down_exps.weight", True)
        vec(il, "SH_GATE_INP", f"{p}.ffn_gate_inp_shexp.weight")
        mat(il, "SH_GATE", f"{p}.ffn_gate_shexp.weight")
        mat(il, "SH_UP", f"{p}.ffn_up_shexp.weight")
        mat(il, "SH_DOWN", f"{p}.ffn_down_shexp.weight")
    m.finalize(ep_rank, ep_world)
    m.gguf = g            # keeps the maps alive for as long as the model
    return m
