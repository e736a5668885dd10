"""Shared test helpers: realise a synthetic model description in the CPU oracle."""
import numpy as np

import oracle


def oracle_cfg(cfg):
    """Copy a pyre_b200.Cfg (same field layout) into the oracle's config struct."""
    oc = oracle.Cfg()
    for name, _ in oracle.Cfg._fields_:
        setattr(oc, name, getattr(cfg, name))
    return oc


def oracle_model(cfg, spec, seed=0, ctx_train=0, indexer=None, ple=None):
    om = oracle.Model(oracle_cfg(cfg))
    if ple:
        om.set_ple(ple["ngram"], ple["per_gram"], ple["conv_k"], ple["eos"], ple["dim"], ple["mult"], ple["off"], ple["vocab"])
    if ctx_train:
        om.set_ctx_train(ctx_train)
    if indexer:
        om.set_indexer(*indexer)
    mats = {}
    for item in spec:
        if item[0] == "mat":
            _, layer, role, t, rows, cols, tid = item
            q = oracle.QMat.synth(t, rows, cols, seed, tid)
            om.set_mat(layer, role, q)
            mats[(layer, role)] = q
        else:
            _, layer, role, arr = item
            om.set_vec(layer, role, arr)
            mats[(layer, role)] = np.asarray(arr, dtype=np.float32)
    return om, mats


def small_cfg(pb, **kw):
    """A scaled-down hybrid config that keeps every structural feature of the full model."""
    base = dict(n_layers=4, d=512, n_head=4, n_kv=2, hd=256, n_rot=64, n_exp=16, top_k=4, ff_exp=256, ff_sh=256,
                lin_nk=2, lin_nv=4, lin_dk=128, lin_dv=128, conv_k=4, full_every=4, vocab=1024, max_ctx=512,
                kv_bits=0, kv_recent=64)
    base.update(kw)
    return pb.make_cfg(**base)


# tensor names of a qwen4exp GGUF (Model::load, src/model/qwen4exp_gguf.rs:492-512) by the library's role names
GGUF_NAMES = {
    "TOKEN_EMBD": "token_embd.weight", "OUTPUT": "output.weight", "OUT_NORM": "output_norm.weight",
    "ATTN_NORM": "attn_norm.weight", "FFN_NORM": "ffn_norm.weight",
    "ATTN_Q": "attn_q.weight", "ATTN_K": "attn_k.weight", "ATTN_V": "attn_v.weight", "ATTN_O": "attn_output.weight",
    "ATTN_Q_NORM": "attn_q_norm.weight", "ATTN_K_NORM": "attn_k_norm.weight",
    "LIN_QKV": "attn_qkv.weight", "LIN_Z": "attn_gate.weight", "LIN_BETA": "ssm_beta.weight", "LIN_ALPHA": "ssm_alpha.weight", "LIN_OUT": "ssm_out.weight",
    "LIN_A": "ssm_a", "LIN_DT": "ssm_dt.bias", "LIN_CONV": "ssm_conv1d.weight", "LIN_NORM": "ssm_norm.weight",
    "ROUTER": "ffn_gate_inp.weight", "EXP_GATE": "ffn_gate_exps.weight", "EXP_UP": "ffn_up_exps.weight", "EXP_DOWN": "ffn_down_exps.weight",
    "SH_GATE_INP": "ffn_gate_inp_shexp.weight", "SH_GATE": "ffn_gate_shexp.weight", "SH_UP": "ffn_up_shexp.weight", "SH_DOWN": "ffn_down_shexp.weight",
    "PLE_TAB": "per_layer_token_embd.weight", "PLE_KEY": "ple_key.weight", "PLE_VALUE": "ple_value.weight", "PLE_NORM_KEY": "ple_norm_key.weight",
    "PLE_NORM_QUERY": "ple_norm_query.weight", "PLE_NORM_CONV": "ple_norm_conv.weight", "PLE_CONV": "ple_conv1d.weight",
    "HCA_NORM": "hc_attn_norm.weight", "HCA_DOWN": "hc_attn_down.weight", "HCA_UP": "hc_attn_up.weight", "HCA_INJECT": "hc_attn_inject.weight",
    "HCF_NORM": "hc_ffn_norm.weight", "HCF_DOWN": "hc_ffn_down.weight", "HCF_UP": "hc_ffn_up.weight", "HCF_INJECT": "hc_ffn_inject.weight",
    "OUT_HC_NORM": "output_hc_norm.weight", "OUT_HC_DOWN": "output_hc_down.weight", "OUT_HC_UP": "output_hc_up.weight",
    "IDX_Q": "indexer.q_proj.weight", "IDX_K": "indexer.k_proj.weight", "IDX_Q_NORM": "indexer.q_norm.weight", "IDX_K_NORM": "indexer.k_norm.weight",
}


def write_synth_gguf(path, cfg, spec, seed, split_after=None, indexer=None, ctx_train=0, ple=None):
    """A synthetic model (pyre_b200.synth.model_spec) as a qwen4exp GGUF file written with gguf-py: metadata keys and tensor
    names as Model::load reads them, quantized tensors as their raw block bytes (the oracle's generator)."""
    import gguf
    from gguf import GGMLQuantizationType as T
    import oracle
    w = gguf.GGUFWriter(str(path), "qwen4exp")
    a = "qwen4exp"
    for key, v in (("block_count", cfg.n_layers), ("embedding_length", cfg.d), ("hyper_connection.count", cfg.hc), ("hyper_connection.low_rank", cfg.hc_lr),
                   ("attention.head_count", cfg.n_head), ("attention.head_count_kv", cfg.n_kv), ("attention.key_length", cfg.hd), ("rope.dimension_count", cfg.n_rot),
                   ("expert_count", cfg.n_exp), ("expert_used_count", cfg.top_k), ("expert_feed_forward_length", cfg.ff_exp), ("ssm.group_count", cfg.lin_nk),
                   ("ssm.time_step_rank", cfg.lin_nv), ("ssm.state_size", cfg.lin_dk), ("ssm.conv_kernel", cfg.conv_k), ("full_attention_interval", cfg.full_every)):
        w.add_uint32(f"{a}.{key}", int(v))
    if indexer:
        budget, ratio, inh, ihd = indexer
        w.add_uint32(f"{a}.attention.indexer.top_k", budget); w.add_uint32(f"{a}.attention.indexer.head_count", inh); w.add_uint32(f"{a}.attention.indexer.key_length", ihd)
        w.add_array(f"{a}.attention.compress_ratios", [1, ratio])
    if ctx_train:
        w.add_uint32(f"{a}.context_length", ctx_train)
    if ple:
        w.add_array(f"{a}.ple.layers", [int(v) for v in ple["layers"]])
        for key, name in (("ngram", "ple.ngram_size"), ("per_gram", "ple.heads_per_ngram"), ("conv_k", "ple.conv_kernel"), ("eos", "ple.eos_token_id"), ("dim", "embedding_length_per_layer_input")):
            w.add_uint32(f"{a}.{name}", int(ple[key]))
        # gguf-py stores a Python int array as int32 unless told otherwise; the multipliers need all 64 bits
        for key, name in (("mult", "ple.layer_multipliers"), ("off", "ple.head_offsets"), ("vocab", "ple.head_vocab_sizes")):
            w.add_key_value(f"{a}.{name}", [int(v) for v in ple[key]], gguf.GGUFValueType.ARRAY, sub_type=gguf.GGUFValueType.UINT64)
    w.add_float32(f"{a}.rope.freq_base", float(cfg.rope_base))
    w.add_float32(f"{a}.attention.layer_norm_rms_epsilon", float(cfg.eps))
    w.add_string("general.name", "synthetic")
    w.add_array("tokenizer.ggml.tokens", ["a", "b", "c"])       # an array of strings in the metadata, as real files have
    for item in spec:
        layer, role = item[1], item[2]
        name = GGUF_NAMES[role] if layer < 0 else f"blk.{layer}.{GGUF_NAMES[role]}"
        if item[0] == "vec":
            arr = np.ascontiguousarray(item[3], dtype=np.float32)
            if role == "LIN_CONV":
                arr = arr.reshape(-1, cfg.conv_k)
            if role == "PLE_CONV":
                arr = arr.reshape(-1, ple["conv_k"])
            w.add_tensor(name, arr)
        else:
            _, _, _, t, rows, cols, tid = item
            if t == oracle.F32:
                w.add_tensor(name, oracle.synth_normal(seed, tid, 0, rows * cols, 0.02).reshape(rows, cols))
            else:
                raw = oracle.synth_rows(t, seed, tid, cols, 0, rows).reshape(rows, -1)
                if role in ("EXP_GATE", "EXP_UP", "EXP_DOWN"):   # fused expert tensors are three-dimensional in real files
                    raw = raw.reshape(cfg.n_exp, rows // cfg.n_exp, -1)
                w.add_tensor(name, raw, raw_dtype=T(t))
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
