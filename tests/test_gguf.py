"""GGUF reader (CPU) and qwen4exp loader (GPU): files written with gguf-py, read by pyre_b200.gguf."""
import struct

import numpy as np
import pytest

import oracle
import pyre_b200 as pb
from pyre_b200 import synth
from pyre_b200.gguf import Gguf, GgufError, load_model, shard_paths
from helpers import small_cfg, write_synth_gguf


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def test_reader_on_a_hand_built_file(tmp_path):
    """A minimal file assembled byte by byte after the GGUF layout (no writer library involved): every scalar metadata type,
    a string, an array of strings, a nested numeric array, a custom alignment, two tensors."""
    kv = [("general.architecture", 8, _s("qwen4exp")), ("general.alignment", 4, struct.pack("<I", 64)),
          ("a.u8", 0, struct.pack("<B", 200)), ("a.i8", 1, struct.pack("<b", -5)), ("a.u16", 2, struct.pack("<H", 60000)), ("a.i16", 3, struct.pack("<h", -300)),
          ("a.i32", 5, struct.pack("<i", -7)), ("a.f32", 6, struct.pack("<f", 0.5)), ("a.bool", 7, b"\x01"), ("a.u64", 10, struct.pack("<Q", 1 << 40)),
          ("a.i64", 11, struct.pack("<q", -(1 << 40))), ("a.f64", 12, struct.pack("<d", 1e-300)),
          ("a.strs", 9, struct.pack("<IQ", 8, 2) + _s("x") + _s("yz")), ("a.nums", 9, struct.pack("<IQ", 4, 3) + struct.pack("<III", 1, 2, 3))]
    t0 = np.arange(6, dtype=np.float32).reshape(2, 3)                 # rows 2, cols 3 -> shape [3, 2]
    t1 = np.random.default_rng(0).integers(0, 256, 110 * 2, dtype=np.uint8)   # one IQ3_S row of 512 columns
    head = b"GGUF" + struct.pack("<IQQ", 3, 2, len(kv))
    for k, t, payload in kv:
        head += _s(k) + struct.pack("<I", t) + payload
    head += _s("w0") + struct.pack("<I", 2) + struct.pack("<QQ", 3, 2) + struct.pack("<IQ", 0, 0)
    head += _s("w1") + struct.pack("<I", 2) + struct.pack("<QQ", 512, 1) + struct.pack("<IQ", 21, 64)
    data0 = -(-len(head) // 64) * 64
    blob = head + b"\0" * (data0 - len(head)) + t0.tobytes() + b"\0" * (64 - 24) + t1.tobytes()
    p = tmp_path / "hand.gguf"
    p.write_bytes(blob)
    g = Gguf.open(p)
    assert g.arch() == "qwen4exp"
    assert g.meta["a.u8"] == 200 and g.meta["a.i8"] == -5 and g.meta["a.u16"] == 60000 and g.meta["a.i16"] == -300 and g.meta["a.i32"] == -7
    assert g.meta["a.f32"] == 0.5 and g.meta["a.bool"] is True and g.meta["a.u64"] == 1 << 40 and g.meta["a.i64"] == -(1 << 40) and g.meta["a.f64"] == 1e-300
    assert g.meta["a.strs"] == ["x", "yz"] and g.meta["a.nums"] == [1, 2, 3]
    ty, rows, cols, raw = g.mat("w0")
    assert (ty, rows, cols) == (0, 2, 3) and np.array_equal(raw.view(np.float32).reshape(2, 3), t0)
    ty, rows, cols, raw = g.mat("w1")
    assert (ty, rows, cols) == (21, 1, 512) and np.array_equal(raw, t1)
    assert g.shape("w1") == [512, 1] and g.has("w0") and not g.has("w2")
    with pytest.raises(GgufError):
        g.mat("w2")
    g.close()
    (tmp_path / "short.gguf").write_bytes(blob[:len(head) - 10])
    with pytest.raises(GgufError):
        Gguf.open(tmp_path / "short.gguf")
    (tmp_path / "cut.gguf").write_bytes(blob[:-100])                   # tensor data runs past the end
    with pytest.raises(GgufError):
        Gguf.open(tmp_path / "cut.gguf").mat("w1")
    (tmp_path / "bad.gguf").write_bytes(b"GGML" + blob[4:])
    with pytest.raises(GgufError):
        Gguf.open(tmp_path / "bad.gguf")


def test_reader_against_gguf_py_writer_and_shards(tmp_path):
    """A synthetic qwen4exp file written by gguf-py: metadata, three-dimensional expert tensors flattened to matrices, raw
    block bytes unchanged; shard names."""
    pytest.importorskip("gguf")
    cfg = small_cfg(pb, n_layers=4, n_exp=8, top_k=2)
    spec = synth.model_spec(cfg, 5)
    p = tmp_path / "m.gguf"
    write_synth_gguf(p, cfg, spec, 5)
    g = Gguf.open(p)
    assert g.arch() == "qwen4exp" and g.meta["qwen4exp.block_count"] == 4 and g.meta["qwen4exp.expert_count"] == 8
    assert abs(g.meta["qwen4exp.rope.freq_base"] - cfg.rope_base) < 1 and g.meta["tokenizer.ggml.tokens"] == ["a", "b", "c"]
    ty, rows, cols, raw = g.mat("blk.0.ffn_gate_exps.weight")
    assert (ty, rows, cols) == (oracle.IQ3_S, cfg.n_exp * cfg.ff_exp, cfg.d)
    tid = synth.tensor_id(0, "EXP_GATE")
    assert np.array_equal(raw, oracle.synth_rows(oracle.IQ3_S, 5, tid, cfg.d, 0, rows))
    assert g.shape("blk.0.ffn_gate_exps.weight") == [cfg.d, cfg.ff_exp, cfg.n_exp]
    ty, rows, cols, raw = g.mat("blk.0.ssm_conv1d.weight")
    assert (ty, cols) == (0, cfg.conv_k)
    g.close()
    for k in (1, 2, 3):
        (tmp_path / f"big-{k:05d}-of-00003.gguf").write_bytes(b"")
    assert [q.name for q in shard_paths(tmp_path / "big-00002-of-00003.gguf")] == [f"big-{k:05d}-of-00003.gguf" for k in (1, 2, 3)]
    (tmp_path / "big-00003-of-00003.gguf").unlink()
    with pytest.raises(GgufError):
        shard_paths(tmp_path / "big-00001-of-00003.gguf")
    assert shard_paths(p) == [p]


@pytest.mark.gpu
@pytest.mark.parametrize("hc", [0, 2])
def test_loaded_model_decodes_like_the_directly_built_one(ctx, tmp_path, hc):
    """load_model on a synthetic qwen4exp GGUF (names and keys of Model::load) gives the tokens of the same weights
    bound directly, with pre-norm residual and with hyper-connection streams."""
    pytest.importorskip("gguf")
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=256, hc=hc, hc_lr=32 if hc else 0)
    spec = synth.model_spec(cfg, 41)
    p = tmp_path / "model.gguf"
    write_synth_gguf(p, cfg, spec, 41)
    m = load_model(ctx, p, max_ctx=256, kv_bits=4, kv_recent=64)
    assert m.cfg.n_layers == 8 and m.cfg.vocab == cfg.vocab and m.cfg.hc == hc and m.cfg.ff_sh == cfg.ff_sh
    ref = synth.build_model(ctx, cfg, spec, 41)
    a, b = m.new_state(1), ref.new_state(1)
    prompt = np.array([3, 999, 27, 500, 1], np.uint32)
    la, lb = a.forward(prompt), b.forward(prompt)
    assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    assert a.decode_greedy([int(la[0].argmax())], 24)[0].tolist() == b.decode_greedy([int(lb[0].argmax())], 24)[0].tolist()
    a.destroy(); b.destroy(); m.destroy(); ref.destroy()


def test_drafter_file_reader_and_q8_0_quantizer(tmp_path):
    """The MTP drafter's tensor file (safetensors of BF16, src/model/mtp.rs:27-44): names lose their `mtp.` / `layers.0.`
    prefixes, values come back as the BF16 they were stored as; the Q8_0 quantizer gives the bytes gguf-py gives, and
    the oracle decodes them to within half a step."""
    gguf = pytest.importorskip("gguf")
    from pyre_b200 import mtp_loader as ml
    rng = np.random.default_rng(3)
    a = rng.standard_normal((6, 64)).astype(np.float32); b = rng.standard_normal(64).astype(np.float32)
    ml.write_safetensors(tmp_path / "d.safetensors", {"mtp.layers.0.self_attn.q_proj.weight": a, "mtp.pre_fc_norm_embedding.weight": b})
    t = ml.read_safetensors(tmp_path / "d.safetensors")
    assert set(t) == {"self_attn.q_proj.weight", "pre_fc_norm_embedding.weight"}
    bf = lambda x: ((x.view(np.uint32) >> 16) << 16).view(np.float32)
    assert np.array_equal(t["self_attn.q_proj.weight"], bf(a)) and np.array_equal(t["pre_fc_norm_embedding.weight"], bf(b))
    x = (rng.standard_normal((5, 256)) * np.exp(rng.standard_normal((5, 1)))).astype(np.float32)
    x[2, 32:64] = 0.0
    raw = ml.quantize_q8_0(x)
    want = gguf.quants.quantize(x, gguf.GGMLQuantizationType.Q8_0)
    assert np.array_equal(raw, np.ascontiguousarray(want).view(np.uint8).reshape(-1))
    back = oracle.dequant(oracle.Q8_0, raw, x.size).reshape(x.shape)
    step = np.abs(x.reshape(5, 8, 32)).max(axis=2, keepdims=True) / 127.0
    assert np.all(np.abs(back.reshape(5, 8, 32) - x.reshape(5, 8, 32)) <= 0.6 * step + 1e-7)       # half a step, plus what the f16 rounding of the scale moves the largest value
    with pytest.raises(ml.MtpFileError):
        ml.drafter_spec(t, type("C", (), dict(d=64, hc=2))())          # tensors missing


@pytest.mark.gpu
def test_loaded_model_with_indexer_and_trained_context(ctx, tmp_path):
    """A file that carries the sparse-attention indexer (attention.indexer.* keys, blk.N.indexer.* tensors) and a trained
    context shorter than the requested one: the loader hands both to the library, and the loaded model decodes like the
    same weights bound directly with the same indexer geometry and YaRN scaling -- 80 tokens, well past the dense range."""
    pytest.importorskip("gguf")
    indexer = (32, 4, 2, 64)
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=256)
    spec = synth.model_spec(cfg, 43, indexer=indexer)
    p = tmp_path / "model.gguf"
    write_synth_gguf(p, cfg, spec, 43, indexer=indexer, ctx_train=128)
    m = load_model(ctx, p, max_ctx=256, kv_bits=4, kv_recent=64)
    assert m.indexer == indexer
    ref = synth.build_model(ctx, cfg, spec, 43, ctx_train=128, indexer=indexer)
    plain = synth.build_model(ctx, cfg, [it for it in spec if not it[2].startswith("IDX_")], 43)
    a, b, c = m.new_state(1), ref.new_state(1), plain.new_state(1)
    ta, tb, tc = (s.decode_greedy([17], 80)[0].tolist() for s in (a, b, c))
    assert ta == tb and ta != tc
    for s in (a, b, c):
        s.destroy()
    m.destroy(); ref.destroy(); plain.destroy()


def test_ple_keys_and_tensors_are_read_back(tmp_path):
    """The n-gram embedding keys (64-bit multipliers among them) and tensor names of a written file, through the reader."""
    pytest.importorskip("gguf")
    cfg = small_cfg(pb, n_layers=4, max_ctx=64, hc=1, hc_lr=32)
    ple = synth.ple_geometry([1, 3])
    spec = synth.model_spec(cfg, 47, ple=ple)
    p = tmp_path / "ple.gguf"
    write_synth_gguf(p, cfg, spec, 47, ple=ple)
    g = Gguf.open(p)
    assert [int(v) for v in g.meta["qwen4exp.ple.layers"]] == [1, 3]
    assert [int(v) for v in g.meta["qwen4exp.ple.layer_multipliers"]] == ple["mult"] and max(ple["mult"]) > 1 << 63
    assert [int(v) for v in g.meta["qwen4exp.ple.head_vocab_sizes"]] == ple["vocab"]
    assert int(g.meta["qwen4exp.embedding_length_per_layer_input"]) == 256
    ty, rows, cols, raw = g.mat("per_layer_token_embd.weight")
    assert (rows, cols) == (sum(ple["vocab"]), 256)
    assert g.has("blk.1.ple_key.weight") and g.has("blk.3.ple_conv1d.weight") and not g.has("blk.0.ple_key.weight")
    assert g.mat("blk.1.ple_key.weight")[1:3] == (cfg.d, 4 * 256)
    g.close()


@pytest.mark.gpu
def test_loaded_model_with_ngram_embeddings(ctx, tmp_path):
    """A file with per-layer n-gram embeddings (ple.* keys, per_layer_token_embd and blk.N.ple_* tensors) loads into a model that decodes
    like the same weights bound directly, and unlike the model without them."""
    pytest.importorskip("gguf")
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=256, hc=2, hc_lr=32)
    ple = synth.ple_geometry([2, 5])
    spec = synth.model_spec(cfg, 48, ple=ple)
    p = tmp_path / "ple.gguf"
    write_synth_gguf(p, cfg, spec, 48, ple=ple)
    m = load_model(ctx, p, max_ctx=256, kv_bits=4, kv_recent=64)
    ref = synth.build_model(ctx, cfg, spec, 48, ple=ple)
    plain = synth.build_model(ctx, cfg, [it for it in spec if not it[2].startswith("PLE_")], 48)
    a, b, c = m.new_state(1), ref.new_state(1), plain.new_state(1)
    ta, tb, tc = (s.decode_greedy([17], 40)[0].tolist() for s in (a, b, c))
    assert ta == tb and ta != tc
    for s in (a, b, c):
        s.destroy()
    m.destroy(); ref.destroy(); plain.destroy()


@pytest.mark.gpu
def test_mixed_type_file_decodes_like_the_oracle(ctx, tmp_path):
    """A file whose tensors mix the block formats the way the reference's own checkpoint does (routed and shared gate / up in
    IQ3_XXS, IQ2_S, IQ2_XXS or IQ1_M by layer, down in IQ4_NL, projections in IQ4_XS and IQ3_S, Q6_K head, Q4_K embeddings): every tensor
    runs through the streaming kernels in its own format, and the loaded model gives the oracle's greedy tokens."""
    pytest.importorskip("gguf")
    from helpers import oracle_model
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=128)
    spec = []
    for it in synth.model_spec(cfg, 45):
        if it[0] == "mat" and it[3] == pb.IQ3_S:
            _, layer, role, ty, rows, cols, tid = it
            if role in ("EXP_GATE", "EXP_UP", "SH_GATE", "SH_UP"):
                ty = (pb.IQ3_XXS, pb.IQ2_S, pb.IQ2_XXS, pb.IQ1_M)[layer % 4]
            elif role in ("EXP_DOWN", "SH_DOWN"):
                ty = pb.IQ4_NL
            elif role.startswith("ATTN_") or role == "LIN_OUT":
                ty = pb.IQ4_XS
            elif role == "OUTPUT":
                ty = pb.Q6_K
            elif role == "TOKEN_EMBD":
                ty = pb.Q4_K
            it = ("mat", layer, role, ty, rows, cols, tid)
        spec.append(it)
    p = tmp_path / "mixed.gguf"
    write_synth_gguf(p, cfg, spec, 45)
    m = load_model(ctx, p, max_ctx=128, kv_bits=4, kv_recent=64)
    om, _ = oracle_model(cfg, spec, 45)
    st, ost = m.new_state(1), om.new_state()
    prompt = [3, 999, 27, 500, 1]
    lg, lo = st.forward(np.array(prompt, np.uint32))[0], ost.forward(prompt)
    assert np.max(np.abs(lg - lo)) < 1e-3 * np.max(np.abs(lo))
    tok = otok = int(lg.argmax())
    for i in range(32):
        tok = int(st.step_greedy([tok])[0]); otok = oracle.argmax(ost.forward([otok]))
        assert tok == otok, (i, ost.margins())
    st.destroy(); m.destroy()
