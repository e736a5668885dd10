"""CPU tests of the oracle (no GPU): golden vectors, reference-test properties, host logic."""
from pathlib import Path

import numpy as np
import pytest

import oracle
from conftest import rel_err

GOLD = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["Q8_0", "Q4_K", "IQ2_XS", "IQ3_S", "IQ3_XXS", "IQ2_S", "IQ4_NL", "IQ4_XS", "IQ2_XXS", "Q6_K", "Q2_0", "IQ1_M", "Q4_0", "Q5_0", "Q3_K", "Q5_K"])
def test_dequant_matches_gguf_py_golden(name):
    """Bit-for-bit against gguf-py 0.19 output committed as a fixture (tests/golden/make_golden.py; Q2_0, which gguf-py does not
    know, against the reference's two-line rule written in numpy there)."""
    g = np.load(GOLD / f"dequant_{name}.npz")
    rows, cols, t = int(g["rows"]), int(g["cols"]), int(g["type"])
    y = oracle.dequant(t, g["raw"], rows * cols).reshape(rows, cols)
    assert np.array_equal(y.view(np.uint32), g["f32"].view(np.uint32))


def test_dequant_matches_gguf_py_live():
    """Same check against the installed gguf-py on fresh random blocks (skipped if gguf is absent)."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants, GGMLQuantizationType as T
    m = {"Q8_0": T.Q8_0, "Q4_K": T.Q4_K, "IQ2_XS": T.IQ2_XS, "IQ3_S": T.IQ3_S}
    for name, t in oracle.QUANT_TYPES.items():
        el, bs = oracle.geom(t)
        raw = oracle.synth_rows(t, 3, 77, 1024, 0, 32)
        y = oracle.dequant(t, raw, 32 * 1024)
        ref = quants.dequantize(raw.reshape(-1, bs), m[name]).reshape(-1)
        assert np.array_equal(y.view(np.uint32), ref.view(np.uint32)), name
    m2 = {"IQ3_XXS": T.IQ3_XXS, "IQ2_S": T.IQ2_S, "IQ4_NL": T.IQ4_NL, "IQ4_XS": T.IQ4_XS, "IQ2_XXS": T.IQ2_XXS, "Q6_K": T.Q6_K, "IQ1_M": T.IQ1_M, "Q4_0": T.Q4_0, "Q5_0": T.Q5_0, "Q3_K": T.Q3_K, "Q5_K": T.Q5_K}
    rng = np.random.default_rng(99)
    for name, t in oracle.EXTRA_TYPES.items():
        if name not in m2:
            continue
        el, bs = oracle.geom(t)
        b = rng.integers(0, 256, size=(2048 // el * 8, bs), dtype=np.uint8)
        b[:, {"Q6_K": 209, "Q3_K": 109}.get(name, 1)] = rng.integers(0x20, 0x38, b.shape[0])
        if name == "Q5_K":
            b[:, 3] = rng.integers(0x20, 0x38, b.shape[0])
        if name == "IQ1_M":          # exponent nibbles of the scattered f16 scale
            b[:, 55] = (b[:, 55] & 0x0F) | 0x20
        y = oracle.dequant(t, b.reshape(-1), 8 * 2048)
        ref = quants.dequantize(b, m2[name]).reshape(-1)
        assert np.array_equal(y.view(np.uint32), ref.view(np.uint32)), name


def test_geometry():
    # QType::geom, gguf_q.rs:33-41, and the row-byte figures of the hot-path table
    assert oracle.geom(oracle.Q8_0) == (32, 34)
    assert oracle.geom(oracle.Q4_K) == (256, 144)
    assert oracle.geom(oracle.IQ2_XS) == (256, 74)
    assert oracle.geom(oracle.IQ3_S) == (256, 110)
    assert [oracle.row_bytes(t, 2048) for t in (oracle.Q8_0, oracle.Q4_K, oracle.IQ2_XS, oracle.IQ3_S)] == [2176, 1152, 592, 880]
    assert [oracle.geom(t) for t in (oracle.IQ3_XXS, oracle.IQ2_S, oracle.IQ4_NL, oracle.IQ4_XS)] == [(256, 98), (256, 82), (32, 18), (256, 136)]
    assert [oracle.geom(t) for t in (oracle.Q2_0, oracle.IQ2_XXS, oracle.Q6_K, oracle.IQ1_M, oracle.Q4_0, oracle.Q5_0, oracle.Q3_K, oracle.Q5_K)] == [(64, 18), (256, 66), (256, 210), (256, 56), (32, 18), (32, 22), (256, 110), (256, 176)]
    with pytest.raises(ValueError):
        oracle.geom(99)


def test_synth_is_deterministic_and_row_addressable():
    a = oracle.synth_rows(oracle.IQ3_S, 0, 5, 2048, 0, 8)
    b = oracle.synth_rows(oracle.IQ3_S, 0, 5, 2048, 4, 2)
    rb = oracle.row_bytes(oracle.IQ3_S, 2048)
    assert np.array_equal(a[4 * rb:6 * rb], b)
    assert not np.array_equal(a, oracle.synth_rows(oracle.IQ3_S, 1, 5, 2048, 0, 8))
    # block scales follow |N(0, 0.02)| (config 0 of the benchmark)
    d = oracle.synth_rows(oracle.IQ3_S, 0, 9, 2048, 0, 512).reshape(-1, 110)[:, :2].copy().view(np.float16).astype(np.float32)
    assert abs(float(d.mean()) - 0.02 * np.sqrt(2 / np.pi)) < 1e-3
    q = oracle.synth_rows(oracle.Q8_0, 0, 9, 2048, 0, 64).reshape(-1, 34)[:, 2:].view(np.int8)
    assert q.min() == -127 and q.max() == 127


def test_gemv_matches_f64_of_dequant():
    rng = np.random.default_rng(0)
    for t in oracle.QUANT_TYPES.values():
        W = oracle.QMat.synth(t, 64, 2048, 0, 3)
        x = rng.standard_normal((3, 2048)).astype(np.float32)
        y = W.matmul(x)
        ref = x.astype(np.float64) @ W.to_f32().astype(np.float64).T
        assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()


def test_top_k_softmax_over_selection():
    rng = np.random.default_rng(1)
    r = rng.standard_normal(512).astype(np.float32)
    idx, w = oracle.top_k(r, 10)
    order = np.argsort(-r, kind="stable")[:10]
    assert list(idx) == list(order)              # descending logit, the canonical order
    e = np.exp(r[order] - r[order].max())
    assert np.allclose(w, e / e.sum(), rtol=1e-6)
    assert abs(w.sum() - 1) < 1e-6
    r2 = r.copy(); r2[5] = np.nan                # nan_clean: NaN never selected
    idx2, _ = oracle.top_k(r2, 10)
    assert 5 not in idx2
    # ties go to the lower index
    idx3, w3 = oracle.top_k(np.zeros(16, np.float32), 4)
    assert list(idx3) == [0, 1, 2, 3] and np.allclose(w3, 0.25)


def test_argmax_first_max_wins():
    assert oracle.argmax(np.array([1, 3, 3, 2], np.float32)) == 1   # sampler.rs:142-148 (strict >)
    assert oracle.argmax(np.array([5, 3, 3, 2], np.float32)) == 0


def test_kv4_reference_properties():
    """The assertions of src/model/kv4.rs:52-104 on its own input vector."""
    g = np.load(GOLD / "kv4_vector.npz")
    x = g["x"]
    w, s = oracle.kv4_pack(x)
    assert np.array_equal(w, g["words"]) and np.array_equal(s, g["scales"])
    assert w.size == x.size // 8 and s.size == x.size // 32
    y = oracle.kv4_unpack(w, s, x.size)
    assert np.all(np.abs(y - x) <= np.repeat(s, 32) * 0.5 + 1e-6)
    # kvq_roundtrip(..., 4): q = round(v / s) clamped to +-7, times s
    z = np.where(np.repeat(s, 32) > 0, np.clip(np.round(x / np.repeat(s, 32)), -7, 7) * np.repeat(s, 32), 0).astype(np.float32)
    assert np.all(np.abs(y - z) <= 1e-5 * np.maximum(np.abs(z), 1.0))
    w0, s0 = oracle.kv4_pack(np.zeros(32, np.float32))
    assert np.array_equal(oracle.kv4_unpack(w0, s0, 32), np.zeros(32, np.float32))
    ext = np.ones(32, np.float32); ext[31] = -1
    we, se = oracle.kv4_pack(ext)
    assert abs(oracle.kv4_unpack(we, se, 32)[31] + 1.0) < 1e-5
    # nibble_sign_extension
    v = np.zeros(32, np.float32); v[0], v[1] = -0.7, 0.7
    wv, sv = oracle.kv4_pack(v)
    assert (wv[0] & 0xF) >= 8 and ((wv[0] >> 4) & 0xF) < 8
    mae4 = np.abs(y - x).mean()
    assert mae4 < 0.2


def test_rope_inv():
    inv = oracle.rope_inv(64, 1e7)
    assert inv.shape == (32,) and inv[0] == 1.0
    assert np.allclose(inv, 1e7 ** (-(2.0 * np.arange(32)) / 64), rtol=1e-5)


def test_yarn_rope_table_against_transformers():
    """The YaRN table the reference builds past the trained context (src/qn_ctx.rs:160-186), held to vectors computed with
    Hugging Face transformers (tests/golden/make_hf_yarn_golden.py).  The reference blends interpolated and trained
    frequencies with the complementary ramp, so the two tables add up to extrap * (1 + 1 / scale) at every index; mscale
    is the same number.  At or under the trained context the table is the plain one, bit for bit."""
    g = np.load(GOLD / "hf_yarn.npz")
    for i, (n_rot, base, tr, ctx) in enumerate(g["cases"]):
        n_rot, tr, ctx = int(n_rot), int(tr), int(ctx)
        inv, ms = oracle.rope_inv_yarn(n_rot, float(base), tr, ctx)
        extrap = float(base) ** (-(2.0 * np.arange(n_rot // 2)) / n_rot)
        total = extrap * (1.0 + tr / ctx)
        assert np.max(np.abs((inv + g[f"inv{i}"]) - total) / total) < 1e-6, i
        assert abs(ms - float(g[f"att{i}"])) < 1e-6, i
        assert np.all(inv <= extrap * (1 + 1e-6)) and np.all(inv >= extrap * tr / ctx * (1 - 1e-6))
    inv, ms = oracle.rope_inv_yarn(64, 1e7, 4096, 4096)
    assert ms == 1.0 and np.array_equal(inv, oracle.rope_inv(64, 1e7))
    inv, ms = oracle.rope_inv_yarn(64, 1e7, 0, 1 << 20)
    assert ms == 1.0 and np.array_equal(inv, oracle.rope_inv(64, 1e7))


def _qdot_test_block(n: int) -> np.ndarray:
    """The row the reference's own test builds (block, src/model/qdot.rs:1033-1045): bytes from a 64-bit LCG seeded with
    0xC0FFEE ^ n, then a sane f16 scale written over the first two bytes of each of the two 110-byte rows."""
    seed = 0xC0FFEE ^ n
    nbytes = 110 * 2          # row_bytes(256) for IQ3_S, twice
    v = np.zeros(nbytes, dtype=np.uint8)
    s = seed
    for i in range(nbytes):
        s = (s * 6364136223846793005 + 1) % (1 << 64)
        v[i] = (s >> 33) & 0xFF
    d = np.float16(0.05 + (seed % 17) * 0.01)
    v[0:2] = np.frombuffer(d.tobytes(), dtype=np.uint8)
    v[110:112] = np.frombuffer(d.tobytes(), dtype=np.uint8)
    return v


def test_int8_row_dot_by_the_references_own_test_method():
    """check(QType::IQ3S, 512), src/model/qdot.rs:1053-1070: the int8 row dot against the dequantized row times the same
    int8 activations, relative error below 2e-3 -- same block generator, same activation pattern, same bound."""
    n = 512
    row = _qdot_test_block(n)
    x = np.array([((i * 17 + 3) % 11) / 5.0 - 1.0 for i in range(n)], dtype=np.float32)
    q, d = oracle.q8_quantize(x)
    assert q.dtype == np.int8 and int(np.abs(q).max()) == 127 and d.shape == (16,)
    got = oracle.row_dot_q8_iq3s(row, q, d)
    exp = oracle.q8_dot_dequant(oracle.IQ3_S, row, q, d)
    assert abs(got - exp) / max(abs(exp), 1e-3) < 2e-3
    # the int8 activations reproduce x within half a step, and the approximation is close to the f32 product
    assert np.abs(q.astype(np.float32) * np.repeat(d, 32) - x).max() <= d.max() * 0.5 + 1e-7
    f32 = float(oracle.QMat(oracle.IQ3_S, 1, n, row).matmul(x[None])[0, 0])
    assert abs(got - f32) / max(abs(f32), 1e-3) < 2e-2
    # seeded synthetic rows of the benchmark's generator too
    Wo = oracle.QMat.synth(oracle.IQ3_S, 4, 2048, 0, 42)
    xx = np.random.default_rng(1).standard_normal(2048).astype(np.float32)
    qq, dd = oracle.q8_quantize(xx)
    raw = Wo.raw().reshape(4, -1)
    for r in range(4):
        a, b = oracle.row_dot_q8_iq3s(raw[r], qq, dd), oracle.q8_dot_dequant(oracle.IQ3_S, raw[r], qq, dd)
        assert abs(a - b) / max(abs(b), 1e-3) < 2e-3


def test_gated_deltanet_against_transformers_qwen3_next_vectors():
    """The oracle's linear_core against vectors computed with Hugging Face transformers' Qwen3-Next code (conv + SiLU,
    L2 norms, gates, torch_recurrent_gated_delta_rule); tests/golden/make_hf_deltanet_golden.py lines up the two places
    where the reference's model family differs (head map, output gate).  Readout compared after the same weight-1 RMS
    norm with the gate saturated to 1; the final recurrent state directly."""
    g = np.load(Path(__file__).resolve().parent / "golden" / "hf_gated_deltanet.npz")
    nk, nv, dk, dv, K, t = (int(g[k]) for k in ("nk", "nv", "dk", "dv", "conv_k", "t"))
    cfg = oracle.Cfg()
    cfg.lin_nk, cfg.lin_nv, cfg.lin_dk, cfg.lin_dv, cfg.conv_k, cfg.eps = nk, nv, dk, dv, K, 1e-6
    ch = 2 * nk * dk + nv * dv
    conv_state = np.zeros((K - 1, ch), np.float32)
    ssm = np.zeros((nv, dk, dv), np.float32)
    z = np.full((t, nv * dv), 30.0, np.float32)                      # sigmoid(30) == 1.0f
    out = oracle.linear_core(cfg, g["qkv"], z, g["beta_raw"], g["alpha_raw"], g["ssm_a"], g["dt_bias"], g["conv_w"],
                             np.ones(dv, np.float32), conv_state, ssm)
    ref = g["readout"].astype(np.float64)                            # [t][nv][dv], before any norm
    ref = ref / np.sqrt((ref ** 2).mean(axis=-1, keepdims=True) + 1e-6)
    assert rel_err(out.reshape(t, nv, dv), ref) < 1e-5
    assert rel_err(ssm, g["state"]) < 1e-5
    assert np.array_equal(conv_state, g["qkv"][t - (K - 1):])        # the history holds the last K-1 raw inputs


def test_gated_attention_against_transformers_qwen3_next_vectors():
    """The oracle's attn_core (f32 KV) token by token against vectors computed with Hugging Face transformers' Qwen3-Next
    code: zero-centred q / k RMS norms, partial rotary embedding, grouped-query causal softmax attention, sigmoid gate
    (tests/golden/make_hf_attention_golden.py)."""
    g = np.load(Path(__file__).resolve().parent / "golden" / "hf_gated_attention.npz")
    cfg = oracle.Cfg()
    cfg.n_head, cfg.n_kv, cfg.hd, cfg.n_rot, cfg.eps = int(g["n_head"]), int(g["n_kv"]), int(g["hd"]), int(g["n_rot"]), float(g["eps"])
    cfg.kv_bits, cfg.kv_recent, cfg.max_ctx = 0, 1024, 64
    t = int(g["t"]); row = cfg.n_kv * cfg.hd
    inv = oracle.rope_inv(cfg.n_rot, float(g["rope_base"]))
    kc = np.zeros((t, row), np.float32); vc = np.zeros((t, row), np.float32)
    for pos in range(t):
        att = oracle.attn_core(cfg, g["qf"][pos], g["kf"][pos], g["vf"][pos], g["q_norm"], g["k_norm"], inv, kc, vc, pos)
        assert rel_err(att, g["att"][pos]) < 2e-5, pos


def test_qsa_selection_and_sparse_attention_properties():
    """QSA (attn_core, src/model/qwen4exp_gguf.rs:1565-1609) as the oracle restates it: the pooled key is the normed, roped
    mean of a block's raw keys; the dense range ends at budget + ratio - 1 tokens; a query past it takes exactly
    budget / ratio complete blocks, the best-scoring ones by an independent numpy evaluation; attention over a position
    list that holds every position equals dense attention, and dropping a position changes it."""
    cfg = oracle.make_cfg(n_head=4, n_kv=2, hd=64, n_rot=32, max_ctx=128, kv_bits=0)
    budget, ratio, inh, ihd = 16, 4, 3, 32
    rng = np.random.default_rng(11)
    inv = oracle.rope_inv(cfg.n_rot, 1e4)
    ik = rng.standard_normal((80, ihd)).astype(np.float32)
    ikn = (1 + 0.1 * rng.standard_normal(ihd)).astype(np.float32); iqn = (1 + 0.1 * rng.standard_normal(ihd)).astype(np.float32)

    def rope(v, pos):
        half = cfg.n_rot // 2; a = pos * inv.astype(np.float64); o = v.astype(np.float64).copy()
        o[:half] = v[:half] * np.cos(a) - v[half:2 * half] * np.sin(a); o[half:2 * half] = v[half:2 * half] * np.cos(a) + v[:half] * np.sin(a)
        return o

    def norm(v, w):
        v = v.astype(np.float64); return v / np.sqrt((v * v).mean() + cfg.eps) * w

    ib = np.stack([oracle.qsa_pool(cfg, ratio, ik, ikn, inv, b) for b in range(20)])
    for b in (0, 7, 19):
        assert np.allclose(ib[b], rope(norm(ik[b * ratio:(b + 1) * ratio].astype(np.float64).mean(0), ikn), b * ratio), atol=2e-6)
    iq = rng.standard_normal((inh, ihd)).astype(np.float32)
    blocks, _ = oracle.qsa_select(cfg, budget, ratio, iq, iqn, inv, ib, budget + ratio - 2)
    assert blocks.size == 0                                   # budget + ratio - 1 visible tokens: still dense
    pos = 61
    blocks, margin = oracle.qsa_select(cfg, budget, ratio, iq, iqn, inv, ib, pos)
    nb = (pos + 1) // ratio
    qh = np.stack([rope(norm(iq[h], iqn), pos) for h in range(inh)])
    sc = np.maximum(qh @ ib[:nb].astype(np.float64).T, 0).sum(0) / np.sqrt(ihd)
    want = np.sort(np.argsort(-sc, kind="stable")[:budget // ratio])
    assert blocks.tolist() == want.tolist() and margin > 0 and np.all(np.diff(blocks) > 0)
    srt = np.sort(sc)[::-1]
    assert abs(margin - (srt[budget // ratio - 1] - srt[budget // ratio])) < 1e-5
    # attention over a full list == dense; a shorter list differs
    row = cfg.n_kv * cfg.hd; n = 40
    kc = rng.standard_normal((n, row)).astype(np.float32); vc = rng.standard_normal((n, row)).astype(np.float32)
    qf = rng.standard_normal(cfg.n_head * 2 * cfg.hd).astype(np.float32); kf = rng.standard_normal(row).astype(np.float32); vf = rng.standard_normal(row).astype(np.float32)
    qn = np.ones(cfg.hd, np.float32); kn = np.ones(cfg.hd, np.float32)
    dense = oracle.attn_core(cfg, qf, kf, vf, qn, kn, inv, kc.copy(), vc.copy(), n - 1)
    full = oracle.attn_core(cfg, qf, kf, vf, qn, kn, inv, kc.copy(), vc.copy(), n - 1, ps=np.arange(n))
    assert np.array_equal(dense, full)
    part = oracle.attn_core(cfg, qf, kf, vf, qn, kn, inv, kc.copy(), vc.copy(), n - 1, ps=np.arange(1, n))
    assert rel_err(part, dense) > 1e-4


def test_ple_hash_rows_follow_the_reference_rule():
    """ple_rows (qwen4exp_gguf.rs:1394-1403) in Python integers: contexts cut at a missing or end-of-sequence predecessor, n-gram size n
    mixes the first n ids times their multipliers by xor (wrapping 64-bit), each head takes the mix modulo its vocabulary plus its offset."""
    from pyre_b200.synth import ple_geometry
    g = ple_geometry([0], ngram=4, per_gram=2, eos=2)
    om = oracle.Model(oracle.make_cfg(n_layers=1, d=256, vocab=64, max_ctx=16))
    om.set_ple(g["ngram"], g["per_gram"], g["conv_k"], g["eos"], g["dim"], g["mult"], g["off"], g["vocab"])
    M64 = (1 << 64) - 1
    for ctx in ([5, 9, 11, 13], [5, -1, 11, 13], [5, 9, 2, 13], [5, 2, 7, 8], [2, 9, 11, 13], [(1 << 32) - 1, 70000, 3, 4]):
        c, cut = [ctx[0]], False
        for s in range(1, 4):
            none = cut or ctx[s] < 0
            cut = cut or none or ctx[s] == 2
            c.append(2 if cut else ctx[s])
        want = []
        for n in range(2, 5):
            mixed = (c[0] * g["mult"][0]) & M64
            for j in range(1, n):
                mixed ^= (c[j] * g["mult"][j]) & M64
            for gi in range(2):
                h = (n - 2) * 2 + gi
                want.append(mixed % g["vocab"][h] + g["off"][h])
        assert om.ple_hash(ctx).tolist() == want, ctx


def test_ple_by_position_rows_equal_the_reference_ring():
    """The oracle keeps the normalized rows by position; the reference drains and extends a ring of the last (conv_k - 1) * ngram rows
    (ple, qwen4exp_gguf.rs:1409-1434, hist :1432).  The reference's loop, written here in numpy with its ring, gives the same streams."""
    from pyre_b200.synth import ple_geometry
    rng = np.random.default_rng(8)
    d, hc, K, ngram, T = 64, 2, 3, 3, 11
    w = hc * d
    g = ple_geometry([0], ngram=ngram, per_gram=1, conv_k=K, dim=256)
    om = oracle.Model(oracle.make_cfg(n_layers=1, d=d, hc=hc, hc_lr=8, vocab=64, max_ctx=32, eps=1e-6))
    om.set_ple(g["ngram"], g["per_gram"], g["conv_k"], g["eos"], g["dim"], g["mult"], g["off"], g["vocab"])
    nk, nq, nc = (1.0 + 0.1 * rng.standard_normal(w)).astype(np.float32), (1.0 + 0.1 * rng.standard_normal(w)).astype(np.float32), (1.0 + 0.1 * rng.standard_normal(w)).astype(np.float32)
    conv = (0.5 * rng.standard_normal((w, K))).astype(np.float32)
    for role, a in (("PLE_NORM_KEY", nk), ("PLE_NORM_QUERY", nq), ("PLE_NORM_CONV", nc), ("PLE_CONV", conv.reshape(-1))):
        om.set_vec(0, role, a)
    keys = rng.standard_normal((T, w)).astype(np.float32); vals = rng.standard_normal((T, d)).astype(np.float32)
    xs = rng.standard_normal((T, w)).astype(np.float32)
    # the oracle, by position
    nrm_all = np.zeros((32, w), np.float32); xo = xs.copy()
    for t in range(T):
        om.ple_token(0, nrm_all, keys[t], vals[t], xo[t], t)
    # the reference's loop with its ring (float64 accumulation is avoided: same f32 operations, numpy order)
    f32 = np.float32
    def rms(v, wt):
        s = f32(1.0) / np.sqrt(f32(np.sum(v * v, dtype=np.float32)) / f32(len(v)) + f32(1e-6))
        return v * s * wt
    dil, hl = ngram, (K - 1) * ngram
    hist = np.zeros((hl, w), np.float32); xr = xs.copy()
    for t in range(T):
        gated = np.zeros(w, np.float32)
        for s_ in range(hc):
            sl = slice(s_ * d, (s_ + 1) * d)
            kk, q = rms(keys[t, sl], nk[sl]), rms(xr[t, sl], nq[sl])
            sc = f32(np.dot(kk, q)) / f32(np.sqrt(f32(d)))
            gte = f32(1.0) / (f32(1.0) + np.exp(-(np.sign(sc) if sc != 0 else f32(1.0)) * np.sqrt(max(abs(sc), f32(1e-6)))))
            gated[sl] = vals[t] * f32(gte)
        nrm = gated.copy()
        for s_ in range(hc):
            sl = slice(s_ * d, (s_ + 1) * d)
            nrm[sl] = rms(nrm[sl], nc[sl])
        o = conv[:, K - 1] * nrm
        for k in range(K - 1):
            back = (K - 1 - k) * dil
            o = o + conv[:, k] * hist[hl - back]
        xr[t] += gated + o / (1.0 + np.exp(-o))
        hist = np.concatenate([hist[1:], nrm[None]])
    assert np.max(np.abs(xo - xr)) < 2e-5 * max(1.0, float(np.max(np.abs(xr))))
    assert np.max(np.abs(nrm_all[T - hl:T] - hist)) < 2e-5
