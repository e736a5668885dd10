"""CPU tests of the oracle (no GPU): golden vectors, reference-test properties, host logic."""
from pathlib import Path

import numpy as np
import pytest

import oracle

GOLD = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["Q8_0", "Q4_K", "IQ2_XS", "IQ3_S"])
def test_dequant_matches_gguf_py_golden(name):
    """Bit-for-bit against gguf-py 0.19 output committed as a fixture (tests/golden/make_golden.py)."""
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


def test_geometry():
    # QType::geom, gguf_q.rs:33-41, and the row-byte figures of the hot-path table
    assert oracle.geom(oracle.Q8_0) == (32, 34)
    assert oracle.geom(oracle.Q4_K) == (256, 144)
    assert oracle.geom(oracle.IQ2_XS) == (256, 74)
    assert oracle.geom(oracle.IQ3_S) == (256, 110)
    assert [oracle.row_bytes(t, 2048) for t in (oracle.Q8_0, oracle.Q4_K, oracle.IQ2_XS, oracle.IQ3_S)] == [2176, 1152, 592, 880]
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
