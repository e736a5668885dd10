"""QSA block-sparse attention (attn_core, src/model/qwen4exp_gguf.rs:1565-1599) in the token loop: the engine against the CPU oracle."""
import numpy as np
import pytest

import oracle
import pyre_b200 as pb
from pyre_b200 import synth
from conftest import rel_err
from helpers import oracle_model, small_cfg

pytestmark = pytest.mark.gpu

INDEXER = (32, 4, 2, 64)     # budget (tokens), block size, index heads, index head dim: dense up to 35 visible tokens


def _pair(ctx, kv_bits, seed, n_layers=8, max_ctx=320):
    cfg = small_cfg(pb, n_layers=n_layers, kv_bits=kv_bits, kv_recent=64, max_ctx=max_ctx)
    spec = synth.model_spec(cfg, seed, indexer=INDEXER)
    m = synth.build_model(ctx, cfg, spec, seed, indexer=INDEXER)
    om, _ = oracle_model(cfg, spec, seed, indexer=INDEXER)
    return cfg, m, om


@pytest.mark.parametrize("kv_bits,steps", [(0, 72), (4, 200)])
def test_sparse_attention_greedy_identity_vs_oracle(ctx, kv_bits, steps):
    """A 24-token prompt (dense range), then greedy steps far past budget + ratio - 1 = 35 visible tokens, so that nearly
    every step selects blocks; with the 4-bit cache the run also crosses two packing steps, so selected blocks lie in the
    packed region (tensor-core tiles with masked positions) and in the f32 window.  Logits within 1e-3 at every step,
    token ids identical; the oracle's smallest selection margin is reported with a failure."""
    cfg, m, om = _pair(ctx, kv_bits, 21)
    st, ost = m.new_state(1), om.new_state()
    prompt = list(range(300, 324))
    lg, lo = st.forward(np.array(prompt, np.uint32))[0], ost.forward(prompt)
    assert rel_err(lg, lo) < 1e-3 and ost.qsa_margin() == float("inf")
    tok = otok = int(lg.argmax()); worst, min_margin = 0.0, float("inf")
    for i in range(steps):
        lg, lo = st.forward(np.array([tok], np.uint32))[0], ost.forward([otok])
        min_margin = min(min_margin, ost.qsa_margin())
        worst = max(worst, rel_err(lg, lo))
        assert worst < 1e-3, (i, worst, min_margin)
        tok, otok = int(lg.argmax()), oracle.argmax(lo)
        assert tok == otok, (i, min_margin, ost.margins())
    assert min_margin < float("inf")                      # sparse queries did happen
    assert ctx.device_status() == 0
    st.destroy(); m.destroy()


def test_sparse_differs_from_dense_and_batch_matches_single(ctx):
    """The selection is really in force (logits differ from the same weights without an indexer geometry), and a batch of
    three sequences at different tokens equals three single-sequence runs (every sequence has its own keys and mask)."""
    cfg, m, om = _pair(ctx, 4, 22, n_layers=4)
    firsts = [11, 500, 77]
    stb = m.new_state(3)
    outb = stb.decode_greedy(firsts, 90)
    for i, f in enumerate(firsts):
        s1 = m.new_state(1)
        assert s1.decode_greedy([f], 90)[0].tolist() == outb[i].tolist()
        s1.destroy()
    spec = synth.model_spec(cfg, 22, indexer=INDEXER)
    dense = synth.build_model(ctx, cfg, [it for it in spec if not it[2].startswith("IDX_")], 22)
    a, b = m.new_state(1), dense.new_state(1)
    toks = np.arange(100, 170, dtype=np.uint32)
    la = [a.forward(toks[i:i + 1])[0] for i in range(toks.size)][-1]
    lb = [b.forward(toks[i:i + 1])[0] for i in range(toks.size)][-1]
    assert rel_err(la, lb) > 1e-3
    for s in (stb, a, b):
        s.destroy()
    m.destroy(); dense.destroy()


def test_windows_snapshots_and_rollback_with_an_indexer(ctx):
    """Verify windows, kept prefixes and snapshots of a state whose queries are sparse: per-position logits of a window
    equal token-by-token steps; after keeping a prefix the state continues like one that only saw the prefix (a block
    that was pooled with rejected tokens is pooled again when its last token returns); a restored snapshot, whose pooled
    keys are rebuilt from the raw ones, continues with the same tokens; a 70-token prompt (longer than the dense range,
    so its tokens select blocks inside the prompt pass) gives the logits of 70 single steps."""
    cfg, m, om = _pair(ctx, 4, 23, n_layers=4)
    a, b = m.new_state(1), m.new_state(1)
    head = np.arange(200, 260, dtype=np.uint32)
    for t in head:
        a.forward([t]); b.forward([t])
    window = np.array([5, 6, 7, 8, 9, 10], np.uint32)
    lg = a.forward_multi(window)
    for j, tok in enumerate(window):
        assert rel_err(lg[j], b.forward([tok])[0]) < 1e-5
    a.spec_keep(6, 3)                       # position 63: the block of positions 60..63 was pooled with a rejected token
    c = m.new_state(1)
    for t in np.concatenate([head, window[:3]]):
        c.forward([t])
    snap = a.snapshot()
    ta = a.decode_greedy([77], 40)[0].tolist()
    assert ta == c.decode_greedy([77], 40)[0].tolist()
    d = m.new_state(1); d.restore(snap)
    assert d.decode_greedy([77], 40)[0].tolist() == ta
    e, f = m.new_state(1), m.new_state(1)
    prompt = np.arange(400, 470, dtype=np.uint32)
    le = e.forward(prompt)[0]
    for t in prompt:
        lf = f.forward([t])[0]
    assert rel_err(le, lf) < 5e-3           # the prompt's projections take the f16 tensor-core GEMM
    assert int(le.argmax()) == int(lf.argmax())
    assert ctx.device_status() == 0
    for s in (a, b, c, d, e, f):
        s.destroy()
    m.destroy()
