"""Per-layer n-gram embeddings (ple_rows / ple, src/model/qwen4exp_gguf.rs:1390-1434): the token loop, windows, rollbacks, batches and
snapshots of a model whose layers 2 and 6 inject them, against the CPU oracle."""
import numpy as np
import pytest

import oracle
import pyre_b200 as pb
from pyre_b200 import synth
from conftest import rel_err
from helpers import oracle_model, small_cfg

pytestmark = pytest.mark.gpu
EOS = 2


def _build(ctx, hc, seed=61, qtype=None, **geo):
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=320, hc=hc, hc_lr=32)
    ple = synth.ple_geometry([2, 6], eos=EOS, **geo)
    spec = synth.model_spec(cfg, seed, ple=ple) if qtype is None else synth.model_spec(cfg, seed, qtype=qtype, ple=ple)
    m = synth.build_model(ctx, cfg, spec, seed, ple=ple)
    om, _ = oracle_model(cfg, spec, seed, ple=ple)
    return cfg, m, om


@pytest.mark.parametrize("hc", [0, 2])
def test_ple_token_loop_vs_oracle(ctx, hc):
    """Prompt (one window, with an end-of-sequence id inside that cuts the contexts after it) and 48 greedy steps; the injected
    model differs from the same model without the tensors."""
    cfg, m, om = _build(ctx, hc)
    st, ost = m.new_state(1), om.new_state()
    prompt = [3, 999, EOS, 27, 500, 1, 1, 77, 42]
    lg, lo = st.forward(np.array(prompt, np.uint32))[0], ost.forward(prompt)
    assert rel_err(lg, lo) < 1e-3
    tok = otok = int(lg.argmax())
    assert tok == oracle.argmax(lo)
    for i in range(48):
        tok = int(st.step_greedy([tok])[0]); otok = oracle.argmax(ost.forward([otok]))
        assert tok == otok, (i, ost.margins())
    plain_spec = synth.model_spec(cfg, 61)
    plain = synth.build_model(ctx, cfg, plain_spec, 61)
    ps = plain.new_state(1)
    assert rel_err(ps.forward(np.array(prompt, np.uint32))[0], lo) > 1e-2      # the injection matters
    assert ctx.device_status() == 0
    st.destroy(); ps.destroy(); m.destroy(); plain.destroy()


def test_ple_window_rollback_batch_and_snapshot(ctx):
    cfg, m, om = _build(ctx, 2, seed=62)
    prompt = np.array([9, 8, 7, 6, 5, 4], np.uint32)
    window = np.array([100, 200, EOS, 400, 500, 600, 700], np.uint32)
    a = m.new_state(1); a.forward(prompt)
    lg = a.forward_multi(window)
    ost = om.new_state(); ost.forward(prompt.tolist())
    for j, tok in enumerate(window):
        assert rel_err(lg[j], ost.forward([int(tok)])) < 1e-3                  # every position of the window against the oracle's token loop
    a.spec_keep(7, 3)                                                          # accept three, drop four: no checkpoint needed, rows go by position
    c = m.new_state(1); c.forward(np.concatenate([prompt, window[:3]]))
    ta, tc = a.decode_greedy([77], 24)[0].tolist(), c.decode_greedy([77], 24)[0].tolist()
    assert ta == tc
    oc = om.new_state(); oc.forward(np.concatenate([prompt, window[:3]]).tolist())
    otok, ref = 77, []
    for _ in range(24):
        otok = oracle.argmax(oc.forward([otok])); ref.append(otok)
    assert ta == ref
    # a batch of sequences: each equals its own single-sequence run (histories are per sequence)
    s3 = m.new_state(3)
    t3 = s3.decode_greedy([5, 600, 5], 16)
    for i, first in enumerate([5, 600, 5]):
        s1 = m.new_state(1)
        assert s1.decode_greedy([first], 16)[0].tolist() == t3[i].tolist()
        s1.destroy()
    # snapshot / restore carries the last ids and the last normalized rows
    blob = a.snapshot()
    cont = a.decode_greedy([ta[-1]], 12)[0].tolist()
    b = m.new_state(1); b.restore(blob)
    assert b.decode_greedy([ta[-1]], 12)[0].tolist() == cont
    # a reset state starts a fresh history
    a.reset()
    assert a.decode_greedy([5], 16)[0].tolist() == t3[0].tolist()
    assert ctx.device_status() == 0
    for s in (a, b, c, s3):
        s.destroy()
    m.destroy()


def test_ple_long_prompt_chunks_and_other_geometry(ctx):
    """A prompt longer than one prefill chunk (the history crosses chunk boundaries and the ring wraps), 4-grams with one head each,
    a Q8_0 table and projections, two conv taps."""
    cfg, m, om = _build(ctx, 1, seed=63, qtype=pb.Q8_0, ngram=4, per_gram=1, conv_k=2, dim=256)
    rng = np.random.default_rng(5)
    prompt = rng.integers(3, cfg.vocab, 300 - 8).astype(np.uint32)
    st, ost = m.new_state(1), om.new_state()
    lg, lo = st.forward(prompt)[0], ost.forward(prompt.tolist())
    assert rel_err(lg, lo) < 5e-3                                              # prefill chunks of 32 tokens and more take the tcgen05 GEMM
    tok = otok = int(lg.argmax())
    for i in range(8):
        tok = int(st.step_greedy([tok])[0]); otok = oracle.argmax(ost.forward([otok]))
        assert tok == otok, (i, ost.margins())
    st.destroy(); m.destroy()


def test_ple_argument_checks(ctx):
    cfg = small_cfg(pb, n_layers=4, max_ctx=64)
    geo = synth.ple_geometry([1])
    spec = synth.model_spec(cfg, 1, ple=geo)
    with pytest.raises(pb.PyreError):
        synth.build_model(ctx, cfg, spec, 1)                                   # tensors present, geometry never set
    m = pb.model.Model(ctx, cfg)
    with pytest.raises(pb.PyreError):
        m.set_ple(9, 1, 4, EOS, 256, [1] * 9, [0] * 8, [10] * 8)               # 9-grams
    with pytest.raises(pb.PyreError):
        m.set_ple(3, 2, 4, EOS, 100, [1] * 3, [0] * 4, [10] * 4)               # rows of 100 values
    with pytest.raises(pb.PyreError):
        m.set_ple(3, 2, 4, EOS, 256, [1] * 3, [0] * 4, [10, 0, 10, 10])        # an empty head
    m.destroy()
    bad = dict(geo); bad["vocab"] = [v + 50 for v in geo["vocab"]]             # heads reach past the table
    with pytest.raises(pb.PyreError):
        synth.build_model(ctx, cfg, spec, 1, ple=bad)
