"""Batched prompt prefill (256-token chunks on the absolute grid, tcgen05 GEMM for the dense projections, the DeltaNet
recurrence looped inside one kernel) against the CPU oracle and against token-by-token decoding, and the prefix cache."""
import numpy as np
import pytest

import oracle
import pyre_b200 as pb
from pyre_b200 import synth
from pyre_b200.prefix import PrefixCache
from conftest import rel_err
from helpers import oracle_model, small_cfg

pytestmark = pytest.mark.gpu
# The chunked pass rounds the dense projections' weights to f16 once (tensor-core GEMM); the recurrent layers carry that
# noise through the prompt.  The reference's own batched prefill runs its projections on f16 tensor cores as well
# (k_gemm_tc, src/model/qn_cube.rs:153) and is compared with its f32 path at the level of generated tokens.
PREFILL_TOL = 5e-3


def _model(ctx, seed, **kw):
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, **kw)
    spec = synth.model_spec(cfg, seed)
    return cfg, spec, synth.build_model(ctx, cfg, spec, seed)


@pytest.mark.parametrize("n", [40, 300])
def test_prefill_logits_vs_oracle_and_stepwise(ctx, n):
    """A prompt of n tokens (n = 300: a full 256-token chunk and a ragged one): last-position logits against the CPU
    oracle's token loop and against this library's own exact token-by-token path; the greedy continuation agrees."""
    cfg, spec, m = _model(ctx, 21, max_ctx=512)
    om, _ = oracle_model(cfg, spec, 21)
    prompt = np.random.default_rng(n).integers(0, cfg.vocab, size=n).astype(np.uint32)
    st = m.new_state(1)
    lg = st.forward(prompt)[0]
    assert st.pos() == n
    lo = om.new_state().forward([int(t) for t in prompt])
    assert rel_err(lg, lo) < PREFILL_TOL
    one = m.new_state(1)
    for t in prompt:
        l1 = one.forward(np.array([t], np.uint32))[0]
    assert rel_err(l1, lo) < 1e-3                      # the token-by-token path keeps the decode tolerance
    assert rel_err(lg, l1) < PREFILL_TOL
    assert int(lg.argmax()) == int(l1.argmax()) == oracle.argmax(lo)
    # decoding continues from the prefilled state like from the stepped one (first tokens; later ones may drift apart)
    a = st.decode_greedy([int(lg.argmax())], 8)[0]
    b = one.decode_greedy([int(l1.argmax())], 8)[0]
    assert a[0] == b[0]
    assert ctx.device_status() == 0
    st.destroy(); one.destroy(); m.destroy()


def test_prefill_is_deterministic_and_independent_of_the_call_split(ctx):
    """The same prompt in one pb_forward call or in several: the pieces always end on the absolute 256-token grid, so
    the state and the logits are bit-identical."""
    cfg, spec, m = _model(ctx, 22, max_ctx=1024)
    prompt = np.random.default_rng(7).integers(0, cfg.vocab, size=700).astype(np.uint32)
    a = m.new_state(1)
    la = a.forward(prompt)[0]
    b = m.new_state(1)
    b.forward(prompt[:256]); b.forward(prompt[256:512]); lb = b.forward(prompt[512:])[0]
    assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    c = m.new_state(1)
    lc = c.forward(prompt)[0]
    assert np.array_equal(la.view(np.uint32), lc.view(np.uint32))
    assert a.decode_greedy([5], 16)[0].tolist() == b.decode_greedy([5], 16)[0].tolist()
    a.destroy(); b.destroy(); c.destroy(); m.destroy()


def test_prefix_cache_resume_is_bit_identical_to_a_full_prefill(ctx):
    """Snapshots at the grid boundaries; a second prompt sharing 520 tokens resumes from the snapshot at 512 and must
    reach exactly the logits of a prefill from scratch (src/engine_qn.rs:92-139)."""
    cfg, spec, m = _model(ctx, 23, max_ctx=1024)
    rng = np.random.default_rng(9)
    first = rng.integers(0, cfg.vocab, size=600).astype(np.uint32)
    second = np.concatenate([first[:520], rng.integers(0, cfg.vocab, size=90).astype(np.uint32)])
    st = m.new_state(1)
    pc = PrefixCache()
    _, s1 = pc.prefill(st, first)
    assert s1.source == "new" and s1.snapshots_taken == 2 and s1.pieces == [(0, 256), (256, 512), (512, 600)]
    l2, s2 = pc.prefill(st, second)
    assert s2.source == "snapshot" and s2.cached_n == 512 and s2.pieces == [(512, 610)]
    fresh = m.new_state(1)
    lf = fresh.forward(second)[0]
    assert np.array_equal(l2[0].view(np.uint32), lf.view(np.uint32))
    assert st.pos() == fresh.pos() == len(second)
    # and the continuation
    assert st.decode_greedy([int(l2[0].argmax())], 12)[0].tolist() == fresh.decode_greedy([int(lf.argmax())], 12)[0].tolist()
    st.destroy(); fresh.destroy(); m.destroy()


def test_reset_starts_a_fresh_conversation(ctx):
    cfg, spec, m = _model(ctx, 24, max_ctx=512)
    st = m.new_state(1)
    st.forward(np.arange(300, dtype=np.uint32) % cfg.vocab)
    st.reset()
    assert st.pos() == 0
    fresh = m.new_state(1)
    p = np.array([4, 8, 15, 16, 23, 42], np.uint32)
    assert np.array_equal(st.forward(p), fresh.forward(p))
    st.destroy(); fresh.destroy(); m.destroy()
