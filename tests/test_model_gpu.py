"""Token-loop parity: logits and greedy token ids of the engine against the CPU oracle."""
import numpy as np
import pytest

import oracle
import pyre_b200 as pb
from pyre_b200 import synth
from conftest import rel_err
from helpers import oracle_model, small_cfg

pytestmark = pytest.mark.gpu


def _greedy_pair(st, ost, first, n):
    tok = otok = first
    a, b, margins = [], [], []
    for _ in range(n):
        tok = int(st.step_greedy([tok])[0])
        otok = oracle.argmax(ost.forward([otok]))
        a.append(tok); b.append(otok); margins.append(ost.margins())
    return a, b, margins


@pytest.mark.parametrize("kv_bits", [0, 4])
def test_greedy_identity_small_model(ctx, kv_bits):
    """64 greedy steps on a scaled-down hybrid model (3 DeltaNet + 1 attention layer pattern, twice)."""
    cfg = small_cfg(pb, n_layers=8, kv_bits=kv_bits, kv_recent=64, max_ctx=256)
    spec = synth.model_spec(cfg, 1)
    m = synth.build_model(ctx, cfg, spec, 1)
    om, _ = oracle_model(cfg, spec, 1)
    st, ost = m.new_state(1), om.new_state()
    prompt = [3, 999, 27, 500, 1]
    lg, lo = st.forward(np.array(prompt, np.uint32))[0], ost.forward(prompt)
    assert rel_err(lg, lo) < 1e-3
    assert int(lg.argmax()) == oracle.argmax(lo)
    a, b, margins = _greedy_pair(st, ost, int(lg.argmax()), 64)
    assert a == b, f"diverged at step {next(i for i in range(64) if a[i] != b[i])}; oracle margins there {margins}"
    # the same tokens again through the device-resident multi-step path from a fresh state
    st2 = m.new_state(1)
    lg2 = st2.forward(np.array(prompt, np.uint32))[0]
    assert np.array_equal(lg2, lg)                           # deterministic
    assert st2.decode_greedy([int(lg2.argmax())], 64)[0].tolist() == a
    assert st2.pos() == len(prompt) + 64
    assert ctx.device_status() == 0
    st.destroy(); st2.destroy(); m.destroy()


def test_batch_sequences_are_independent(ctx):
    """Batch of 3 sequences fed different tokens equals three single-sequence runs."""
    cfg = small_cfg(pb, n_layers=4, max_ctx=64)
    spec = synth.model_spec(cfg, 2)
    m = synth.build_model(ctx, cfg, spec, 2)
    firsts = [11, 500, 77]
    stb = m.new_state(3)
    outb = stb.decode_greedy(firsts, 12)
    for i, f in enumerate(firsts):
        s1 = m.new_state(1)
        assert s1.decode_greedy([f], 12)[0].tolist() == outb[i].tolist()
        s1.destroy()
    stb.destroy(); m.destroy()


def test_large_batch_matches_single_sequences(ctx):
    """20 sequences with a 4-bit KV cache (tensor-core GEMM tiles of 16 + 4 tokens, pre-split expert hidden
    vectors, fine attention splits) produce the tokens of single-sequence runs."""
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=256)
    spec = synth.model_spec(cfg, 4)
    m = synth.build_model(ctx, cfg, spec, 4)
    rng = np.random.default_rng(12)
    k = rng.standard_normal((150, cfg.n_kv * cfg.hd)).astype(np.float32); v = rng.standard_normal((150, cfg.n_kv * cfg.hd)).astype(np.float32)
    firsts = [(37 * i + 5) % cfg.vocab for i in range(20)]

    def prefilled(batch):
        st = m.new_state(batch)
        for b in range(batch):
            for ai in range(cfg.n_layers // cfg.full_every):
                st.fill_kv(b, ai, k, v)
        st.set_pos(150)
        return st

    stb = prefilled(20)
    outb = stb.decode_greedy(firsts, 16)
    for i in (0, 7, 19):
        s1 = prefilled(1)
        assert s1.decode_greedy([firsts[i]], 16)[0].tolist() == outb[i].tolist(), i
        s1.destroy()
    assert ctx.device_status() == 0
    stb.destroy(); m.destroy()


def test_context_limit_and_bad_calls(ctx):
    cfg = small_cfg(pb, n_layers=4, max_ctx=8)
    spec = synth.model_spec(cfg, 0)
    m = synth.build_model(ctx, cfg, spec, 0)
    st = m.new_state(1)
    st.forward(np.arange(8, dtype=np.uint32))
    with pytest.raises(pb.PyreError):
        st.step_greedy([1])                                   # context full
    with pytest.raises(pb.PyreError):
        st.deltanet_step(3, np.zeros((1, cfg.d), np.float32)) # layer 3 is an attention layer
    with pytest.raises(pb.PyreError):
        pb.model.Model(ctx, small_cfg(pb, hc=4))              # hyper-connections are not built
    st.destroy(); m.destroy()


def test_verify_and_keep_roll_back(ctx):
    """forward_multi / spec_keep (:2365-2515): per-position logits agree with token-by-token forward (the
    window streams each weight once for all its tokens on the tensor-core path, so summation order differs:
    1e-5, not bit for bit); keeping a prefix of the window leaves the state as if only that prefix had been fed."""
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=256)
    spec = synth.model_spec(cfg, 4)
    m = synth.build_model(ctx, cfg, spec, 4)
    om, _ = oracle_model(cfg, spec, 4)
    prompt = np.array([9, 8, 7, 6, 5, 4], np.uint32)
    window = np.array([100, 200, 300, 400, 500], np.uint32)
    a = m.new_state(1); a.forward(prompt)
    lg = a.forward_multi(window)
    assert lg.shape == (5, cfg.vocab) and a.pos() == 11
    b = m.new_state(1); b.forward(prompt)
    ost = om.new_state(); ost.forward(prompt.tolist())
    for j, tok in enumerate(window):
        assert rel_err(lg[j], b.forward([tok])[0]) < 1e-5                    # batched window vs one token at a time
        assert rel_err(lg[j], ost.forward([int(tok)])) < 1e-3               # and the oracle agrees
    a.spec_keep(5, 2)                                                        # accept 100, 200; drop the rest
    assert a.pos() == 8
    c = m.new_state(1); c.forward(np.concatenate([prompt, window[:2]]))
    assert a.decode_greedy([77], 24)[0].tolist() == c.decode_greedy([77], 24)[0].tolist()
    # keeping the whole window is a no-op; mismatched calls fail loudly
    a.forward_multi(window[:3]); a.spec_keep(3, 3)
    with pytest.raises(pb.PyreError):
        a.spec_keep(3, 1)                                                    # no window pending
    with pytest.raises(pb.PyreError):
        a.forward_multi(np.arange(9, dtype=np.uint32))                       # window larger than 8
    for s in (a, b, c):
        s.destroy()
    m.destroy()


@pytest.mark.parametrize("kv_bits", [0, 4])
def test_snapshot_restore(ctx, kv_bits):
    """snapshot / restore (Snap :3277-3298): a restored state continues with identical tokens."""
    cfg = small_cfg(pb, n_layers=8, kv_bits=kv_bits, kv_recent=64, max_ctx=400)
    spec = synth.model_spec(cfg, 6)
    m = synth.build_model(ctx, cfg, spec, 6)
    a = m.new_state(1)
    first = a.decode_greedy([3], 150)[0]                  # crosses the first 4-bit repack boundary at 128
    blob = a.snapshot()
    cont = a.decode_greedy([int(first[-1])], 40)[0]
    b = m.new_state(1)
    b.restore(blob)
    assert b.pos() == 150
    assert b.decode_greedy([int(first[-1])], 40)[0].tolist() == cont.tolist()
    with pytest.raises(pb.PyreError):
        b.restore(blob[:100])                              # truncated
    with pytest.raises(pb.PyreError):
        m.new_state(2).restore(blob)                       # different batch
    a.destroy(); b.destroy(); m.destroy()


def test_snapshot_after_rollback_across_repack_boundary(ctx):
    """A verify window that crosses a 64-position repack boundary moves the packed boundary of the 4-bit cache
    forward; rolling the window back (spec_keep) does not move it back.  A snapshot taken then must carry the
    boundary the device holds, and a state restored from it must continue exactly like the original."""
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=400)
    spec = synth.model_spec(cfg, 8)
    m = synth.build_model(ctx, cfg, spec, 8)
    a = m.new_state(1)
    a.forward((np.arange(121, dtype=np.uint32) * 7 + 3) % cfg.vocab)       # pos 121; ring capacity 64 + 64
    a.forward_multi(np.array([5, 6, 7, 8, 9, 10, 11, 12], np.uint32))       # len reaches 129: positions 0..63 packed
    a.spec_keep(8, 1)                                                      # back to pos 122, boundary stays at 64
    assert a.pos() == 122
    blob = a.snapshot()
    b = m.new_state(1)
    b.restore(blob)
    assert b.pos() == 122
    ta = a.decode_greedy([77], 48)[0].tolist()
    tb = b.decode_greedy([77], 48)[0].tolist()
    assert ta == tb
    with pytest.raises(pb.PyreError) as e:
        a.set_pos(10)                                                      # below the packed boundary
    assert e.value.status == pb.PB_ERR_STATE
    for s in (a, b):
        s.destroy()
    m.destroy()


def test_rewound_state_equals_fresh_state(ctx):
    """set_pos(0) starts a new sequence in a used state: the packed boundary goes back to 0, so new f32 rows are not
    mistaken for packed ones.  With the DeltaNet state cleared the tokens equal those of a fresh state."""
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=400)
    spec = synth.model_spec(cfg, 9)
    m = synth.build_model(ctx, cfg, spec, 9)
    a = m.new_state(1)
    a.decode_greedy([3], 200)                                              # boundary at 128 by now
    a.set_pos(0)
    ch = 2 * cfg.lin_nk * cfg.lin_dk + cfg.lin_nv * cfg.lin_dv
    for il in range(cfg.n_layers):
        if (il + 1) % cfg.full_every:
            a.set_lin(il, np.zeros((1, cfg.conv_k - 1, ch), np.float32), np.zeros((1, cfg.lin_nv, cfg.lin_dk, cfg.lin_dv), np.float32))
    f = m.new_state(1)
    assert a.decode_greedy([9], 150)[0].tolist() == f.decode_greedy([9], 150)[0].tolist()
    a.destroy(); f.destroy(); m.destroy()


def test_step_graph_captured_early_serves_a_long_context(ctx):
    """The step graph is captured on the second step.  Captured at an almost empty context and replayed after the
    cache was filled to thousands of positions, it must still give the tokens of a graph captured at that length:
    the split of attention work between packed and f32 positions is made on the device from the current length."""
    cfg = small_cfg(pb, n_layers=4, kv_bits=4, kv_recent=64, max_ctx=4400)
    spec = synth.model_spec(cfg, 10)
    m = synth.build_model(ctx, cfg, spec, 10)
    rng = np.random.default_rng(5)
    k = rng.standard_normal((4000, cfg.n_kv * cfg.hd)).astype(np.float32); v = rng.standard_normal((4000, cfg.n_kv * cfg.hd)).astype(np.float32)
    early = m.new_state(1)
    early.decode_greedy([1], 4)                                            # graph captured at positions 1..3
    early.set_pos(0)
    for il in range(cfg.n_layers):
        if (il + 1) % cfg.full_every:
            ch = 2 * cfg.lin_nk * cfg.lin_dk + cfg.lin_nv * cfg.lin_dv
            early.set_lin(il, np.zeros((1, cfg.conv_k - 1, ch), np.float32), np.zeros((1, cfg.lin_nv, cfg.lin_dk, cfg.lin_dv), np.float32))
    late = m.new_state(1)
    for s in (early, late):
        s.fill_kv(0, 0, k, v); s.set_pos(4000)
    assert early.decode_greedy([2], 24)[0].tolist() == late.decode_greedy([2], 24)[0].tolist()
    early.destroy(); late.destroy(); m.destroy()


def test_contexts_on_two_devices_in_one_process():
    """One process may hold a context per GPU: kernel attributes (shared-memory limits) are kept per context and
    every entry point makes its context's GPU current."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    outs = []
    ctxs = [pb.Ctx(0), pb.Ctx(1)]
    x = np.random.default_rng(0).standard_normal((1, 2048)).astype(np.float32)
    mats = [pb.QMat.synth(c, pb.IQ3_S, 4096, 2048, 0, 5) for c in ctxs]
    for _ in range(2):                                                     # alternate, so the current device keeps changing
        for W in mats:
            outs.append(W.matmul(x))
    assert all(np.array_equal(outs[0], o) for o in outs[1:])
    for W in mats:
        W.free()
    for c in ctxs:
        c.close()


def _fused_cfg(**kw):
    """A scaled-down hybrid model whose every matrix has a re-coded copy, so that a batch-1 state takes its steps
    through the fused step kernel when PYRE_B200_FUSED=1 asks for it (expert width 512; hidden 512)."""
    base = dict(n_layers=8, ff_exp=512, ff_sh=512, kv_bits=4, kv_recent=64, max_ctx=256)
    base.update(kw)
    return small_cfg(pb, **base)


def test_fused_step_matches_per_operation_kernels_bit_for_bit(ctx, monkeypatch):
    """The fused step kernel runs the arithmetic of the per-operation kernels: logits and tokens must be identical,
    not merely close.  PYRE_B200_FUSED=1 (read at a state's first step) puts a state on the fused path."""
    cfg = _fused_cfg()
    spec = synth.model_spec(cfg, 11)
    m = synth.build_model(ctx, cfg, spec, 11)
    fused, plain = m.new_state(1), m.new_state(1)
    monkeypatch.setenv("PYRE_B200_FUSED", "1")
    lf = fused.forward([5])[0]                                   # first step decides the path of `fused`
    monkeypatch.delenv("PYRE_B200_FUSED")
    lp = plain.forward([5])[0]
    assert fused.stats().kernels_launched < plain.stats().kernels_launched   # the fused path really ran
    assert np.array_equal(lf.view(np.uint32), lp.view(np.uint32))
    tok = int(lf.argmax())
    for _ in range(6):                                           # eager step, captured graph, replays
        lf, lp = fused.forward([tok])[0], plain.forward([tok])[0]
        assert np.array_equal(lf.view(np.uint32), lp.view(np.uint32))
        tok = int(lf.argmax())
    assert fused.decode_greedy([tok], 150)[0].tolist() == plain.decode_greedy([tok], 150)[0].tolist()   # crosses a KV repack boundary
    assert ctx.device_status() == 0
    fused.destroy(); plain.destroy(); m.destroy()


def test_fused_step_greedy_identity_vs_oracle(ctx, monkeypatch):
    monkeypatch.setenv("PYRE_B200_FUSED", "1")
    cfg = _fused_cfg()
    spec = synth.model_spec(cfg, 12)
    m = synth.build_model(ctx, cfg, spec, 12)
    om, _ = oracle_model(cfg, spec, 12)
    st, ost = m.new_state(1), om.new_state()
    tok = otok = 17
    for i in range(64):
        lg = st.forward([tok])[0]
        lo = ost.forward([otok])
        assert rel_err(lg, lo) < 1e-3, i
        tok, otok = int(lg.argmax()), oracle.argmax(lo)
        assert tok == otok, (i, ost.margins())
    assert ctx.device_status() == 0
    st.destroy(); m.destroy()


@pytest.mark.parametrize("hc", [1, 2])
def test_hyper_connection_greedy_identity_vs_oracle(ctx, hc):
    """The reference's own residual form: hc parallel streams mixed before every block and recombined after it
    (hc_mix / hc_combine, src/model/qwen4exp_gguf.rs:1357-1388), low rank 32.  Prompt logits and 64 greedy tokens
    against the CPU oracle; the verify window and the batched form agree with the token loop."""
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=256, hc=hc, hc_lr=32)
    spec = synth.model_spec(cfg, 31)
    m = synth.build_model(ctx, cfg, spec, 31)
    om, _ = oracle_model(cfg, spec, 31)
    st, ost = m.new_state(1), om.new_state()
    prompt = [3, 999, 27, 500, 1]
    lg, lo = st.forward(np.array(prompt, np.uint32))[0], ost.forward(prompt)
    assert rel_err(lg, lo) < 1e-3
    assert int(lg.argmax()) == oracle.argmax(lo)
    a, b, margins = _greedy_pair(st, ost, int(lg.argmax()), 64)
    assert a == b, f"diverged at step {next(i for i in range(64) if a[i] != b[i])}; oracle margins there {margins}"
    # two sequences in one batch: each equals its own single-sequence run
    s2 = m.new_state(2)
    t2 = s2.decode_greedy([5, 600], 12)
    for i, first in enumerate([5, 600]):
        s1 = m.new_state(1)
        assert s1.decode_greedy([first], 12)[0].tolist() == t2[i].tolist()
        s1.destroy()
    # a verify window: per-position logits against the oracle's token loop
    w = m.new_state(1); ow = om.new_state()
    win = np.array([7, 8, 9, 10, 11], np.uint32)
    lw = w.forward_multi(win)
    for j, tok in enumerate(win):
        assert rel_err(lw[j], ow.forward([int(tok)])) < 1e-3
    assert ctx.device_status() == 0
    for x in (st, s2, w):
        x.destroy()
    m.destroy()


@pytest.mark.parametrize("kv_bits", [0, 4])
def test_yarn_scaled_context_greedy_identity_vs_oracle(ctx, kv_bits):
    """A context of 256 positions on a model trained on 64: the rope table is YaRN-scaled for the whole run (frequencies
    and mscale on cos and sin, Model::load :490-517).  Prompt logits within 1e-3 and 48 greedy ids identical to the oracle;
    and the scaling is really in effect (the logits differ from the same model without a trained-context limit)."""
    cfg = small_cfg(pb, n_layers=8, kv_bits=kv_bits, kv_recent=64, max_ctx=256)
    spec = synth.model_spec(cfg, 5)
    m = synth.build_model(ctx, cfg, spec, 5, ctx_train=64)
    om, _ = oracle_model(cfg, spec, 5, ctx_train=64)
    st, ost = m.new_state(1), om.new_state()
    prompt = list(range(40, 64))     # 24 tokens: below the size from which prompts take the f16 tensor-core GEMM
    lg, lo = st.forward(np.array(prompt, np.uint32))[0], ost.forward(prompt)
    assert rel_err(lg, lo) < 1e-3
    assert int(lg.argmax()) == oracle.argmax(lo)
    a, b, margins = _greedy_pair(st, ost, int(lg.argmax()), 48)
    assert a == b, f"diverged at step {next(i for i in range(48) if a[i] != b[i])}; oracle margins there {margins}"
    m0 = synth.build_model(ctx, cfg, spec, 5)
    st0 = m0.new_state(1)
    lg0 = st0.forward(np.array(prompt, np.uint32))[0]
    assert rel_err(lg0, lg) > 1e-3
    with pytest.raises(pb.PyreError):
        m.set_ctx_train(128)          # after finalize
    assert ctx.device_status() == 0
    st.destroy(); st0.destroy(); m.destroy(); m0.destroy()


@pytest.mark.parametrize("name", ["Q8_0", "Q4_K", "IQ2_XS", "IQ3_XXS", "IQ2_S", "IQ4_NL", "IQ4_XS", "IQ2_XXS", "Q6_K", "Q2_0", "IQ1_M", "Q4_0", "Q5_0", "Q3_K", "Q5_K"])
def test_other_quant_formats_greedy_identity_vs_oracle(ctx, name):
    """The token loop with every matrix in one of the other streaming formats (the per-operation kernels; the fused step
    kernel is for re-coded IQ3_S): prompt logits within 1e-3 and 32 greedy ids identical to the oracle.  Q8_0 rows are the
    widest (34 bytes per 32 weights): the expert kernels then take fewer rows per chunk than they have consumer warps."""
    qt = getattr(pb, name)
    cfg = small_cfg(pb, n_layers=4, kv_bits=4, kv_recent=64, max_ctx=128)
    spec = synth.model_spec(cfg, 7, qtype=qt)
    m = synth.build_model(ctx, cfg, spec, 7)
    om, _ = oracle_model(cfg, spec, 7)
    st, ost = m.new_state(1), om.new_state()
    prompt = [5, 900, 31, 77]
    lg, lo = st.forward(np.array(prompt, np.uint32))[0], ost.forward(prompt)
    assert rel_err(lg, lo) < 1e-3
    a, b, margins = _greedy_pair(st, ost, int(lg.argmax()), 32)
    assert a == b, (name, margins)
    assert ctx.device_status() == 0
    st.destroy(); m.destroy()


def test_forward_into_page_locked_buffer(ctx):
    """pb_forward / pb_verify write straight into a destination from pb_host_alloc: same logits as through a pageable array."""
    cfg = small_cfg(pb, n_layers=4, kv_bits=4, kv_recent=64, max_ctx=128)
    spec = synth.model_spec(cfg, 5)
    m = synth.build_model(ctx, cfg, spec, 5)
    a, b = m.new_state(1), m.new_state(1)
    out = ctx.pinned_empty((1, cfg.vocab))
    for tok in (3, 400, 9):
        la = a.forward([tok], out=out)
        assert la is out
        assert np.array_equal(la, b.forward([tok]))
    with pytest.raises(ValueError):
        a.forward([1], out=np.empty((2, cfg.vocab), np.float32))
    del out, la
    assert ctx.device_status() == 0
    a.destroy(); b.destroy(); m.destroy()
