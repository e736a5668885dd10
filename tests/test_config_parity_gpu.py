"""Parity at the benchmark's own configurations (the shapes bench.py times), through the C ABI:

  * gated attention of config 4: 32768 pre-filled positions in a 4-bit cache with a 1024-position f32
    window, decode steps that cross a 64-position repack boundary, 1 and 4 sequences;
  * Gated DeltaNet of config 2: 64 sequences, 256 sequential steps;
  * MoE block of config 3 at 128 tokens;
  * the full 48-layer model: 64 greedy tokens identical to the CPU oracle's (committed fixture,
    tests/golden/make_full_model_golden.py).

Tolerance: 1e-3 of the largest reference magnitude (f32 accumulate), greedy ids identical.
"""
import sys
from pathlib import Path

import numpy as np
import pytest

import oracle
import pyre_b200 as pb
from pyre_b200 import synth
from conftest import rel_err
from helpers import oracle_cfg, oracle_model

pytestmark = pytest.mark.gpu
TOL = 1e-3
GOLDEN = Path(__file__).resolve().parent / "golden"


def _attn_case(ctx, batch):
    """One attention layer of config-4 shape at a 32768-token context; steps run across len = 32768, where
    (len - 1024) / 64 grows and 64 more positions are re-packed to 4 bits."""
    n0, steps = 32740, 40
    cfg = pb.make_cfg(n_layers=4, full_every=4, vocab=1024, max_ctx=32768 + 64, kv_bits=4, kv_recent=1024, n_exp=16, top_k=2)
    spec = synth.model_spec(cfg, 0)
    m = synth.build_model(ctx, cfg, spec, 0)
    _, mats = oracle_model(cfg, spec, 0)
    ocfg = oracle_cfg(cfg)
    layer, row = 3, cfg.n_kv * cfg.hd
    st = m.new_state(batch)
    rng = np.random.default_rng(40 + batch)
    kc = [np.zeros((cfg.max_ctx, row), np.float32) for _ in range(batch)]
    vc = [np.zeros((cfg.max_ctx, row), np.float32) for _ in range(batch)]
    for b in range(batch):
        kc[b][:n0] = rng.standard_normal((n0, row)); vc[b][:n0] = rng.standard_normal((n0, row))
        st.fill_kv(b, 0, kc[b][:n0], vc[b][:n0])
    st.set_pos(n0)
    inv = oracle.rope_inv(cfg.n_rot, cfg.rope_base)
    q4n = ((n0 - cfg.kv_recent) // 64) * 64
    packed = [(*oracle.kv4_pack(kc[b][:q4n]), *oracle.kv4_pack(vc[b][:q4n])) for b in range(batch)]
    worst, crossed = 0.0, False
    for step in range(steps):
        pos = n0 + step
        x = rng.standard_normal((batch, cfg.d)).astype(np.float32)
        y = st.attn_step(layer, x)
        st.set_pos(pos + 1)
        want = ((pos + 1 - cfg.kv_recent) // 64) * 64          # kv_push :1520
        for b in range(batch):
            qf, kf, vf = (mats[(layer, r)].matmul(x[b])[0] for r in ("ATTN_Q", "ATTN_K", "ATTN_V"))
            if want > q4n:
                packed[b] = (*oracle.kv4_pack(kc[b][:want]), *oracle.kv4_pack(vc[b][:want]))
            att = oracle.attn_core(ocfg, qf, kf, vf, mats[(layer, "ATTN_Q_NORM")], mats[(layer, "ATTN_K_NORM")], inv, kc[b], vc[b], pos,
                                   packed[b], max(want, q4n))
            worst = max(worst, rel_err(y[b], mats[(layer, "ATTN_O")].matmul(att)[0]))
        if want > q4n:
            q4n, crossed = want, True
    assert crossed and q4n == 31744
    assert ctx.device_status() == 0
    st.destroy(); m.destroy()
    return worst


@pytest.mark.parametrize("batch", [1, 4])
def test_attention_config4_context(ctx, batch):
    assert _attn_case(ctx, batch) < TOL


def test_sparse_attention_config4_context(ctx):
    """The same layer with the QSA indexer at the reference's defaults (budget 2048 tokens in blocks of 4, index heads of
    128): 32740 pre-filled positions with their raw index keys, then decode steps of two sequences.  Every query scores
    8185 pooled block keys, takes the best 512 plus the tail, and attends to them in the 4-bit region (tensor-core tiles
    with masked positions, untouched tiles skipped) and in the f32 window; outputs within 1e-3 of the oracle, which makes
    its own selection from its own keys; the smallest selection margin met is checked to be resolvable in f32."""
    n0, steps, batch = 32740, 10, 2
    indexer = (2048, 4, 4, 128)
    budget, ratio, inh, ihd = indexer
    cfg = pb.make_cfg(n_layers=4, full_every=4, vocab=1024, max_ctx=32768 + 64, kv_bits=4, kv_recent=1024, n_exp=16, top_k=2)
    spec = synth.model_spec(cfg, 0, indexer=indexer)
    m = synth.build_model(ctx, cfg, spec, 0, indexer=indexer)
    _, mats = oracle_model(cfg, spec, 0, indexer=indexer)
    ocfg = oracle_cfg(cfg)
    layer, row = 3, cfg.n_kv * cfg.hd
    st = m.new_state(batch)
    rng = np.random.default_rng(77)
    inv = oracle.rope_inv(cfg.n_rot, cfg.rope_base)
    kc, vc, ik, ib, packed = [], [], [], [], []
    q4n = ((n0 - cfg.kv_recent) // 64) * 64
    for b in range(batch):
        kc.append(np.zeros((cfg.max_ctx, row), np.float32)); vc.append(np.zeros((cfg.max_ctx, row), np.float32)); ik.append(np.zeros((cfg.max_ctx, ihd), np.float32))
        kc[b][:n0] = rng.standard_normal((n0, row)); vc[b][:n0] = rng.standard_normal((n0, row)); ik[b][:n0] = rng.standard_normal((n0, ihd))
        st.fill_kv(b, 0, kc[b][:n0], vc[b][:n0]); st.fill_index_keys(b, 0, ik[b][:n0])
        ib.append(np.zeros((cfg.max_ctx // ratio + 1, ihd), np.float32))
        for blk in range(n0 // ratio):
            ib[b][blk] = oracle.qsa_pool(ocfg, ratio, ik[b], mats[(layer, "IDX_K_NORM")], inv, blk)
        packed.append((*oracle.kv4_pack(kc[b][:q4n]), *oracle.kv4_pack(vc[b][:q4n])))
    st.set_pos(n0)
    worst, min_margin = 0.0, float("inf")
    for step in range(steps):
        pos = n0 + step
        x = rng.standard_normal((batch, cfg.d)).astype(np.float32)
        y = st.attn_step(layer, x)
        st.set_pos(pos + 1)
        assert ((pos + 1 - cfg.kv_recent) // 64) * 64 == q4n       # no packing step inside this run
        for b in range(batch):
            qf, kf, vf, iq, ikf = (mats[(layer, r)].matmul(x[b])[0] for r in ("ATTN_Q", "ATTN_K", "ATTN_V", "IDX_Q", "IDX_K"))
            ik[b][pos] = ikf
            if (pos + 1) % ratio == 0:
                ib[b][pos // ratio] = oracle.qsa_pool(ocfg, ratio, ik[b], mats[(layer, "IDX_K_NORM")], inv, pos // ratio)
            blocks, margin = oracle.qsa_select(ocfg, budget, ratio, iq.reshape(inh, ihd), mats[(layer, "IDX_Q_NORM")], inv, ib[b], pos)
            assert blocks.size == budget // ratio
            min_margin = min(min_margin, margin)
            ps = np.concatenate([(blocks[:, None] * ratio + np.arange(ratio)[None]).reshape(-1), np.arange(((pos + 1) // ratio) * ratio, pos + 1)])
            att = oracle.attn_core(ocfg, qf, kf, vf, mats[(layer, "ATTN_Q_NORM")], mats[(layer, "ATTN_K_NORM")], inv, kc[b], vc[b], pos, packed[b], q4n, ps=ps)
            worst = max(worst, rel_err(y[b], mats[(layer, "ATTN_O")].matmul(att)[0]))
    assert min_margin > 1e-6, min_margin
    assert worst < TOL, (worst, min_margin)
    assert ctx.device_status() == 0
    st.destroy(); m.destroy()


def test_deltanet_config2_batch64_256_steps(ctx):
    """Config 2 verbatim: 64 sequences, state N(0, 0.1), 256 sequential steps.  The sequences are independent, so the
    oracle follows a sample of them (first, last and two inside); their outputs are checked at every step and
    their states every 32 steps."""
    cfg = pb.make_cfg(n_layers=1, full_every=0, vocab=1024, max_ctx=512, n_exp=16, top_k=2)
    spec = synth.model_spec(cfg, 0)
    m = synth.build_model(ctx, cfg, spec, 0)
    _, mats = oracle_model(cfg, spec, 0)
    ocfg = oracle_cfg(cfg)
    B, steps, watch = 64, 256, [0, 21, 42, 63]
    rng = np.random.default_rng(64)
    ch = 2 * cfg.lin_nk * cfg.lin_dk + cfg.lin_nv * cfg.lin_dv
    conv = np.zeros((B, cfg.conv_k - 1, ch), np.float32)
    ssm = (0.1 * rng.standard_normal((B, cfg.lin_nv, cfg.lin_dk, cfg.lin_dv))).astype(np.float32)
    st = m.new_state(B)
    st.set_lin(0, conv, ssm)
    oconv = {b: np.ascontiguousarray(conv[b]) for b in watch}
    ossm = {b: np.ascontiguousarray(ssm[b]) for b in watch}
    worst = 0.0
    for step in range(steps):
        x = rng.standard_normal((B, cfg.d)).astype(np.float32)
        y = st.deltanet_step(0, x)
        st.set_pos(st.pos() + 1)
        xs = x[watch]
        proj = [mats[(0, r)].matmul(xs) for r in ("LIN_QKV", "LIN_Z", "LIN_BETA", "LIN_ALPHA")]
        o = np.concatenate([oracle.linear_core(ocfg, proj[0][i], proj[1][i], proj[2][i], proj[3][i], mats[(0, "LIN_A")], mats[(0, "LIN_DT")],
                                               mats[(0, "LIN_CONV")], mats[(0, "LIN_NORM")], oconv[b], ossm[b]) for i, b in enumerate(watch)])
        worst = max(worst, rel_err(y[watch], mats[(0, "LIN_OUT")].matmul(o)))
        if (step + 1) % 32 == 0:
            gconv, gssm = st.get_lin(0)
            for b in watch:
                assert rel_err(gssm[b], ossm[b]) < TOL, (step, b)
                assert rel_err(gconv[b], oconv[b]) < 1e-6, (step, b)
        assert worst < TOL, step
    assert ctx.device_status() == 0
    st.destroy(); m.destroy()


def test_moe_config3_128_tokens(ctx):
    cfg = pb.make_cfg(n_layers=1, full_every=0, vocab=1024, max_ctx=64)
    spec = synth.model_spec(cfg, 0)
    m = synth.build_model(ctx, cfg, spec, 0)
    _, mats = oracle_model(cfg, spec, 0)
    t = 128
    st = m.new_state(t)
    x = np.random.default_rng(128).standard_normal((t, cfg.d)).astype(np.float32)
    y, sel = st.moe_forward(0, x)
    yo, selo, _ = oracle.moe(oracle_cfg(cfg), mats[(0, "ROUTER")], mats[(0, "EXP_GATE")], mats[(0, "EXP_UP")], mats[(0, "EXP_DOWN")],
                             mats[(0, "SH_GATE")], mats[(0, "SH_UP")], mats[(0, "SH_DOWN")], mats[(0, "SH_GATE_INP")], x)
    assert rel_err(y, yo) < TOL
    assert np.array_equal(np.sort(sel, axis=1), np.sort(selo, axis=1))
    assert ctx.device_status() == 0
    st.destroy(); m.destroy()


@pytest.mark.parametrize("name,t", [("Q8_0", 1), ("Q8_0", 8), ("Q4_K", 8), ("IQ2_XS", 8), ("IQ3_XXS", 1), ("IQ3_XXS", 8), ("IQ2_S", 8), ("IQ4_NL", 8), ("IQ4_XS", 1), ("IQ4_XS", 8),
                                    ("IQ2_XXS", 1), ("IQ2_XXS", 8), ("Q6_K", 8), ("Q2_0", 1), ("Q2_0", 8), ("IQ1_M", 1), ("IQ1_M", 8), ("Q4_0", 8), ("Q5_0", 1), ("Q5_0", 8), ("Q3_K", 1), ("Q3_K", 8), ("Q5_K", 1), ("Q5_K", 8)])
def test_moe_full_width_other_formats(ctx, name, t):
    """The MoE block at full width (2048 x 512 experts of 512) in the other streaming formats; Q8_0 rows of 2048 columns are
    2176 bytes, where a chunk of the gate / up kernel holds fewer rows than it has consumer warps."""
    cfg = pb.make_cfg(n_layers=1, full_every=0, vocab=1024, max_ctx=64)
    spec = synth.model_spec(cfg, 3, qtype=getattr(pb, name))
    m = synth.build_model(ctx, cfg, spec, 3)
    _, mats = oracle_model(cfg, spec, 3)
    st = m.new_state(t)
    x = np.random.default_rng(t).standard_normal((t, cfg.d)).astype(np.float32)
    y, sel = st.moe_forward(0, x)
    yo, selo, _ = oracle.moe(oracle_cfg(cfg), mats[(0, "ROUTER")], mats[(0, "EXP_GATE")], mats[(0, "EXP_UP")], mats[(0, "EXP_DOWN")],
                             mats[(0, "SH_GATE")], mats[(0, "SH_UP")], mats[(0, "SH_DOWN")], mats[(0, "SH_GATE_INP")], x)
    assert rel_err(y, yo) < TOL
    assert np.array_equal(np.sort(sel, axis=1), np.sort(selo, axis=1))
    assert ctx.device_status() == 0
    st.destroy(); m.destroy()


def test_full_model_greedy_identity_64_steps(ctx):
    """The whole 48-layer, 512-expert, 151936-token model: prompt, then 64 greedy tokens, against the oracle's
    recorded run.  A mismatch reports the oracle's margins at that step: a top-2 logit margin or a 10th/11th
    router margin at the level of f32 summation noise (< 1e-4) marks a near-tie, anything larger a bug."""
    sys.path.insert(0, str(GOLDEN))
    import make_full_model_golden as g

    gold = np.load(GOLDEN / "full_model_greedy.npz")
    cfg = pb.make_cfg(**g.CFG)
    spec = synth.model_spec(cfg, g.SEED)
    m = synth.build_model(ctx, cfg, spec, g.SEED)
    st = m.new_state(1)
    for ai in range(cfg.n_layers // cfg.full_every):
        k, v = g.prefill_rows(cfg, ai)
        st.fill_kv(0, ai, k, v)
    st.set_pos(g.PREFILL)
    lg = st.forward(np.array(g.PROMPT, np.uint32))[0]
    assert rel_err(lg[::g.LOGIT_STRIDE], gold["logit_samples"][0]) < TOL
    tok = int(lg.argmax())
    assert tok == int(gold["first"])
    toks = []
    for i in range(g.STEPS):
        lg = st.forward(np.array([tok], np.uint32))[0]
        tok = int(lg.argmax())
        toks.append(tok)
        assert tok == int(gold["tokens"][i]), (
            f"step {i}: token {tok}, oracle {int(gold['tokens'][i])}; oracle top-2 logit margin {gold['logit_margin'][i]:.3g}, "
            f"smallest router margin {gold['router_margin'][i]:.3g}")
        assert rel_err(lg[::g.LOGIT_STRIDE], gold["logit_samples"][i + 1]) < TOL, i
    # the device-resident loop produces the same tokens from a fresh state
    st2 = m.new_state(1)
    for ai in range(cfg.n_layers // cfg.full_every):
        k, v = g.prefill_rows(cfg, ai)
        st2.fill_kv(0, ai, k, v)
    st2.set_pos(g.PREFILL)
    first = int(st2.forward(np.array(g.PROMPT, np.uint32))[0].argmax())
    assert st2.decode_greedy([first], g.STEPS)[0].tolist() == toks
    assert ctx.device_status() == 0
    st.destroy(); st2.destroy(); m.destroy()
