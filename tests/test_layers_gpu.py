"""GPU parity of the decode-path blocks (MoE, Gated DeltaNet, gated attention with f32 and
4-bit KV) against the CPU oracle, through the layer-level C-ABI entry points."""
import numpy as np
import pytest

import oracle
import pyre_b200 as pb
from pyre_b200 import synth
from conftest import rel_err
from helpers import oracle_cfg, oracle_model, small_cfg

pytestmark = pytest.mark.gpu
TOL = 1e-3   # relative to the largest reference magnitude, f32 accumulate (north-star tolerance)


@pytest.fixture(scope="module")
def small(ctx):
    cfg = small_cfg(pb)
    spec = synth.model_spec(cfg, 0)
    m = synth.build_model(ctx, cfg, spec, 0)
    om, mats = oracle_model(cfg, spec, 0)
    yield cfg, m, om, mats
    m.destroy()


def _moe_ref(cfg, mats, layer, x):
    return oracle.moe(oracle_cfg(cfg), mats[(layer, "ROUTER")], mats[(layer, "EXP_GATE")], mats[(layer, "EXP_UP")], mats[(layer, "EXP_DOWN")],
                      mats[(layer, "SH_GATE")], mats[(layer, "SH_UP")], mats[(layer, "SH_DOWN")], mats[(layer, "SH_GATE_INP")], x)


@pytest.mark.parametrize("t", [1, 3, 32])
def test_moe_block(ctx, small, t):
    cfg, m, _, mats = small
    st = m.new_state(t)
    x = np.random.default_rng(t).standard_normal((t, cfg.d)).astype(np.float32)
    y, sel = st.moe_forward(1, x)
    yo, selo, _ = _moe_ref(cfg, mats, 1, x)
    assert rel_err(y, yo) < TOL
    assert np.array_equal(np.sort(sel, axis=1), np.sort(selo, axis=1))      # same experts
    assert np.all(np.diff(sel, axis=1) > 0)                                  # accumulated in ascending expert id
    assert ctx.device_status() == 0
    st.destroy()


def test_moe_block_full_width(ctx):
    """Config 3 shapes: hidden 2048, 512 experts top-10, ff 512, one layer, batch 1 and 32."""
    cfg = pb.make_cfg(n_layers=1, full_every=0, vocab=1024, max_ctx=64)
    spec = [s for s in synth.model_spec(cfg, 0)]
    m = synth.build_model(ctx, cfg, spec, 0)
    _, mats = oracle_model(cfg, spec, 0)
    for t in (1, 32):
        st = m.new_state(t)
        x = np.random.default_rng(100 + t).standard_normal((t, cfg.d)).astype(np.float32)
        y, sel = st.moe_forward(0, x)
        yo, selo, _ = _moe_ref(cfg, mats, 0, x)
        assert rel_err(y, yo) < TOL
        assert np.array_equal(np.sort(sel, axis=1), np.sort(selo, axis=1))
        st.destroy()
    m.destroy()


def test_moe_router_edge_cases(ctx, small):
    """Zero input: all router logits tie, the selection is the lowest expert ids with uniform weights."""
    cfg, m, _, mats = small
    st = m.new_state(2)
    x = np.zeros((2, cfg.d), np.float32)
    y, sel = st.moe_forward(0, x)
    assert np.array_equal(sel, np.tile(np.arange(cfg.top_k, dtype=np.int32), (2, 1)))
    assert np.all(y == 0)
    st.destroy()


def _lin_ref_step(cfg, mats, layer, x, conv, ssm):
    ocfg = oracle_cfg(cfg)
    y = np.zeros_like(x)
    for b in range(x.shape[0]):
        proj = [mats[(layer, r)].matmul(x[b]) for r in ("LIN_QKV", "LIN_Z", "LIN_BETA", "LIN_ALPHA")]
        cs, ss = np.ascontiguousarray(conv[b]), np.ascontiguousarray(ssm[b])
        o = oracle.linear_core(ocfg, *proj, mats[(layer, "LIN_A")], mats[(layer, "LIN_DT")], mats[(layer, "LIN_CONV")], mats[(layer, "LIN_NORM")], cs, ss)
        conv[b], ssm[b] = cs, ss
        y[b] = mats[(layer, "LIN_OUT")].matmul(o)[0]
    return y


@pytest.mark.parametrize("batch", [1, 3])
def test_deltanet_steps(ctx, small, batch):
    """Sequential steps from a random N(0, 0.1) state; outputs and final state within tolerance."""
    cfg, m, _, mats = small
    rng = np.random.default_rng(7 + batch)
    ch = 2 * cfg.lin_nk * cfg.lin_dk + cfg.lin_nv * cfg.lin_dv
    conv = (0.1 * rng.standard_normal((batch, cfg.conv_k - 1, ch))).astype(np.float32)
    ssm = (0.1 * rng.standard_normal((batch, cfg.lin_nv, cfg.lin_dk, cfg.lin_dv))).astype(np.float32)
    st = m.new_state(batch)
    st.set_lin(0, conv, ssm)
    c0, s0 = st.get_lin(0)
    assert np.array_equal(c0, conv) and np.array_equal(s0, ssm)            # set/get round trip
    for step in range(24):
        x = rng.standard_normal((batch, cfg.d)).astype(np.float32)
        y = st.deltanet_step(0, x)
        st.set_pos(st.pos() + 1)
        assert rel_err(y, _lin_ref_step(cfg, mats, 0, x, conv, ssm)) < TOL, step
    c1, s1 = st.get_lin(0)
    assert rel_err(s1, ssm) < TOL and rel_err(c1, conv) < 1e-6
    assert ctx.device_status() == 0
    st.destroy()


def test_deltanet_full_width(ctx):
    """Config 2 shapes: 16 QK heads, 32 V heads of 128, conv k=4, hidden 2048, batch 8, a run of steps."""
    cfg = pb.make_cfg(n_layers=1, full_every=0, vocab=1024, max_ctx=512, n_exp=16, top_k=2)
    spec = synth.model_spec(cfg, 0)
    m = synth.build_model(ctx, cfg, spec, 0)
    _, mats = oracle_model(cfg, spec, 0)
    rng = np.random.default_rng(3)
    B = 8
    ch = 2 * cfg.lin_nk * cfg.lin_dk + cfg.lin_nv * cfg.lin_dv
    conv = np.zeros((B, cfg.conv_k - 1, ch), np.float32)
    ssm = (0.1 * rng.standard_normal((B, cfg.lin_nv, cfg.lin_dk, cfg.lin_dv))).astype(np.float32)
    st = m.new_state(B)
    st.set_lin(0, conv, ssm)
    for step in range(6):
        x = rng.standard_normal((B, cfg.d)).astype(np.float32)
        y = st.deltanet_step(0, x)
        st.set_pos(st.pos() + 1)
        assert rel_err(y, _lin_ref_step(cfg, mats, 0, x, conv, ssm)) < TOL
    assert rel_err(st.get_lin(0)[1], ssm) < TOL
    st.destroy(); m.destroy()


def _attn_run(ctx, cfg, m, mats, n0, steps, seed):
    ocfg = oracle_cfg(cfg)
    rng = np.random.default_rng(seed)
    layer = cfg.full_every - 1
    row = cfg.n_kv * cfg.hd
    st = m.new_state(1)
    kc = np.zeros((cfg.max_ctx, row), np.float32); vc = np.zeros((cfg.max_ctx, row), np.float32)
    if n0:
        kc[:n0] = rng.standard_normal((n0, row)); vc[:n0] = rng.standard_normal((n0, row))
        st.fill_kv(0, 0, kc[:n0], vc[:n0]); st.set_pos(n0)
    inv = oracle.rope_inv(cfg.n_rot, cfg.rope_base)
    q4n, packed, worst = 0, None, 0.0
    for step in range(steps):
        pos = n0 + step
        x = rng.standard_normal((1, cfg.d)).astype(np.float32)
        y = st.attn_step(layer, x)
        st.set_pos(pos + 1)
        qf, kf, vf = (mats[(layer, r)].matmul(x)[0] for r in ("ATTN_Q", "ATTN_K", "ATTN_V"))
        if cfg.kv_bits == 4:
            want = ((pos + 1 - cfg.kv_recent) // 64) * 64 if pos + 1 > cfg.kv_recent else 0   # kv_push :1520
            if want > q4n:
                q4n = want
                packed = (*oracle.kv4_pack(kc[:q4n]), *oracle.kv4_pack(vc[:q4n]))
        att = oracle.attn_core(ocfg, qf, kf, vf, mats[(layer, "ATTN_Q_NORM")], mats[(layer, "ATTN_K_NORM")], inv, kc, vc, pos, packed if q4n else None, q4n)
        worst = max(worst, rel_err(y, mats[(layer, "ATTN_O")].matmul(att)))
    st.destroy()
    return worst, q4n


def test_attention_f32_kv_from_empty(ctx, small):
    cfg, m, _, mats = small
    worst, _ = _attn_run(ctx, cfg, m, mats, 0, 40, 1)      # first token attends to itself only
    assert worst < TOL


def test_attention_f32_kv_prefilled(ctx, small):
    cfg, m, _, mats = small
    worst, _ = _attn_run(ctx, cfg, m, mats, 333, 10, 2)    # ragged: not a multiple of the 32-position tile
    assert worst < TOL


def test_attention_kv4(ctx):
    """4-bit KV: packed region + f32 recent window, crossing two 64-position repack boundaries."""
    cfg = small_cfg(pb, kv_bits=4, kv_recent=64, max_ctx=512)
    spec = synth.model_spec(cfg, 0)
    m = synth.build_model(ctx, cfg, spec, 0)
    _, mats = oracle_model(cfg, spec, 0)
    worst, q4n = _attn_run(ctx, cfg, m, mats, 300, 100, 3)
    assert worst < TOL
    assert q4n == ((300 + 100 - 64) // 64) * 64
    worst, q4n = _attn_run(ctx, cfg, m, mats, 0, 140, 4)   # starts empty, begins packing at 128 positions
    assert worst < TOL and q4n == 64
    assert ctx.device_status() == 0
    m.destroy()


def test_kv4_pack_matches_reference_rule(ctx):
    """kv4::pack / unpack on the device equal the oracle bit for bit, including the reference's own vector."""
    from pathlib import Path
    g = np.load(Path(__file__).resolve().parent / "golden" / "kv4_vector.npz")
    w, s = ctx.kv4_pack(g["x"])
    assert np.array_equal(w, g["words"]) and np.array_equal(s, g["scales"])
    assert np.array_equal(ctx.kv4_unpack(w, s, 256), g["unpacked"])
    x = np.random.default_rng(0).standard_normal(64 * 512).astype(np.float32)
    x[:32] = 0; x[40] = np.inf                       # zero block, non-finite block (scale 0, kv4.rs:18)
    w, s = ctx.kv4_pack(x)
    wo, so = oracle.kv4_pack(x)
    assert np.array_equal(w, wo) and np.array_equal(s, so)
    with pytest.raises(pb.PyreError):
        ctx.kv4_pack(np.zeros(33, np.float32))       # kv4.rs:13 asserts a multiple of 32
