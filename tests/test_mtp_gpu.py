"""The MTP drafter (src/model/mtp.rs, Model::mtp_draft src/model/qwen4exp_gguf.rs:2177-2278): the engine's pb_draft against
the CPU oracle's drafter cell driven by the same bookkeeping, and speculative decoding with it against plain greedy decoding."""
import numpy as np
import pytest

import oracle
import pyre_b200 as pb
from pyre_b200 import synth
from pyre_b200.model import Model
from conftest import rel_err
from helpers import oracle_model, small_cfg

pytestmark = pytest.mark.gpu
WINDOW = 16
N_IDS = 256


def _drafter_spec(cfg_d, seed):
    """A drafter layer: the tensors of one attention layer with hyper-connections and a MoE block, the final mixer and the
    draft-vocabulary head (synthetic rows), plus the input stage; no embeddings of its own."""
    rng = np.random.default_rng(seed + 1000)
    spec = [it for it in synth.model_spec(cfg_d, seed) if it[2] != "TOKEN_EMBD"]
    d, hc = cfg_d.d, cfg_d.hc
    spec.append(("mat", -1, "MTP_FC_E", pb.Q8_0, d, d, synth.tensor_id(-1, "MTP_FC_E")))
    spec.append(("mat", -1, "MTP_FC_H", pb.Q8_0, d, d, synth.tensor_id(-1, "MTP_FC_H")))
    spec.append(("vec", -1, "MTP_PRE_E", (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)))
    spec.append(("vec", -1, "MTP_PRE_H", (1.0 + 0.1 * rng.standard_normal(hc * d)).astype(np.float32)))
    return spec


def _build(ctx, kv_bits=4):
    cfg = small_cfg(pb, n_layers=8, kv_bits=kv_bits, kv_recent=64, max_ctx=256, hc=2, hc_lr=32)
    spec = synth.model_spec(cfg, 51)
    m = synth.build_model(ctx, cfg, spec, 51)
    om, mats = oracle_model(cfg, spec, 51)
    cfg_d = small_cfg(pb, n_layers=1, full_every=1, kv_bits=0, max_ctx=256, hc=2, hc_lr=32, vocab=N_IDS, n_exp=8, top_k=2)
    spec_d = _drafter_spec(cfg_d, 52)
    dm = Model(ctx, cfg_d)
    for item in spec_d:
        if item[0] == "mat":
            _, layer, role, t, rows, cols, tid = item
            dm.set_tensor(layer, role, pb.QMat.synth(ctx, t, rows, cols, 52, tid))
        else:
            dm.set_vec(item[1], item[2], item[3])
    dm.set_mtp(WINDOW)
    dm.finalize()
    odm, dmats = oracle_model(cfg_d, spec_d, 52)
    ids = (np.arange(N_IDS, dtype=np.uint32) * 3 + 5) % cfg.vocab          # the draft vocabulary: some subset of the tokens
    return cfg, m, om, mats, cfg_d, dm, odm, dmats, ids


class OracleDrafter:
    """mtp_draft_in's bookkeeping (:2179-2278) around the oracle's drafter cell."""

    def __init__(self, om, mats, odm, dmats, ids, window):
        self.om, self.odm, self.dmats, self.ids, self.window = om, odm, dmats, ids, window
        self.embd = mats[(-1, "TOKEN_EMBD")].to_f32()
        self.ds = odm.new_state()
        self.tokens, self.R, self.c0, self.end = [], {}, 0, 0

    def fed(self, ost, ids):
        rows = ost.last_residual()
        assert rows.shape[0] == len(ids)
        for j, t in enumerate(ids):
            self.R[len(self.tokens)] = rows[j]
            self.tokens.append(int(t))

    def rollback(self, n):
        self.tokens = self.tokens[:n]
        self.R = {p: r for p, r in self.R.items() if p < n}
        self.end = min(self.end, n); self.c0 = min(self.c0, self.end)

    def draft(self, pending, k, min_p, pick=None):
        n = len(self.tokens)
        if n == 0 or (n - 1) not in self.R:
            return [], []
        self.end = min(self.end, n - 1); self.c0 = min(self.c0, self.end)
        first = n - 1
        while (first - 1) in self.R:
            first -= 1
        cont = self.end > self.c0 and self.end >= first
        lo = self.end if cont else max(first, n - 1 - self.window)
        lo = max(lo, 0)
        if not cont:
            self.c0 = self.end = lo
        for i in range(lo, n - 1):
            self.ds.mtp_cell(self.R[i], self.embd[self.tokens[i + 1]], i, self.c0, self.window, False)
            self.end = i + 1
        r, tok, out, probs = self.R[n - 1], pending, [], []
        for j in range(k):
            s, rr = self.ds.mtp_cell(r, self.embd[tok], n - 1 + j, self.c0, self.window, True)
            if j == 0:
                self.end = n
            lg = self.dmats[(-1, "OUTPUT")].matmul(s)[0]
            bi = int(np.argmax(lg)); p = float(1.0 / np.exp(lg.astype(np.float64) - lg[bi]).sum())
            if j > 0 and p < min_p:
                break
            tid = int(self.ids[bi]) if pick is None else int(pick(lg, self.ids))
            out.append(tid); probs.append(p)
            r, tok = rr, tid
        return out, probs


def test_drafts_match_the_oracle_through_prompts_windows_and_rollbacks(ctx):
    """Prompt, then rounds of: draft three tokens, verify the pending token and the drafts in one window, keep a varying
    prefix.  After every step the engine's drafts (ids and probabilities) equal those of the oracle's drafter, which is fed
    the oracle model's residual rows: through the catch-up of the prompt's cells (more than the window), kept prefixes that
    shorten the drafter's cells, and min_p gating."""
    cfg, m, om, mats, cfg_d, dm, odm, dmats, ids = _build(ctx)
    st, ost = m.new_state(1), om.new_state()
    st.attach_drafter(dm, ids)
    od = OracleDrafter(om, mats, odm, dmats, ids, WINDOW)
    prompt = list(range(700, 730))                      # 30 cells to catch up, window 16
    lg = st.forward(np.array(prompt, np.uint32))[0]
    lo = ost.forward(prompt); od.fed(ost, prompt)
    assert rel_err(lg, lo) < 5e-3
    fed = list(prompt)
    pending = int(np.argmax(lo))
    keeps = [4, 1, 2, 4, 3, 1, 4, 2]
    for rnd, keep in enumerate(keeps):
        min_p = 0.0 if rnd % 2 == 0 else 0.02
        g_ids, g_p = st.draft(pending, 3, min_p)
        o_ids, o_p = od.draft(pending, 3, min_p)
        assert g_ids.tolist() == o_ids, (rnd, g_ids, o_ids, g_p, o_p)
        assert np.allclose(g_p, o_p, rtol=2e-3, atol=1e-6), (rnd, g_p, o_p)
        assert len(o_ids) >= 1
        window = [pending] + o_ids
        keep = min(keep, len(window))
        lgw = st.forward_multi(np.array(window, np.uint32))
        st.spec_keep(len(window), keep)
        fed += window[:keep]
        ost = om.new_state(); ost.forward(fed[:-1]) if len(fed) > 1 else None      # the oracle has no rollback: replay
        lo = ost.forward([fed[-1]])
        # residual rows: the replay holds them for every fed position again
        od.rollback(len(fed) - keep)
        o2 = om.new_state(); o2.forward(fed[:len(fed) - keep]) if len(fed) > keep else None
        for tkn in window[:keep]:
            o2.forward([tkn]); od.fed(o2, [tkn])
        assert rel_err(lgw[keep - 1], lo) < 1e-3, rnd
        pending = int(np.argmax(lo))
    assert ctx.device_status() == 0
    st.destroy(); m.destroy(); dm.destroy()


def test_speculative_decoding_with_the_drafter_equals_plain_greedy(ctx):
    """spec.rs's loop with the model drafter: draft, verify [pending + drafts], accept the longest prefix the verify pass
    agrees with.  Every emitted token comes from the verify pass, so the output equals plain greedy decoding token for token
    (the drafts only decide how many tokens a pass yields); a state without a drafter answers PB_UNSUPPORTED."""
    cfg, m, om, mats, cfg_d, dm, odm, dmats, ids = _build(ctx, kv_bits=0)
    prompt = np.arange(40, 60, dtype=np.uint32)
    plain = m.new_state(1)
    first = int(plain.forward(prompt)[0].argmax())
    want = [first] + plain.decode_greedy([first], 47)[0].tolist()
    st = m.new_state(1)
    with pytest.raises(pb.PyreError):
        st.draft(1, 2)
    st.attach_drafter(dm, ids)
    pending = int(st.forward(prompt)[0].argmax())
    out, passes, accepted = [pending], 0, 0
    while len(out) < 48:
        drafts, _ = st.draft(pending, 3, 0.0)
        window = [pending] + drafts.tolist()
        lg = st.forward_multi(np.array(window, np.uint32))
        nxt = lg.argmax(axis=1)
        keep = 1
        while keep < len(window) and int(nxt[keep - 1]) == window[keep]:
            keep += 1
        st.spec_keep(len(window), keep)
        out += window[1:keep] + [int(nxt[keep - 1])]
        pending = int(nxt[keep - 1]); passes += 1; accepted += keep - 1
    assert out[:48] == want[:48], (passes, accepted)
    assert ctx.device_status() == 0
    plain.destroy(); st.destroy(); m.destroy(); dm.destroy()


def test_drafter_loaded_from_its_tensor_file_matches_the_oracle(ctx, tmp_path):
    """Mtp::load's host side (pyre_b200/mtp_loader.py): a synthetic drafter file in the reference's format (BF16
    safetensors, `mtp.` names, fused gate_up_proj, norms stored without their 1) is read, quantized to Q8_0 and bound
    under the library's roles, the head gathered from the main model's output matrix; the loaded drafter drafts what an
    oracle drafter built from the same bytes drafts."""
    from pyre_b200 import mtp_loader as ml
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=256, hc=2, hc_lr=32)
    spec = synth.model_spec(cfg, 61)
    m = synth.build_model(ctx, cfg, spec, 61)
    om, mats = oracle_model(cfg, spec, 61)
    d, hc, lr, ne, ff, nh, nkv, hd = cfg.d, cfg.hc, 16, 8, 256, cfg.n_head, cfg.n_kv, cfg.hd
    rng = np.random.default_rng(62)
    g = lambda *sh: (0.05 * rng.standard_normal(sh)).astype(np.float32)
    tensors = {"mtp.pre_fc_norm_embedding.weight": g(d), "mtp.pre_fc_norm_hidden.weight": g(hc * d),
               "mtp.fc_embedding.weight": g(d, d), "mtp.fc_hidden.weight": g(d, d),
               "mtp.layers.0.self_attn.q_proj.weight": g(nh * 2 * hd, d), "mtp.layers.0.self_attn.k_proj.weight": g(nkv * hd, d),
               "mtp.layers.0.self_attn.v_proj.weight": g(nkv * hd, d), "mtp.layers.0.self_attn.o_proj.weight": g(d, nh * hd),
               "mtp.layers.0.self_attn.q_norm.weight": g(hd), "mtp.layers.0.self_attn.k_norm.weight": g(hd),
               "mtp.layers.0.mlp.gate.weight": g(ne, d), "mtp.layers.0.mlp.experts.gate_up_proj": g(ne, 2 * ff, d), "mtp.layers.0.mlp.experts.down_proj": g(ne, d, ff),
               "mtp.layers.0.mlp.shared_expert.gate_proj.weight": g(ff, d), "mtp.layers.0.mlp.shared_expert.up_proj.weight": g(ff, d),
               "mtp.layers.0.mlp.shared_expert.down_proj.weight": g(d, ff), "mtp.layers.0.mlp.shared_expert_gate.weight": g(1, d)}
    for pre, inj in (("mtp.layers.0.attn_hyper_connection", True), ("mtp.layers.0.mlp_hyper_connection", True), ("mtp.hyper_connection_mixer", False)):
        tensors[f"{pre}.hc_norm.weight"] = g(hc * d); tensors[f"{pre}.input_mix_weight_down.weight"] = g(lr, hc * d); tensors[f"{pre}.input_mix_weight_up.weight"] = g(hc * d, lr)
        if inj:
            tensors[f"{pre}.block_inject_weight.weight"] = g(hc, hc * d)
    path = tmp_path / "mtp.safetensors"
    ml.write_safetensors(path, tensors)
    ids = (np.arange(N_IDS, dtype=np.uint32) * 3 + 5) % cfg.vocab
    head = pb.QMat.synth(ctx, pb.IQ3_S, cfg.vocab, d, 61, synth.tensor_id(-1, "OUTPUT"))        # the main model's output matrix again
    dm = ml.load_drafter(ctx, path, cfg, head, ids, window=WINDOW)
    assert dm.cfg.n_exp == ne and dm.cfg.ff_exp == ff and dm.cfg.hc_lr == lr and dm.cfg.vocab == N_IDS
    # the oracle's drafter from the same bytes
    cfgkw, items = ml.drafter_spec(ml.read_safetensors(path), cfg)
    from helpers import oracle_cfg
    ocfg = oracle_cfg(pb.make_cfg(vocab=N_IDS, **cfgkw))
    odm = oracle.Model(ocfg); dmats = {}
    for it in items:
        if it[0] == "mat":
            _, layer, role, ty, rows, cols, raw = it
            q = oracle.QMat(ty, rows, cols, raw); odm.set_mat(layer, role, q); dmats[(layer, role)] = q
        else:
            odm.set_vec(it[1], it[2], it[3])
    hq = oracle.QMat(oracle.IQ3_S, N_IDS, d, np.concatenate([head.raw_rows(int(i), 1) for i in ids]))
    odm.set_mat(-1, "OUTPUT", hq); dmats[(-1, "OUTPUT")] = hq
    st, ost = m.new_state(1), om.new_state()
    st.attach_drafter(dm, ids)
    od = OracleDrafter(om, mats, odm, dmats, ids, WINDOW)
    prompt = list(range(100, 112))
    st.forward(np.array(prompt, np.uint32)); lo = ost.forward(prompt); od.fed(ost, prompt)
    pending = int(np.argmax(lo))
    for rnd in range(4):
        g_ids, g_p = st.draft(pending, 3, 0.0)
        o_ids, o_p = od.draft(pending, 3, 0.0)
        assert g_ids.tolist() == o_ids and np.allclose(g_p, o_p, rtol=2e-3, atol=1e-6), (rnd, g_ids, o_ids, g_p, o_p)
        st.forward(np.array([pending], np.uint32)); lo = ost.forward([pending]); od.fed(ost, [pending])
        pending = int(np.argmax(lo))
    assert ctx.device_status() == 0
    head.free(); st.destroy(); m.destroy(); dm.destroy()


def _qsample(temperature, rng):
    """mtp_qsample (qwen4exp_gguf.rs:3321-3331): softmax at the temperature over the 64 largest logits, one uniform draw."""
    def pick(lg, ids):
        n = min(len(lg), len(ids)); kk = min(64, n)
        ix = np.argsort(-lg[:n], kind="stable")[:kk]
        w = np.exp((lg[ix] - lg[ix].max()) / max(temperature, 1e-3)); q = w / w.sum()
        u, choice = rng.random(), int(ids[ix[0]])
        for i, pr in zip(ix, q):
            choice = int(ids[i])
            if u < pr:
                break
            u -= pr
        return choice
    return pick


def test_sampled_drafts_follow_the_callers_sampler(ctx):
    """pb_draft_sampled hands the drafter's logits to the caller's sampler after the gate; with the same sampler and the same random
    draws the engine and the oracle's drafter produce the same drafts, and they differ from the greedy drafts."""
    cfg, m, om, mats, cfg_d, dm, odm, dmats, ids = _build(ctx)
    st, ost = m.new_state(1), om.new_state()
    st.attach_drafter(dm, ids)
    od = OracleDrafter(om, mats, odm, dmats, ids, WINDOW)
    prompt = list(range(300, 312))
    st.forward(np.array(prompt, np.uint32))
    lo = ost.forward(prompt); od.fed(ost, prompt)
    pending = int(np.argmax(lo))
    greedy, _ = st.draft(pending, 4, 0.0)
    seen = []

    def spy(lg, vid):
        seen.append((lg.copy(), vid.copy()))
        return _qsample(1.5, np.random.default_rng(100 + len(seen)))(lg, vid)

    g_ids, g_p = st.draft_sampled(pending, 4, 0.0, spy)
    calls = [0]

    def opick(lg, vid):
        calls[0] += 1
        return _qsample(1.5, np.random.default_rng(100 + calls[0]))(seen[calls[0] - 1][0], vid)   # the engine's logits: same draw, same token

    o_ids, o_p = od.draft(pending, 4, 0.0, opick)
    assert g_ids.tolist() == o_ids and len(o_ids) == 4
    assert np.allclose(g_p, o_p, rtol=2e-3, atol=1e-6)
    assert np.array_equal(seen[0][1], ids) and seen[0][0].shape == (N_IDS,)
    # the oracle's own logits of the first step agree with the ones the sampler was handed
    s0, _ = od.ds.mtp_cell(od.R[len(prompt) - 1], od.embd[pending], len(prompt) - 1, od.c0, WINDOW, True)
    assert rel_err(seen[0][0], dmats[(-1, "OUTPUT")].matmul(s0)[0]) < 2e-3
    assert g_ids.tolist() != greedy.tolist()
    with pytest.raises(pb.PyreError):
        st.draft_sampled(pending, 2, 0.0, lambda lg, vid: cfg.vocab + 5)      # a sampler that answers outside the vocabulary
    assert ctx.device_status() == 0
