#!/usr/bin/env python3
"""Writes tests/golden/full_model_greedy.npz: 64 greedy decode steps of the CPU oracle on the FULL
benchmark model (48 layers, hidden 2048, 512 experts top-10, vocabulary 151936, IQ3_S weights from
the seeded block generator), with a 4-bit KV cache pre-filled with 150 positions per attention layer.

The oracle needs about four seconds per step on eight cores, so the GPU test compares the engine with
this fixture instead of running the oracle again.  Recorded per step: the chosen token, the top-2
logit margin and the smallest 10th/11th router-logit margin over the layers (a later mismatch can
then be classed as a near-tie or a bug), and a strided sample of the logits for a tolerance check.

    python tests/golden/make_full_model_golden.py            (from the repository root, ~6 minutes)

Inputs are regenerated from the constants below by the test, so only outputs are stored.
"""
from __future__ import annotations

import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

SEED = 0
PREFILL = 150          # positions per attention layer before the prompt
PROMPT = [3, 999, 27]
STEPS = 64
LOGIT_STRIDE = 97      # every 97th logit of each step is stored
CFG = dict(n_layers=48, max_ctx=256, kv_bits=4, kv_recent=64)   # everything else: the benchmark's config 4


def prefill_rows(cfg, ai):
    """K and V rows [PREFILL][n_kv * hd] of attention layer ai (already normed and roped, N(0,1))."""
    rng = np.random.default_rng(1000 + ai)
    row = cfg.n_kv * cfg.hd
    return rng.standard_normal((PREFILL, row)).astype(np.float32), rng.standard_normal((PREFILL, row)).astype(np.float32)


def main():
    import oracle
    import pyre_b200 as pb
    from pyre_b200 import synth
    from helpers import oracle_model

    cfg = pb.make_cfg(**CFG)
    spec = synth.model_spec(cfg, SEED)
    om, _ = oracle_model(cfg, spec, SEED)
    ost = om.new_state()
    for ai in range(cfg.n_layers // cfg.full_every):
        k, v = prefill_rows(cfg, ai)
        ost.fill_kv(ai, k, v)
    ost.set_pos(PREFILL)
    t0 = time.time()
    lg = ost.forward(PROMPT)
    toks, lmargin, rmargin, samples = [], [], [], [lg[::LOGIT_STRIDE].copy()]
    tok = oracle.argmax(lg)
    first = tok
    for i in range(STEPS):
        lg = ost.forward([tok])
        tok = oracle.argmax(lg)
        a, b = ost.margins()
        toks.append(tok); lmargin.append(a); rmargin.append(b); samples.append(lg[::LOGIT_STRIDE].copy())
        print(f"step {i}: token {tok} logit margin {a:.4g} router margin {b:.4g} ({time.time() - t0:.0f} s)", flush=True)
    out = Path(__file__).resolve().parent / "full_model_greedy.npz"
    np.savez_compressed(out, first=np.uint32(first), tokens=np.array(toks, np.uint32), logit_margin=np.array(lmargin, np.float32),
                        router_margin=np.array(rmargin, np.float32), logit_samples=np.stack(samples).astype(np.float32))
    print("wrote", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
