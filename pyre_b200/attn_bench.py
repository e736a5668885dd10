"""Decode steps of a short stack of benchmark-shaped layers at a long context, with or without the QSA indexer.

    python -m pyre_b200.attn_bench --batch 32 --indexer          # 3 DeltaNet + 1 attention layer, 32768 positions of 4-bit KV
    python -m pyre_b200.attn_bench --batch 1

Prints one JSON line with the time per step; used with `ncu --metrics gpu__time_duration.sum` for per-kernel times of the
attention path (KV append, indexer, split attention, combine).
"""
import argparse
import json
import time

import numpy as np

import pyre_b200 as pb
from pyre_b200 import synth


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--indexer", action="store_true", help="QSA: budget 2048 tokens, blocks of 4, 8 index heads of 128")
    a = ap.parse_args()
    ctx = pb.Ctx(0)
    cfg = pb.make_cfg(n_layers=a.layers, max_ctx=a.ctx + 256, kv_bits=4, kv_recent=1024)
    idx = (2048, 4, 8, 128) if a.indexer else None
    spec = synth.model_spec(cfg, 0, indexer=idx)
    m = synth.build_model(ctx, cfg, spec, 0, indexer=idx)
    st = m.new_state(a.batch)
    for ai in range(cfg.n_layers // cfg.full_every):
        st.fill_kv_synth(ai, a.ctx, 1)
    st.set_pos(a.ctx)
    st.decode_greedy(np.arange(a.batch, dtype=np.uint32) + 1, 3)
    ctx.sync()
    t = time.time()
    st.decode_greedy(np.arange(a.batch, dtype=np.uint32) + 7, a.steps)
    ctx.sync()
    print(json.dumps({"batch": a.batch, "layers": a.layers, "context": a.ctx, "indexer": bool(a.indexer), "ms_per_step": round((time.time() - t) / a.steps * 1e3, 4)}))
    st.destroy(); m.destroy()


if __name__ == "__main__":
    main()
