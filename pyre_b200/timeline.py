"""Phase timeline of one decode step from the kernels' own clock stamps.

    python -m pyre_b200.timeline [--layers 8] [--ctx 32768] [--out file.md]

Builds the benchmark model (config-4 shapes, `--layers` of its 48 layers), pre-fills the 4-bit KV cache,
turns stamp tracing on (pb_ctx_stamps_enable), decodes a few steps and prints, per kind of launch, the
median time between the stamps of its first CTA:

    launch gap   previous launch's last store -> this launch's entry
    set-up       entry -> barriers / tables initialised
    dep wait     -> predecessor's data visible (griddepcontrol.wait returned)
    prologue     -> activations normalised and split
    first bytes  -> first weight stage landed in shared memory
    stream       -> last store of the first CTA
    tail         -> last store of the last CTA

For the fused step kernel (one launch per step) the stamps are one per phase and the table lists the
phases instead.  Stamps come from %globaltimer (nanoseconds, one clock for the whole GPU).
"""
from __future__ import annotations

import argparse
import sys
from collections import defaultdict

import numpy as np

KNAMES = {1: "gemv", 2: "router", 3: "expert gate/up", 4: "expert down", 5: "deltanet", 6: "attention",
          101: "fused: gemv", 102: "fused: deltanet", 103: "fused: router", 104: "fused: expert gate/up", 105: "fused: expert down"}


def launches_table(st: np.ndarray, ids: np.ndarray, label_of=None) -> str:
    """st [n][8] stamps of consecutive launches of one step (stream order), ids [n]."""
    rows = defaultdict(list)
    prev_end = None
    for i in range(len(ids)):
        w = st[i].astype(np.int64)
        if w[0] == 0:
            prev_end = None
            continue
        end_first = w[5] if w[5] else w[0]
        end_last = max(w[7], end_first)
        name = KNAMES.get(int(ids[i]), str(ids[i])) if label_of is None else label_of(i)

        def d(a, b):
            return float(b - a) / 1e3 if a and b and b >= a else 0.0
        t1 = w[1] if w[1] else w[0]
        t2 = w[2] if w[2] else t1
        t3 = w[3] if w[3] else t2
        t4 = w[4] if w[4] else t3
        rows[name].append((d(prev_end, w[0]) if prev_end else 0.0, d(w[0], t1), d(t1, t2), d(t2, t3), d(t3, t4), d(max(t3, t4), end_first), d(end_first, end_last),
                           d(w[0], end_last)))
        prev_end = end_last
    out = ["| launch | n | launch gap | set-up | dep wait | prologue | first bytes | stream | tail | entry -> end |", "|---|---|---|---|---|---|---|---|---|---|"]
    for name, v in rows.items():
        a = np.median(np.array(v), axis=0)
        out.append(f"| {name} | {len(v)} | " + " | ".join(f"{x:.2f}" for x in a) + " |")
    return "\n".join(out)


def main():
    import pyre_b200 as pb
    from pyre_b200 import synth

    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    ctx = pb.Ctx(0)
    cfg = pb.make_cfg(n_layers=a.layers, max_ctx=a.ctx + 256, kv_bits=4, kv_recent=1024)
    spec = synth.model_spec(cfg, 0)
    m = synth.build_model(ctx, cfg, spec, 0)
    st = m.new_state(1)
    for ai in range(cfg.n_layers // cfg.full_every):
        st.fill_kv_synth(ai, a.ctx, 1)
    st.set_pos(a.ctx)
    ctx.stamps_enable(8192)
    st.decode_greedy([1], 6)                 # eager step, captured step, replays (the replays overwrite the captured step's slots)
    stamps, ids = ctx.stamps_read()
    per_step = int(st.stats().kernels_launched)
    text = [f"decode step, {a.layers} layers, context {a.ctx}, {per_step} launches per step, {len(ids)} traced launches (all times in microseconds, medians)"]
    fused = bool(len(ids)) and int(ids.max()) > 100
    if fused:   # the operations of the fused step kernel keep the slots they were given when the list was built
        text.append("operations of the fused step kernel (launch gap = end of the previous operation in CTA 0 -> start of this one; dep wait = grid barrier)")
        n = 0
    else:
        n = len(ids) // 2
    text.append(launches_table(stamps[n:], ids[n:]))
    step = stamps[n:]
    nz = step[step > 0]
    if nz.size:
        text.append(f"\nfirst stamp -> last stamp of the step: {(int(nz.max()) - int(nz.min())) / 1e3:.1f} us")
    s = "\n".join(text)
    print(s)
    if a.out:
        open(a.out, "w").write(s + "\n")
    st.destroy(); m.destroy(); ctx.close()


if __name__ == "__main__":
    sys.exit(main())
