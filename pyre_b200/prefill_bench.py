"""Prompt prefill timing: a prompt of N tokens through pb_forward on the benchmark model shapes.

    python -m pyre_b200.prefill_bench [--layers 48] [--tokens 4096] [--reps 2]

Builds the synthetic model (`--layers` of the 48 layers of the benchmark shapes, 4-bit KV cache), feeds a seeded
random prompt from an empty context and prints wall-clock milliseconds and tokens per second per repetition.  The
prompt runs in 256-token chunks on the absolute grid; the first repetition includes the eager chunk and the capture of
the chunk graph.  With a small `--layers` and `--tokens 256` this is the command to put under a profiler for the launch
list of one chunk.
"""
from __future__ import annotations

import argparse
import time

import numpy as np


def main():
    import torch
    import pyre_b200 as pb
    from pyre_b200 import synth

    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--reps", type=int, default=2)
    a = ap.parse_args()
    ctx = pb.Ctx(0)
    cfg = pb.make_cfg(n_layers=a.layers, max_ctx=max(2048, a.tokens + 256), kv_bits=4, kv_recent=1024)
    m = synth.build_model(ctx, cfg, synth.model_spec(cfg, 0), 0)
    st = m.new_state(1)
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, size=a.tokens).astype(np.uint32)
    for rep in range(a.reps):
        st.reset()
        torch.cuda.synchronize()
        t0 = time.time()
        st.forward(prompt)
        torch.cuda.synchronize()
        dt = time.time() - t0
        print(f"prefill {a.tokens} tokens, {a.layers} layers: {dt * 1e3:.1f} ms, {a.tokens / dt:.0f} tok/s", flush=True)
    st.destroy(); m.destroy(); ctx.close()


if __name__ == "__main__":
    main()
