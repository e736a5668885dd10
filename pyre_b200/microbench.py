"""Dequant-GEMV micro-benchmark (config 1 of the benchmark: mixed-quant GEMV sweep).

    python -m pyre_b200.microbench                      # the full sweep, one line per case
    python -m pyre_b200.microbench --type IQ3_S --rows 151936 --cols 2048 --t 1 --iters 3

For each (format, shape, batch) it times `pb_gemv_dev` with CUDA events on the launching
stream and reports achieved GB/s over the algorithmic bytes
(rows * row_bytes + 4 * t * (cols + rows)).  Between timed launches a buffer larger than the
L2 is rewritten unless the matrix itself exceeds the L2 (the lm-head shape).
"""
from __future__ import annotations

import argparse
import json

import numpy as np

import pyre_b200 as pb

SHAPES = [(2048, 512), (1024, 2048), (4096, 2048), (151936, 2048)]
TYPES = ["Q8_0", "Q4_K", "IQ2_XS", "IQ3_S"]
L2_BYTES = 126 << 20


def time_case(ctx, torch, stream, tname, rows, cols, t, iters, flush):
    W = pb.QMat.synth(ctx, pb.TYPE_NAMES[tname], rows, cols, 0, 4242)
    x = torch.randn(t, cols, device="cuda")
    y = torch.empty(t, rows, device="cuda")
    big = W.nbytes() > L2_BYTES
    times = []
    with torch.cuda.stream(stream):
        for _ in range(3):
            W.matmul_dev(x.data_ptr(), t, y.data_ptr())
        for _ in range(iters):
            if not big:
                flush.add_(1.0)          # rewrite > L2 bytes so the weights come from HBM
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            W.matmul_dev(x.data_ptr(), t, y.data_ptr())
            e1.record(stream)
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
    W.free()
    us = float(np.median(times))
    alg = rows * (cols // pb.type_geom(pb.TYPE_NAMES[tname])[0]) * pb.type_geom(pb.TYPE_NAMES[tname])[1] + 4 * t * (cols + rows)
    return {"type": tname, "rows": rows, "cols": cols, "t": t, "us": round(us, 2), "gbs": round(alg / us / 1e3, 1), "bytes": alg}


def main():
    import torch

    ap = argparse.ArgumentParser()
    ap.add_argument("--type", default=None)
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--cols", type=int, default=None)
    ap.add_argument("--t", type=int, default=None)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    ctx = pb.Ctx(0)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    flush = torch.zeros((L2_BYTES * 2) // 4, device="cuda")
    types = [a.type] if a.type else TYPES
    shapes = [(a.rows, a.cols)] if a.rows else SHAPES
    ts = [a.t] if a.t else [1, 4, 16]
    for tname in types:
        for rows, cols in shapes:
            for t in ts:
                print(json.dumps(time_case(ctx, torch, stream, tname, rows, cols, t, a.iters, flush)), flush=True)
    ctx.own_stream()
    ctx.close()


if __name__ == "__main__":
    main()
