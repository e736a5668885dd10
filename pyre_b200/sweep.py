"""Timing sweep of the dequant-GEMV / GEMM kernels on device-resident operands.

    python -m pyre_b200.sweep                      # the mixed-quant sweep: four formats x four shapes x batch 1, 4, 16
    python -m pyre_b200.sweep --gemm               # IQ3_S at 16, 64, 256 tokens (tensor-core GEMM)
    python -m pyre_b200.sweep --type IQ3_S --rows 12288 --cols 2048 --tokens 256 --reps 3   # one case (e.g. under a profiler)

Shapes (out x in) are those of the model's matrices: 2048 x 512 (expert down), 1024 x 2048 (expert gate + up),
4096 x 2048 (attention q / gate projection), 151936 x 2048 (lm-head).  Weights are synthetic (seeded block fields),
activations N(0, 1).  Each case is timed with CUDA events on the launching stream after three warm-up launches;
between the timed launches of the small shapes a 256 MB buffer is rewritten so that the weights come from HBM, not L2.
Reported: microseconds per launch, weight bytes / time (GB/s, against the measured copy bandwidth if the file
MEASURED_PEAKS.json is present next to the package), and for GEMM cases 2 * rows * cols * tokens / time (TFLOP/s).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

SHAPES = [(2048, 512), (1024, 2048), (4096, 2048), (151936, 2048)]


def time_case(pb, torch, ctx, stream, tname, rows, cols, tokens, reps, flush):
    t = getattr(pb, tname)
    W = pb.QMat.synth(ctx, t, rows, cols, 0, 77)
    xd = torch.randn(tokens, cols, device="cuda")
    yd = torch.empty(tokens, rows, device="cuda")
    big = W.nbytes() > 200e6
    with torch.cuda.stream(stream):
        for _ in range(3):
            W.matmul_dev(xd.data_ptr(), tokens, yd.data_ptr())
        tot = 0.0
        for _ in range(reps):
            if not big and flush is not None:
                flush.add_(1.0)                      # evicts the weights from L2
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            W.matmul_dev(xd.data_ptr(), tokens, yd.data_ptr())
            e1.record(stream)
            e1.synchronize()
            tot += e0.elapsed_time(e1)
    us = tot * 1e3 / reps
    nbytes = W.nbytes()
    W.free()
    return us, nbytes


def main():
    import torch
    import pyre_b200 as pb

    ap = argparse.ArgumentParser()
    ap.add_argument("--gemm", action="store_true")
    ap.add_argument("--type", default=None)
    ap.add_argument("--rows", type=int, default=0)
    ap.add_argument("--cols", type=int, default=0)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args()
    ctx = pb.Ctx(0)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    peak = None
    pk = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    if pk.exists():
        peak = float(json.load(open(pk)).get("hbm_gbs", 0)) or None
    flush = torch.zeros(64 << 20, device="cuda")     # 256 MB > the 126 MB L2
    if a.type:
        cases = [(a.type, a.rows, a.cols, a.tokens)]
    elif a.gemm:
        cases = [("IQ3_S", r, c, t) for (r, c) in SHAPES + [(12288, 2048), (2048, 4096)] for t in (16, 64, 256) if r * t <= 151936 * 64]
    else:
        cases = [(n, r, c, t) for n in ("Q8_0", "Q4_K", "IQ2_XS", "IQ3_S") for (r, c) in SHAPES for t in (1, 4, 16)]
    out = []
    for (n, r, c, t) in cases:
        us, nb = time_case(pb, torch, ctx, stream, n, r, c, t, a.reps, flush)
        rec = {"type": n, "rows": r, "cols": c, "tokens": t, "us": round(us, 2), "weight_gbs": round(nb / us / 1e3, 1)}
        if peak:
            rec["frac_of_measured_hbm"] = round(nb / us / 1e3 / peak, 3)
        if t >= 16:
            rec["tflops"] = round(2.0 * r * c * t / us / 1e6, 1)
        out.append(rec)
        if not a.json:
            print(" ".join(f"{k}={v}" for k, v in rec.items()), flush=True)
    if a.json:
        print(json.dumps(out))
    ctx.close()


if __name__ == "__main__":
    main()
