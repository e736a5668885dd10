#!/usr/bin/env python3
"""Regenerate the golden fixtures in this directory.

dequant_<TYPE>.npz : `raw` = four rows of 512 columns of seeded block bytes, `f32` = their
dequantization by gguf-py 0.19 (`gguf.quants.dequantize`), the tool the reference's
authors checked their decoder against (docs/development-log.md:434-436 of the reference).
The bytes come from the oracle's synthetic generator plus fully random bytes with a sane
f16 scale (the construction of src/model/qdot.rs:1033-1047).
kv4_vector.npz     : the input vector of src/model/kv4.rs:55-58 and its packed words/scales from the
oracle, with the properties that test asserts checked at generation time.
Run from the repository root:  python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402
from gguf import quants, GGMLQuantizationType as T  # noqa: E402

HERE = Path(__file__).resolve().parent
# Q2_0 (ggml id 42 of the reference, src/model/gguf_q.rs:80-81) is not a gguf-py type: its fixture is the two-line rule of that file written in numpy
GG = {"IQ2_XXS": T.IQ2_XXS, "Q6_K": T.Q6_K, "IQ1_M": T.IQ1_M, "Q4_0": T.Q4_0, "Q5_0": T.Q5_0, "Q3_K": T.Q3_K, "Q5_K": T.Q5_K, "Q8_0": T.Q8_0, "Q4_K": T.Q4_K, "IQ2_XS": T.IQ2_XS, "IQ3_S": T.IQ3_S, "IQ3_XXS": T.IQ3_XXS, "IQ2_S": T.IQ2_S, "IQ4_NL": T.IQ4_NL, "IQ4_XS": T.IQ4_XS}


def q2_0_numpy(blocks):
    """[nb][18] bytes -> [nb][64] f32: value (two-bit field j of byte 2 + k) - 1, times the f16 at byte 0, for weight 4k + j."""
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)                       # [nb][1]
    f = (blocks[:, 2:, None] >> (2 * np.arange(4, dtype=np.uint8))[None, None, :]) & 3     # [nb][16][4]
    return (f.astype(np.int32) - 1).astype(np.float32).reshape(-1, 64) * d


def main():
    only = set(sys.argv[1:])          # names to (re)write; none = all
    for name, t in oracle.QUANT_TYPES.items():
        if only and name not in only:
            continue
        el, bs = oracle.geom(t)
        cols, rows = 512, 4
        a = oracle.synth_rows(t, 0, 11, cols, 0, rows // 2)
        rng = np.random.default_rng(1234 + t)
        nb = (rows // 2) * cols // el
        b = rng.integers(0, 256, size=(nb, bs), dtype=np.uint8)
        b[:, 1] = rng.integers(0x20, 0x38, nb)  # f16 exponent byte: scales of about 0.01 .. 0.5
        if name == "Q4_K":
            b[:, 3] = rng.integers(0x20, 0x38, nb)
        raw = np.concatenate([a, b.reshape(-1)])
        f32 = quants.dequantize(raw.reshape(-1, bs), GG[name]).reshape(rows, cols).astype(np.float32)
        np.savez_compressed(HERE / f"dequant_{name}.npz", raw=raw, f32=f32, rows=rows, cols=cols, type=t)
        print(name, raw.size, "bytes")
    for name, t in oracle.EXTRA_TYPES.items():     # the loader's further formats: random bytes with a sane f16 scale only
        if only and name not in only:
            continue
        el, bs = oracle.geom(t)
        cols, rows = 512, 4
        rng = np.random.default_rng(4321 + t)
        nb = rows * cols // el
        b = rng.integers(0, 256, size=(nb, bs), dtype=np.uint8)
        b[:, {"Q6_K": 209, "Q3_K": 109}.get(name, 1)] = rng.integers(0x20, 0x38, nb)      # Q6_K and Q3_K keep their f16 scale in the last two bytes
        if name == "Q5_K":
            b[:, 3] = rng.integers(0x20, 0x38, nb)
        if name == "IQ1_M":            # its f16 scale is spread over the top nibbles of the four scale words (bytes 49, 51, 53, 55)
            hi = rng.integers(0x20, 0x38, nb)
            b[:, 53] = (b[:, 53] & 0x0F) | ((hi & 0xF) << 4).astype(np.uint8)
            b[:, 55] = (b[:, 55] & 0x0F) | (hi & 0xF0).astype(np.uint8)
        raw = b.reshape(-1)
        if name == "Q2_0":
            f32 = q2_0_numpy(raw.reshape(-1, bs)).reshape(rows, cols)
        else:
            f32 = quants.dequantize(raw.reshape(-1, bs), GG[name]).reshape(rows, cols).astype(np.float32)
        np.savez_compressed(HERE / f"dequant_{name}.npz", raw=raw, f32=f32, rows=rows, cols=cols, type=t)
        print(name, raw.size, "bytes")
    if only and "kv4" not in only:
        return
    x = np.array([(i * np.float32(0.017) - np.float32(1.3)) * (np.float32(4.0) if i % 32 == 7 else np.float32(0.15)) for i in range(256)], dtype=np.float32)
    w, s = oracle.kv4_pack(x)
    y = oracle.kv4_unpack(w, s, 256)
    assert np.all(np.abs(y - x) <= np.repeat(s, 32) * 0.5 + 1e-6)
    np.savez_compressed(HERE / "kv4_vector.npz", x=x, words=w, scales=s, unpacked=y)
    print("kv4 ok")


if __name__ == "__main__":
    main()
