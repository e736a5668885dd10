"""GPU parity of dequantization and dequant-GEMV against the CPU oracle, through the C ABI."""
from pathlib import Path

import numpy as np
import pytest

import oracle
import pyre_b200 as pb
from conftest import rel_err

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
TYPES = {"Q8_0": pb.Q8_0, "Q4_K": pb.Q4_K, "IQ2_XS": pb.IQ2_XS, "IQ3_S": pb.IQ3_S}
EXTRA = {"IQ3_XXS": pb.IQ3_XXS, "IQ2_S": pb.IQ2_S, "IQ4_NL": pb.IQ4_NL, "IQ4_XS": pb.IQ4_XS,   # the GGUF loader's further formats
         "Q2_0": pb.Q2_0, "IQ2_XXS": pb.IQ2_XXS, "Q6_K": pb.Q6_K, "IQ1_M": pb.IQ1_M, "Q4_0": pb.Q4_0, "Q5_0": pb.Q5_0, "Q3_K": pb.Q3_K, "Q5_K": pb.Q5_K}
GEMV_TOL = 1e-3   # relative, f32 accumulate (north-star tolerance)


@pytest.mark.parametrize("name", list(TYPES))
def test_dequant_golden_bit_exact(ctx, name):
    g = np.load(GOLD / f"dequant_{name}.npz")
    rows, cols = int(g["rows"]), int(g["cols"])
    W = pb.QMat.upload(ctx, TYPES[name], rows, cols, g["raw"])
    y = W.to_f32()
    assert np.array_equal(y.view(np.uint32), g["f32"].view(np.uint32))
    assert np.array_equal(W.raw_rows(1, 2), g["raw"].reshape(rows, -1)[1:3].reshape(-1))
    W.free()


@pytest.mark.parametrize("name", list(EXTRA))
def test_extra_formats_dequant_golden_and_gemv(ctx, name):
    """The further formats: dequantization bit-for-bit against the gguf-py fixture, and the GEMV over the
    fixture's bytes against the oracle."""
    g = np.load(GOLD / f"dequant_{name}.npz")
    rows, cols = int(g["rows"]), int(g["cols"])
    W = pb.QMat.upload(ctx, EXTRA[name], rows, cols, g["raw"])
    assert np.array_equal(W.to_f32().view(np.uint32), g["f32"].view(np.uint32))
    x = np.random.default_rng(3).standard_normal((5, cols)).astype(np.float32)
    ref = oracle.QMat(EXTRA[name], rows, cols, g["raw"]).matmul(x)
    assert rel_err(W.matmul(x), ref) < GEMV_TOL
    W.free()


@pytest.mark.parametrize("name", list(TYPES))
def test_dequant_bit_exact_vs_oracle_config0_shape(ctx, name):
    """Config 0: 4096 x 2048 from seed 0; the device generator must also reproduce the oracle's bytes."""
    t = TYPES[name]
    W = pb.QMat.synth(ctx, t, 4096, 2048, 0, 1)
    Wo = oracle.QMat.synth(t, 4096, 2048, 0, 1)
    assert np.array_equal(W.raw_rows(0, 4096), Wo.raw())
    assert np.array_equal(W.to_f32().view(np.uint32), Wo.to_f32().view(np.uint32))
    W.free()


def test_synth_f32_matches_oracle(ctx):
    W = pb.QMat.synth(ctx, pb.F32, 512, 2048, 7, 3)
    ref = oracle.synth_normal(7, 3, 0, 512 * 2048, 0.02).reshape(512, 2048)
    assert np.array_equal(W.to_f32().view(np.uint32), ref.view(np.uint32))
    assert abs(float(ref.std()) - 0.02) < 5e-4
    W.free()


def test_config0_iq3s_gemv(ctx):
    """Config 0: W 4096x2048 IQ3_S seed 0, x ~ N(0,1), batch 1; y within 1e-3 relative."""
    W = pb.QMat.synth(ctx, pb.IQ3_S, 4096, 2048, 0, 1)
    x = np.random.default_rng(0).standard_normal((1, 2048)).astype(np.float32)
    y = W.matmul(x)
    ref = oracle.QMat.synth(oracle.IQ3_S, 4096, 2048, 0, 1).matmul(x)
    assert rel_err(y, ref) < GEMV_TOL
    # element-wise form of the tolerance: |y - ref| <= 1e-3 |ref| + 1e-3 rms(ref)
    assert np.all(np.abs(y - ref) <= GEMV_TOL * np.abs(ref) + GEMV_TOL * np.sqrt(np.mean(ref ** 2)))
    W.free()


@pytest.mark.parametrize("name", list(TYPES) + list(EXTRA) + ["F32"])
@pytest.mark.parametrize("shape", [(2048, 512), (1024, 2048), (4096, 2048), (515, 2048), (200, 4096), (300, 256), (40, 768)])
def test_gemv_sweep(ctx, name, shape):
    """Config 1 shapes (lm-head covered separately) and ragged row counts, batch 1 / 4 / 16 and odd batches."""
    t = pb.F32 if name == "F32" else (TYPES[name] if name in TYPES else EXTRA[name])
    rows, cols = shape
    W = pb.QMat.synth(ctx, t, rows, cols, 0, 42)
    Wo = oracle.QMat.synth(t, rows, cols, 0, 42)
    rng = np.random.default_rng(rows * 31 + cols)
    for tt in (1, 3, 4, 16, 19):
        x = rng.standard_normal((tt, cols)).astype(np.float32)
        y = W.matmul(x)
        assert y.shape == (tt, rows)
        assert rel_err(y, Wo.matmul(x)) < GEMV_TOL, (name, shape, tt)
    assert ctx.device_status() == 0
    W.free()


_IMMA_SHAPES = [(2048, 512), (1024, 1024), (515, 2048), (4096, 2048), (33, 512), (6000, 2048)]
_IMMA_SCRIPT = r"""
import sys, numpy as np
import pyre_b200 as pb
ctx = pb.Ctx()
out = {}
for rows, cols in %r:
    W = pb.QMat.synth(ctx, pb.IQ3_S, rows, cols, 0, 9)
    rng = np.random.default_rng(rows + 7 * cols)
    x = rng.standard_normal((2, cols)).astype(np.float32)
    x[0, :32] *= 1e4
    x[1, 64:96] *= 1e-6
    x[1, 256:512] = 0.0
    out[f"x_{rows}x{cols}"] = x
    out[f"y2_{rows}x{cols}"] = W.matmul(x)
    out[f"y1_{rows}x{cols}"] = W.matmul(x[:1])
    out[f"launches_{rows}x{cols}"] = np.array(ctx.device_status())
    W.free()
np.savez(sys.argv[1], **out)
""" % (_IMMA_SHAPES,)


def test_int8_tensor_core_gemv_vs_oracle(tmp_path):
    """The int8 tensor-core kernel (pb_gemvi.cu), forced for every size and for one token too (by default it takes two
    tokens of large matrices): row widths of 2, 4 and 8 blocks of 256, ragged row counts, activations with groups of
    very different magnitude (its levels share one scale per 256 values) and an all-zero block; 3e-6 against the
    oracle, far inside the 1e-3 of the contract."""
    import os
    import subprocess
    import sys
    f = tmp_path / "imma.npz"
    env = dict(os.environ, PYRE_B200_IMMA_MIN="1", PYRE_B200_IMMA_MIN_WEIGHTS="0")
    root = str(Path(__file__).resolve().parent.parent)
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    subprocess.run([sys.executable, "-c", _IMMA_SCRIPT, str(f)], check=True, env=env, cwd=root, timeout=300)
    res = dict(np.load(f))
    for rows, cols in _IMMA_SHAPES:
        Wo = oracle.QMat.synth(oracle.IQ3_S, rows, cols, 0, 9)
        x = res[f"x_{rows}x{cols}"]
        ref = Wo.matmul(x)
        assert res[f"y2_{rows}x{cols}"].shape == (2, rows)
        assert rel_err(res[f"y2_{rows}x{cols}"], ref) < 3e-6, (rows, cols)
        assert rel_err(res[f"y1_{rows}x{cols}"], ref[:1]) < 3e-6, (rows, cols)
        assert int(res[f"launches_{rows}x{cols}"]) == 0


def test_gemv_lm_head_linearity(ctx):
    """Full-size lm-head (151936 x 2048 IQ3_S): oracle on a row sample, linearity on all rows."""
    rows, cols = 151936, 2048
    W = pb.QMat.synth(ctx, pb.IQ3_S, rows, cols, 0, 2)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, cols)).astype(np.float32)
    y = W.matmul(x)
    ysum = W.matmul((x[0] + x[1])[None])
    assert rel_err(ysum[0], y[0] + y[1]) < 1e-4
    for r0 in (0, 75000, rows - 64):
        Wo = oracle.QMat(oracle.IQ3_S, 64, cols, oracle.synth_rows(oracle.IQ3_S, 0, 2, cols, r0, 64))
        assert rel_err(y[:, r0:r0 + 64], Wo.matmul(x)) < GEMV_TOL
    W.free()


def test_gemv_zero_and_extreme_inputs(ctx):
    W = pb.QMat.synth(ctx, pb.IQ3_S, 256, 2048, 0, 8)
    Wo = oracle.QMat.synth(oracle.IQ3_S, 256, 2048, 0, 8)
    assert np.all(W.matmul(np.zeros((1, 2048), np.float32)) == 0)
    x = np.zeros((1, 2048), np.float32); x[0, 100] = 1e4; x[0, 1999] = -3e-5
    assert rel_err(W.matmul(x), Wo.matmul(x)) < GEMV_TOL
    W.free()


def test_bad_arguments_fail_loudly(ctx):
    with pytest.raises(pb.PyreError):
        pb.QMat.upload(ctx, 99, 4, 256, np.zeros(16, np.uint8))          # unknown ggml type
    with pytest.raises(pb.PyreError):
        pb.QMat.upload(ctx, pb.IQ3_S, 4, 250, np.zeros(440, np.uint8))   # row not a multiple of the block
    with pytest.raises(pb.PyreError):
        pb.QMat.upload(ctx, pb.IQ3_S, 4, 256, np.zeros(100, np.uint8))   # truncated data
    W = pb.QMat.synth(ctx, pb.IQ3_S, 4, 256, 0, 1)
    with pytest.raises(pb.PyreError):
        W.raw_rows(2, 5)
    W.free()


_NATIVE_SCRIPT = r"""
import sys, numpy as np
import pyre_b200 as pb
ctx = pb.Ctx()
out = {}
for rows, cols, t in [(4096, 2048, 1), (2048, 512, 2), (515, 2048, 1), (200, 4096, 1), (1024, 2048, 8), (515, 2048, 15), (200, 4096, 5), (2048, 512, 12)]:
    W = pb.QMat.synth(ctx, pb.IQ3_S, rows, cols, 0, 5)
    x = np.random.default_rng(rows + cols).standard_normal((t, cols)).astype(np.float32)
    out[f"{rows}x{cols}x{t}"] = W.matmul(x)
    W.free()
np.savez(sys.argv[1], **out)
"""


def test_iq3s_recoded_and_native_kernels_agree_bit_for_bit(ctx, tmp_path):
    """IQ3_S matrices are streamed from a copy re-coded into 4-bit codes (weight = 2c - 15).  The
    re-coding is lossless and the offset is removed in integers, so the GEMV through the re-coded copy
    must equal the GEMV over the native GGUF blocks (PYRE_B200_REPACK=0) bit for bit -- on the dp4a path
    (1-2 tokens; two tokens of matrices above ten million weights go to the int8 tensor-core kernel, which has its
    own test) and on the warp-level tensor-core path (3 to 15 tokens; 16 and more go to the tcgen05 GEMM, which
    exists only for the re-coded copy and is compared with the oracle in test_gemmtc_gpu.py)."""
    import os
    import subprocess
    import sys
    res = {}
    for mode in ("1", "0"):
        f = tmp_path / f"gemv_repack{mode}.npz"
        env = dict(os.environ, PYRE_B200_REPACK=mode)
        root = str(Path(__file__).resolve().parent.parent)
        env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
        subprocess.run([sys.executable, "-c", _NATIVE_SCRIPT, str(f)], check=True, env=env, cwd=root, timeout=300)
        res[mode] = dict(np.load(f))
    assert set(res["0"]) == set(res["1"]) and len(res["0"]) == 8
    for k in res["0"]:
        assert np.array_equal(res["0"][k].view(np.uint32), res["1"][k].view(np.uint32)), k
    # and both against the oracle
    x = np.random.default_rng(4096 + 2048).standard_normal((1, 2048)).astype(np.float32)
    ref = oracle.QMat.synth(oracle.IQ3_S, 4096, 2048, 0, 5).matmul(x)
    assert rel_err(res["1"]["4096x2048x1"], ref) < GEMV_TOL
