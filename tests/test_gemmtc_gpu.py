"""tcgen05 dequant-GEMM (16 and more tokens, IQ3_S): parity with the CPU oracle through the C-ABI (pb_gemv)."""
import os

import numpy as np
import pytest

import oracle
import pyre_b200 as pb
from conftest import rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _tc_from_16_tokens(monkeypatch):
    """The dispatcher prefers the warp-level kernel below 32 tokens (it is faster there); these tests run the tcgen05
    kernel from its own lower limit."""
    monkeypatch.setenv("PYRE_B200_TC_MIN", "16")

GEMM_TOL = 1e-3   # relative to the largest output, f32 accumulate (the tolerance of the GEMV configurations)


@pytest.mark.parametrize("shape", [(2048, 512), (1024, 2048), (4096, 2048), (515, 2048), (200, 4096), (300, 256)])
@pytest.mark.parametrize("tt", [16, 64, 256])
def test_gemm_sweep_vs_oracle(ctx, shape, tt):
    """The GEMV sweep's shapes (out x in) and ragged row counts at 16, 64 and 256 tokens."""
    rows, cols = shape
    W = pb.QMat.synth(ctx, pb.IQ3_S, rows, cols, 0, 42)
    Wo = oracle.QMat.synth(oracle.IQ3_S, rows, cols, 0, 42)
    x = np.random.default_rng(rows * 31 + cols + tt).standard_normal((tt, cols)).astype(np.float32)
    y = W.matmul(x)
    assert y.shape == (tt, rows)
    assert rel_err(y, Wo.matmul(x)) < GEMM_TOL, (shape, tt)
    assert ctx.device_status() == 0
    W.free()


@pytest.mark.parametrize("tt", [17, 100, 129, 300])
def test_gemm_ragged_token_counts(ctx, tt):
    """Token counts that are no multiple of 16 or of the 128-token block; every output row of every token is written."""
    W = pb.QMat.synth(ctx, pb.IQ3_S, 384, 1024, 3, 7)
    Wo = oracle.QMat.synth(oracle.IQ3_S, 384, 1024, 3, 7)
    x = np.random.default_rng(tt).standard_normal((tt, 1024)).astype(np.float32)
    y = W.matmul(x)
    assert rel_err(y, Wo.matmul(x)) < GEMM_TOL
    # per token, not only against the largest output of the whole batch
    ref = Wo.matmul(x)
    for b in (0, tt // 2, tt - 1):
        assert rel_err(y[b], ref[b]) < GEMM_TOL
    W.free()


def test_gemm_matches_the_single_token_kernel(ctx):
    """The same matrix through the integer GEMV (one token at a time) and through the tensor-core GEMM (all at once)."""
    W = pb.QMat.synth(ctx, pb.IQ3_S, 1024, 2048, 1, 5)
    x = np.random.default_rng(2).standard_normal((64, 2048)).astype(np.float32)
    y = W.matmul(x)
    y1 = np.concatenate([W.matmul(x[i:i + 1]) for i in range(0, 64, 9)])
    assert rel_err(y[::9], y1) < 5e-4
    W.free()


def test_gemm_extreme_scales_and_inputs(ctx):
    """Block scales spanning the f16 range and activations spanning many orders of magnitude: the per-tile shift of the
    weights and the per-token prescale of the activations keep f16 operands in range."""
    rows, cols = 256, 512
    Wo = oracle.QMat.synth(oracle.IQ3_S, rows, cols, 0, 11)
    raw = Wo.raw().reshape(rows, cols // 256, 110).copy()
    d = raw[:, :, :2].view(np.float16)
    d[::2] = np.float16(120.0)        # d * 465 alone overflows f16
    d[1::2] = np.float16(3e-4)
    Wbig = oracle.QMat(oracle.IQ3_S, rows, cols, raw.reshape(-1))
    W = pb.QMat.upload(ctx, pb.IQ3_S, rows, cols, raw.reshape(-1))
    x = np.random.default_rng(4).standard_normal((32, cols)).astype(np.float32)
    x[3] *= 1e6; x[7] *= 1e-6; x[9] = 0
    y, ref = W.matmul(x), Wbig.matmul(x)
    assert np.all(np.isfinite(y))
    for b in range(32):
        assert rel_err(y[b], ref[b]) < GEMM_TOL or np.abs(ref[b]).max() == 0
    assert np.all(y[9] == 0)
    W.free()


def test_many_tokens_on_a_matrix_wider_than_the_streaming_kernels_take(ctx):
    """8192 columns are outside the integer / tensor-core kernels (4096 at most): pb_gemv must cut 64 tokens into pieces
    the generic kernel accepts instead of handing it all 64."""
    W = pb.QMat.synth(ctx, pb.IQ3_S, 256, 8192, 0, 3)
    Wo = oracle.QMat.synth(oracle.IQ3_S, 256, 8192, 0, 3)
    x = np.random.default_rng(8).standard_normal((64, 8192)).astype(np.float32)
    assert rel_err(W.matmul(x), Wo.matmul(x)) < GEMM_TOL
    W.free()
