"""pb_gemv_static: the GEMV entry point for hosts that cannot allocate device memory.

Collected last on purpose.  It goes through the C ABI and compares the allocation-free
variant (x and y staged in the fixed array compiled into the library) with pb_gemv (staging
buffer from cudaMalloc): same kernels, so the outputs must be identical; two calls in a row
show that bytes left in the shared array by one call do not leak into the next.
"""
import numpy as np
import pytest

import pyre_b200 as pb

pytestmark = pytest.mark.gpu


def test_static_staging_matches_allocating_entry_point(ctx):
    rng = np.random.default_rng(11)
    W = pb.QMat.synth(ctx, pb.IQ3_S, 4096, 2048, 0, 77)
    W2 = pb.QMat.synth(ctx, pb.Q4_K, 1000, 512, 0, 78)
    x1 = rng.standard_normal((4, 2048)).astype(np.float32)
    x2 = rng.standard_normal((1, 512)).astype(np.float32)
    # first call: larger problem, fills much of the array; second call: smaller, different matrix
    y1 = W.matmul_static(x1)
    y2 = W2.matmul_static(x2)
    assert np.array_equal(y1, W.matmul(x1))
    assert np.array_equal(y2, W2.matmul(x2))
    # and again in the opposite order
    assert np.array_equal(W2.matmul_static(x2), y2)
    assert np.array_equal(W.matmul_static(x1), y1)
    assert ctx.device_status() == 0
    W.free(); W2.free()


def test_static_staging_rejects_oversized_requests(ctx):
    W = pb.QMat.synth(ctx, pb.IQ3_S, 151936, 2048, 0, 79)      # t=8: 8 * (2048 + 151936) * 4 bytes > 4 MiB
    with pytest.raises(pb.PyreError) as e:
        W.matmul_static(np.zeros((8, 2048), np.float32))
    assert e.value.status == pb.PB_ERR_ARG and "4194304" in str(e.value)
    y = W.matmul_static(np.ones((1, 2048), np.float32))          # t=1 fits (616 KB)
    assert y.shape == (1, 151936)
    W.free()


def test_static_staging_allocates_no_device_memory(ctx):
    """The property the entry point exists for: after a warm-up call (which loads the kernels' module and resolves
    the array's address), further calls -- other shapes, other matrices -- leave the free device memory untouched."""
    import torch
    torch.cuda.mem_get_info(0)                                   # torch's own lazy initialisation happens here, not below
    rng = np.random.default_rng(12)
    mats = [pb.QMat.synth(ctx, pb.IQ3_S, 4096, 2048, 0, 80), pb.QMat.synth(ctx, pb.Q8_0, 2048, 512, 0, 81), pb.QMat.synth(ctx, pb.IQ3_S, 151936, 2048, 0, 82)]
    xs = [rng.standard_normal((t, W.cols)).astype(np.float32) for W, t in zip(mats, (16, 3, 1))]
    for W, x in zip(mats, xs):
        W.matmul_static(x)                                       # warm-up: every kernel instance used below has run once
    ctx.sync()
    free0 = torch.cuda.mem_get_info(0)[0]
    for _ in range(3):
        for W, x in zip(mats, xs):
            W.matmul_static(x)
    ctx.sync()
    assert torch.cuda.mem_get_info(0)[0] == free0
    for W in mats:
        W.free()


def test_static_staging_limit_is_exact(ctx):
    """4 tokens of 2048 columns take 32768 bytes; with 260096 rows the outputs fill the rest of the 4 MiB exactly."""
    W = pb.QMat.synth(ctx, pb.IQ3_S, 260096, 2048, 0, 83)
    x = np.random.default_rng(13).standard_normal((4, 2048)).astype(np.float32)
    assert np.array_equal(W.matmul_static(x), W.matmul(x))
    W.free()
    W = pb.QMat.synth(ctx, pb.IQ3_S, 260096 + 16, 2048, 0, 84)    # 256 bytes over
    with pytest.raises(pb.PyreError) as e:
        W.matmul_static(x)
    assert e.value.status == pb.PB_ERR_ARG
    W.free()
