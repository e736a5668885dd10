"""Expert parallelism: host logic on CPU (gloo, world size 2) and, where two GPUs exist, token identity."""
import socket
import tempfile

import numpy as np
import pytest

from pyre_b200 import parallel


def _port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _spawn(fn, world, out_dir):
    import torch.multiprocessing as mp
    mp.spawn(fn, args=(world, _port(), out_dir), nprocs=world, join=True)


def test_ep_range_and_owner():
    assert parallel.ep_range(512, 0, 8) == (0, 64) and parallel.ep_range(512, 7, 8) == (448, 512)
    assert [parallel.owner_of(e, 512, 8) for e in (0, 63, 64, 511)] == [0, 0, 1, 7]
    assert parallel.ep_range(512, 0, 1) == (0, 512)
    with pytest.raises(ValueError):
        parallel.ep_range(512, 0, 3)          # experts must divide evenly
    with pytest.raises(ValueError):
        parallel.ep_range(512, 8, 8)


def test_exact_gather_world2_gloo():
    import ep_worker
    with tempfile.TemporaryDirectory() as d:
        _spawn(ep_worker.cpu_exact_gather, 2, d)
        assert np.load(f"{d}/full.npy").shape[1] == 3


@pytest.mark.gpu
def test_expert_parallel_tokens_identical_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import ep_worker
    with tempfile.TemporaryDirectory() as d:
        _spawn(ep_worker.gpu_ep_tokens, 2, d)
        a, b, s = np.load(f"{d}/ep0.npy"), np.load(f"{d}/ep1.npy"), np.load(f"{d}/single.npy")
        assert np.array_equal(a, b) and np.array_equal(a, s)


def test_sharded_exchange_world2_gloo():
    import ep_worker
    with tempfile.TemporaryDirectory() as d:
        _spawn(ep_worker.cpu_sharded_bookkeeping, 2, d)
        assert np.load(f"{d}/ok.npy")[0] == 1


@pytest.mark.gpu
def test_sharded_tokens_identical_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import ep_worker
    with tempfile.TemporaryDirectory() as d:
        _spawn(ep_worker.gpu_sharded_tokens, 2, d)
        a, b, s = np.load(f"{d}/sh0.npy"), np.load(f"{d}/sh1.npy"), np.load(f"{d}/single.npy")
        assert np.array_equal(np.concatenate([a, b]), s)


def test_flag_protocol_world2_bounded_wait():
    import ep_worker
    with tempfile.TemporaryDirectory() as d:
        _spawn(ep_worker.cpu_flag_protocol, 2, d)
        assert np.load(f"{d}/flag_ok.npy")[0] == 1


@pytest.mark.gpu
def test_peer_wait_that_nobody_answers_returns_device_error():
    """A hand-shake whose partner never posts its flag: the kernel's bounded wait runs out, the call returns
    PB_ERR_DEVICE, and the context serves the next call."""
    import pyre_b200 as pb
    ctx = pb.Ctx(0)
    with pytest.raises(pb.PyreError) as e:
        ctx.ep_probe_wait_timeout(2000)
    assert e.value.status == pb.PB_ERR_DEVICE
    assert ctx.device_status() == 0
    W = pb.QMat.synth(ctx, pb.IQ3_S, 64, 256, 0, 1)     # the next call on the same context works
    x = np.random.default_rng(0).standard_normal((1, 256)).astype(np.float32)
    y = W.matmul(x)
    assert np.allclose(y, x @ W.to_f32().T, rtol=2e-3, atol=2e-3)
    with pytest.raises(pb.PyreError):
        ctx.ep_probe_wait_timeout(500)                   # and a second timeout is reported again
    assert W.matmul(x).shape == (1, 64)
    W.free(); ctx.close()
