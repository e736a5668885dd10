"""Worker functions for the expert-parallel tests (spawned as separate processes)."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def _init(rank, world, port, backend):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group(backend, rank=rank, world_size=world)
    return dist


def cpu_exact_gather(rank, world, port, out_dir):
    """gloo, CPU: per-rank partial MoE outputs (zero where the expert is remote) all-reduced with
    sum equal the single-process result bit for bit; the unique-id hand-off delivers rank 0's bytes."""
    import torch
    import oracle
    import pyre_b200 as pb
    from pyre_b200 import parallel, synth
    from helpers import oracle_cfg, oracle_model, small_cfg
    dist = _init(rank, world, port, "gloo")
    uid = parallel.share_unique_id(dist, lambda: bytes(range(128)), rank)
    assert uid == bytes(range(128))
    cfg = small_cfg(pb, d=256, ff_exp=256, ff_sh=256, n_exp=8, top_k=3, n_layers=1, full_every=0, vocab=256)
    spec = synth.model_spec(cfg, 5)
    _, mats = oracle_model(cfg, spec, 5)
    x = np.random.default_rng(9).standard_normal((4, cfg.d)).astype(np.float32)
    ocfg = oracle_cfg(cfg)
    y_ref, sel, selw = oracle.moe(ocfg, mats[(0, "ROUTER")], mats[(0, "EXP_GATE")], mats[(0, "EXP_UP")], mats[(0, "EXP_DOWN")],
                                  mats[(0, "SH_GATE")], mats[(0, "SH_UP")], mats[(0, "SH_DOWN")], mats[(0, "SH_GATE_INP")], x)
    lo, hi = parallel.ep_range(cfg.n_exp, rank, world)
    order = np.argsort(sel, axis=1)                      # accumulation order: ascending expert id
    part = np.zeros((4, cfg.top_k, cfg.d), np.float32)
    silu = lambda v: v * (np.float32(1) / (np.float32(1) + np.exp(-v)))
    G, U, D = (mats[(0, r)].to_f32() for r in ("EXP_GATE", "EXP_UP", "EXP_DOWN"))
    for t in range(4):
        for slot, j in enumerate(order[t]):
            e = int(sel[t, j])
            assert parallel.owner_of(e, cfg.n_exp, world) == (rank if lo <= e < hi else parallel.owner_of(e, cfg.n_exp, world))
            if lo <= e < hi:
                g = G[e * cfg.ff_exp:(e + 1) * cfg.ff_exp] @ x[t]; u = U[e * cfg.ff_exp:(e + 1) * cfg.ff_exp] @ x[t]
                part[t, slot] = selw[t, j] * (D[e * cfg.d:(e + 1) * cfg.d] @ (silu(g) * u).astype(np.float32))
    local = part.copy()
    tt = torch.from_numpy(part)
    dist.all_reduce(tt)
    full = tt.numpy()
    # exact gather: wherever this rank produced a row the reduced row has the same bits
    mine = np.abs(local).sum(axis=2) > 0
    assert np.array_equal(full[mine].view(np.uint32), local[mine].view(np.uint32))
    assert np.all(np.abs(full).sum(axis=2) > 0)          # every (token, slot) was produced by someone
    if rank == 0:
        np.save(Path(out_dir) / "full.npy", full)
        # routed sum in slot order matches the oracle's routed contribution within f32 matmul noise
        sg = 1 / (1 + np.exp(-(x @ mats[(0, "SH_GATE_INP")])))
        xs = [mats[(0, r)] for r in ("SH_GATE", "SH_UP", "SH_DOWN")]
        sh = xs[2].matmul((silu(xs[0].matmul(x)) * xs[1].matmul(x)).astype(np.float32)) * sg[:, None].astype(np.float32)
        y = sh + full.sum(axis=1)
        assert np.abs(y - y_ref).max() <= 1e-4 * np.abs(y_ref).max()
    dist.barrier(); dist.destroy_process_group()


def gpu_ep_tokens(rank, world, port, out_dir):
    """NCCL, one GPU per rank: expert-parallel greedy tokens are identical to a single-GPU run."""
    import torch
    import pyre_b200 as pb
    from pyre_b200 import parallel, synth
    from helpers import small_cfg
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist = _init(rank, world, port, "gloo")
    ctx = pb.Ctx(rank)
    parallel.init_expert_parallel(ctx, dist, rank, world)
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=256)
    spec = synth.model_spec(cfg, 3)
    m = synth.build_model(ctx, cfg, spec, 3, rank, world)
    st = m.new_state(2)
    toks = st.decode_greedy([5, 600], 40)
    np.save(Path(out_dir) / f"ep{rank}.npy", toks)
    st.destroy(); m.destroy()
    if rank == 0:
        ctx1 = pb.Ctx(0)
        m1 = synth.build_model(ctx1, cfg, spec, 3)
        s1 = m1.new_state(2)
        np.save(Path(out_dir) / "single.npy", s1.decode_greedy([5, 600], 40))
        s1.destroy(); m1.destroy(); ctx1.close()
    dist.barrier(); ctx.close(); dist.destroy_process_group()


def gpu_sharded_tokens(rank, world, port, out_dir):
    """NCCL, one GPU per rank, sharded tokens: rank r decodes sequences [2r, 2r+2) of a global batch of
    2 * world; dense layers see only the local sequences, MoE blocks all-gather / reduce-scatter.  The
    tokens equal a single-GPU run of the whole batch."""
    import torch
    import pyre_b200 as pb
    from pyre_b200 import parallel, synth
    from helpers import small_cfg
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist = _init(rank, world, port, "gloo")
    ctx = pb.Ctx(rank)
    parallel.init_expert_parallel(ctx, dist, rank, world)
    cfg = small_cfg(pb, n_layers=8, kv_bits=4, kv_recent=64, max_ctx=256)
    spec = synth.model_spec(cfg, 3)
    m = synth.build_model(ctx, cfg, spec, 3, rank, world)
    first = np.array([5, 600, 77, 1000, 9, 321, 42, 800], np.uint32)[:2 * world]
    st = m.new_state(2, sharded=True)             # default: in-kernel peer exchange
    toks = st.decode_greedy(first[2 * rank:2 * rank + 2], 40)
    np.save(Path(out_dir) / f"sh{rank}.npy", toks)
    assert st.stats().exchange_ns > 0             # the peer hand-shakes ran (they account their own time)
    os.environ["PYRE_B200_EP_EXCHANGE"] = "nccl"  # the same through NCCL all-gather + reduce-scatter
    st2 = m.new_state(2, sharded=True)
    toks2 = st2.decode_greedy(first[2 * rank:2 * rank + 2], 40)
    del os.environ["PYRE_B200_EP_EXCHANGE"]
    assert st2.stats().exchange_ns == 0
    assert np.array_equal(toks, toks2)
    # both states alive at once, stepping alternately: each owns its exchange block and sequence counter
    a = st.decode_greedy(toks[:, -1].copy(), 8); b = st2.decode_greedy(toks2[:, -1].copy(), 8)
    assert np.array_equal(a, b)
    st2.destroy(); st.destroy(); m.destroy()
    if rank == 0:
        ctx1 = pb.Ctx(0)
        m1 = synth.build_model(ctx1, cfg, spec, 3)
        # the single-GPU run steps each rank's share in a state of the same batch size: kernels are chosen by batch size
        # (dp4a / tensor cores, attention splits), and bit-identical results need the same ones on both sides
        single = []
        for r in range(world):
            s1 = m1.new_state(2)
            single.append(s1.decode_greedy(first[2 * r:2 * r + 2], 40))
            s1.destroy()
        np.save(Path(out_dir) / "single.npy", np.concatenate(single))
        m1.destroy(); ctx1.close()
    dist.barrier(); ctx.close(); dist.destroy_process_group()


def cpu_sharded_bookkeeping(rank, world, port, out_dir):
    """gloo, CPU: the exchange of a sharded MoE block -- all-gather of the local rows, per-rank partial
    rows for the local experts of every token, reduce-scatter to the owners -- returns to every rank
    exactly the rows a single process computes for its tokens."""
    import torch
    from pyre_b200 import parallel
    dist = _init(rank, world, port, "gloo")
    t, d, top_k, n_exp = 3, 8, 2, 4
    rng = np.random.default_rng(11)
    x_all = rng.standard_normal((world * t, d)).astype(np.float32)           # same on every rank
    sel = np.stack([np.sort(rng.choice(n_exp, top_k, replace=False)) for _ in range(world * t)])
    W = rng.standard_normal((n_exp, d, d)).astype(np.float32)
    ref = np.stack([[W[e] @ x_all[tok] for e in sel[tok]] for tok in range(world * t)]).astype(np.float32)
    mine = torch.from_numpy(x_all[rank * t:(rank + 1) * t].copy())
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    xg = torch.cat(gathered).numpy()
    assert np.array_equal(xg, x_all)
    lo, hi = parallel.ep_range(n_exp, rank, world)
    part = np.zeros((world * t, top_k, d), np.float32)
    for tok in range(world * t):
        for slot, e in enumerate(sel[tok]):
            if lo <= e < hi:
                part[tok, slot] = W[e] @ xg[tok]
    # gloo has no reduce_scatter: all-reduce, then keep the local slice (the same sum of one row and zeros)
    full = torch.from_numpy(part.copy()); dist.all_reduce(full); out = full[rank * t:(rank + 1) * t]
    assert np.array_equal(out.numpy().view(np.uint32), ref[rank * t:(rank + 1) * t].view(np.uint32))
    if rank == 0:
        np.save(Path(out_dir) / "ok.npy", np.ones(1))
    dist.barrier(); dist.destroy_process_group()


def cpu_flag_protocol(rank, world, port, out_dir):
    """CPU, two processes over one memory-mapped flag array: the sequence-numbered hand-shake of the peer exchange.
    Exchange 1 and 2 complete on both ranks (rank 1 runs ahead and posts 2 before rank 0 looked at 1); rank 1 then
    stops posting, and rank 0's bounded wait for exchange 3 reports a timeout instead of blocking."""
    import time
    from pyre_b200 import parallel
    dist = _init(rank, world, port, "gloo")
    path = Path(out_dir) / "flags.bin"
    if rank == 0:
        np.zeros((world, 2, world), np.uint64).tofile(path)
    dist.barrier()
    flags = np.memmap(path, dtype=np.uint64, mode="r+", shape=(world, 2, world))
    fx = parallel.FlagExchange(flags, rank, world, spin_limit=400, pause=lambda: time.sleep(0.005))
    res = []
    if rank == 1:
        fx.post(0, 1); fx.post(0, 2); flags.flush()          # a fast peer: two exchanges announced back to back
        res = [fx.wait(0, 1), fx.wait(0, 2)]
        assert res == [True, True]
    else:
        time.sleep(0.2)                                       # a slow rank: it first sees the value 2
        res = [fx.exchange(0, 1), fx.exchange(0, 2)]
        assert res == [True, True]
        short = parallel.FlagExchange(flags, rank, world, spin_limit=40, pause=lambda: time.sleep(0.005))
        assert short.exchange(0, 3) is False                  # rank 1 never posts 3: the wait gives up
        assert short.exchange(1, 1) is False                  # the other kind has its own counters
        np.save(Path(out_dir) / "flag_ok.npy", np.ones(1))
    dist.barrier(); dist.destroy_process_group()
