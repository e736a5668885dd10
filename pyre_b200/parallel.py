"""Host-side plumbing of expert parallelism: shard ranges and the NCCL unique-id exchange.

One process per GPU.  `torch.distributed` (NCCL on GPUs, gloo in CPU tests) is used only to
hand rank 0's 128-byte NCCL id to the other ranks; the data path runs inside the library.
"""
from __future__ import annotations


def ep_range(n_exp: int, rank: int, world: int) -> tuple[int, int]:
    """Experts [lo, hi) held by `rank`: contiguous blocks of n_exp / world (pb_model_finalize uses the same rule)."""
    if world < 1 or not (0 <= rank < world) or n_exp % world:
        raise ValueError(f"rank {rank} of {world} with {n_exp} experts")
    per = n_exp // world
    return rank * per, (rank + 1) * per


def owner_of(expert: int, n_exp: int, world: int) -> int:
    return expert // (n_exp // world)


def share_unique_id(dist, make_id, rank: int, device=None) -> bytes:
    """Rank 0 creates the id with `make_id()`; everyone returns the same 128 bytes."""
    import torch

    t = torch.zeros(128, dtype=torch.uint8, device=device)
    if rank == 0:
        uid = make_id()
        assert len(uid) == 128
        t = torch.tensor(list(uid), dtype=torch.uint8, device=device)
    dist.broadcast(t, src=0)
    return bytes(t.cpu().tolist())


def init_expert_parallel(ctx, dist, rank: int, world: int, device=None):
    """Create the library's NCCL communicator on `ctx` for this rank."""
    uid = share_unique_id(dist, ctx.ep_unique_id, rank, device)
    ctx.ep_init(uid, rank, world)
