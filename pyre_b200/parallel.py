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


class FlagExchange:
    """Host model of the flag protocol the peer-exchange kernels run on the device (csrc/pb_ep.cu).

    `flags` is one shared array [world][kinds][world] of unsigned 64-bit counters (on the device: one [kinds][world]
    array in every rank's memory, mapped into every rank).  flags[dst][kind][src] holds the sequence number of the
    last exchange of `kind` that `src` completed towards `dst`.  Sequence numbers only grow, so a waiter compares with
    `>=` and a fast peer that is already one exchange ahead never makes a slow one miss a value.  A wait is bounded:
    after `spin_limit` polls it gives up and reports a timeout instead of blocking (the device kernel then records a
    status that makes the host call return PB_ERR_DEVICE).
    """

    def __init__(self, flags, rank: int, world: int, spin_limit: int = 100000, pause=None):
        self.flags, self.rank, self.world, self.spin_limit, self.pause = flags, rank, world, spin_limit, pause

    def post(self, kind: int, seq: int):
        for p in range(self.world):
            self.flags[p, kind, self.rank] = seq

    def wait(self, kind: int, seq: int) -> bool:
        """True once every peer announced exchange `seq` of `kind`; False when the bounded wait ran out."""
        for p in range(self.world):
            ok = False
            for _ in range(self.spin_limit):
                if int(self.flags[self.rank, kind, p]) >= seq:
                    ok = True
                    break
                if self.pause:
                    self.pause()
            if not ok:
                return False
        return True

    def exchange(self, kind: int, seq: int) -> bool:
        self.post(kind, seq)
        return self.wait(kind, seq)
