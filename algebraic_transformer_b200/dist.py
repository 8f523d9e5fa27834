"""Rank bootstrap and the two partitioning rules of the multi-GPU path.

One process per GPU (`torch.distributed`, NCCL over NVLink/NVSwitch on GPUs, gloo on
CPU for the host-logic tests).  Attention shards by (batch, head) units with no
communication; the Alg-CE head shards the vocabulary in 128-column tiles and exchanges
one (2, N) fp32 all-reduce of per-row partials.  The reference itself is data-parallel
only (src/algebraic/train.py:199, 245-246); this partitioning is the B200 design.
"""

import os
from typing import Tuple

VOCAB_TILE = 128


def vocab_shard(vocab_total: int, rank: int, world: int, tile: int = VOCAB_TILE) -> Tuple[int, int]:
    """(first_row, row_count) of `rank`'s contiguous vocabulary range.  Whole tiles are dealt
    out as evenly as possible (the first `ntiles % world` ranks get one more); the last
    range ends at `vocab_total`, so a ragged final tile is owned by exactly one rank."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    ntiles = -(-vocab_total // tile)
    base, extra = divmod(ntiles, world)
    first_tile = rank * base + min(rank, extra)
    count_tiles = base + (1 if rank < extra else 0)
    lo = min(first_tile * tile, vocab_total)
    hi = min((first_tile + count_tiles) * tile, vocab_total)
    return lo, hi - lo


def unit_shard(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """(first_unit, count) of `rank`'s contiguous block of independent units
    ((batch, head) pairs for attention, sequences for prefill)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    base, extra = divmod(n_units, world)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def init_from_env(backend: str = None):
    """Join the process group described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_*.
    Returns (rank, world, local_rank).  A single process (no WORLD_SIZE) is world 1 and
    creates no group."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        kw = {"device_id": torch.device("cuda", local)} if backend == "nccl" else {}
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kw)
    return rank, world, local


class HeadExchange:
    """Peer-mapped exchange regions for the fused vocabulary-sharded head
    (`alg_head_fwd_exchange`): one symmetric-memory allocation per rank, mapped on every GPU
    of the group, into which the head's exchange kernel stores per-row partials directly over
    NVLink.  Create it once per (group, capacity); every rank must create it collectively."""

    def __init__(self, group, n_capacity: int, device):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        from . import _lib as L
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_capacity = int(n_capacity)
        nbytes = L.load().alg_head_exchange_region_bytes(self.world, self.n_capacity)
        if nbytes == 0:
            raise ValueError("bad world size or capacity for the head exchange")
        self.buf = symm.empty(int(nbytes), dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buf, group)
        self.buf.zero_()                       # call counter, flags and data start at zero
        torch.cuda.synchronize(device)
        dist.barrier(group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.ptrs) != self.world:
            raise RuntimeError("symmetric memory returned an unexpected number of peer pointers")
