"""Output-row sharding of a Q4_K matrix over the ranks of one node.

Rows are independent (out[row] depends on W[row, :] and x only), so each rank keeps a contiguous
run of row groups (8 rows, the unit of the split-tile layout), quantises the replicated
activations itself, and the [m, rows] output slices are gathered: by the projection kernel itself,
which stores into every rank's buffer (q4k_q8_project_gather over a symmetric_pool allocation), or by
an NCCL all-gather of the slices.  No other exchange."""
from __future__ import annotations

from typing import List, Tuple


def row_shard(n: int, world: int, rank: int) -> Tuple[int, int, int]:
    """(first row, rows, rows per full shard) of `rank`.  Shards are multiples of 8 rows; the
    last ranks may hold fewer rows (or none) when n/8 does not divide evenly."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("rank outside the world")
    per = (((n + 7) // 8) + world - 1) // world * 8
    row0 = min(n, rank * per)
    return row0, min(n, row0 + per) - row0, per


def gathered_to_token_major(gathered, n: int):
    """gathered: [world, m, per] as written by all_gather_into_tensor (rank g's slice in
    gathered[g]).  Returns the [m, n] token-major view-or-copy: out[t, g*per + j] = gathered[g, t, j]."""
    world, m, per = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, world * per)[:, :n]


def symmetric_pool(words: int, device, group=None):
    """A zeroed fp32 buffer of `words` elements allocated on every rank with
    torch.distributed._symmetric_memory.  Returns (local tensor, [device address of rank g's buffer in
    this process], handle); keep the handle alive as long as the addresses are used."""
    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm

    group = group or dist.group.WORLD
    buf = symm.empty(words, dtype=torch.float32, device=device)
    buf.zero_()
    handle = symm.rendezvous(buf, group.group_name)
    torch.cuda.synchronize(device)
    dist.barrier(group)
    return buf, [int(handle.buffer_ptrs[g]) for g in range(dist.get_world_size(group))], handle
