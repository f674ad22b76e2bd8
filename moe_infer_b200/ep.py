"""Host-side helpers of the expert-parallel path.

`plan` mirrors, in numpy, what `ep_plan_kernel` derives on the device from the
table of per-rank expert histograms: where a rank's rows land inside the owner's
receive buffer and which (expert, tile) work items the owner runs.  It exists so
that the partition logic can be tested on CPU ranks; the product path computes
the same thing on the GPU.
"""
from __future__ import annotations

from typing import List, Tuple

import numpy as np

TILE = 256  # tokens per GEMM tile (kNT in csrc/grouped.cu)


def owner_of(expert: int, num_experts: int, world: int) -> int:
    return expert // (num_experts // world)


def plan(counts_all: np.ndarray, me: int, n_local: int, tile: int = TILE):
    """counts_all int [world, E]: rows rank s sends to expert e.

    Returns (base_send [E], total_recv, tiles) where base_send[e] is the first slot,
    inside the owner's buffer, of this rank's rows for expert e, and tiles is the
    owner's list of (expert, first slot, rows); the shared expert (id E) covers the
    rank's own n_local tokens stored after the received rows.
    """
    world, E = counts_all.shape
    eloc = E // world
    tot = counts_all.sum(axis=0)
    before = counts_all[:me].sum(axis=0) if me > 0 else np.zeros(E, np.int64)
    estart = np.zeros(E, np.int64)
    for d in range(world):
        seg = tot[d * eloc:(d + 1) * eloc]
        estart[d * eloc:(d + 1) * eloc] = np.concatenate([[0], np.cumsum(seg)[:-1]])
    base_send = estart + before
    total_recv = int(tot[me * eloc:(me + 1) * eloc].sum())
    tiles: List[Tuple[int, int, int]] = []
    for i in range(eloc):
        e = me * eloc + i
        c = int(tot[e])
        for j in range(0, c, tile):
            tiles.append((e, int(estart[e]) + j, min(tile, c - j)))
    for j in range(0, n_local, tile):
        tiles.append((E, total_recv + j, min(tile, n_local - j)))
    return base_send.astype(np.int64), total_recv, tiles


def exchange_handles(handle: bytes) -> bytes:
    """All-gathers the 64-byte buffer handles in rank order with torch.distributed."""
    import torch.distributed as dist
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, handle)
    return b"".join(out)
