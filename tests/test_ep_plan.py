"""CPU, two gloo ranks: the expert-parallel partition / slot-offset logic."""
import os
import sys

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    from moe_infer_b200 import ep
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    E, K, n = 16, 4, 23 + 9 * rank
    rng = np.random.default_rng(100 + rank)
    idx = np.stack([rng.choice(E, size=K, replace=False) for _ in range(n)])
    counts = np.bincount(idx.ravel(), minlength=E).astype(np.int64)
    gathered = [None] * world
    dist.all_gather_object(gathered, counts)
    counts_all = np.stack(gathered)
    base_send, total_recv, tiles = ep.plan(counts_all, rank, n, tile=8)
    # every (token, k) row gets a slot at its owner: collect (owner, slot, expert) triples from all ranks
    cursor = np.zeros(E, np.int64)
    rows = []
    for e in idx.ravel():
        rows.append((ep.owner_of(int(e), E, world), int(base_send[e] + cursor[e]), int(e)))
        cursor[e] += 1
    all_rows = [None] * world
    dist.all_gather_object(all_rows, rows)
    mine = sorted((s, e) for rr in all_rows for (o, s, e) in rr if o == rank)
    ok = [s for s, _ in mine] == list(range(total_recv))                      # slots are a permutation of 0..total-1
    ok = ok and all(mine[i][1] <= mine[i + 1][1] for i in range(len(mine) - 1))  # grouped by expert
    covered = np.zeros(total_recv + n, bool)
    for e, s0, c in tiles:
        ok = ok and c <= 8 and not covered[s0:s0 + c].any()
        covered[s0:s0 + c] = True
        if e < E:
            ok = ok and all(ex == e for (s, ex) in mine[s0:s0 + c]) and ep.owner_of(e, E, world) == rank
    ok = ok and covered.all()
    handles = ep.exchange_handles(bytes([rank]) * 64)
    ok = ok and handles == b"".join(bytes([r]) * 64 for r in range(world))
    ret[rank] = bool(ok)
    dist.destroy_process_group()


def test_ep_plan_two_gloo_ranks():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
