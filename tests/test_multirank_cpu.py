"""The several-rank scheme on CPU ranks (gloo, world size 2 and 3).

No GPU is present here, so the ranks run the same partitioned semi-naive evaluation the library
runs with world > 1 — relations hash-partitioned on the join key, one exchange per join step,
head tuples sent to their home rank, an all-reduced emptiness vote — with the CPU oracle as each
rank's operator engine and xlog_b200.dist as the exchange layer.  The gathered shards must equal
the single-rank result, shards must be disjoint, and every tuple must sit on its owner.
"""
import os
import socket

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _pack(c0, c1):
    return (c0.astype(np.uint64) << np.uint64(32)) | c1.astype(np.uint64)


def _rank_main(rank, world, port, edges, out_dir):
    import sys
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    from oracle import oracle as O
    from xlog_b200 import dist as D

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c0, c1 = edges
        lo, hi = D.shard_bounds(len(c0), rank, world)
        mine = _pack(c0[lo:hi], c1[lo:hi])
        M = np.uint64(0xFFFFFFFF)
        S = np.uint64(32)
        # edge index: partitioned by its join column (column 0)
        edge = np.unique(D.exchange_by_owner(mine, mine >> S, world))
        assert np.all(D.owner_of(edge >> S, world) == rank)
        erel = O.OracleRel.from_columns([(edge >> S).astype(np.uint32), (edge & M).astype(np.uint32)])
        # reach is homed on column 1, the column its delta is probed by
        seed = np.unique(D.exchange_by_owner(mine, mine & M, world))
        full = seed
        delta = seed
        iters = 0
        while True:
            iters += 1
            # delta rows already sit on owner(Y): the join with edge(Y, Z) is local
            drel = O.OracleRel.from_columns([(delta >> S).astype(np.uint32), (delta & M).astype(np.uint32)])
            j = O.hash_join(drel, erel, [1], [0]).columns()
            cand = _pack(j[0], j[3]) if len(j[0]) else np.zeros(0, np.uint64)
            cand = D.exchange_by_owner(cand, cand & M, world)          # to the home rank of (X, Z)
            novel = np.setdiff1d(np.unique(cand), full, assume_unique=True)
            if D.allreduce_sum(len(novel)) == 0:
                break
            full = np.union1d(full, novel)
            delta = novel
            assert iters < 1000
        assert np.all(D.owner_of(full & M, world) == rank)
        got = D.gather_shards([(full >> S).astype(np.uint32), (full & M).astype(np.uint32)])
        sizes = [None] * world
        dist.all_gather_object(sizes, len(full))
        if rank == 0:
            np.savez(os.path.join(out_dir, "out.npz"), c0=got[0], c1=got[1], sizes=np.array(sizes), iters=iters)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_partitioned_fixpoint_equals_single_rank(oracle, tmp_path, world):
    from xlog_b200 import programs, workloads
    c0, c1 = workloads.uniform_digraph(120, 300, 11)
    want, ex = oracle.run_program(programs.transitive_closure(), {"edge": [c0, c1]}, ["reach"])
    mp.spawn(_rank_main, args=(world, _free_port(), (c0, c1), str(tmp_path)), nprocs=world, join=True)
    out = np.load(tmp_path / "out.npz")
    assert np.array_equal(out["c0"], want["reach"][0]) and np.array_equal(out["c1"], want["reach"][1])
    assert int(out["sizes"].sum()) == len(want["reach"][0])      # shards are disjoint
    assert int(out["iters"]) == ex.iterations                     # the vote ends every rank in the same round


def _bad_count_rank(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    from xlog_b200 import dist as D

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows = np.arange(100 * rank, 100 * rank + 50, dtype=np.uint64)
        wrong = None
        if rank == 1:                      # this rank claims one row more for rank 0 than it has
            wrong = np.bincount(D.owner_of(rows, world), minlength=world)
            wrong[0] += 1
        try:
            D.exchange_by_owner(rows, rows, world, _send_counts=wrong)
            outcome = "exchanged"
        except D.ExchangeCountError as e:
            outcome = str(e)
        # the ranks are still in step: a second, correct exchange goes through
        got = D.exchange_by_owner(rows, rows, world)
        assert np.all(D.owner_of(got, world) == rank)
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write(outcome)
    finally:
        dist.destroy_process_group()


def test_a_wrong_send_count_fails_every_rank_the_same_way(tmp_path):
    """Failure made on the host: one rank's count row does not add up.  Every rank must see it in
    the gathered matrix and raise before the all-to-all, none may hang, and the group stays usable."""
    world = 3
    mp.spawn(_bad_count_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    outcomes = [open(tmp_path / f"rank{r}.txt").read() for r in range(world)]
    assert all("rank(s) [1]" in o for o in outcomes), outcomes
