"""Several GPUs: one process and one context per GPU, NCCL exchange inside the library.

Runs only where at least two GPUs are visible.  Every rank loads a slice of each input, all
ranks run the same plan, and the gathered shards must equal the CPU oracle's single-rank result
bit for bit; shards must be disjoint and the derived-tuple count must be the global one.

Every program runs in each way the library evaluates a component on several ranks:
  replicated   heads of a small dense domain live on every rank as bitmaps; one OR of the ranks'
               candidate bitmaps per iteration (the default for these small inputs);
  sliced       the same with the large stored relation left in slices (forced here by lowering
               the size from which a relation counts as large);
  broadcast    hash-partitioned heads, stored relations copied to every rank (XLB_FLAG_NO_DENSE
               switches the bitmaps off);
  shuffle      everything hash-partitioned, an all-to-all per join step (XLB_FLAG_SHUFFLE_ONLY);
               once more with the heads kept as hash sets (bitmaps off), and once with neither, so
               that candidates are sorted and subtracted by merging; and once with a small bound
               on join candidates, so that the ranks agree on several chunks per rule variant.
"""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _triangle_plan():
    from xlog_b200 import _abi as A
    from xlog_b200.plan import CompiledRule, ExecutionPlan, Join, Project, Scan, Scc
    body = Project(Join(Join(Scan(0), Scan(0), [1], [0]), Scan(0), [3, 0], [0, 1]), [0])   # tri(X): nodes on a triangle
    return ExecutionPlan([Scc(0, False, [CompiledRule("tri", body, (A.U32,))])], {"edge": 0, "tri": 1})


def _cases():
    from xlog_b200 import programs, workloads
    c0, c1 = workloads.uniform_digraph(400, 1500, 13)
    r0, r1 = workloads.rmat_graph(13, 16)
    t0, t1, _ = workloads.tree_dag(800, 0.05, 9)
    return [
        ("tc", programs.transitive_closure(), {"edge": [c0, c1]}, "reach"),
        ("tc_nonlinear", programs.transitive_closure_nonlinear(), {"edge": [c0[:600], c1[:600]]}, "reach"),
        ("tc_left", programs.transitive_closure_left_linear(), {"edge": [c0[:600], c1[:600]]}, "reach"),
        ("reach0", programs.reach_from_source(0), {"edge": [r0, r1]}, "r"),
        ("sg", programs.same_generation(), {"edge": [t0, t1]}, "sg"),
        ("andersen", programs.andersen(), {k: list(v) for k, v in workloads.andersen_program(0.0002).items()}, "pt"),
        ("triangle", _triangle_plan(), {"edge": [c0, c1]}, "tri"),
        ("negation", programs.unreachable_nodes(int(c0[0])), {"edge": [c0, c1], "node": [np.arange(400, dtype=np.uint32)]}, "un"),
    ]


def _modes():
    """(name, context flags, XLB_REPL_SLICE_MIN or None, join_chunk_tuples)"""
    from xlog_b200 import _abi as A
    return [("replicated", 0, None, 0), ("sliced", 0, "64", 0), ("broadcast", A.FLAG_NO_DENSE, None, 0),
            ("shuffle", A.FLAG_SHUFFLE_ONLY, None, 0), ("shuffle_set", A.FLAG_SHUFFLE_ONLY | A.FLAG_NO_DENSE, None, 0),
            ("shuffle_sorted", A.FLAG_SHUFFLE_ONLY | A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET, None, 0),
            # a small bound on join candidates: from the second iteration on the ranks agree on several
            # chunks per rule variant, and every rank runs that many rounds of exchanges
            ("shuffle_chunked", A.FLAG_SHUFFLE_ONLY | A.FLAG_NO_DENSE, None, 1500)]


def _rank_main(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("XLB_COMM_TIMEOUT_S", "60")
    import torch
    import torch.distributed as dist
    from xlog_b200 import dist as D
    from xlog_b200.executor import Executor
    from xlog_b200.provider import KernelProvider

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        results = {}
        for mode, flags, slice_min, chunk in _modes():
          if slice_min is None:
              os.environ.pop("XLB_REPL_SLICE_MIN", None)
          else:
              os.environ["XLB_REPL_SLICE_MIN"] = slice_min
          for case, plan, inputs, out in _cases():
            name = f"{mode}/{case}"
            prov = KernelProvider(device=rank, flags=flags, join_chunk_tuples=chunk)
            D.init_comm(prov, rank, world)
            ex = Executor(prov)
            for rel, rid in plan.rel_ids.items():
                ex.register_relation(rid, rel)
            for rel, cols in inputs.items():
                lo, hi = D.shard_bounds(len(cols[0]), rank, world)
                ex.put_relation(rel, prov.create_buffer_from_slices([np.asarray(c)[lo:hi] for c in cols]))
            stats = ex.execute_plan(plan)
            shard = prov.download(ex.get(out))
            sizes = [None] * world
            dist.all_gather_object(sizes, len(shard[0]))
            full = D.gather_shards(shard)
            if rank == 0:
                results[name] = {"cols": full, "sizes": sizes, "derived": stats["derived_tuples"],
                                 "iterations": stats["iterations"], "exchange_bytes": stats["exchange_bytes"]}
            prov.close()
        if rank == 0:
            np.save(os.path.join(out_dir, "results.npy"), results, allow_pickle=True)
    finally:
        dist.destroy_process_group()


def test_sharded_fixpoints_match_the_oracle(oracle, tmp_path):
    import torch
    import torch.multiprocessing as mp
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    results = np.load(tmp_path / "results.npy", allow_pickle=True).item()
    for case, plan, inputs, out in _cases():
      want, ex = oracle.run_program(plan, inputs, [out])
      for mode, _, _, _ in _modes():
        name = f"{mode}/{case}"
        if name not in results:
            continue
        got = results[name]
        assert len(got["cols"]) == len(want[out])
        for g, w in zip(got["cols"], want[out]):
            assert np.array_equal(g, w), f"{name}: gathered shards differ from the oracle"
        assert sum(got["sizes"]) == len(want[out][0]), f"{name}: shards overlap"
        if case != "negation":      # derived_tuples counts every head of the plan; that plan has three
            assert got["derived"] == len(want[out][0]), name
        if case not in ("negation", "triangle"):
            assert got["iterations"] == ex.iterations, f"{name}: the ranks stopped in another round than one rank does"
        assert got["exchange_bytes"] > 0, name


def _rank_wide(rank, world, port, out_dir, scale):
    import sys
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("XLB_COMM_TIMEOUT_S", "60")
    import torch
    import torch.distributed as dist
    from xlog_b200 import dist as D
    from xlog_b200 import programs, workloads
    from xlog_b200.executor import Executor
    from xlog_b200.provider import KernelProvider

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c0, c1 = workloads.rmat_dag(scale, 8)
        plan = programs.transitive_closure()
        prov = KernelProvider(device=rank, profile=True)
        D.init_comm(prov, rank, world)
        prov.profile_enable("*")
        ex = Executor(prov)
        for rel, rid in plan.rel_ids.items():
            ex.register_relation(rid, rel)
        lo, hi = D.shard_bounds(len(c0), rank, world)
        ex.put_relation("edge", prov.create_buffer_from_slices([c0[lo:hi], c1[lo:hi]]))
        stats = ex.execute_plan(plan)
        mine = {"digest": prov.checksum(ex.get("reach")), "derived": stats["derived_tuples"], "kernels": sorted(prov.profile_read())}
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        prov.close()
        if rank == 0:
            np.save(os.path.join(out_dir, "wide.npy"), everyone, allow_pickle=True)
    finally:
        dist.destroy_process_group()


def test_closure_over_a_domain_of_28_bits_on_several_ranks(tmp_path):
    # hash-partitioned heads that move from hash sets to bitmaps of their own shard once an
    # iteration brings enough candidates: the shards' digests must add up to the digest of the
    # closure computed on the host from bit rows, and the marking join must have run
    import torch
    import torch.multiprocessing as mp
    from xlog_b200 import digest, workloads
    n_gpus = torch.cuda.device_count()
    if n_gpus < 2:
        pytest.skip("needs at least two GPUs")
    scale, world = 14, 2
    mp.spawn(_rank_wide, args=(world, _free_port(), str(tmp_path), scale), nprocs=world, join=True)
    got = np.load(tmp_path / "wide.npy", allow_pickle=True).tolist()

    c0, c1 = workloads.rmat_dag(scale, 8)
    n = 1 << scale
    rows = np.zeros((n, n // 64), dtype=np.uint64)
    order = np.argsort(c0, kind="stable")
    dst, starts = c1[order], np.searchsorted(c0[order], np.arange(n + 1))
    for v in range(n - 1, -1, -1):
        kids = dst[starts[v]:starts[v + 1]]
        if len(kids):
            row = np.bitwise_or.reduce(rows[kids], axis=0)
            np.bitwise_or.at(row, kids >> 6, np.uint64(1) << (kids & 63).astype(np.uint64))
            rows[v] = row
    bits = np.unpackbits(rows.view(np.uint8), axis=1, bitorder="little")
    a, b = np.nonzero(bits)
    want = digest.result_checksum([a.astype(np.uint32), b.astype(np.uint32)])
    assert digest.checksum_text([g["digest"] for g in got]) == digest.checksum_text([want])
    assert all(g["derived"] == len(a) for g in got)
    assert all("expand_mark" in g["kernels"] for g in got)
