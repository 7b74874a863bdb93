#!/usr/bin/env python
"""Benchmark of the semi-naive fixpoint data plane.

  python bench.py --gpus N --steps K --warmup W            # the CUDA path (libxlb.so)
  python bench.py --impl reference --steps K --warmup W    # the CPU restatement of the reference

Headline workload (config 2): single-source reachability r(Y) :- edge(0,Y). r(Z) :- r(Y), edge(Y,Z).
over a seeded R-MAT graph, scale 20, edge factor 16 (a=.57 b=.19 c=.19 d=.05), self-loops and
duplicates removed.  One step is one complete fixpoint: from the edge relation resident as
column-major u32 columns to the final relation, sorted, on the device.  Metric: derived tuples per
second (final tuple count divided by the fixpoint time).  With N > 1 ranks every rank holds 1/N of
the edge rows (total work fixed: strong scaling).

The same line carries a `secondary` object: the full transitive closure of the banded R-MAT DAG of
config 5 at a reduced scale (16 instead of 24: the stated scale derives about 5e12 tuples), which
is the workload that runs the join probes and expansions, the wide-bitmap and hash-set dedup, the
radix sort and, on several ranks, the tuple exchange.  It reports its own time, the per-iteration
exchange, the rooflines of `radix_scatter`, `hash_probe` and `expand_mark` (whichever of them the
evaluation mode at hand launches), and a checksum of the result that is the same at every N.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
# stdout carries exactly one JSON line: everything else that libraries print there (NCCL's version
# banner, for one) is sent to stderr by pointing file descriptor 1 at stderr until the line is due
_REAL_STDOUT = os.dup(1)
os.dup2(2, 1)


def emit(line: dict) -> None:
    sys.stdout.flush()
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


METRIC = "derived_tuples_per_sec"
UNIT = "tuples/s"
L2_NOTE = "256 MB buffer written between steps"
TIMING_NOTE = "CUDA events on the library's stream around xlb_execute_plan, max over ranks"
# algorithmic bytes per launch are counted by the library (xlb_profile_read); the DRAM traffic of
# one launch was measured with ncu on a small case of the same kernel and grows with the rows of a
# launch, so it is scaled from the algorithmic bytes: the summary that holds the capture is named
TRAFFIC = {"radix_scatter": (13.2 / 16.0, "profiles/radix_scatter_sort_16M_keys.md"),
           "scan_join_mark": (0.90, "profiles/frontier_scan_c2.md")}


def make_workload(name: str, scale: int):
    from xlog_b200 import programs, workloads
    if name == "c2":
        c0, c1 = workloads.rmat_graph(scale, 16)
        return programs.reach_from_source(0), {"edge": [c0, c1]}, "r", \
            f"single-source reachability, R-MAT scale {scale} edge factor 16 ({len(c0)} edges)"
    if name == "c1":
        c0, c1 = workloads.uniform_digraph()
        return programs.transitive_closure(), {"edge": [c0, c1]}, "reach", "transitive closure, 2000 nodes / 10000 uniform edges"
    if name == "c5":
        c0, c1 = workloads.rmat_dag(scale, 8)
        return programs.transitive_closure(), {"edge": [c0, c1]}, "reach", \
            f"transitive closure, banded R-MAT DAG scale {scale} edge factor 8 ({len(c0)} edges)"
    if name == "c3":
        c0, c1, _ = workloads.tree_dag(scale, 0.05)
        return programs.same_generation(), {"edge": [c0, c1]}, "sg", \
            f"same generation, tree of {scale} nodes (2-6 children) plus 5% forward edges ({len(c0)} edges)"
    raise SystemExit(f"unknown workload {name}")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(gpu_index)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


from xlog_b200.digest import checksum_text, result_checksum  # noqa: E402


def roofline_of(prof: dict, kernel: str, peak: float, peak_kind: str):
    k = prof.get(kernel)
    if not k or k["ms"] <= 0 or not k["launches"]:
        return None
    achieved = k["bytes"] / (k["ms"] / 1e3) / 1e9
    per_alg, source = TRAFFIC.get(kernel, (None, None))
    return {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
            "frac": achieved / peak, "traffic": (k["bytes"] / k["launches"]) * per_alg if per_alg else None,
            "traffic_source": source, "launches": k["launches"], "avg_launch_us": 1e3 * k["ms"] / k["launches"],
            "algorithmic_bytes_per_launch": k["bytes"] / k["launches"]}


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's evaluation of the same program
    (the reference itself is Rust + CUDA and cannot be built without a Rust toolchain), on all
    host cores, timed by wall clock."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    plan, inputs, out_name, desc = make_workload(args.workload, args.scale)
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    times, derived, ex, out = [], 0, None, None
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        out, ex = O.run_program(plan, inputs, [out_name])
        dt = time.perf_counter() - t0
        derived = len(out[out_name][0])
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = derived / (ms / 1e3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u32", "data": "synthetic",
        "config": {"workload": desc, "derived_tuples": derived, "iterations": int(ex.iterations),
                   "candidate_tuples": int(ex.candidates), "l2": L2_NOTE, "timing": TIMING_NOTE},
        "checksum": checksum_text([result_checksum(out[out_name])]),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "the whole fixpoint of the same workload, once per step"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "secondary": None,
        "note": "wall clock of the CPU port of the reference's semi-naive loop (config keys l2 / timing describe the CUDA arm); "
                "the secondary workload is not run on the CPU port: its 9e8 join candidates take minutes there",
    }
    emit(line)


class Job:
    """One context on this rank's GPU with a workload loaded: runs device-resident and end-to-end
    steps of one fixpoint."""

    def __init__(self, env, workload: str, scale: int, flags: int = 0):
        import torch
        from xlog_b200.executor import Executor
        from xlog_b200.provider import KernelProvider
        self.env = env
        self.torch = torch
        self.plan, inputs, self.out_name, self.desc = make_workload(workload, scale)
        self.edge_name = next(iter(inputs))
        cols = inputs[self.edge_name]
        self.inputs = inputs
        n_rows = len(cols[0])
        lo, hi = n_rows * env.rank // env.world, n_rows * (env.rank + 1) // env.world
        # this rank's slice of the input, in pinned host memory (the end-to-end path copies from here)
        self.pinned = [torch.empty(hi - lo, dtype=torch.int32).pin_memory() for _ in cols]
        self.host_cols = []
        for t, c in zip(self.pinned, cols):
            a = t.numpy().view(np.uint32)
            a[:] = c[lo:hi]
            self.host_cols.append(a)
        self.prov = KernelProvider(device=env.local, flags=flags)
        if env.world > 1:
            from xlog_b200 import dist as D
            D.init_comm(self.prov, env.rank, env.world, device="cuda")
        self.ex = Executor(self.prov)
        for name, rid in self.plan.rel_ids.items():
            self.ex.register_relation(rid, name)
        self.master = self.prov.create_buffer_from_slices(self.host_cols)
        self.cplan = self.plan.compile()

    def _drop_result(self):
        try:
            self.ex.remove(self.out_name)
        except Exception:
            pass

    def device_step(self, salt: int = 1):
        self._drop_result()
        self.ex.put_relation(self.edge_name, self.prov.clone_buffer(self.master))
        self.env.flush.fill_(self.env.rank + salt)
        self.env.barrier()
        return self.ex.execute_plan(self.cplan)

    def e2e_step(self):
        """Host buffers in, host result out: the copies are inside the timed region."""
        self._drop_result()
        self.env.flush.fill_(self.env.rank + 3)
        self.env.barrier()
        t0 = time.perf_counter()
        self.ex.put_relation(self.edge_name, self.prov.create_buffer_from_slices(self.host_cols))
        self.ex.execute_plan(self.cplan)
        res = self.prov.download(self.ex.get(self.out_name))
        self.torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3, sum(c.nbytes for c in res)

    def result(self):
        return self.prov.download(self.ex.get(self.out_name))

    def result_digest(self):
        """Digest of this rank's shard, computed on the device (no download)."""
        buf = self.ex.get(self.out_name)
        return self.prov.checksum(buf), buf.num_rows()

    def close(self):
        self.prov.close()


class Env:
    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
        torch.cuda.set_device(self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, dtype=self.torch.float64, device="cuda")
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t

    def gather(self, obj):
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj)
        return out


def timed_steps(env, job, steps, kernels):
    """`steps` device-resident fixpoints with the launches of `kernels` bracketed by CUDA events."""
    job.prov.profile_enable(kernels)
    ms, host, stats, launches = [], [], None, 0
    env.barrier()
    for _ in range(steps):
        stats = job.device_step()
        host.append([round(stats["ms_host_total"], 3), round(stats["ms_host_wait"], 3), round(stats["ms_host_alloc"], 3)])
        ms.append(stats["ms_total"])
        launches += stats["kernel_launches"]
    env.barrier()
    prof = job.prov.profile_read()
    job.prov.profile_enable(None)
    return env.max_over_ranks(ms), host, stats, launches, prof


def secondary_block(env, args, peak, peak_kind, flags, label):
    """The sort / probe / exchange workload at reduced scale, in one evaluation mode."""
    from xlog_b200 import _abi as A
    job = Job(env, "c5", args.secondary_scale, flags | A.FLAG_PROFILE)   # phase timers on: they give the exchange time
    for _ in range(args.secondary_warmup):
        job.device_step()
    ms_t, _, stats, launches, prof = timed_steps(env, job, args.secondary_steps, "radix_scatter,hash_probe,expand_mark")
    ms = float(ms_t.mean().item())
    digest, shard_rows = job.result_digest()
    parts = env.gather((digest, shard_rows, stats["ms_exchange"], stats["exchange_bytes"],
                        stats["ms_sort"], stats["ms_join"], stats["ms_setops"]))
    job.close()
    if env.rank != 0:
        return None
    derived, iters = stats["derived_tuples"], max(stats["iterations"], 1)
    sizes = [p[1] for p in parts]
    ex_ms = [p[2] for p in parts]
    ex_bytes = [p[3] for p in parts]
    return {
        "mode": label,
        "workload": job.desc + " (config 5 at a reduced scale)",
        "metric": METRIC, "unit": UNIT, "value": derived / (ms / 1e3), "ms_per_step": ms,
        "steps": args.secondary_steps, "warmup": args.secondary_warmup, "ms_steps": [round(float(x), 3) for x in ms_t.tolist()],
        "derived_tuples": derived, "iterations": stats["iterations"], "candidate_tuples": stats["candidate_tuples"],
        "checksum": checksum_text([p[0] for p in parts]),
        "shards": {"max": max(sizes), "mean": sum(sizes) / len(sizes)},
        # device time between the events around every exchange step of the last timed fixpoint
        # (partition by owner, count all-gather, all-to-all, vote), and the bytes a rank sent
        "exchange": {"ms_per_step_max": max(ex_ms), "ms_per_step_mean": sum(ex_ms) / len(ex_ms),
                     "ms_per_iteration_max": max(ex_ms) / iters,
                     "bytes_sent_per_rank_per_iteration_max": max(ex_bytes) / iters,
                     "bytes_sent_per_rank_per_step_max": max(ex_bytes)},
        "phases_ms_rank0": {"sort": round(parts[0][4], 3), "join": round(parts[0][5], 3), "setops": round(parts[0][6], 3),
                            "exchange": round(parts[0][2], 3)},
        "gpu_launches": int(launches),
        "roofline": {k: roofline_of(prof, k, peak, peak_kind) for k in ("radix_scatter", "hash_probe", "expand_mark")},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="xlb", choices=["xlb", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c5"])
    ap.add_argument("--scale", type=int, default=20, help="R-MAT scale (c2, c5) or number of tree nodes (c3)")
    ap.add_argument("--kernel", default="auto",
                    help="kernel whose launches are timed for the roofline object (auto: the one with the most device time in the last warm-up step)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (large results)")
    ap.add_argument("--no-clocks", action="store_true", help="do not run nvidia-smi beside the timed region")
    ap.add_argument("--no-secondary", action="store_true", help="skip the reduced-scale config 5 block")
    ap.add_argument("--secondary-scale", type=int, default=16)
    ap.add_argument("--secondary-steps", type=int, default=5)
    ap.add_argument("--secondary-warmup", type=int, default=3)
    ap.add_argument("--shuffle-only", action="store_true", help="headline workload with XLB_FLAG_SHUFFLE_ONLY (several ranks: no replicated relations)")
    ap.add_argument("--flags", type=int, default=0, help="extra XLB_FLAG_* bits for the headline workload's context (A/B runs)")
    ap.add_argument("--phases", action="store_true", help="time the executor's phases with events (fills phases_last_step; adds event records to the timed steps)")
    ap.add_argument("--breakdown", action="store_true", help="extra untimed pass with every kernel timed, to stderr")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    if args.impl == "reference":
        run_reference(args)
        return

    from xlog_b200 import _abi as A
    env = Env(args)
    world, rank = env.world, env.rank
    flags = (A.FLAG_PROFILE if args.phases else 0) | (A.FLAG_SHUFFLE_ONLY if args.shuffle_only else 0) | args.flags
    job = Job(env, args.workload, args.scale, flags)
    prov = job.prov

    # ---- device-resident steps: warm-up, then K timed steps ---------------------------------
    # clocks are sampled from the first warm-up step to the last end-to-end step: the timed region
    # alone lasts tens of milliseconds, less than one nvidia-smi sampling period
    sampler = ClockSampler(env.local) if rank == 0 and not args.no_clocks else None
    if sampler:
        time.sleep(1.0)  # let nvidia-smi finish starting up: its first query stalls CUDA calls for milliseconds
    for w in range(args.warmup):
        if args.kernel == "auto" and w == args.warmup - 1:
            prov.profile_enable("*")  # untimed step: find the kernel that dominates this workload
        job.device_step()
    if args.kernel == "auto":
        seen = {k: v for k, v in prov.profile_read().items() if v["bytes"]}
        prov.profile_enable(None)
        mine = max(seen, key=lambda k: seen[k]["ms"]) if seen else "radix_scatter"
        args.kernel = env.gather(mine)[0]   # every rank times rank 0's choice
    ms_t, host_steps, stats, launches, prof = timed_steps(env, job, args.steps, args.kernel)
    ms_per_step = float(ms_t.mean().item())
    derived = stats["derived_tuples"]
    value = derived / (ms_per_step / 1e3)
    digest = checksum_text([p for p in env.gather(job.result_digest()[0])])  # computed on the device, shard by shard

    # ---- end to end: host buffers in, host result out, copies inside the timed region ------
    e2e_ms, d2h_bytes = [], 0
    for i in range(0 if args.no_e2e else args.warmup + args.steps):
        dt, d2h_bytes = job.e2e_step()
        if i >= args.warmup:
            e2e_ms.append(dt)
    clocks = sampler.stop() if sampler else None
    e2e_ms_per_step = float(env.max_over_ranks(e2e_ms).mean().item()) if e2e_ms else float("nan")

    if args.breakdown and rank == 0 and world == 1:
        prov.profile_enable("*")
        for _ in range(3):
            job.device_step()
        full = prov.profile_read()
        prov.profile_enable(None)
        tot = sum(v["ms"] for v in full.values())
        print(f"# kernel breakdown over 3 steps (device ms inside kernels: {tot:.3f}; steps took {3 * ms_per_step:.3f})", file=sys.stderr)
        for k, v in sorted(full.items(), key=lambda kv: -kv[1]["ms"]):
            gbs = v["bytes"] / v["ms"] / 1e6 if v["ms"] > 0 and v["bytes"] else 0.0
            print(f"#   {k:20s} launches {v['launches']:5d}  ms {v['ms']:9.3f}  share {100 * v['ms'] / tot:5.1f}%  alg GB/s {gbs:8.1f}", file=sys.stderr)

    h2d_bytes = int(sum(c.nbytes for c in job.host_cols))
    plan, inputs, out_name, desc = job.plan, job.inputs, job.out_name, job.desc
    job.close()

    peak, peak_kind = measured_peak_gbs()
    secondary = None
    if not args.no_secondary and args.workload == "c2":
        secondary = secondary_block(env, args, peak, peak_kind, 0, "one rank" if world == 1 else
                                    "stored relation copied to every rank, closure placed by its carried column: no tuple exchange")
        if world > 1:
            shuffle = secondary_block(env, args, peak, peak_kind, A.FLAG_SHUFFLE_ONLY,
                                      "hash-partitioned on the join key, all-to-all per iteration (XLB_FLAG_SHUFFLE_ONLY)")
            if rank == 0:
                secondary["shuffle"] = shuffle

    if rank != 0:
        if world > 1:
            env.dist.destroy_process_group()
        return

    roof = roofline_of(prof, args.kernel, peak, peak_kind)

    cpu = None
    if not args.no_cpu_baseline and world == 1:
        from oracle import oracle as O
        cores = os.cpu_count() or 1
        O.set_threads(cores)
        t0 = time.perf_counter()
        out, _ = O.run_program(plan, inputs, [out_name])
        dt = time.perf_counter() - t0
        cpu = {"value": len(out[out_name][0]) / dt, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": "one whole fixpoint of the same workload", "seconds": dt,
               "checksum": checksum_text([result_checksum(out[out_name])])}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u32", "data": "synthetic", "ms_steps": [round(float(x), 4) for x in ms_t.tolist()],
        "config": {"workload": desc, "derived_tuples": derived, "iterations": stats["iterations"],
                   "candidate_tuples": stats["candidate_tuples"], "l2": L2_NOTE, "timing": TIMING_NOTE},
        "checksum": digest,
        "e2e": None if args.no_e2e else {"value": derived / (e2e_ms_per_step / 1e3), "unit": UNIT, "ms_per_step": e2e_ms_per_step,
                                         "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": int(d2h_bytes)},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roof,
        "cpu_baseline": cpu,
        "host_last_step": {k: stats[k] for k in ("host_syncs", "ms_host_wait", "ms_host_total")},
        # device time per phase in the last step (rank 0; only with --phases, else zeros) and exchanged bytes
        "phases_last_step": {k: round(stats[k], 4) if isinstance(stats[k], float) else stats[k]
                             for k in ("ms_join", "ms_sort", "ms_setops", "ms_exchange", "exchange_bytes")},
        "host_ms_total_wait_alloc_per_step": host_steps,
        "secondary": secondary,
    }
    emit(line)
    if world > 1:
        env.dist.destroy_process_group()


if __name__ == "__main__":
    main()
