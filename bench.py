#!/usr/bin/env python
"""Benchmark of the semi-naive fixpoint data plane.

  python bench.py --gpus N --steps K --warmup W            # the CUDA path (libxlb.so)
  python bench.py --impl reference --steps K --warmup W    # the CPU restatement of the reference

Workload: single-source reachability r(Y) :- edge(0,Y). r(Z) :- r(Y), edge(Y,Z). over a seeded
R-MAT graph, scale 20, edge factor 16 (a=.57 b=.19 c=.19 d=.05), self-loops and duplicates removed.
One step is one complete fixpoint: from the edge relation resident as column-major u32 columns to
the final relation, sorted, on the device.  Metric: derived tuples per second (final tuple count
divided by the fixpoint time).  With N > 1 ranks every rank holds 1/N of the edge rows; relations
are hash-partitioned and exchanged by all-to-all inside the fixpoint (total work fixed: strong
scaling).  One JSON line is printed by rank 0.
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


def make_workload(args):
    from xlog_b200 import programs, workloads
    if args.workload == "c2":
        c0, c1 = workloads.rmat_graph(args.scale, 16)
        return programs.reach_from_source(0), {"edge": [c0, c1]}, "r", \
            f"single-source reachability, R-MAT scale {args.scale} edge factor 16 ({len(c0)} edges)"
    if args.workload == "c1":
        c0, c1 = workloads.uniform_digraph()
        return programs.transitive_closure(), {"edge": [c0, c1]}, "reach", "transitive closure, 2000 nodes / 10000 uniform edges"
    if args.workload == "c5":
        c0, c1 = workloads.rmat_dag(args.scale, 8)
        return programs.transitive_closure(), {"edge": [c0, c1]}, "reach", \
            f"transitive closure, banded R-MAT DAG scale {args.scale} edge factor 8 ({len(c0)} edges)"
    raise SystemExit(f"unknown workload {args.workload}")


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


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's evaluation of the same program
    (the reference itself is Rust + CUDA and cannot be built without a Rust toolchain), on all
    host cores, timed by wall clock."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    plan, inputs, out_name, desc = make_workload(args)
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    times, derived = [], 0
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
        "config": {"workload": desc, "derived_tuples": derived},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "the whole fixpoint of the same workload, once per step"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="xlb", choices=["xlb", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c5"])
    ap.add_argument("--scale", type=int, default=20)
    ap.add_argument("--kernel", default="auto",
                    help="kernel whose launches are timed for the roofline object (auto: the one with the most device time in the last warm-up step)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (large results)")
    ap.add_argument("--no-clocks", action="store_true", help="do not run nvidia-smi beside the timed region")
    ap.add_argument("--phases", action="store_true", help="time the executor's phases with events (fills phases_last_step; adds event records to the timed steps)")
    ap.add_argument("--breakdown", action="store_true", help="extra untimed pass with every kernel timed, to stderr")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from xlog_b200.executor import Executor
    from xlog_b200.provider import KernelProvider
    from xlog_b200 import _abi as A

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    plan, inputs, out_name, desc = make_workload(args)
    edge_name = next(iter(inputs))
    cols = inputs[edge_name]
    n_rows = len(cols[0])
    lo, hi = n_rows * rank // world, n_rows * (rank + 1) // world
    # this rank's slice of the input, in pinned host memory (the end-to-end path copies from here)
    pinned = [torch.empty(hi - lo, dtype=torch.int32).pin_memory() for _ in cols]
    host_cols = []
    for t, c in zip(pinned, cols):
        a = t.numpy().view(np.uint32)
        a[:] = c[lo:hi]
        host_cols.append(a)

    prov = KernelProvider(device=local, flags=A.FLAG_PROFILE if args.phases else 0)
    if world > 1:
        from xlog_b200 import dist as D
        D.init_comm(prov, rank, world, device="cuda")

    ex = Executor(prov)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    master = prov.create_buffer_from_slices(host_cols)
    cplan = plan.compile()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2

    def reset_store():
        try:
            ex.remove(out_name)
        except Exception:
            pass
        ex.put_relation(edge_name, prov.clone_buffer(master))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def device_step():
        reset_store()
        flush.fill_(rank + 1)
        barrier()
        return ex.execute_plan(cplan)

    # ---- device-resident steps: warm-up, then K timed steps ---------------------------------
    # clocks are sampled from the first warm-up step to the last end-to-end step: the timed region
    # alone lasts tens of milliseconds, less than one nvidia-smi sampling period
    sampler = ClockSampler(local) if rank == 0 and not args.no_clocks else None
    if sampler:
        time.sleep(1.0)  # let nvidia-smi finish starting up: its first query stalls CUDA calls for milliseconds
    for w in range(args.warmup):
        if args.kernel == "auto" and w == args.warmup - 1:
            prov.profile_enable("*")  # untimed step: find the kernel that dominates this workload
        device_step()
    if args.kernel == "auto":
        seen = {k: v for k, v in prov.profile_read().items() if v["bytes"]}
        prov.profile_enable(None)
        args.kernel = max(seen, key=lambda k: seen[k]["ms"]) if seen else "radix_scatter"
    prov.profile_enable(args.kernel)
    ms_steps, host_steps, stats = [], [], None
    launches = 0
    barrier()
    for _ in range(args.steps):
        stats = device_step()
        host_steps.append([round(stats["ms_host_total"], 3), round(stats["ms_host_wait"], 3), round(stats["ms_host_alloc"], 3)])
        ms_steps.append(stats["ms_total"])
        launches += stats["kernel_launches"]
    barrier()
    prof = prov.profile_read()
    prov.profile_enable(None)
    ms_t = torch.tensor(ms_steps, dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms_t.mean().item())
    derived = stats["derived_tuples"]
    value = derived / (ms_per_step / 1e3)

    # ---- end to end: host buffers in, host result out, copies inside the timed region ------
    e2e_ms, d2h_bytes = [], 0
    for i in range(0 if args.no_e2e else args.warmup + args.steps):
        try:
            ex.remove(out_name)
        except Exception:
            pass
        flush.fill_(rank + 3)
        barrier()
        t0 = time.perf_counter()
        ex.put_relation(edge_name, prov.create_buffer_from_slices(host_cols))
        ex.execute_plan(cplan)
        res = prov.download(ex.get(out_name))
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) * 1e3
        d2h_bytes = sum(c.nbytes for c in res)
        if i >= args.warmup:
            e2e_ms.append(dt)
    clocks = sampler.stop() if sampler else None
    e2e_t = torch.tensor(e2e_ms, dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = float(e2e_t.mean().item()) if e2e_ms else float("nan")

    if args.breakdown and rank == 0 and world == 1:
        prov.profile_enable("*")
        for _ in range(3):
            device_step()
        full = prov.profile_read()
        prov.profile_enable(None)
        tot = sum(v["ms"] for v in full.values())
        print(f"# kernel breakdown over 3 steps (device ms inside kernels: {tot:.3f}; steps took {3 * ms_per_step:.3f})", file=sys.stderr)
        for k, v in sorted(full.items(), key=lambda kv: -kv[1]["ms"]):
            gbs = v["bytes"] / v["ms"] / 1e6 if v["ms"] > 0 and v["bytes"] else 0.0
            print(f"#   {k:20s} launches {v['launches']:5d}  ms {v['ms']:9.3f}  share {100 * v['ms'] / tot:5.1f}%  alg GB/s {gbs:8.1f}", file=sys.stderr)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak_gbs()
    roof = None
    k = prof.get(args.kernel)
    if k and k["ms"] > 0 and k["launches"]:
        achieved = k["bytes"] / (k["ms"] / 1e3) / 1e9
        # DRAM bytes per launch: ncu captures of these kernels measured 13.2 B per key against 16
        # algorithmic for one radix pass over 16 M keys, and 1.0 x the algorithmic bytes for the
        # scan join over the 16 M edge rows; both grow with the rows of a launch, so they are
        # scaled to the rows an average launch of this run processed
        per_alg = {"radix_scatter": 13.2 / 16.0, "scan_join_mark": 1.0}.get(args.kernel)
        traffic = (k["bytes"] / k["launches"]) * per_alg if per_alg else None
        roof = {"bound": "hbm", "kernel": args.kernel, "achieved": achieved, "peak": peak, "peak_kind": peak_kind,
                "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                "launches": k["launches"], "avg_launch_us": 1e3 * k["ms"] / k["launches"],
                "algorithmic_bytes_per_launch": k["bytes"] / k["launches"]}

    cpu = None
    if not args.no_cpu_baseline and world == 1:
        from oracle import oracle as O
        cores = os.cpu_count() or 1
        O.set_threads(cores)
        t0 = time.perf_counter()
        out, _ = O.run_program(plan, inputs, [out_name])
        dt = time.perf_counter() - t0
        cpu = {"value": len(out[out_name][0]) / dt, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": "one whole fixpoint of the same workload", "seconds": dt}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u32", "data": "synthetic", "ms_steps": [round(float(x), 4) for x in ms_t.tolist()],
        "config": {"workload": desc, "derived_tuples": derived, "iterations": stats["iterations"],
                   "candidate_tuples": stats["candidate_tuples"], "l2": "256 MB buffer written between steps",
                   "timing": "CUDA events on the library's stream around xlb_execute_plan, max over ranks"},
        "e2e": None if args.no_e2e else {"value": derived / (e2e_ms_per_step / 1e3), "unit": UNIT, "ms_per_step": e2e_ms_per_step,
                                         "h2d_bytes_per_step": int(sum(c.nbytes for c in host_cols)), "d2h_bytes_per_step": int(d2h_bytes)},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roof,
        "cpu_baseline": cpu,
        "host_last_step": {k: stats[k] for k in ("host_syncs", "ms_host_wait", "ms_host_total")},
        # device time per phase in the last step (rank 0; only with XLB_FLAG_PROFILE, else zeros) and exchanged bytes
        "phases_last_step": {k: round(stats[k], 4) if isinstance(stats[k], float) else stats[k]
                             for k in ("ms_join", "ms_sort", "ms_setops", "ms_exchange", "exchange_bytes")},
        "host_ms_total_wait_alloc_per_step": host_steps,
    }
    emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
