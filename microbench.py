"""Kernel microbenchmarks through the C ABI: one operator on seeded keys, every kernel timed with
CUDA events (xlb_profile_enable) and reported against its algorithmic bytes.

  python microbench.py sort  --rows 32000000 --bits 32
  python microbench.py setops --rows 32000000 --bits 24
  python microbench.py join  --rows 16000000 --bits 20 --probe 4000000

These are the small cases that ncu captures of single kernels run; the figures the benchmark
reports come from bench.py.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from xlog_b200.provider import KernelProvider  # noqa: E402
from xlog_b200.workloads import splitmix64  # noqa: E402


def _cols(n, bits, seed):
    sh = np.uint64(64 - bits)
    return [(splitmix64(seed, 0, n) >> sh).astype(np.uint32), (splitmix64(seed + 1, 0, n) >> sh).astype(np.uint32)]


def _peak():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _report(prof, reps):
    peak, kind = _peak()
    tot = sum(v["ms"] for v in prof.values())
    print(f"{'kernel':18s} {'launches':>8s} {'us/launch':>10s} {'share':>6s} {'alg GB/s':>9s} {'of ' + kind + ' peak':>16s}")
    for k, v in sorted(prof.items(), key=lambda kv: -kv[1]["ms"]):
        if not v["launches"]:
            continue
        gbs = v["bytes"] / v["ms"] / 1e6 if v["ms"] > 0 and v["bytes"] else 0.0
        frac = f"{gbs / peak:6.3f}" if gbs else "     -"
        print(f"{k:18s} {v['launches'] // reps:8d} {1e3 * v['ms'] / v['launches']:10.1f} {100 * v['ms'] / tot:5.1f}% {gbs:9.1f} {frac:>16s}")
    print(f"device time in kernels per repetition: {tot / reps:.3f} ms")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["sort", "setops", "join"])
    ap.add_argument("--rows", type=float, default=3.2e7)
    ap.add_argument("--bits", type=int, default=32, help="random bits per 32-bit column")
    ap.add_argument("--probe", type=float, default=4e6)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args()
    n = int(args.rows)
    p = KernelProvider(device=args.device)
    a = p.create_buffer_from_slices(_cols(n, args.bits, 1))

    if args.what == "sort":            # full-row dedup = radix sort + adjacent-compare compaction
        def run():
            return [p.dedup(a)]
    elif args.what == "setops":        # difference and union of two canonical relations
        da = p.dedup(a)
        db = p.dedup(p.create_buffer_from_slices(_cols(n // 4, args.bits, 7)))

        def run():
            return [p.diff_gpu(da, db), p.union_gpu(da, db)]
    else:                              # hash join: build on `a` column 0, probe with --probe rows
        m = int(args.probe)
        b = p.create_buffer_from_slices(_cols(m, args.bits, 11))

        def run():
            return [p.hash_join_v2(b, a, [1], [0])]

    for _ in range(2):
        for o in run():
            o.free()
    p.profile_enable("*")
    outs = []
    for i in range(args.reps):
        for o in outs:
            o.free()
        outs = run()
    prof = p.profile_read()
    p.profile_enable(None)
    print(f"{args.what}: rows {n}, {args.bits} random bits per column, output rows {[o.num_rows() for o in outs]}")
    _report(prof, args.reps)
    if args.what == "sort" and n <= 40_000_000:
        cols = p.download(outs[0])
        k = (cols[0].astype(np.uint64) << np.uint64(32)) | cols[1]
        assert np.all(k[1:] > k[:-1]), "result is not sorted and unique"
        print("checked: sorted and unique")
    p.close()


if __name__ == "__main__":
    main()
