#!/usr/bin/env python
"""Writes tests/golden/operators.json, tests/golden/programs.json and tests/golden/groupby.json.

Every case is a known-answer test transcribed from the reference's own test suite (cited per
case by path inside the reference project).  Operator cases carry the literal inputs and the
literal expected outputs the reference asserts.  Program cases carry the reference's literal
input facts; where the reference test states the expected rows they are copied, and where it
computes them with an in-test oracle (a BTreeSet closure), `expected` is computed here by
`naive_fixpoint`, an independent, deliberately simple Python evaluator of the same rules
(`expected_source` says which).  Nothing in this script uses the repository's oracle or CUDA
code, so the fixtures can pin both.

Run:  python tests/golden/make_golden.py
"""
import itertools
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
SO = "crates/xlog-cuda/tests/set_ops_tests.rs"
FR = "crates/xlog-cuda/tests/test_full_row_set_algebra.rs"
JV = "crates/xlog-cuda/tests/join_v2_tests.rs"
JC = "crates/xlog-cuda/tests/join_collision_test.rs"
ST = "crates/xlog-cuda/tests/sort_tests.rs"
GB = "crates/xlog-cuda/tests/groupby_tests.rs"
SD = "crates/xlog-cuda/tests/test_sort_dedup_u64.rs"
TCOV = "crates/xlog-cuda/tests/type_coverage_tests.rs"


def rows1(xs):
    return [[x] for x in xs]


def operators():
    c = []

    def add(op, cite, expected, **kw):
        c.append({"op": op, "cite": cite, "expected": expected, **kw})

    # ---- sort (stable, lexicographic) ----------------------------------------------------------
    add("sort", ST + ":7-25", rows1([1, 2, 3, 5, 8, 9]), types=["u32"], a=rows1([5, 2, 8, 1, 9, 3]), keys=[0])
    add("sort", ST + ":28-54", [[1, 10], [2, 20], [3, 30]], types=["u32", "u32"], a=[[3, 30], [1, 10], [2, 20]], keys=[0])
    add("sort", ST + ":57-68", [], types=["u32"], a=[], keys=[0])
    add("sort", ST + ":71-87", rows1([1, 2, 3, 4, 5]), types=["u32"], a=rows1([1, 2, 3, 4, 5]), keys=[0])
    add("sort", ST + ":90-108", rows1([1, 1, 2, 2, 3, 3]), types=["u32"], a=rows1([3, 1, 2, 1, 3, 2]), keys=[0])
    add("sort", ST + ":136-154", rows1([1, 2, 3, 4, 5]), types=["u32"], a=rows1([5, 4, 3, 2, 1]), keys=[0])
    # ---- full-row dedup matrix on (u32, u32) ---------------------------------------------------
    t2 = ["u32", "u32"]
    add("dedup", FR + ":63-69", [[1, 10], [2, 20], [3, 30]], types=t2, a=[[1, 10], [2, 20], [3, 30]])
    add("dedup", FR + ":71-77", [[1, 10]], types=t2, a=[[1, 10], [1, 10], [1, 10]])
    add("dedup", FR + ":79-85", [[1, 10], [1, 20], [2, 20]], types=t2, a=[[1, 10], [1, 10], [1, 20], [2, 20], [2, 20]])
    add("dedup", FR + ":87-95", [[1, 10], [1, 20], [1, 30]], types=t2, a=[[1, 10], [1, 20], [1, 30]])
    add("dedup", FR + ":97-105", [], types=t2, a=[])
    add("dedup", FR + ":107-113", [[7, 8]], types=t2, a=[[7, 8]])
    # ---- full-row difference on (u32, u32) -----------------------------------------------------
    add("diff", FR + ":119-127", [[1, 20]], types=t2, a=[[1, 10], [1, 10], [1, 20]], b=[[1, 10]])
    add("diff", FR + ":129-139", [[1, 20], [2, 30]], types=t2, a=[[1, 20], [1, 20], [2, 30]], b=[[1, 10]])
    add("diff", FR + ":141-148", [], types=t2, a=[[1, 10], [2, 20]], b=[[2, 20], [1, 10]])
    add("diff", FR + ":150-157", [[1, 10], [2, 20]], types=t2, a=[[1, 10], [1, 10], [2, 20]], b=[[3, 30]])
    add("diff", FR + ":159-167", [[1, 20], [2, 10]], types=t2, a=[[1, 10], [1, 20], [2, 10]], b=[[1, 10]])
    # ---- union / union_many, one u32 column ----------------------------------------------------
    u1 = ["u32"]
    add("union", SO + ":184-207", rows1([1, 2, 3, 4, 5]), types=u1, ins=[rows1([1, 2, 3]), rows1([3, 4, 5])])
    add("union", SO + ":248-271", rows1([1, 2, 3, 4]), types=u1, ins=[rows1([1, 2]), rows1([3, 4])])
    add("union", SO + ":274-297", rows1([1, 2, 3]), types=u1, ins=[rows1([1, 2, 3]), rows1([1, 2, 3])])
    add("union", SO + ":300-320", rows1([1, 2]), types=u1, ins=[[], rows1([1, 2])])
    add("union", SO + ":323-343", rows1([1, 2]), types=u1, ins=[rows1([1, 2]), []])
    add("union", SO + ":346-362", [], types=u1, ins=[[], []])
    add("union", SO + ":365-388", rows1([1, 2, 3]), types=u1, ins=[rows1([1, 1, 2]), rows1([2, 3, 3])])
    add("union", SO + ":412-449", rows1([1, 2, 3, 4, 5, 6, 7, 8, 9]), types=u1,
        ins=[rows1([5, 1, 5, 9]), rows1([2, 9, 3]), rows1([7, 1, 8, 8]), rows1([4, 3, 6])])
    add("union", SO + ":481-521", rows1([1, 2, 3, 4, 5]), types=u1,
        ins=[rows1(x) for x in ([1, 2, 3], [2, 3, 4], [3, 4, 5], [4, 5, 1], [5, 1, 2], [1, 3, 5], [2, 4, 1], [5, 2, 3])])
    add("union", SO + ":621-636 (a single input is deduplicated)", rows1([1, 2, 3]), types=u1, ins=[rows1([3, 1, 2, 1, 3])])
    add("union_error", SO + ":922-929 (no inputs)", None, types=u1, ins=[])
    add("union_error", SO + ":952-969 (incompatible schemas)", None, types=None,
        typed_ins=[{"types": ["u32"], "rows": rows1([1])}, {"types": ["u32", "u32"], "rows": [[1, 2]]}])
    # ---- difference, one u32 column -------------------------------------------------------------
    add("diff", SO + ":1024-1047", rows1([1, 3]), types=u1, a=rows1([1, 2, 3, 4]), b=rows1([2, 4]))
    add("diff", SO + ":1050-1073", rows1([1, 2, 3]), types=u1, a=rows1([1, 2, 3]), b=rows1([4, 5, 6]))
    add("diff", SO + ":1076-1098", [], types=u1, a=rows1([1, 2, 3]), b=rows1([1, 2, 3]))
    add("diff", SO + ":1101-1120", [], types=u1, a=[], b=rows1([1, 2]))
    add("diff", SO + ":1123-1143", rows1([1, 2, 3]), types=u1, a=rows1([1, 2, 3]), b=[])
    add("diff", SO + ":1146-1168", [], types=u1, a=rows1([2, 3]), b=rows1([1, 2, 3, 4, 5]))
    add("diff", SO + ":1171-1196", rows1([1, 3]), types=u1, a=rows1([4, 1, 3, 2]), b=rows1([2, 4]))
    add("diff", SO + ":1199-1222", rows1([1, 3]), types=u1, a=rows1([1, 1, 2, 2, 3]), b=rows1([2]))
    # ---- one u64 column --------------------------------------------------------------------------
    u8 = ["u64"]
    add("union", SO + ":1227-1249", rows1([1, 2, 3, 4]), types=u8, ins=[rows1([1, 2, 3]), rows1([2, 3, 4])])
    add("union", SO + ":1252-1275", rows1([1, 2, 3]), types=u8, ins=[rows1([1, 1, 2]), rows1([2, 3, 3])])
    add("union", SO + ":1278-1299", rows1([1, 2, 3]), types=u8, ins=[[], rows1([1, 2, 3])])
    add("diff", SO + ":1302-1324", rows1([1, 3]), types=u8, a=rows1([1, 2, 3, 4]), b=rows1([2, 4]))
    add("diff", SO + ":1327-1349", rows1([1, 2, 3]), types=u8, a=rows1([1, 2, 3]), b=rows1([4, 5, 6]))
    add("diff", SO + ":1352-1373", [], types=u8, a=rows1([1, 2, 3]), b=rows1([1, 2, 3]))
    add("diff", SO + ":1376-1397", rows1([1, 2, 3]), types=u8, a=rows1([1, 2, 3]), b=[])
    # three-column rows (the reference uses i64 triples; the non-negative rows keep their order as u64)
    add("union", SO + ":452-478 (rows shifted to non-negative values)", [[0, 12, 13], [6, 7, 8], [8, 35, 4], [14, 5, 1]],
        types=["u64", "u64", "u64"],
        ins=[[[8, 35, 4], [0, 12, 13]], [[6, 7, 8], [8, 35, 4]], [[0, 12, 13], [14, 5, 1], [6, 7, 8]]])
    # ---- typed order: signed integers and floats ------------------------------------------------
    i8, f8, i4 = ["i64"], ["f64"], ["i32"]
    add("union", SO + ":1400-1423", rows1([-10, -5, 0, 5, 10, 20]), types=i8, ins=[rows1([-10, -5, 0, 5]), rows1([-5, 0, 10, 20])])
    add("union", SO + ":1426-1450", rows1([-5, 0, 5]), types=i8, ins=[rows1([-5, -5, 0]), rows1([0, 5, 5])])
    add("union", SO + ":1453-1475", rows1([1.5, 2.5, 3.5, 4.5]), types=f8, ins=[rows1([1.5, 2.5, 3.5]), rows1([2.5, 3.5, 4.5])])
    add("union", SO + ":1478-1502", rows1([1.5, 2.5, 3.5]), types=f8, ins=[rows1([1.5, 1.5, 2.5]), rows1([2.5, 3.5, 3.5])])
    add("diff", SO + ":1505-1527", rows1([-10, 0, 10]), types=i8, a=rows1([-10, -5, 0, 5, 10]), b=rows1([-5, 5]))
    add("diff", SO + ":1530-1554", rows1([-10, -5, 0]), types=i8, a=rows1([-10, -5, 0]), b=rows1([5, 10, 15]))
    add("diff", SO + ":1557-1579", rows1([1.5, 3.5]), types=f8, a=rows1([1.5, 2.5, 3.5, 4.5]), b=rows1([2.5, 4.5]))
    add("diff", SO + ":1582-1604", rows1([1.5, 2.5, 3.5]), types=f8, a=rows1([1.5, 2.5, 3.5]), b=rows1([4.5, 5.5, 6.5]))
    add("union", SO + ":452-478 (i64 triples, signed order)", [[-5, 7, 8], [1, 2, 3], [3, 30, -1], [9, 0, -4]], types=["i64"] * 3,
        ins=[[[3, 30, -1], [-5, 7, 8]], [[1, 2, 3], [3, 30, -1]], [[-5, 7, 8], [9, 0, -4], [1, 2, 3]]])
    add("dedup", FR + ":170-183", rows1([-2, -1, 0, 1]), types=i4, a=rows1([-2, -1, 0, 1, -1, -2, 0]))
    add("diff", FR + ":185-201", rows1([-3, 0, 3]), types=i4, a=rows1([-3, -1, 0, 1, 3]), b=rows1([-1, 1]))
    # f32 rows are given as bit patterns; the reference compares these as sets of bit patterns
    fb = ["f32bits"]
    NAN_A, NAN_B, ONE, PZ, NZ, PINF, NINF = 0x7FC00001, 0x7FC00002, 0x3F800000, 0x00000000, 0x80000000, 0x7F800000, 0xFF800000
    add("dedup", FR + ":234-245 (NaNs collapse only when bit-identical)", rows1(sorted([NAN_A, ONE])), types=fb, a=rows1([NAN_A, NAN_A, ONE]), compare="set")
    add("dedup", FR + ":247-258", rows1(sorted([NAN_A, NAN_B])), types=fb, a=rows1([NAN_A, NAN_B]), compare="set")
    add("dedup", FR + ":260-272 (signed zeros are distinct)", rows1(sorted([PZ, NZ])), types=fb, a=rows1([PZ, NZ, PZ]), compare="set")
    add("dedup", FR + ":274-286", rows1(sorted([PINF, NINF, ONE])), types=fb, a=rows1([PINF, NINF, PINF, ONE]), compare="set")
    add("diff", FR + ":288-298", rows1([NAN_A]), types=fb, a=rows1([NAN_A]), b=rows1([NAN_B]), compare="set")
    add("diff", FR + ":300-310", rows1([PZ]), types=fb, a=rows1([PZ]), b=rows1([NZ]), compare="set")
    # ---- joins -----------------------------------------------------------------------------------
    add("join", JV + ":14-48 (2 rows, arity 4)", [[2, 20, 2, 200], [3, 30, 3, 300]], types=t2, rtypes=t2,
        a=[[1, 10], [2, 20], [3, 30]], b=[[2, 200], [3, 300], [4, 400]], lk=[0], rk=[0], join="inner")
    add("join", JV + ":50-80", rows1([2, 4]), types=u1, rtypes=u1, a=rows1([1, 2, 3, 4]), b=rows1([2, 4]), lk=[0], rk=[0], join="semi")
    add("join", JV + ":83-112", rows1([1, 3]), types=u1, rtypes=u1, a=rows1([1, 2, 3, 4]), b=rows1([2, 4]), lk=[0], rk=[0], join="anti")
    add("join", JV + ":115-140", [], types=u1, rtypes=u1, a=rows1([1, 2, 3]), b=rows1([4, 5, 6]), lk=[0], rk=[0], join="inner")
    add("join", JV + ":143-171 (bag semantics: 4 rows)", [[2, 2]] * 4, types=u1, rtypes=u1, a=rows1([1, 2, 2]), b=rows1([2, 2]),
        lk=[0], rk=[0], join="inner")
    add("join", JV + ":174-217", [[2, 20], [3, 30]], types=t2, rtypes=u1, a=[[1, 10], [2, 20], [3, 30]], b=rows1([2, 3, 4]),
        lk=[0], rk=[0], join="semi")
    add("join", JV + ":304-353 (two key columns, 3 matches)",
        [[1, 10, 100, 1, 10, 1000], [1, 20, 200, 1, 20, 3000], [2, 10, 300, 2, 10, 2000]], types=["u32"] * 3, rtypes=["u32"] * 3,
        a=[[1, 10, 100], [1, 20, 200], [2, 10, 300]], b=[[1, 10, 1000], [2, 10, 2000], [1, 20, 3000]], lk=[0, 1], rk=[0, 1], join="inner")
    add("join", JC + ":19-53 (different keys never join, whatever their hashes)", [], types=t2, rtypes=t2,
        a=[[100, 1]], b=[[200, 2]], lk=[0], rk=[0], join="inner")
    add("join", JC + ":57-82", [[200, 2, 200, 10]], types=t2, rtypes=t2, a=[[100, 1], [200, 2]], b=[[200, 10], [300, 20]],
        lk=[0], rk=[0], join="inner")
    add("join", JC + ":85-130 (second key column differs)", [], types=["u32"] * 3, rtypes=["u32"] * 3,
        a=[[1, 2, 100]], b=[[1, 3, 200]], lk=[0, 1], rk=[0, 1], join="inner")
    add("join", JC + ":132-162", [], types=u1, rtypes=u1, a=rows1([100, 200]), b=rows1([300, 400]), lk=[0], rk=[0], join="semi")
    add("join", JC + ":165-194", rows1([100, 200]), types=u1, rtypes=u1, a=rows1([100, 200]), b=rows1([300, 400]), lk=[0], rk=[0], join="anti")
    # ---- u64 keys: both halves of the key take part in the order ---------------------------------
    big = (1 << 32)
    add("sort", SD + ":253-270", rows1(list(range(1, 10))), types=["u64"], a=rows1([5, 2, 8, 1, 9, 3, 7, 4, 6]), keys=[0])
    add("sort", SD + ":273-287", [[10, 100], [20, 200], [30, 300], [40, 400]], types=["u64", "u32"],
        a=[[30, 300], [10, 100], [20, 200], [40, 400]], keys=[0])
    add("sort", SD + ":290-302", [], types=["u64"], a=[], keys=[0])
    add("sort", SD + ":305-318", rows1([1, 2, 3, 5, 8, 13, 21]), types=["u64"], a=rows1([1, 2, 3, 5, 8, 13, 21]), keys=[0])
    above = [big + 7, 2, big, big + 2, 7, (1 << 64) - 1, big - 1]
    add("sort", SD + ":321-356 (keys above u32::MAX)", rows1(sorted(above)), types=["u64"], a=rows1(above), keys=[0])
    d64 = [[big, 5], [1, 2], [1, 2], [big, 5], [big, 4], [1, 3]]
    add("dedup", SD + ":363-387", [list(t) for t in sorted({tuple(r) for r in d64})], types=["u64", "u64"], a=d64)
    add("dedup", SD + ":390-407", [[1, 2], [1, 3], [big, 1], [big, 2]], types=["u64", "u64"], a=[[1, 2], [1, 3], [big, 1], [big, 2]])
    # ---- the u32 matrix of the type-coverage suite -----------------------------------------------
    add("sort", TCOV + ":128-149", [[1, 10], [2, 20], [3, 30], [5, 50], [8, 80], [9, 90]], types=t2,
        a=[[5, 50], [2, 20], [8, 80], [1, 10], [9, 90], [3, 30]], keys=[0])
    add("sort", TCOV + ":153-170", rows1([1, 1, 2, 2, 3, 3]), types=u1, a=rows1([3, 1, 2, 1, 3, 2]), keys=[0])
    add("join", TCOV + ":209-237", rows1([2, 4]), types=u1, rtypes=u1, a=rows1([1, 2, 3, 4]), b=rows1([2, 4]), lk=[0], rk=[0], join="semi")
    add("join", TCOV + ":240-268", rows1([1, 3]), types=u1, rtypes=u1, a=rows1([1, 2, 3, 4]), b=rows1([2, 4]), lk=[0], rk=[0], join="anti")
    add("union", TCOV + ":368-390", rows1([1, 2, 3, 4, 5]), types=u1, ins=[rows1([1, 2, 3]), rows1([3, 4, 5])])
    add("union", TCOV + ":394-415", rows1([1, 2, 3, 4]), types=u1, ins=[rows1([1, 2]), rows1([3, 4])])
    add("diff", TCOV + ":421-443", rows1([1, 3]), types=u1, a=rows1([1, 2, 3, 4]), b=rows1([2, 4]))
    add("diff", TCOV + ":447-468", rows1([1, 2, 3]), types=u1, a=rows1([1, 2, 3]), b=rows1([4, 5, 6]))
    add("sort", TCOV + ":707-724", rows1([42]), types=u1, a=rows1([42]), keys=[0])
    return c


# ---- an independent naive evaluator -------------------------------------------------------------
def naive_fixpoint(rules, facts):
    """rules: list of (head, head_vars, body atoms [(rel, vars)], filters [(op, x, y)]).
    Variables are strings, constants ints.  Re-evaluates every rule on the whole database until
    nothing new appears (the textbook naive fixpoint)."""
    db = {k: set(map(tuple, v)) for k, v in facts.items()}
    for r in rules:
        db.setdefault(r[0], set())

    def solve(atoms, env):
        if not atoms:
            yield env
            return
        rel, vs = atoms[0]
        for row in db.get(rel, ()):
            e = dict(env)
            ok = True
            for v, x in zip(vs, row):
                if isinstance(v, int):
                    ok = v == x
                elif v in e:
                    ok = e[v] == x
                else:
                    e[v] = x
                if not ok:
                    break
            if ok:
                yield from solve(atoms[1:], e)

    while True:
        new = {}
        for head, hv, body, filters in rules:
            for env in solve(body, {}):
                if all({"!=": env[x] != env[y], "==": env[x] == env[y]}[op] for op, x, y in filters):
                    t = tuple(env[v] for v in hv)
                    if t not in db[head]:
                        new.setdefault(head, set()).add(t)
        if not new:
            break
        for k, v in new.items():
            db[k] |= v
    return {k: sorted(v) for k, v in db.items()}


TC = [("q", ["X", "Y"], [("edge", ["X", "Y"])], []), ("q", ["X", "Z"], [("q", ["X", "Y"]), ("edge", ["Y", "Z"])], [])]
TC_LEFT = [TC[0], ("q", ["X", "Z"], [("edge", ["X", "Y"]), ("q", ["Y", "Z"])], [])]
TC_NONLIN = [TC[0], ("q", ["X", "Z"], [("q", ["X", "Y"]), ("q", ["Y", "Z"])], [])]
TC_SWAP = [("q", ["Y", "X"], [("edge", ["X", "Y"])], []), ("q", ["Z", "X"], [("q", ["Y", "X"]), ("edge", ["Y", "Z"])], [])]
SG = [("sg", ["X", "Y"], [("edge", ["P", "X"]), ("edge", ["P", "Y"])], [("!=", "X", "Y")]),
      ("sg", ["X", "Y"], [("edge", ["A", "X"]), ("sg", ["A", "B"]), ("edge", ["B", "Y"])], [])]
PT = [("points_to", ["P", "T"], [("addr_of", ["P", "T"])], []),
      ("points_to", ["D", "T"], [("copy", ["D", "S"]), ("points_to", ["S", "T"])], [])]
ANDERSEN = [("pt", ["V", "O"], [("addressOf", ["V", "O"])], []),
            ("pt", ["V", "O"], [("assign", ["V", "W"]), ("pt", ["W", "O"])], []),
            ("pt", ["V", "O"], [("load", ["V", "P"]), ("pt", ["P", "Q"]), ("pt", ["Q", "O"])], []),
            ("pt", ["Q", "O"], [("store", ["P", "V"]), ("pt", ["P", "Q"]), ("pt", ["V", "O"])], [])]
REACH0 = [("r", ["Y"], [("edge", [0, "Y"])], []), ("r", ["Z"], [("r", ["Y"]), ("edge", ["Y", "Z"])], [])]

IRREGULAR = [(0, 1), (1, 2), (2, 0), (3, 4), (3, 5), (4, 6), (5, 6), (6, 7), (8, 0), (8, 3), (8, 7), (8, 9), (9, 9), (3, 4), (11, 1)]
SPIKE = "crates/xlog-integration/tests/test_factorized_delta_spike.rs"
E2E = "crates/xlog-integration/tests/test_factorized_delta_e2e.rs"


def block_cycle(k, b):
    return [(i * b + u, ((i + 1) % k) * b + v) for i in range(k) for u in range(b) for v in range(b)]


def programs():
    c = []

    def add(name, program, cite, facts, rules, out, expected=None, source=None, check=None):
        got = naive_fixpoint(rules, facts)[out]
        if expected is not None:
            assert [list(t) for t in got] == [list(t) for t in expected], name
        c.append({"name": name, "program": program, "cite": cite, "facts": {k: [list(t) for t in v] for k, v in facts.items()},
                  "output": out, "expected": [list(t) for t in got],
                  "expected_source": source or "naive_fixpoint in this script (the reference test computes it with an in-test oracle)"})
        if check:
            check(got)

    add("tc_chain3", "tc", "crates/xlog-integration/tests/e2e_integration_tests.rs:256-315; README.md:56-89",
        {"edge": [(1, 2), (2, 3), (3, 4)]}, TC, "q",
        expected=[(1, 2), (1, 3), (1, 4), (2, 3), (2, 4), (3, 4)],
        source="the reference asserts reach(1, {2,3,4}) and 6 rows; rows written out here")
    add("tc_irregular", "tc", SPIKE + ":257-275,322-343; " + E2E + ":310-322", {"edge": IRREGULAR}, TC, "q")
    add("tc_irregular_left_linear", "tc_left", E2E + ":324-336", {"edge": IRREGULAR}, TC_LEFT, "q")
    add("tc_irregular_nonlinear", "tc_nonlinear", E2E + ":338-350", {"edge": IRREGULAR}, TC_NONLIN, "q")
    add("tc_irregular_swapped_head", "tc_swapped", E2E + ":352-363", {"edge": IRREGULAR}, TC_SWAP, "q")
    add("tc_chain200", "tc", E2E + ":365-377", {"edge": [(i, i + 1) for i in range(200)]}, TC, "q",
        check=lambda rows: None if len(rows) == 200 * 201 // 2 else (_ for _ in ()).throw(AssertionError("chain count")))
    add("tc_block_cycle_3x4", "tc", SPIKE + ":424-437 (|TC| = (k*b)^2)", {"edge": block_cycle(3, 4)}, TC, "q",
        check=lambda rows: None if len(rows) == 144 else (_ for _ in ()).throw(AssertionError("block cycle count")))
    add("points_to_copy", "points_to_copy", "crates/xlog-integration/tests/real_world_tests.rs:753-815; "
        "examples/xlog/50-program-analysis/01_points_to_copy.xlog", {"addr_of": [(3, 1), (4, 2)], "copy": [(5, 3), (6, 5)]}, PT, "points_to",
        expected=[(3, 1), (4, 2), (5, 1), (6, 1)], source="rows asserted by the reference test")
    # the benchmark programs on tiny inputs (no reference fixture exists for them: the naive evaluator is the pin)
    tree = [(0, 1), (0, 2), (1, 3), (1, 4), (2, 5), (2, 6), (3, 7), (5, 8), (6, 9), (1, 6), (2, 7)]
    add("same_generation_tiny", "same_generation", "benchmark configuration 3 program; operator semantics as in "
        "crates/xlog-integration/tests/test_same_generation_gpu.rs:168-290", {"edge": tree}, SG, "sg")
    add("andersen_tiny", "andersen", "benchmark configuration 4 program",
        {"addressOf": [(0, 10), (1, 11), (2, 12)], "assign": [(3, 0), (4, 3), (1, 4)], "load": [(5, 3), (6, 1)], "store": [(0, 1), (4, 2)]},
        ANDERSEN, "pt")
    add("reach_from_0", "reach_from_source", "benchmark configuration 2 program (bound first argument; "
        "crates/xlog-logic/tests/test_v085_magic_sets.rs:22-58 for the bound form)", {"edge": IRREGULAR}, REACH0, "r")
    return c


# one semi-naive step with a given delta and full relation (lex-sorted, deduplicated emit order)
def novel_step():
    delta = [(0, 1), (0, 1), (2, 0), (8, 3), (7, 7), (3, 6)]
    full = [(0, 2), (2, 1), (8, 4)]
    succ = {}
    for y, z in IRREGULAR:
        succ.setdefault(y, set()).add(z)
    novel = sorted({(x, z) for x, y in delta for z in succ.get(y, ()) if (x, z) not in set(full)})
    return {"cite": SPIKE + ":278-320", "edge": [list(t) for t in IRREGULAR], "delta": [list(t) for t in delta],
            "full": [list(t) for t in full], "expected": [list(t) for t in novel],
            "expected_source": "set comprehension restating oracle_novel_step (" + SPIKE + ":159-180)"}


def groupby():
    """Literal inputs and asserted outputs of the reference's group-by tests.  `aggs`: (value
    column, op) with op in count / sum / min / max; expected columns = keys, then aggregates."""
    c = []

    def add(cite, cols, keys, aggs, expected, types=None):
        c.append({"cite": cite, "types": types or ["u32"] * len(cols), "cols": cols, "keys": keys, "aggs": aggs, "expected": expected})

    kv = [[1, 1, 2, 2, 2], [10, 20, 5, 15, 25]]
    add(GB + ":19-53", kv, [0], [[1, "count"]], [[1, 2], [2, 3]])
    add(GB + ":56-89", kv, [0], [[1, "sum"]], [[1, 2], [30, 45]])
    add(GB + ":92-123", kv, [0], [[1, "min"]], [[1, 2], [10, 5]])
    add(GB + ":124-135", kv, [0], [[1, "max"]], [[1, 2], [20, 25]])
    add(GB + ":138-188", kv, [0], [[1, "sum"], [1, "count"], [1, "min"], [1, "max"]], [[1, 2], [30, 45], [2, 3], [10, 5], [20, 25]])
    add(GB + ":191-209", [[], []], [0], [[1, "sum"]], [[], []])
    add(GB + ":212-244", [[5, 5, 5, 5], [10, 20, 30, 40]], [0], [[1, "sum"], [1, "count"]], [[5], [100], [4]])
    add(GB + ":247-281", [[2, 1, 2, 1, 2], [5, 10, 15, 20, 25]], [0], [[1, "sum"]], [[1, 2], [30, 45]])
    add(GB + ":284-317", [[1, 1, 2, 2], [10, 10, 20, 20], [5, 7, 11, 13]], [0, 1], [[2, "sum"]], [[1, 2], [10, 20], [12, 24]])
    add(GB + ":331-367", [[5, 3, 1, 4, 2], [50, 30, 10, 40, 20]], [0], [[1, "sum"], [1, "count"]],
        [[1, 2, 3, 4, 5], [10, 20, 30, 40, 50], [1, 1, 1, 1, 1]])
    add(TCOV + ":301-326", [[1, 1, 2, 2, 2, 3], [10, 20, 30, 40, 50, 60]], [0], [[1, "count"]], [[1, 2, 3], [2, 3, 1]])
    add(TCOV + ":542-585", [[1, 1, 2, 2, 2, 3], [10, 20, 5, 15, 25, 100]], [0], [[1, "count"], [1, "sum"], [1, "min"], [1, "max"]],
        [[1, 2, 3], [2, 3, 1], [30, 45, 100], [10, 5, 100], [20, 25, 100]])
    return c


if __name__ == "__main__":
    with open(os.path.join(HERE, "groupby.json"), "w") as f:
        json.dump(groupby(), f, separators=(",", ":"))
    with open(os.path.join(HERE, "operators.json"), "w") as f:
        json.dump(operators(), f, separators=(",", ":"))
    with open(os.path.join(HERE, "programs.json"), "w") as f:
        json.dump({"programs": programs(), "novel_step": novel_step()}, f, separators=(",", ":"))
    print("wrote operators.json, programs.json, groupby.json")
