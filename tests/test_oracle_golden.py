"""The CPU oracle against the known-answer fixtures transcribed from the reference's tests."""
import json
import os

import numpy as np
import pytest

from xlog_b200 import programs

HERE = os.path.dirname(os.path.abspath(__file__))
OPS = json.load(open(os.path.join(HERE, "golden", "operators.json")))
PROGS = json.load(open(os.path.join(HERE, "golden", "programs.json")))

DT = {"u32": np.uint32, "u64": np.uint64, "i32": np.int32, "i64": np.int64, "f64": np.float64, "f32bits": np.float32}
PLANS = {"tc": programs.transitive_closure, "tc_left": programs.transitive_closure_left_linear,
         "tc_nonlinear": programs.transitive_closure_nonlinear, "tc_swapped": programs.transitive_closure_swapped_head,
         "points_to_copy": programs.points_to_copy, "same_generation": programs.same_generation,
         "andersen": programs.andersen, "reach_from_source": programs.reach_from_source}
# names the fixtures use for the relations of each plan builder
RENAME = {"tc": {"q": "reach"}, "tc_left": {"q": "reach"}, "tc_nonlinear": {"q": "reach"}, "tc_swapped": {"q": "reach"},
          "points_to_copy": {"addr_of": "alloc", "copy": "assign"}}


def cols_of(rows, types):
    out = []
    for i, t in enumerate(types):
        vals = [r[i] for r in rows]
        if t == "f32bits":          # rows carry IEEE bit patterns
            out.append(np.array(vals, dtype=np.uint32).view(np.float32))
        else:
            out.append(np.array(vals, dtype=DT[t]))
    return out


def rows_of(cols):
    if not cols or not len(cols[0]):
        return []
    lists = [c.view(np.uint32).tolist() if c.dtype == np.float32 else c.tolist() for c in cols]
    return [list(t) for t in zip(*lists)]


def expected_of(case, got):
    """(got, want) in comparable form: joins and bit-pattern cases compare as sorted sets."""
    if case["op"] == "join" or case.get("compare") == "set":
        return sorted(got), sorted(case["expected"])
    return got, case["expected"]


def run_operator_case(case, make, ops):
    """make(rows, types) -> relation; ops: object with sort/dedup/union_many/diff/hash_join/rows."""
    op = case["op"]
    if op == "sort":
        return ops.rows(ops.sort(make(case["a"], case["types"]), case["keys"]))
    if op == "dedup":
        return ops.rows(ops.dedup(make(case["a"], case["types"])))
    if op == "union":
        return ops.rows(ops.union_many([make(r, case["types"]) for r in case["ins"]]))
    if op == "diff":
        return ops.rows(ops.diff(make(case["a"], case["types"]), make(case["b"], case["types"])))
    if op == "join":
        jt = {"inner": 0, "semi": 1, "anti": 2}[case["join"]]
        out = ops.hash_join(make(case["a"], case["types"]), make(case["b"], case["rtypes"]), case["lk"], case["rk"], jt)
        return ops.rows(out)
    raise AssertionError(op)


class OracleOps:
    def __init__(self, O):
        self.O = O

    def make(self, rows, types):
        return self.O.OracleRel.from_columns(cols_of(rows, types), arity=len(types)) if rows else \
            self.O.OracleRel.from_columns([np.zeros(0, dtype=DT[t]) for t in types], arity=len(types))

    def rows(self, r):
        return rows_of(r.columns())

    def sort(self, r, keys):
        return self.O.sort(r, keys)

    def dedup(self, r):
        return self.O.dedup(r)

    def union_many(self, rs):
        return self.O.union_many(rs)

    def diff(self, a, b):
        return self.O.diff(a, b)

    def hash_join(self, a, b, lk, rk, jt):
        return self.O.hash_join(a, b, lk, rk, jt)


@pytest.mark.parametrize("case", [c for c in OPS if not c["op"].endswith("_error")], ids=lambda c: c["op"] + "@" + c["cite"].split(" ")[0])
def test_oracle_operator_kat(oracle, case):
    ops = OracleOps(oracle)
    got, want = expected_of(case, run_operator_case(case, ops.make, ops))
    assert got == want, case["cite"]


def test_oracle_union_errors(oracle):
    ops = OracleOps(oracle)
    with pytest.raises(ValueError):
        oracle.union_many([])
    with pytest.raises(ValueError):
        oracle.union_many([ops.make([[1]], ["u32"]), ops.make([[1, 2]], ["u32", "u32"])])


def program_inputs(case):
    ren = RENAME.get(case["program"], {})
    facts = {ren.get(k, k): cols_of(v, ["u32"] * len(v[0])) for k, v in case["facts"].items()}
    return PLANS[case["program"]](), facts, ren.get(case["output"], case["output"])


@pytest.mark.parametrize("case", PROGS["programs"], ids=lambda c: c["name"])
def test_oracle_program_kat(oracle, case):
    plan, facts, out = program_inputs(case)
    got, _ = oracle.run_program(plan, facts, [out])
    assert rows_of(got[out]) == case["expected"], case["cite"]


def test_oracle_novel_step(oracle):
    ns = PROGS["novel_step"]
    ops = OracleOps(oracle)
    t2 = ["u32", "u32"]
    joined = oracle.hash_join(ops.make(ns["delta"], t2), ops.make(ns["edge"], t2), [1], [0], 0)
    c = joined.columns()
    cand = oracle.OracleRel.from_columns([c[0], c[3]])
    novel = oracle.diff(cand, ops.make(ns["full"], t2))
    assert rows_of(novel.columns()) == ns["expected"]      # emitted lex-sorted and deduplicated
    assert novel.canonical


def test_oracle_iteration_limit(oracle):
    c0 = np.arange(0, 50, dtype=np.uint32)
    with pytest.raises(RuntimeError, match="iteration limit"):
        oracle.run_program(programs.transitive_closure(), {"edge": [c0, c0 + 1]}, ["reach"], max_iterations=3)


def _reachable(c0, c1, source):
    seen, frontier = set(), {int(y) for x, y in zip(c0.tolist(), c1.tolist()) if x == source}
    adj = {}
    for x, y in zip(c0.tolist(), c1.tolist()):
        adj.setdefault(x, []).append(y)
    while frontier:
        seen |= frontier
        frontier = {z for y in frontier for z in adj.get(y, ())} - seen
    return seen


def stratified_case():
    from xlog_b200 import workloads
    c0, c1 = workloads.uniform_digraph(80, 160, 3)
    source = int(c0[0])
    node = np.arange(80, dtype=np.uint32)
    reach = _reachable(c0, c1, source)
    return programs.unreachable_nodes(source), {"edge": [c0, c1], "node": [node]}, reach, set(range(80)) - reach


def test_oracle_stratified_negation_and_union_body(oracle):
    plan, inputs, reach, unreach = stratified_case()
    out, _ = oracle.run_program(plan, inputs, ["r", "un", "either"])
    assert out["r"][0].tolist() == sorted(reach) and len(reach) > 3
    assert out["un"][0].tolist() == sorted(unreach)
    assert out["either"][0].tolist() == list(range(80))
