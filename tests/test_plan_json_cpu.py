"""The plan importer (serialized xlog_ir::ExecutionPlan -> plan descriptor) without a GPU: the
imported plans are evaluated by the CPU oracle and compared with the hand-built ones."""
import json

import numpy as np
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import plan_json as PJ
from xlog_b200 import programs, workloads
from xlog_b200.lib import XlbError
from xlog_b200.plan import Filter, Join, Project, Scan

# The serialized form of one plan is kept as a fixture: tests/golden/plan_tc_serde.json (its note
# says what it is a reading of, and that no Rust toolchain has produced it yet).
import os

with open(os.path.join(os.path.dirname(__file__), "golden", "plan_tc_serde.json")) as _f:
    TC_FIXTURE = json.load(_f)
TC_JSON = json.dumps(TC_FIXTURE["plan"])


def test_transitive_closure_known_answer(oracle):
    plan = PJ.plan_from_json(TC_JSON, rel_names={int(k): v for k, v in TC_FIXTURE["rel_names"].items()})
    edge = [np.array(col, np.uint32) for col in TC_FIXTURE["input"]["edge"]]
    out, _ = oracle.run_program(plan, {"edge": edge}, ["reach"])
    assert [list(t) for t in zip(*[c.tolist() for c in out["reach"]])] == TC_FIXTURE["expect"]["reach"]
    assert plan.sccs[0].is_recursive and plan.rel_ids == {"edge": 0, "reach": 1}
    assert isinstance(plan.sccs[0].rules[1].body, Project)      # the ChainJoin's fallback tree


@pytest.mark.parametrize("builder", [programs.transitive_closure, programs.transitive_closure_left_linear,
                                     programs.transitive_closure_nonlinear, programs.transitive_closure_swapped_head,
                                     programs.reach_from_source, programs.same_generation, programs.andersen,
                                     programs.points_to_copy, programs.unreachable_nodes])
def test_every_program_round_trips(builder):
    plan = builder()
    back = PJ.plan_from_json(PJ.plan_to_json(plan))
    assert back.rel_ids == plan.rel_ids and len(back.sccs) == len(plan.sccs)
    for a, b in zip(back.sccs, plan.sccs):
        assert (a.id, bool(a.is_recursive)) == (b.id, bool(b.is_recursive))
        assert [(r.head, r.body, tuple(r.head_types)) for r in a.rules] == [(r.head, r.body, tuple(r.head_types)) for r in b.rules]


def test_imported_program_gives_the_same_fixpoint(oracle):
    c0, c1, _ = workloads.tree_dag(300, 0.05, 5)
    plan = programs.same_generation()
    want, _ = oracle.run_program(plan, {"edge": [c0, c1]}, ["sg"])
    got, _ = oracle.run_program(PJ.plan_from_json(PJ.plan_to_json(plan)), {"edge": [c0, c1]}, ["sg"])
    assert all(np.array_equal(g, w) for g, w in zip(got["sg"], want["sg"]))


def test_filters_constants_and_conjunctions():
    pred = {"And": [{"Compare": {"left": {"Const": {"U32": 5}}, "op": "Lt", "right": {"Column": 1}}},
                    {"Compare": {"left": {"Column": 0}, "op": "Ne", "right": {"Column": 1}}}]}
    node = PJ.node_from_json({"Filter": {"input": {"Scan": {"rel": 3}}, "predicate": pred}})
    # 5 < c1  is  c1 > 5; the conjunction nests
    assert node == Filter(Filter(Scan(3), A.GT, 1, 5, True), A.NE, 0, 1, False)
    semi = PJ.node_from_json({"Join": {"left": {"Scan": {"rel": 0}}, "right": {"Scan": {"rel": 1}}, "left_keys": [0],
                                      "right_keys": [0], "join_type": "Anti"}})
    assert semi == Join(Scan(0), Scan(1), [0], [0], A.JOIN_ANTI)


def test_strata_order_is_the_evaluation_order():
    doc = json.loads(PJ.plan_to_json(programs.unreachable_nodes()))
    ids = [s["id"] for s in doc["sccs"]]
    assert len(ids) >= 2
    # list the SCCs in reverse, keep the strata: the importer follows the strata
    doc["sccs"].reverse()
    doc["rules_by_scc"].reverse()
    plan = PJ.plan_from_json(doc)
    assert [s.id for s in plan.sccs] == ids


@pytest.mark.parametrize("body,what", [
    ({"GroupBy": {"input": {"Scan": {"rel": 0}}, "key_cols": [0], "aggs": []}}, "RirNode::GroupBy"),
    ({"Project": {"input": {"Scan": {"rel": 0}}, "columns": [{"Computed": [{"Column": 0}, "U32"]}]}}, "ProjectExpr::Computed"),
    ({"Filter": {"input": {"Scan": {"rel": 0}}, "predicate": {"Not": {"Column": 0}}}}, "Expr::Not"),
    ({"Join": {"left": {"Scan": {"rel": 0}}, "right": {"Scan": {"rel": 0}}, "left_keys": [0], "right_keys": [0],
               "join_type": "LeftOuter"}}, "JoinType::LeftOuter"),
    ({"Filter": {"input": {"Scan": {"rel": 0}}, "predicate": {"Compare": {"left": {"Column": 0}, "op": "Eq",
                                                                       "right": {"Const": {"Symbol": "a"}}}}}}, "Symbol constant"),
])
def test_constructs_outside_the_subset_are_named(body, what):
    with pytest.raises(XlbError, match=what.replace("::", "::")) as e:
        PJ.node_from_json(body)
    assert e.value.status == A.ERR_UNSUPPORTED


def test_malformed_documents_are_errors():
    with pytest.raises(XlbError, match="rel_names"):
        PJ.plan_from_json(TC_JSON)
    with pytest.raises(XlbError, match="same length"):
        PJ.plan_from_json({"sccs": [], "rules_by_scc": [[]]}, rel_names={0: "e"})
    bad = json.loads(TC_JSON)
    bad["strata"] = [{"id": 0, "sccs": [7]}]
    with pytest.raises(XlbError, match="unknown SCC 7"):
        PJ.plan_from_json(bad, rel_names={0: "edge", 1: "reach"})
    bad = json.loads(TC_JSON)
    bad["rules_by_scc"][0][0]["head"] = "nobody"
    with pytest.raises(XlbError, match="no RelId"):
        PJ.plan_from_json(bad, rel_names={0: "edge", 1: "reach"})


def test_diff_and_distinct_round_trip(oracle):
    """RirNode::Diff and RirNode::Distinct survive export and import, and the imported plan computes
    what the hand-built one does."""
    from xlog_b200.plan import CompiledRule, Diff, Distinct, ExecutionPlan, Scc
    one_way = CompiledRule("one_way", Diff(Scan(0), Project(Scan(0), [1, 0])), (A.U32, A.U32))
    first = CompiledRule("first", Distinct(Scan(0), [0]), (A.U32, A.U32))
    plan = ExecutionPlan([Scc(0, False, [one_way]), Scc(1, False, [first])], {"edge": 0, "one_way": 1, "first": 2})
    back = PJ.plan_from_json(PJ.plan_to_json(plan))
    assert isinstance(back.sccs[0].rules[0].body, Diff) and isinstance(back.sccs[1].rules[0].body, Distinct)
    assert list(back.sccs[1].rules[0].body.key_cols) == [0]
    c0, c1 = workloads.uniform_digraph(40, 160, 3)
    want, _ = oracle.run_program(plan, {"edge": [c0, c1]}, ["one_way", "first"])
    got, _ = oracle.run_program(back, {"edge": [c0, c1]}, ["one_way", "first"])
    for name in ("one_way", "first"):
        assert all(np.array_equal(g, w) for g, w in zip(got[name], want[name]))
    pairs = set(zip(c0.tolist(), c1.tolist()))
    assert set(zip(*[c.tolist() for c in want["one_way"]])) == {p for p in pairs if (p[1], p[0]) not in pairs}
