"""Execution plans of the benchmark programs, in the shape the reference's lowering emits.

A two-atom rule ``h(X,Z) :- l(X,Y), r(Y,Z)`` lowers to
``Project(Join(Scan l, Scan r, [1], [0]), [0, 3])`` — the ``fallback`` tree of the promoted
ChainJoin (crates/xlog-logic/src/promote.rs:2035-2073).  Three-atom bodies lower to a binary
join tree whose leaf order is the output column layout (crates/xlog-logic/src/lower.rs:1270-1292).
"""
from __future__ import annotations

from . import _abi as A
from .plan import CompiledRule, ExecutionPlan, Filter, Join, Project, Scan, Scc

U2 = (A.U32, A.U32)


def transitive_closure(edge: str = "edge", reach: str = "reach") -> ExecutionPlan:
    """reach(X,Y) :- edge(X,Y).  reach(X,Z) :- reach(X,Y), edge(Y,Z).
    (examples/xlog/00-basics/01_tc_reachability.xlog)"""
    ids = {edge: 0, reach: 1}
    base = CompiledRule(reach, Scan(ids[edge]), U2)
    rec = CompiledRule(reach, Project(Join(Scan(ids[reach]), Scan(ids[edge]), [1], [0]), [0, 3]), U2)
    return ExecutionPlan([Scc(0, True, [base, rec])], ids)


def transitive_closure_left_linear(edge="edge", reach="reach") -> ExecutionPlan:
    """reach(X,Z) :- edge(X,Y), reach(Y,Z)."""
    ids = {edge: 0, reach: 1}
    base = CompiledRule(reach, Scan(ids[edge]), U2)
    rec = CompiledRule(reach, Project(Join(Scan(ids[edge]), Scan(ids[reach]), [1], [0]), [0, 3]), U2)
    return ExecutionPlan([Scc(0, True, [base, rec])], ids)


def transitive_closure_nonlinear(edge="edge", reach="reach") -> ExecutionPlan:
    """reach(X,Z) :- reach(X,Y), reach(Y,Z)."""
    ids = {edge: 0, reach: 1}
    base = CompiledRule(reach, Scan(ids[edge]), U2)
    rec = CompiledRule(reach, Project(Join(Scan(ids[reach]), Scan(ids[reach]), [1], [0]), [0, 3]), U2)
    return ExecutionPlan([Scc(0, True, [base, rec])], ids)


def transitive_closure_swapped_head(edge="edge", reach="reach") -> ExecutionPlan:
    """reach(Y,X) :- edge(X,Y).  reach(Z,X) :- reach(Y,X), edge(Y,Z)  (head columns swapped)."""
    ids = {edge: 0, reach: 1}
    base = CompiledRule(reach, Project(Scan(ids[edge]), [1, 0]), U2)
    rec = CompiledRule(reach, Project(Join(Scan(ids[reach]), Scan(ids[edge]), [0], [0]), [3, 1]), U2)
    return ExecutionPlan([Scc(0, True, [base, rec])], ids)


def reach_from_source(source: int = 0, edge="edge", reach="r") -> ExecutionPlan:
    """Single-source reachability as a seeded frontier:
    r(Y) :- edge(source, Y).  r(Z) :- r(Y), edge(Y, Z).
    The bound-first-argument form that the magic-set rewrite reduces ``?- reach(source, N)`` to
    (crates/xlog-logic/src/magic_sets.rs), without the guard atom."""
    ids = {edge: 0, reach: 1}
    base = CompiledRule(reach, Project(Filter(Scan(ids[edge]), A.EQ, 0, source, True), [1]), (A.U32,))
    rec = CompiledRule(reach, Project(Join(Scan(ids[reach]), Scan(ids[edge]), [0], [0]), [2]), (A.U32,))
    return ExecutionPlan([Scc(0, True, [base, rec])], ids)


def same_generation(edge="edge", sg="sg") -> ExecutionPlan:
    """sg(X,Y) :- edge(P,X), edge(P,Y), X != Y.
    sg(X,Y) :- edge(A,X), sg(A,B), edge(B,Y)."""
    ids = {edge: 0, sg: 1}
    e, s = ids[edge], ids[sg]
    base = CompiledRule(sg, Project(Filter(Join(Scan(e), Scan(e), [0], [0]), A.NE, 1, 3), [1, 3]), U2)
    # ((edge(A,X) join sg(A,B)) on A) join edge(B,Y) on B: columns A X A B B Y
    rec = CompiledRule(sg, Project(Join(Join(Scan(e), Scan(s), [0], [0]), Scan(e), [3], [0]), [1, 5]), U2)
    return ExecutionPlan([Scc(0, True, [base, rec])], ids)


def andersen() -> ExecutionPlan:
    """pt(V,O) :- addressOf(V,O).            pt(V,O) :- assign(V,W), pt(W,O).
    pt(V,O) :- load(V,P), pt(P,Q), pt(Q,O).  pt(Q,O) :- store(P,V), pt(P,Q), pt(V,O)."""
    ids = {"addressOf": 0, "assign": 1, "load": 2, "store": 3, "pt": 4}
    ao, asg, ld, st, pt = (ids[k] for k in ("addressOf", "assign", "load", "store", "pt"))
    r0 = CompiledRule("pt", Scan(ao), U2)
    r1 = CompiledRule("pt", Project(Join(Scan(asg), Scan(pt), [1], [0]), [0, 3]), U2)
    # load(V,P) pt(P,Q) pt(Q,O): columns V P P Q Q O
    r2 = CompiledRule("pt", Project(Join(Join(Scan(ld), Scan(pt), [1], [0]), Scan(pt), [3], [0]), [0, 5]), U2)
    # store(P,V) pt(P,Q) pt(V,O): columns P V P Q V O ; head (Q, O)
    r3 = CompiledRule("pt", Project(Join(Join(Scan(st), Scan(pt), [0], [0]), Scan(pt), [1], [0]), [3, 5]), U2)
    return ExecutionPlan([Scc(0, True, [r0, r1, r2, r3])], ids)


def points_to_copy() -> ExecutionPlan:
    """points_to(V,O) :- alloc(V,O).  points_to(V,O) :- assign(V,W), points_to(W,O).
    (examples/xlog/50-program-analysis/01_points_to_copy.xlog)"""
    ids = {"alloc": 0, "assign": 1, "points_to": 2}
    r0 = CompiledRule("points_to", Scan(0), U2)
    r1 = CompiledRule("points_to", Project(Join(Scan(1), Scan(2), [1], [0]), [0, 3]), U2)
    return ExecutionPlan([Scc(0, True, [r0, r1])], ids)


def unreachable_nodes(source: int = 0) -> ExecutionPlan:
    """Two strata: r(Y) :- edge(source,Y). r(Z) :- r(Y), edge(Y,Z).   then
    un(X) :- node(X), not r(X).   (negation lowered to an anti join against the lower stratum)
    and  either(X) :- r(X).  either(X) :- un(X).  written as one rule with a Union body."""
    from .plan import Union
    ids = {"edge": 0, "r": 1, "node": 2, "un": 3, "either": 4}
    base = CompiledRule("r", Project(Filter(Scan(0), A.EQ, 0, source, True), [1]), (A.U32,))
    rec = CompiledRule("r", Project(Join(Scan(1), Scan(0), [0], [0]), [2]), (A.U32,))
    un = CompiledRule("un", Join(Scan(2), Scan(1), [0], [0], A.JOIN_ANTI), (A.U32,))
    either = CompiledRule("either", Union([Scan(1), Scan(3)]), (A.U32,))
    return ExecutionPlan([Scc(0, True, [base, rec]), Scc(1, False, [un]), Scc(2, False, [either])], ids)
