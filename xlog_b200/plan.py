"""Execution plans: a Python mirror of the reference's relational IR subset.

The classes mirror ``RirNode::{Scan, Filter, Project, Join, Union}``
(crates/xlog-ir/src/rir.rs:339-541), ``CompiledRule``, ``Scc`` and ``ExecutionPlan``
(crates/xlog-ir/src/plan.rs:8-70).  ``ExecutionPlan.compile()`` lowers the tree to the C
structs of include/xlb.h; the returned object keeps every allocation alive.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Sequence

from . import _abi as A


class RirNode:
    def arity(self, arities: dict[int, int]) -> int:
        raise NotImplementedError


@dataclass
class Scan(RirNode):
    rel: int

    def arity(self, arities):
        return arities[self.rel]


@dataclass
class Filter(RirNode):
    """``input`` rows where ``column(lhs) <cmp> rhs`` (rhs: column index or constant)."""
    input: RirNode
    cmp: int
    lhs_col: int
    rhs: int
    rhs_is_const: bool = False

    def arity(self, arities):
        return self.input.arity(arities)


@dataclass
class Project(RirNode):
    input: RirNode
    columns: Sequence[int]

    def arity(self, arities):
        return len(self.columns)


@dataclass
class Join(RirNode):
    left: RirNode
    right: RirNode
    left_keys: Sequence[int]
    right_keys: Sequence[int]
    join_type: int = A.JOIN_INNER   # JOIN_SEMI / JOIN_ANTI keep the left columns only

    def arity(self, arities):
        if self.join_type != A.JOIN_INNER:
            return self.left.arity(arities)
        return self.left.arity(arities) + self.right.arity(arities)


@dataclass
class Union(RirNode):
    inputs: Sequence[RirNode]

    def arity(self, arities):
        return self.inputs[0].arity(arities)


@dataclass
class Diff(RirNode):
    """``left`` minus ``right`` with set semantics on full rows (``RirNode::Diff``)."""
    left: RirNode
    right: RirNode

    def arity(self, arities):
        return self.left.arity(arities)


@dataclass
class Distinct(RirNode):
    """One row per distinct value of ``key_cols`` (``RirNode::Distinct``); no key columns = full rows."""
    input: RirNode
    key_cols: Sequence[int] = ()

    def arity(self, arities):
        return self.input.arity(arities)


@dataclass
class CompiledRule:
    head: str
    body: RirNode
    head_types: Sequence[int] = (A.U32, A.U32)


@dataclass
class Scc:
    id: int
    is_recursive: bool
    rules: Sequence[CompiledRule]


@dataclass
class ExecutionPlan:
    """SCCs in evaluation order plus the RelId -> name table the caller registers
    (``Compiler::rel_ids()`` in the reference's tests)."""
    sccs: Sequence[Scc]
    rel_ids: dict[str, int] = field(default_factory=dict)

    def compile(self) -> "CompiledPlan":
        return CompiledPlan(self)


class CompiledPlan:
    def __init__(self, plan: ExecutionPlan):
        self._keep: list = []
        sccs = (A.Scc * len(plan.sccs))()
        for i, s in enumerate(plan.sccs):
            rules = (A.Rule * len(s.rules))()
            for j, r in enumerate(s.rules):
                rules[j].head = r.head.encode()
                rules[j].body = C.pointer(self._node(r.body))
                rules[j].head_schema = A.Schema.of(list(r.head_types))
            self._keep.append(rules)
            sccs[i].id = s.id
            sccs[i].is_recursive = 1 if s.is_recursive else 0
            sccs[i].rules = rules
            sccs[i].n_rules = len(s.rules)
        self._keep.append(sccs)
        self.c = A.Plan(sccs, len(plan.sccs))
        self.plan = plan

    def _node(self, n: RirNode) -> A.Node:
        c = A.Node()
        self._keep.append(c)
        if isinstance(n, Scan):
            c.kind, c.rel_id = A.NODE_SCAN, n.rel
        elif isinstance(n, Filter):
            c.kind = A.NODE_FILTER
            c.input = C.pointer(self._node(n.input))
            c.cmp, c.cmp_lhs_col = n.cmp, n.lhs_col
            c.cmp_rhs_is_const, c.cmp_rhs = int(n.rhs_is_const), n.rhs
        elif isinstance(n, Project):
            c.kind = A.NODE_PROJECT
            c.input = C.pointer(self._node(n.input))
            c.n_cols = len(n.columns)
            for i, x in enumerate(n.columns):
                c.cols[i] = x
        elif isinstance(n, Join):
            c.kind = A.NODE_JOIN
            c.left = C.pointer(self._node(n.left))
            c.right = C.pointer(self._node(n.right))
            c.n_keys = len(n.left_keys)
            c.join_type = n.join_type
            for i, (a, b) in enumerate(zip(n.left_keys, n.right_keys)):
                c.left_keys[i], c.right_keys[i] = a, b
        elif isinstance(n, Union):
            c.kind = A.NODE_UNION
            arr = (C.POINTER(A.Node) * len(n.inputs))()
            for i, x in enumerate(n.inputs):
                arr[i] = C.pointer(self._node(x))
            self._keep.append(arr)
            c.inputs, c.n_inputs = arr, len(n.inputs)
        elif isinstance(n, Diff):
            c.kind = A.NODE_DIFF
            c.left = C.pointer(self._node(n.left))
            c.right = C.pointer(self._node(n.right))
        elif isinstance(n, Distinct):
            c.kind = A.NODE_DISTINCT
            c.input = C.pointer(self._node(n.input))
            c.n_cols = len(n.key_cols)
            for i, x in enumerate(n.key_cols):
                c.cols[i] = x
        else:
            raise TypeError(f"unsupported plan node {n!r}")
        return c
