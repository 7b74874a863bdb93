"""Import a serialized ``xlog_ir::ExecutionPlan`` so that the reference's planner can drive this
executor: the caller side of the path.

The reference has no serializer for its plan types; the format read here is what
``#[derive(Serialize)]`` with serde's default (externally tagged) representation gives for them,
so a maintainer adds the derive and ``serde_json::to_string(&plan)``:

* ``ExecutionPlan`` (crates/xlog-ir/src/plan.rs:52-70): ``{"sccs": [Scc], "strata": [Stratum],
  "rules_by_scc": [[CompiledRule]], "rel_arities": {...}, ...}``; ``Scc`` = ``{"id", "predicates",
  "is_recursive"}`` (plan.rs:9-16); ``CompiledRule`` = ``{"head", "body", "meta"}`` (plan.rs:29-36,
  ``meta`` ignored).
* ``RirNode`` (crates/xlog-ir/src/rir.rs:339-470) as ``{"Variant": {fields}}``: ``Scan{rel}``,
  ``Filter{input, predicate}``, ``Project{input, columns}``, ``Join{left, right, left_keys,
  right_keys, join_type}``, ``Union{inputs}``; ``ChainJoin`` and ``MultiWayJoin`` stand for their
  ``fallback`` tree.  ``RelId`` is a newtype over u32 and serializes as the number.
* ``Expr`` (rir.rs:20-60): a ``Compare{left, op, right}`` between ``Column(i)`` and ``Column(j)``
  or ``Const(ConstValue)``; ``And([...])`` of such comparisons becomes nested filters.
  ``ProjectExpr::Column(i)`` only.

Two things the plan does not carry are given beside it, as the reference's callers hold them too:
``rel_names`` (RelId -> name: ``Compiler::rel_ids()``, registered through
``Executor::register_relation``) and, optionally, ``head_types`` (name -> list of column type names;
default: u32 columns, one per column of the rule body).  They may sit in the JSON object under
those keys or be passed as arguments.

Anything outside the built subset raises ``XlbError(UNSUPPORTED)`` naming the construct: nothing is
dropped silently.
"""
from __future__ import annotations

import json
from typing import Any, Mapping

from . import _abi as A
from .lib import XlbError
from .plan import CompiledRule, Diff, Distinct, ExecutionPlan, Filter, Join, Project, RirNode, Scan, Scc, Union

_CMP = {"Eq": A.EQ, "Ne": A.NE, "Lt": A.LT, "Le": A.LE, "Gt": A.GT, "Ge": A.GE}
_FLIP = {A.EQ: A.EQ, A.NE: A.NE, A.LT: A.GT, A.LE: A.GE, A.GT: A.LT, A.GE: A.LE}
_JOIN = {"Inner": A.JOIN_INNER, "Semi": A.JOIN_SEMI, "Anti": A.JOIN_ANTI}
_TYPES = {"U32": A.U32, "U64": A.U64, "I32": A.I32, "I64": A.I64, "F32": A.F32, "F64": A.F64, "Bool": A.BOOL,
          "Symbol": A.SYMBOL}


def _unsupported(what: str):
    raise XlbError(A.ERR_UNSUPPORTED, f"plan import: {what} is not built")


def _invalid(what: str):
    raise XlbError(A.ERR_INVALID, f"plan import: {what}")


def _variant(obj: Any, what: str) -> tuple[str, Any]:
    """An externally tagged enum value: ``"Unit"`` or ``{"Variant": payload}``."""
    if isinstance(obj, str):
        return obj, None
    if isinstance(obj, dict) and len(obj) == 1:
        (k, v), = obj.items()
        return k, v
    _invalid(f"{what}: expected an enum value, got {json.dumps(obj)[:80]}")


def _operand(e: Any) -> tuple[str, int]:
    kind, v = _variant(e, "Expr")
    if kind == "Column":
        return "col", int(v)
    if kind == "Const":
        ckind, cv = _variant(v, "ConstValue")
        if ckind in ("U32", "U64") or (ckind in ("I32", "I64") and int(cv) >= 0):
            return "const", int(cv)
        _unsupported(f"a {ckind} constant in a filter")
    _unsupported(f"Expr::{kind} as a comparison operand")


def _filters(node: RirNode, pred: Any) -> RirNode:
    kind, v = _variant(pred, "Expr")
    if kind == "And":
        for p in v:
            node = _filters(node, p)
        return node
    if kind != "Compare":
        _unsupported(f"Expr::{kind} as a filter predicate")
    op = _CMP.get(v["op"] if isinstance(v["op"], str) else _variant(v["op"], "CompareOp")[0])
    if op is None:
        _invalid(f"unknown CompareOp {v['op']!r}")
    (lk, lv), (rk, rv) = _operand(v["left"]), _operand(v["right"])
    if lk == "const" and rk == "col":      # c op X  ==  X flipped-op c
        (lk, lv), (rk, rv), op = (rk, rv), (lk, lv), _FLIP[op]
    if lk != "col":
        _unsupported("a comparison between two constants")
    return Filter(node, op, lv, rv, rhs_is_const=(rk == "const"))


def node_from_json(obj: Any) -> RirNode:
    kind, v = _variant(obj, "RirNode")
    if kind == "Scan":
        return Scan(int(v["rel"]))
    if kind == "Filter":
        return _filters(node_from_json(v["input"]), v["predicate"])
    if kind == "Project":
        cols = []
        for c in v["columns"]:
            ck, cv = _variant(c, "ProjectExpr")
            if ck != "Column":
                _unsupported(f"ProjectExpr::{ck}")
            cols.append(int(cv))
        return Project(node_from_json(v["input"]), cols)
    if kind == "Join":
        jt = v.get("join_type", "Inner")
        jt = jt if isinstance(jt, str) else _variant(jt, "JoinType")[0]
        if jt not in _JOIN:
            _unsupported(f"JoinType::{jt}")
        return Join(node_from_json(v["left"]), node_from_json(v["right"]), [int(k) for k in v["left_keys"]],
                    [int(k) for k in v["right_keys"]], _JOIN[jt])
    if kind == "Union":
        return Union([node_from_json(i) for i in v["inputs"]])
    if kind == "Diff":
        return Diff(node_from_json(v["left"]), node_from_json(v["right"]))
    if kind == "Distinct":
        return Distinct(node_from_json(v["input"]), [int(k) for k in v.get("key_cols", [])])
    if kind in ("ChainJoin", "MultiWayJoin"):
        return node_from_json(v["fallback"])   # the promoted forms keep the plain tree they came from
    _unsupported(f"RirNode::{kind}")


def _arity(node: RirNode, arities: Mapping[int, int]) -> int:
    try:
        return node.arity(arities)
    except KeyError as e:
        _invalid(f"no arity known for relation id {e.args[0]} (rel_arities)")


def plan_from_json(text: str | bytes | Mapping[str, Any], rel_names: Mapping[int, str] | None = None,
                   head_types: Mapping[str, list] | None = None) -> ExecutionPlan:
    """-> ``ExecutionPlan`` (``xlog_b200.plan``) with SCCs in the order of ``sccs`` /
    ``rules_by_scc``; when ``strata`` is present its order of SCC ids is the evaluation order
    (executor/mod.rs:1404-1469 walks strata, then their SCCs)."""
    doc = json.loads(text) if isinstance(text, (str, bytes)) else dict(text)
    names = {int(k): str(n) for k, n in (rel_names or doc.get("rel_names") or {}).items()}
    if not names:
        _invalid("rel_names (RelId -> relation name) is required")
    htypes = head_types or doc.get("head_types") or {}
    arities = {int(k): int(a) for k, a in (doc.get("rel_arities") or {}).items()}
    sccs_doc, rules_doc = doc.get("sccs"), doc.get("rules_by_scc")
    if not isinstance(sccs_doc, list) or not isinstance(rules_doc, list) or len(sccs_doc) != len(rules_doc):
        _invalid("sccs and rules_by_scc must be lists of the same length")
    by_name = {n: i for i, n in names.items()}
    # arities of derived relations that rel_arities lacks: taken from the first rule that defines them
    parsed = [[(r["head"], node_from_json(r["body"])) for r in rules] for rules in rules_doc]
    for _ in range(len(names) + 1):
        grew = False
        for rules in parsed:
            for head, body in rules:
                hid = by_name.get(head)
                if hid is None:
                    _invalid(f"head {head!r} has no RelId in rel_names")
                if hid in arities:
                    continue
                try:
                    arities[hid] = body.arity(arities)
                    grew = True
                except KeyError:
                    pass
        if not grew:
            break
    order = list(range(len(sccs_doc)))
    if doc.get("strata"):
        pos = {int(s["id"]): i for i, s in enumerate(sccs_doc)}
        order = []
        for st in doc["strata"]:
            for sid in st["sccs"]:
                if int(sid) not in pos:
                    _invalid(f"stratum {st.get('id')} names an unknown SCC {sid}")
                order.append(pos[int(sid)])
        if sorted(order) != list(range(len(sccs_doc))):
            _invalid("strata must name every SCC exactly once")
    sccs = []
    for i in order:
        s, rules = sccs_doc[i], []
        for head, body in parsed[i]:
            if head in htypes:
                types = [_TYPES[t] if isinstance(t, str) else int(t) for t in htypes[head]]
                try:
                    n = body.arity(arities)
                except KeyError:
                    n = len(types)  # an input's arity is not in rel_arities: nothing to check against
                if len(types) != n:
                    _invalid(f"head_types of {head!r} has {len(types)} columns, its rule bodies give {n}")
            else:
                types = [A.U32] * _arity(body, arities)
            rules.append(CompiledRule(head, body, tuple(types)))
        sccs.append(Scc(int(s["id"]), bool(s["is_recursive"]), rules))
    return ExecutionPlan(sccs, {n: i for i, n in names.items()})


# ---- the other direction: what the derive would print ------------------------------------------
_CMP_NAME = {v: k for k, v in _CMP.items()}
_JOIN_NAME = {v: k for k, v in _JOIN.items()}
_TYPE_NAME = {v: k for k, v in _TYPES.items()}


def node_to_json(n: RirNode) -> Any:
    if isinstance(n, Scan):
        return {"Scan": {"rel": n.rel}}
    if isinstance(n, Filter):
        rhs = {"Const": {"U64" if n.rhs > 0xFFFFFFFF else "U32": int(n.rhs)}} if n.rhs_is_const else {"Column": int(n.rhs)}
        pred = {"Compare": {"left": {"Column": n.lhs_col}, "op": _CMP_NAME[n.cmp], "right": rhs}}
        return {"Filter": {"input": node_to_json(n.input), "predicate": pred}}
    if isinstance(n, Project):
        return {"Project": {"input": node_to_json(n.input), "columns": [{"Column": int(c)} for c in n.columns]}}
    if isinstance(n, Join):
        return {"Join": {"left": node_to_json(n.left), "right": node_to_json(n.right), "left_keys": list(n.left_keys),
                         "right_keys": list(n.right_keys), "join_type": _JOIN_NAME[n.join_type]}}
    if isinstance(n, Union):
        return {"Union": {"inputs": [node_to_json(i) for i in n.inputs]}}
    if isinstance(n, Diff):
        return {"Diff": {"left": node_to_json(n.left), "right": node_to_json(n.right)}}
    if isinstance(n, Distinct):
        return {"Distinct": {"input": node_to_json(n.input), "key_cols": [int(k) for k in n.key_cols]}}
    raise TypeError(f"not a plan node: {n!r}")


def plan_to_json(plan: ExecutionPlan, indent: int | None = None) -> str:
    """The plan in the format ``plan_from_json`` reads (one stratum per SCC, in order)."""
    heads: dict[str, list] = {}
    doc = {"sccs": [], "strata": [], "rules_by_scc": [], "rel_names": {str(i): n for n, i in plan.rel_ids.items()}}
    for k, s in enumerate(plan.sccs):
        preds = sorted({r.head for r in s.rules})
        doc["sccs"].append({"id": s.id, "predicates": preds, "is_recursive": bool(s.is_recursive)})
        doc["strata"].append({"id": k, "sccs": [s.id]})
        doc["rules_by_scc"].append([{"head": r.head, "body": node_to_json(r.body)} for r in s.rules])
        for r in s.rules:
            heads[r.head] = [_TYPE_NAME[t] for t in r.head_types]
    doc["head_types"] = heads
    return json.dumps(doc, indent=indent)
