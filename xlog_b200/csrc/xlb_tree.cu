// The general evaluator behind xlb_execute_plan: a rule body is walked node by node, every node
// producing a column-major relation of any arity (up to XLB_MAX_ARITY columns), the way the
// reference's interpreter does (Executor::execute_node, crates/xlog-runtime/src/executor/
// node_dispatch.rs:98-319: Scan, Filter, Project, Join with `left.arity + right.arity` output
// columns, Union), with the semi-naive loop of execute_recursive_scc around it
// (executor/recursive.rs:447-957; one delta variant per recursive scan occurrence,
// executor/rewrite.rs:413-470).
//
// It takes the components the packed pipelines of xlb_exec.cu cannot: rules that keep more than
// two variables live, relations and heads of three and more columns, join keys of two columns as
// real joins, a Union below the top of a body, semi / anti joins against an arbitrary subtree.
// Scans are views (no copy), projections share column buffers, and every set operation is the
// operator the C ABI exports (rel_join, rel_union_many, rel_difference).  One rank only.
#include <map>
#include <memory>
#include <set>

#include "xlb_ops.h"
#include "xlb_tree.h"

namespace {

using RelPtr = std::unique_ptr<xlb_rel>;

struct Tree {
    xlb_ctx* c;
    xlb_run_stats* st;
    std::map<const xlb_node*, std::string> subst;  // one scan read from another relation (a delta)
};

xlb_rel* stored(xlb_ctx* c, const std::string& name) {
    auto it = c->store.find(name);
    return it == c->store.end() ? nullptr : it->second;
}

void store(xlb_ctx* c, const std::string& name, xlb_rel* rel) {
    auto it = c->store.find(name);
    if (it != c->store.end()) delete it->second;
    c->store[name] = rel;
    c->versions[name]++;
}

void unstore(xlb_ctx* c, const std::string& name) {
    auto it = c->store.find(name);
    if (it == c->store.end()) return;
    delete it->second;
    c->store.erase(it);
    c->versions[name]++;
}

RelPtr eval(Tree& t, const xlb_node* n) {
    xlb_ctx* c = t.c;
    if (!n) xlb_fail(XLB_ERR_INVALID, "plan node is null");
    switch (n->kind) {
        case XLB_NODE_SCAN: {
            std::string name;
            auto s = t.subst.find(n);
            if (s != t.subst.end()) name = s->second;
            else {
                auto nm = c->rel_names.find(n->rel_id);
                if (nm == c->rel_names.end()) xlb_fail(XLB_ERR_INVALID, "scan of unregistered relation id %u", n->rel_id);
                name = nm->second;
            }
            xlb_rel* r = stored(c, name);
            if (!r) xlb_fail(XLB_ERR_NOT_FOUND, "Missing relation: %s", name.c_str());
            return RelPtr(rel_view(c, r));
        }
        case XLB_NODE_FILTER: {
            RelPtr in = eval(t, n->input);
            if (n->cmp_lhs_col >= in->schema.arity || (!n->cmp_rhs_is_const && n->cmp_rhs >= in->schema.arity)) xlb_fail(XLB_ERR_INVALID, "filter column out of range");
            return RelPtr(rel_filter(c, in.get(), n->cmp, n->cmp_lhs_col, n->cmp_rhs_is_const != 0, n->cmp_rhs));
        }
        case XLB_NODE_PROJECT: {
            RelPtr in = eval(t, n->input);
            if (n->n_cols > XLB_MAX_ARITY) xlb_fail(XLB_ERR_INVALID, "projection of more than %u columns", XLB_MAX_ARITY);
            for (uint32_t i = 0; i < n->n_cols; ++i)
                if (n->cols[i] >= in->schema.arity) xlb_fail(XLB_ERR_INVALID, "projection column %u out of range", n->cols[i]);
            return RelPtr(rel_project(c, in.get(), n->cols, n->n_cols));
        }
        case XLB_NODE_JOIN: {
            if (n->join_type > XLB_JOIN_ANTI) xlb_fail(XLB_ERR_UNSUPPORTED, "join type %u is not built", n->join_type);
            RelPtr l = eval(t, n->left), r = eval(t, n->right);
            return RelPtr(rel_join(c, l.get(), r.get(), n->left_keys, n->right_keys, n->n_keys, (xlb_join_type)n->join_type));
        }
        case XLB_NODE_UNION: {
            if ((!n->inputs && n->n_inputs) || n->n_inputs == 0) xlb_fail(XLB_ERR_INVALID, "Union node without inputs");
            std::vector<RelPtr> parts;
            std::vector<const xlb_rel*> ptrs;
            for (uint32_t i = 0; i < n->n_inputs; ++i) {
                parts.push_back(eval(t, n->inputs[i]));
                ptrs.push_back(parts.back().get());
                if (parts.back()->schema.arity != parts[0]->schema.arity) xlb_fail(XLB_ERR_TYPE, "Union inputs differ in arity");
            }
            return RelPtr(rel_concat(c, ptrs.data(), (uint32_t)ptrs.size()));  // RirNode::Union concatenates; the head's union removes duplicates
        }
        case XLB_NODE_DIFF: {
            RelPtr l = eval(t, n->left), r = eval(t, n->right);
            return RelPtr(rel_difference(c, l.get(), r.get()));
        }
        case XLB_NODE_DISTINCT: {
            RelPtr in = eval(t, n->input);
            if (n->n_cols > XLB_MAX_ARITY) xlb_fail(XLB_ERR_INVALID, "more than %u key columns", XLB_MAX_ARITY);
            return RelPtr(rel_distinct(c, in.get(), n->cols, n->n_cols));
        }
    }
    xlb_fail(XLB_ERR_INVALID, "unknown plan node kind %u", n->kind);
}

void collect_scans(const xlb_node* n, std::vector<const xlb_node*>& out) {
    if (!n) return;
    switch (n->kind) {
        case XLB_NODE_SCAN: out.push_back(n); break;
        case XLB_NODE_FILTER:
        case XLB_NODE_DISTINCT:
        case XLB_NODE_PROJECT: collect_scans(n->input, out); break;
        case XLB_NODE_DIFF:
        case XLB_NODE_JOIN: collect_scans(n->left, out); collect_scans(n->right, out); break;
        case XLB_NODE_UNION:
            for (uint32_t i = 0; n->inputs && i < n->n_inputs; ++i) collect_scans(n->inputs[i], out);
            break;
    }
}

// One rule body evaluated; the result takes the head's column types (names and types of the
// body's columns are the plan's business: only widths must agree).
RelPtr eval_rule(Tree& t, const xlb_rule& rule) {
    RelPtr r = eval(t, rule.body);
    if (r->schema.arity != rule.head_schema.arity)
        xlb_fail(XLB_ERR_INVALID, "rule for %s: body yields %u columns, head has %u", rule.head, r->schema.arity, rule.head_schema.arity);
    for (uint32_t i = 0; i < r->schema.arity; ++i)
        if (type_width(r->schema.types[i]) != type_width(rule.head_schema.types[i]))
            xlb_fail(XLB_ERR_TYPE, "rule for %s: column %u does not have the width the head declares", rule.head, i);
    r->schema = rule.head_schema;
    t.st->candidate_tuples += r->rows;
    return r;
}

RelPtr union_of(xlb_ctx* c, const std::vector<RelPtr>& parts, const xlb_rel* first) {
    std::vector<const xlb_rel*> ins;
    if (first) ins.push_back(first);
    for (auto& p : parts) ins.push_back(p.get());
    return RelPtr(rel_union_many(c, ins.data(), (uint32_t)ins.size()));
}

}  // namespace

void run_scc_tree(xlb_ctx* c, const xlb_scc& scc, xlb_run_stats& st) {
    if (c->world > 1) xlb_fail(XLB_ERR_UNSUPPORTED, "rules over more than two live columns run on one rank");
    if (c->flags & XLB_FLAG_KEEP_DELTAS) xlb_fail(XLB_ERR_UNSUPPORTED, "XLB_FLAG_KEEP_DELTAS with rules over more than two live columns is not built");
    Tree t{c, &st, {}};
    std::vector<std::string> preds;
    std::map<std::string, xlb_schema> schema;
    for (uint32_t i = 0; i < scc.n_rules; ++i) {
        if (!scc.rules[i].head || !scc.rules[i].body) xlb_fail(XLB_ERR_INVALID, "rule %u of SCC %u is incomplete", i, scc.id);
        std::string h = scc.rules[i].head;
        if (!schema.count(h)) {
            preds.push_back(h);
            schema[h] = scc.rules[i].head_schema;
        }
    }
    std::sort(preds.begin(), preds.end());
    for (auto& p : preds)
        if (!stored(c, p)) store(c, p, rel_empty(c, schema[p]));  // recursive.rs:471-486
    auto delta_name = [](const std::string& p) { return "__delta_" + p; };
    for (auto& p : preds) unstore(c, delta_name(p));  // this evaluator always seeds: no resuming

    // every rule once on the stored relations (recursive.rs:308-438 for a non-recursive
    // component, :516-609 for the seeding pass of a recursive one)
    std::map<std::string, std::vector<RelPtr>> seeded;
    for (uint32_t i = 0; i < scc.n_rules; ++i) seeded[scc.rules[i].head].push_back(eval_rule(t, scc.rules[i]));
    for (auto& p : preds) {
        xlb_rel* full_old = stored(c, p);
        RelPtr full_new = union_of(c, seeded[p], full_old);
        if (scc.is_recursive) {
            RelPtr d0(full_old->rows == 0 ? rel_view(c, full_new.get()) : rel_difference(c, full_new.get(), full_old));
            store(c, delta_name(p), d0.release());
        }
        store(c, p, full_new.release());
    }
    seeded.clear();
    if (!scc.is_recursive) return;

    struct DropDeltas {  // the deltas are this loop's own: they never outlive it
        xlb_ctx* c;
        const std::vector<std::string>& preds;
        ~DropDeltas() {
            for (auto& p : preds) unstore(c, "__delta_" + p);
        }
    } drop{c, preds};
    bool fix = false;
    for (uint64_t it = 0; it < c->max_iterations; ++it) {  // recursive.rs:619-937
        st.iterations++;
        std::map<std::string, std::vector<RelPtr>> raw;
        for (uint32_t i = 0; i < scc.n_rules; ++i) {
            const xlb_rule& rule = scc.rules[i];
            std::vector<const xlb_node*> scans;
            collect_scans(rule.body, scans);
            for (const xlb_node* s : scans) {  // one variant per recursive scan occurrence (:636-664)
                auto nm = c->rel_names.find(s->rel_id);
                if (nm == c->rel_names.end() || !schema.count(nm->second)) continue;
                xlb_rel* d = stored(c, delta_name(nm->second));
                if (!d || d->rows == 0) continue;
                t.subst = {{s, delta_name(nm->second)}};
                raw[rule.head].push_back(eval_rule(t, rule));
                t.subst.clear();
            }
        }
        bool changed = false;
        for (auto& p : preds) {  // :735-858
            RelPtr dn;
            if (raw[p].empty()) dn.reset(rel_empty(c, schema[p]));
            else {
                RelPtr draw = union_of(c, raw[p], nullptr);
                dn.reset(draw->rows == 0 ? rel_empty(c, schema[p]) : rel_difference(c, draw.get(), stored(c, p)));  // :790
            }
            changed |= dn->rows != 0;
            store(c, delta_name(p), dn.release());
        }
        if (!changed) {  // :861-865
            fix = true;
            break;
        }
        for (auto& p : preds) {  // :868-937
            xlb_rel* d = stored(c, delta_name(p));
            if (d->rows == 0) continue;
            const xlb_rel* both[2] = {stored(c, p), d};
            store(c, p, rel_union_many(c, both, 2));
        }
    }
    if (!fix) xlb_fail(XLB_ERR_ITER_LIMIT, "Recursive SCC iteration limit (%llu) exceeded", (unsigned long long)c->max_iterations);
}
