// The executor behind xlb_execute_plan: relation store, rule flattening, join pipelines and
// the semi-naive loop of Executor::execute_recursive_scc
// (crates/xlog-runtime/src/executor/recursive.rs:447-957), host control in C++, all data on
// the device.
//
// Differences from the reference's control flow that do not change any result:
//   - a rule body (a tree of Scan/Join/Project/Filter nodes) is flattened to a conjunctive
//     query and evaluated as a left-deep pipeline that starts at the delta atom, so every
//     join probes with the small side and builds on a cached index;
//   - scans are views, never copies (the reference deep-copies, node_dispatch.rs:68-83);
//   - full relations stay sorted and unique, so the per-iteration difference and union are
//     merges, never a re-sort of the full relation (relational.rs:976-999 re-sorts).
#include <algorithm>
#include <atomic>
#include <cstring>
#include <deque>
#include <functional>
#include <set>
#include <tuple>

#include "xlb_comm.h"
#include "xlb_ops.h"
#include "xlb_tree.h"

void xlb_resolve_phase_timers(xlb_ctx* c);

// ------------------------------------------------------------------------------ store
struct CachedIndex {
    Index ix;
    uint64_t version = 0;   // store version of the relation the rows came from
    bool table_ok = false;  // hash table matches ix.S
    bool local = false;     // several ranks: built over the rows this rank holds, not over its hash partition
};
struct IndexCache {
    std::map<std::pair<std::string, int>, CachedIndex> m;
};

static IndexCache& cache(xlb_ctx* c) {
    if (!c->indexes) c->indexes = new IndexCache;
    return *c->indexes;
}

static void store_put(xlb_ctx* c, const std::string& name, xlb_rel* rel) {
    auto it = c->store.find(name);
    if (it != c->store.end()) delete it->second;
    c->store[name] = rel;
    c->versions[name]++;
}

static xlb_rel* store_get(xlb_ctx* c, const std::string& name) {
    auto it = c->store.find(name);
    return it == c->store.end() ? nullptr : it->second;
}

void xlb_exec_teardown(xlb_ctx* c) {
    for (auto& kv : c->store) delete kv.second;
    c->store.clear();
    delete c->indexes;
    c->indexes = nullptr;
    comm_destroy(c);
}

#define API_BEGIN(ctxp) \
    xlb_ctx* ctx__ = (ctxp); \
    try {
#define API_END()                                                \
    }                                                            \
    catch (const XlbError& e) {                                  \
        if (ctx__) ctx__->last_error = e.msg;                    \
        return e.st;                                             \
    }                                                            \
    catch (const std::bad_alloc&) {                              \
        if (ctx__) ctx__->last_error = "host allocation failed"; \
        return XLB_ERR_RESOURCE_EXHAUSTED;                       \
    }                                                            \
    return XLB_OK;

extern "C" xlb_status xlb_register_relation(xlb_ctx* c, uint32_t rel_id, const char* name) {
    if (!c || !name) return XLB_ERR_INVALID;
    c->rel_names[rel_id] = name;
    return XLB_OK;
}

extern "C" xlb_status xlb_store_put(xlb_ctx* c, const char* name, xlb_rel* rel) {
    if (!c || !name || !rel) return XLB_ERR_INVALID;
    API_BEGIN(c)
    if (rel->ctx != c) xlb_fail(XLB_ERR_INVALID, "relation belongs to another context");
    store_put(c, name, rel);
    API_END()
}

extern "C" xlb_status xlb_store_get(xlb_ctx* c, const char* name, const xlb_rel** rel) {
    if (!c || !name || !rel) return XLB_ERR_INVALID;
    xlb_rel* r = store_get(c, name);
    if (!r) {
        c->last_error = std::string("Missing relation: ") + name;
        return XLB_ERR_NOT_FOUND;
    }
    *rel = r;
    return XLB_OK;
}

extern "C" xlb_status xlb_store_remove(xlb_ctx* c, const char* name) {
    if (!c || !name) return XLB_ERR_INVALID;
    auto it = c->store.find(name);
    if (it == c->store.end()) return XLB_ERR_NOT_FOUND;
    delete it->second;
    c->store.erase(it);
    c->versions[name]++;
    return XLB_OK;
}

// ------------------------------------------------------------------------------ flattening
struct Atom {
    std::string rel;
    uint32_t arity;
    int var[2];
};
struct FilterC {
    uint32_t cmp;
    int lhs;
    bool rhs_const;
    uint64_t rhs;  // constant, or a variable id
    bool applied;
};
struct CheckC {  // semi / anti join against a stored relation: keep rows whose variable has / lacks a match
    std::string rel;
    int kc;
    int var;
    bool anti;
    bool applied;
};
struct FlatRule {
    std::string head;
    xlb_schema hs;
    std::vector<Atom> atoms;
    std::vector<FilterC> filters;
    std::vector<CheckC> checks;
    std::vector<int> head_vars;
    std::vector<char> start_ok;  // per atom: a pipeline that starts there keeps at most two columns live throughout
};

struct Flattener {
    xlb_ctx* c;
    std::vector<int> parent;
    FlatRule fr;
    int fresh() {
        parent.push_back((int)parent.size());
        return (int)parent.size() - 1;
    }
    int find(int x) {
        while (parent[x] != x) x = parent[x] = parent[parent[x]];
        return x;
    }
    void unite(int a, int b) { parent[find(a)] = find(b); }

    std::vector<int> walk(const xlb_node* n) {
        if (!n) xlb_fail(XLB_ERR_INVALID, "plan node is null");
        switch (n->kind) {
            case XLB_NODE_SCAN: {
                auto nm = c->rel_names.find(n->rel_id);
                if (nm == c->rel_names.end()) xlb_fail(XLB_ERR_INVALID, "scan of unregistered relation id %u", n->rel_id);
                xlb_rel* r = store_get(c, nm->second);
                if (!r) xlb_fail(XLB_ERR_NOT_FOUND, "Missing relation: %s", nm->second.c_str());
                if (!rel_packable(r->schema))
                    xlb_fail(XLB_ERR_UNSUPPORTED, "relation %s: plans take relations of one or two 32-bit columns", nm->second.c_str());
                Atom a;
                a.rel = nm->second;
                a.arity = r->schema.arity;
                std::vector<int> cols;
                for (uint32_t i = 0; i < a.arity; ++i) {
                    a.var[i] = fresh();
                    cols.push_back(a.var[i]);
                }
                fr.atoms.push_back(a);
                return cols;
            }
            case XLB_NODE_FILTER: {
                auto cols = walk(n->input);
                if (n->cmp_lhs_col >= cols.size() || (!n->cmp_rhs_is_const && n->cmp_rhs >= cols.size()))
                    xlb_fail(XLB_ERR_INVALID, "filter column out of range");
                FilterC f{n->cmp, cols[n->cmp_lhs_col], n->cmp_rhs_is_const != 0,
                          n->cmp_rhs_is_const ? n->cmp_rhs : (uint64_t)cols[n->cmp_rhs], false};
                fr.filters.push_back(f);
                return cols;
            }
            case XLB_NODE_PROJECT: {
                auto cols = walk(n->input);
                std::vector<int> out;
                for (uint32_t i = 0; i < n->n_cols; ++i) {
                    if (n->cols[i] >= cols.size()) xlb_fail(XLB_ERR_INVALID, "projection column %u out of range", n->cols[i]);
                    out.push_back(cols[n->cols[i]]);
                }
                return out;
            }
            case XLB_NODE_JOIN: {
                if (n->join_type == XLB_JOIN_SEMI || n->join_type == XLB_JOIN_ANTI) {
                    auto l = walk(n->left);
                    if (!n->right || n->right->kind != XLB_NODE_SCAN || n->n_keys != 1)
                        xlb_fail(XLB_ERR_UNSUPPORTED, "a semi / anti join takes a scanned relation on the right and one key column");
                    auto nm = c->rel_names.find(n->right->rel_id);
                    if (nm == c->rel_names.end()) xlb_fail(XLB_ERR_INVALID, "scan of unregistered relation id %u", n->right->rel_id);
                    xlb_rel* r = store_get(c, nm->second);
                    if (!r) xlb_fail(XLB_ERR_NOT_FOUND, "Missing relation: %s", nm->second.c_str());
                    if (!rel_packable(r->schema)) xlb_fail(XLB_ERR_UNSUPPORTED, "relation %s: plans take relations of one or two 32-bit columns", nm->second.c_str());
                    if (n->left_keys[0] >= l.size() || n->right_keys[0] >= r->schema.arity) xlb_fail(XLB_ERR_INVALID, "join key column out of range");
                    fr.checks.push_back(CheckC{nm->second, (int)n->right_keys[0], l[n->left_keys[0]], n->join_type == XLB_JOIN_ANTI, false});
                    return l;
                }
                if (n->join_type != XLB_JOIN_INNER) xlb_fail(XLB_ERR_UNSUPPORTED, "join type %u is not built", n->join_type);
                auto l = walk(n->left);
                auto r = walk(n->right);
                if (n->n_keys < 1 || n->n_keys > XLB_MAX_KEYS) xlb_fail(XLB_ERR_INVALID, "join needs 1..%u keys", XLB_MAX_KEYS);
                for (uint32_t i = 0; i < n->n_keys; ++i) {
                    if (n->left_keys[i] >= l.size() || n->right_keys[i] >= r.size()) xlb_fail(XLB_ERR_INVALID, "join key column out of range");
                    unite(l[n->left_keys[i]], r[n->right_keys[i]]);
                }
                l.insert(l.end(), r.begin(), r.end());
                return l;
            }
            case XLB_NODE_UNION:
            case XLB_NODE_DIFF:
            case XLB_NODE_DISTINCT:
                xlb_fail(XLB_ERR_UNSUPPORTED, "Union below the top of a body, Diff and Distinct nodes run on the general evaluator");
        }
        xlb_fail(XLB_ERR_INVALID, "unknown plan node kind %u", n->kind);
    }

    FlatRule run(const xlb_rule& rule) {
        fr.head = rule.head;
        fr.hs = rule.head_schema;
        fr.head_vars = walk(rule.body);
        for (auto& a : fr.atoms)
            for (uint32_t i = 0; i < a.arity; ++i) a.var[i] = find(a.var[i]);
        for (auto& f : fr.filters) {
            f.lhs = find(f.lhs);
            if (!f.rhs_const) f.rhs = (uint64_t)find((int)f.rhs);
        }
        for (auto& k : fr.checks) k.var = find(k.var);
        for (auto& v : fr.head_vars) v = find(v);
        if (fr.head_vars.size() != rule.head_schema.arity)
            xlb_fail(XLB_ERR_INVALID, "rule for %s: body yields %zu columns, head has %u", rule.head, fr.head_vars.size(), rule.head_schema.arity);
        if (!rel_packable(rule.head_schema))
            xlb_fail(XLB_ERR_UNSUPPORTED, "head %s: derived relations of one or two 32-bit columns are built", rule.head);
        return fr;
    }
};

// ------------------------------------------------------------------------------ indexes
struct RunState {
    xlb_run_stats st{};
    std::map<std::string, DenseState> dense;  // per head relation: its tuples as a bitmap, while they fit one
    std::map<std::string, TupleSet> tset;     // per head relation too wide for a bitmap: its tuples as a hash set
    // The new tuples a hash set hands back are unique but in no order.  They are sorted only for
    // heads whose sorted list a rule reads (`ordered_heads`); for the others an iteration's new
    // tuples stay a bag (`bag_novel` names the heads for which that holds right now) and the whole
    // relation is sorted once, when the component is done.
    std::set<std::string> ordered_heads, bag_novel;
    // Deltas of a head whose merge into the stored sorted list is put off: while the bitmap serves
    // the set difference and no rule reads the list, merging it every iteration is wasted work.
    struct Pending {
        std::vector<Keys> deltas;
        uint64_t rows = 0, bound = 0;
        bool bags = false;  // some of the deltas are in no order
    };
    std::map<std::string, Pending> pending;
    std::map<std::string, xlb_schema> head_schema;
    std::map<std::pair<std::string, int>, int> scans;  // scan joins run so far per (relation, key column)
    // rows of a stored relation with column `col` equal to `value`, collected while the relation was packed
    std::map<std::tuple<std::string, int, uint64_t>, Keys> prefiltered;
    // heads of 28 to 32 bits that moved from the hash set to bitmaps: an iteration brought more
    // candidates than a 256th of the domain, from where on passes over the bitmaps are the cheaper dedup
    std::set<std::string> wide_dense;
    std::set<std::string> keep_cols;  // stored relations a frontier loop will stream over as columns: not packed ahead of it
    // Several ranks.  Relations whose rows every rank holds in full while the running component is
    // evaluated: full copies of small stored relations (kept in the store under an alias name) and,
    // in replicated mode, the component's own heads.  A join against one of them needs no exchange.
    std::set<std::string> replicated;
    std::vector<std::string> aliases;  // alias names to remove from the store when the component is done
    // Replicated mode: the component's heads fit a small dense domain, so every rank keeps all of
    // their tuples (a bitmap and the sorted list), evaluates its share of every rule variant into a
    // candidate bitmap, and one OR over the ranks' bitmaps per head and iteration replaces the
    // counted all-to-all, the per-rank sort and the termination vote.
    struct Repl {
        bool on = false;
        uint32_t rank = 0, world = 1;
        int vb = 1;                             // bit length of the largest value any column holds, agreed by all ranks
        std::map<std::string, DenseSet> cand;   // per head: this iteration's candidate bitmap, shared by its rule variants
        std::set<std::string> sliced;           // stored relations of which every rank joins only its own rows
    } repl;
    // Partitioned mode: join chunks per rule variant, agreed by all ranks with the termination vote
    // of the iteration before (every rank runs the same number of exchanges).
    uint64_t agreed_chunks = 1, max_cand_local = 0;
};

static bool local_build(xlb_ctx* c, const RunState& rs, const std::string& name) {
    return c->comm_world > 1 && (c->world == 1 || rs.replicated.count(name));
}

// Rows of relation `name` arranged for a join on column kc: (key << 32) | other, sorted.
// kc 0 / 1: join index on that column.  kc == ROW_INDEX: the whole row is the key (membership of a
// pair whose two columns are both bound, as in the closing atom of a triangle).
constexpr int ROW_INDEX = 2;

static Keys index_rows(xlb_ctx* c, const xlb_rel* r, int kc) {
    Keys k = ops_rel_packed(c, r);
    if (kc == ROW_INDEX) {
        if (r->canonical) return k;
        Keys s = k;
        ops_sort(c, s, /*keep_input=*/true);
        return s;
    }
    if (r->schema.arity == 1) {
        Keys s = ops_remap(c, k, SRC_LO, SRC_ZERO);
        if (!r->canonical) ops_sort(c, s);
        return s;
    }
    if (kc == 0) {
        if (r->canonical) return k;  // a canonical relation is already ordered by its first column
        Keys s = k;
        ops_sort_by_high_half(c, s, /*keep_input=*/true);
        return s;
    }
    Keys s = ops_remap(c, k, SRC_LO, SRC_HI);
    if (r->canonical) ops_sort(c, s);           // kept fully sorted: later deltas are merged in
    else ops_sort_by_high_half(c, s);           // an index only needs its rows grouped by key
    return s;
}

// Is a current index of `name` on column kc in the cache?
static bool index_ready(xlb_ctx* c, const std::string& name, int kc, const RunState& rs) {
    auto it = cache(c).m.find({name, kc});
    return it != cache(c).m.end() && it->second.version == c->versions[name] && it->second.ix.built() && it->second.local == local_build(c, rs, name);
}

static const Index& get_index(xlb_ctx* c, const std::string& name, int kc, RunState& rs) {
    xlb_rel* r = store_get(c, name);
    if (!r) xlb_fail(XLB_ERR_NOT_FOUND, "Missing relation: %s", name.c_str());
    CachedIndex& ci = cache(c).m[{name, kc}];
    uint64_t ver = c->versions[name];
    PhaseTimer t(c, &rs.st.ms_join);
    // With several ranks an index is either over this rank's hash partition of the relation (rows
    // exchanged by their key first) or over the rows this rank holds (replicated relations, and
    // everything while a component runs in replicated mode): one kind never stands in for the other.
    const bool local = local_build(c, rs, name);
    const bool exchange = c->world > 1 && !local;
    if (ci.local != local) {
        ci = CachedIndex();
        ci.local = local;
    }
    if ((ci.version != ver || !ci.ix.built()) && (kc == 0 || kc == 1) && r->schema.arity == 2 && !r->canonical && !exchange && !(c->flags & XLB_FLAG_NO_DENSE)) {
        // A stored relation in no particular order whose join keys come from a small dense domain:
        // group its rows by counting instead of sorting them, and address the groups directly.
        Keys rows = ops_rel_packed(c, r);
        const uint64_t kb = rows.bound == ~0ull ? ~0ull : (kc == 0 ? rows.bound >> 32 : rows.bound & 0xFFFFFFFFull);
        int bits = 0;
        while (bits < 32 && (kb >> bits)) ++bits;
        if (kb != ~0ull && bits <= 26 && (1ull << bits) <= 4 * rows.n + 4096) {
            ci.ix = ops_index_build_direct(c, rows, kc == 0 ? SRC_HI : SRC_LO, bits);
            ci.version = ver;
            ci.table_ok = true;
            return ci.ix;
        }
    }
    if (ci.version != ver || !ci.ix.built()) {
        Keys part = index_rows(c, r, kc);
        if (exchange) part = comm_repartition(c, part, SRC_HI, /*sorted_unique_result=*/true, rs.st);
        ci.ix = Index();
        ci.ix.S = part.buf;
        ci.ix.n = part.n;
        ci.ix.bound = part.bound;
        ci.version = ver;
        ci.table_ok = false;
    }
    if (!ci.table_ok) {
        uint64_t b = ci.ix.bound;
        ci.ix = ops_index_build(c, ci.ix.S, ci.ix.n, kc == ROW_INDEX ? 0 : 32, Buf());
        ci.ix.bound = b;
        ci.table_ok = true;
    }
    return ci.ix;
}

// The full relation `name` grew by `delta` (disjoint from it): bring cached indexes along by
// merging instead of re-sorting.  Called before the store is updated; `new_full` is the merged
// relation that is about to be stored under a new version.
static void indexes_on_merge(xlb_ctx* c, const std::string& name, const xlb_rel* new_full, const Keys& delta, uint64_t new_version, RunState& rs) {
    for (auto& kv : cache(c).m) {
        if (kv.first.first != name) continue;
        CachedIndex& ci = kv.second;
        if (ci.version + 1 != new_version || !ci.ix.S) continue;  // stale already: rebuilt on demand
        int kc = kv.first.second;
        PhaseTimer t(c, &rs.st.ms_join);
        if (c->world > 1) {
            // the index copy is partitioned by its own key column: route the new rows there
            Keys d = new_full->schema.arity == 1 ? ops_remap(c, delta, SRC_LO, SRC_ZERO) : (kc != 1 ? delta : ops_remap(c, delta, SRC_LO, SRC_HI));
            if (d.buf == delta.buf) d = ops_copy(c, d);
            d = comm_repartition(c, d, SRC_HI, true, rs.st);
            Keys old;
            old.buf = ci.ix.S;
            old.n = ci.ix.n;
            old.bound = ci.ix.bound;
            Keys extra = ops_diff(c, d, old);
            Keys m = ops_merge_disjoint(c, old, extra);
            ci.ix = Index();
            ci.ix.S = m.buf;
            ci.ix.n = m.n;
            ci.ix.bound = m.bound;
        } else if (new_full->schema.arity == 2 && (kc == 0 || kc == ROW_INDEX)) {
            ci.ix = Index();
            ci.ix.S = new_full->packed;  // alias: canonical order is key order
            ci.ix.n = new_full->rows;
            ci.ix.bound = new_full->or_bound;
        } else {
            Keys d = new_full->schema.arity == 1 ? ops_remap(c, delta, SRC_LO, SRC_ZERO) : ops_remap(c, delta, SRC_LO, SRC_HI);
            if (new_full->schema.arity == 2) ops_sort(c, d);
            Keys old;
            old.buf = ci.ix.S;
            old.n = ci.ix.n;
            old.bound = ci.ix.bound;
            Keys m = ops_merge_disjoint(c, old, d);
            ci.ix = Index();
            ci.ix.S = m.buf;
            ci.ix.n = m.n;
            ci.ix.bound = m.bound;
        }
        ci.version = new_version;
        ci.table_ok = false;
    }
}

// ------------------------------------------------------------------------------ pipelines
struct ChunkTooBig {};

struct Bag {
    Keys k;
    int hi = -1, lo = -1;  // variable in each half (-1: none)
    int part = -1;         // several ranks: the variable whose owner rank holds each row (-1: unknown)
};

static int src_of(const Bag& b, int var) { return var == b.hi ? SRC_HI : SRC_LO; }

static void apply_ready_filters(xlb_ctx* c, FlatRule& fr, Bag& b, RunState& rs) {
    for (auto& k : fr.checks) {  // semi / anti joins whose variable is bound now
        if (k.applied || (k.var != b.hi && k.var != b.lo)) continue;
        const Index& ix = get_index(c, k.rel, k.kc, rs);
        int keysel = src_of(b, k.var);
        if (c->world > 1 && b.part != k.var && !rs.replicated.count(k.rel)) {  // the index is partitioned by its key: take the rows there
            b.k = comm_repartition(c, b.k, keysel, false, rs.st);
            b.part = k.var;
        }
        b.k = ops_semi_filter(c, b.k, keysel, ix, k.anti);
        k.applied = true;
    }
    for (auto& f : fr.filters) {
        if (f.applied) continue;
        bool lhs_ok = f.lhs == b.hi || f.lhs == b.lo;
        bool rhs_ok = f.rhs_const || (int)f.rhs == b.hi || (int)f.rhs == b.lo;
        if (!lhs_ok || !rhs_ok) continue;
        b.k = ops_filter(c, b.k, f.cmp, src_of(b, f.lhs), f.rhs_const, f.rhs_const ? f.rhs : (uint64_t)src_of(b, (int)f.rhs));
        f.applied = true;
    }
}

// Variables still needed once the atoms in `done` are consumed.
static std::set<int> needed_vars(const FlatRule& fr, const std::vector<bool>& done) {
    std::set<int> s;
    for (size_t i = 0; i < fr.atoms.size(); ++i)
        if (!done[i])
            for (uint32_t j = 0; j < fr.atoms[i].arity; ++j) s.insert(fr.atoms[i].var[j]);
    for (auto& f : fr.filters)
        if (!f.applied) {
            s.insert(f.lhs);
            if (!f.rhs_const) s.insert((int)f.rhs);
        }
    for (auto& k : fr.checks)
        if (!k.applied) s.insert(k.var);
    for (int v : fr.head_vars) s.insert(v);
    return s;
}

// The next atom a pipeline joins: the first one with exactly one column bound by the bag (hi, lo)
// such that what must stay live afterwards fits two columns.  pick = -1: there is none.
static void pick_next_atom(const FlatRule& fr, std::vector<bool>& done, int hi, int lo, int* pick_out, int* kc_out, std::set<int>* keep_out) {
    int pick = -1, kc = -1;
    std::set<int> keep;
    for (size_t i = 0; i < fr.atoms.size() && pick < 0; ++i) {
        if (done[i]) continue;
        const Atom& a = fr.atoms[i];
        int bound = 0, which = -1;
        for (uint32_t j = 0; j < a.arity; ++j)
            if (a.var[j] == hi || a.var[j] == lo) { bound++; which = (int)j; }
        if (a.arity == 2 && a.var[0] == a.var[1]) continue;
        if (bound != 1) continue;
        done[i] = true;
        std::set<int> need = needed_vars(fr, done);
        done[i] = false;
        std::set<int> avail{hi, lo};
        if (a.arity == 2) avail.insert(a.var[1 - which]);
        avail.erase(-1);
        std::set<int> k2;
        for (int v : need)
            if (avail.count(v)) k2.insert(v);
        if (k2.size() > 2) continue;
        pick = (int)i;
        kc = which;
        keep = k2;
    }
    *pick_out = pick;
    *kc_out = kc;
    *keep_out = keep;
}

// Would run_pipeline, started at atom `start`, get through the rule?  The same walk without data.
static bool pipeline_feasible(FlatRule fr /*by value: filter flags*/, size_t start) {
    std::vector<bool> done(fr.atoms.size(), false);
    const Atom& sa = fr.atoms[start];
    int hi = -1, lo = -1;
    if (sa.arity == 2) { hi = sa.var[0]; lo = sa.var[1]; }
    else lo = sa.var[0];
    done[start] = true;
    if (sa.arity == 2 && sa.var[0] == sa.var[1]) hi = -1;
    auto ready = [&]() {
        for (auto& k : fr.checks)
            if (!k.applied && (k.var == hi || k.var == lo)) k.applied = true;
        for (auto& f : fr.filters) {
            if (f.applied) continue;
            bool lhs_ok = f.lhs == hi || f.lhs == lo;
            bool rhs_ok = f.rhs_const || (int)f.rhs == hi || (int)f.rhs == lo;
            if (lhs_ok && rhs_ok) f.applied = true;
        }
    };
    ready();
    size_t remaining = fr.atoms.size() - 1;
    while (remaining) {
        bool filtered = false;
        for (size_t i = 0; i < fr.atoms.size(); ++i) {
            const Atom& a = fr.atoms[i];
            if (done[i] || a.arity != 2 || a.var[0] == a.var[1]) continue;
            bool b0 = a.var[0] == hi || a.var[0] == lo, b1 = a.var[1] == hi || a.var[1] == lo;
            if (!b0 || !b1) continue;
            done[i] = true;
            remaining--;
            filtered = true;
        }
        if (filtered) {
            ready();
            continue;
        }
        int pick = -1, kc = -1;
        std::set<int> keep;
        pick_next_atom(fr, done, hi, lo, &pick, &kc, &keep);
        if (pick < 0) return false;
        const Atom& a = fr.atoms[pick];
        done[pick] = true;
        remaining--;
        const int othervar = a.arity == 2 ? a.var[1 - kc] : -1;
        bool pending = false;
        for (auto& f : fr.filters) pending |= !f.applied;
        for (auto& k : fr.checks) pending |= !k.applied;
        int out_hi = -1, out_lo = -1;
        if (remaining == 0 && !pending) {
            if (fr.head_vars.size() == 2) { out_hi = fr.head_vars[0]; out_lo = fr.head_vars[1]; }
            else out_lo = fr.head_vars[0];
        } else {
            std::vector<int> kv(keep.begin(), keep.end());
            if (kv.size() == 2) { out_hi = kv[0]; out_lo = kv[1]; }
            else if (kv.size() == 1) out_lo = kv[0];
        }
        for (int v : {out_hi, out_lo})
            if (v >= 0 && v != hi && v != lo && v != othervar) return false;
        hi = out_hi;
        lo = out_lo;
        ready();
    }
    for (auto& f : fr.filters)
        if (!f.applied) return false;
    for (auto& k : fr.checks)
        if (!k.applied) return false;
    for (int v : fr.head_vars)
        if (v != hi && v != lo) return false;
    return true;
}

// Evaluate the rule with atom `start` read from `start_rows` (the delta, a chunk of it, or a
// full relation) and every other atom from the store.  Returns candidate head tuples (a bag).
// `sink`: when the last join writes the head layout directly and the head fits a dense domain, its
// output is marked into sink->set instead of being materialised (sink->used says so; the returned
// Keys then carries only the tuple count).
struct DenseSink {
    std::string head;
    const Keys* full = nullptr;   // the head relation before this iteration
    const Keys* novel = nullptr;  // what the iteration has found for it so far (disjoint from full)
    bool used = false;
    int home_var = -1;            // several ranks on hash partitions: the head variable whose value decides a tuple's owner
    DenseSet set;
    DenseState* state = nullptr;
    Keys known() const {  // stands for full + novel: row count and OR bound
        Keys k;
        k.n = full->n + novel->n;
        k.bound = (full->n ? full->bound : 0) | (novel->n ? novel->bound : 0);
        return k;
    }
};

static void install_full(xlb_ctx* c, const std::string& pred, const xlb_schema& hs, const Keys& full_new, const Keys* delta, RunState& rs);

// Row count and OR bound of a head relation with the deltas whose merge is put off; the buffer is
// the stored list, which lacks them: read it only through real_full.
static Keys full_view(xlb_ctx* c, RunState& rs, const std::string& head) {
    Keys k = ops_rel_packed(c, store_get(c, head));
    auto it = rs.pending.find(head);
    if (it != rs.pending.end() && it->second.rows) {
        k.bound = (k.n ? k.bound : 0) | it->second.bound;
        k.n += it->second.rows;
    }
    return k;
}

// Bring the stored list of `head` up to date: read it off the bitmap when that holds exactly the
// relation, else merge the deltas in.
static void materialize_full(xlb_ctx* c, RunState& rs, const std::string& head) {
    auto it = rs.pending.find(head);
    if (it == rs.pending.end() || it->second.rows == 0) return;
    RunState::Pending pd = std::move(it->second);
    rs.pending.erase(it);
    PhaseTimer t(c, &rs.st.ms_setops);
    Keys full = ops_rel_packed(c, store_get(c, head));
    const DenseState& ds = rs.dense[head];
    Keys merged;
    if (ds.valid && ds.rows == full.n + pd.rows) {
        merged = ops_dense_state_rows(c, ds, (full.n ? full.bound : 0) | pd.bound);
    } else {
        // the deltas are sorted and pairwise disjoint: two are merged, more are sorted together once
        Keys acc = pd.deltas[0];
        if (pd.deltas.size() == 2 && !pd.bags) acc = ops_merge_disjoint(c, acc, pd.deltas[1]);
        else if (pd.deltas.size() > 2 || pd.bags) {
            if (pd.deltas.size() > 1) acc = ops_concat(c, pd.deltas);
            else if (acc.buf.use_count() > 2) acc = ops_copy(c, acc);  // the sort below may scribble on its input: not on a stored delta
            pd.deltas.clear();
            ops_sort(c, acc);
        }
        merged = full.n ? ops_merge_disjoint(c, full, acc) : acc;
    }
    install_full(c, head, rs.head_schema[head], merged, nullptr, rs);
}

static Keys real_full(xlb_ctx* c, RunState& rs, const std::string& head) {
    materialize_full(c, rs, head);
    return ops_rel_packed(c, store_get(c, head));
}

// Widest domain (bits of both columns together) the bitmap route takes for `head`.
constexpr int DENSE_BITS = 27, WIDE_DENSE_BITS = 32;
static int dense_max_bits(const RunState& rs, const std::string& head) { return rs.wide_dense.count(head) ? WIDE_DENSE_BITS : DENSE_BITS; }

// The bitmap of `head` = full + novel over a domain of at least (hb, lb) bits, built or rebuilt
// when it is missing, too narrow, or out of step with the rows (a route that does not keep it up
// to date has added tuples).
static DenseState* dense_state(xlb_ctx* c, RunState& rs, const std::string& head, int hb, int lb, const Keys& full, const Keys& novel) {
    DenseState& ds = rs.dense[head];
    if (ds.valid && ds.hi_bits >= hb && ds.lo_bits >= lb && ds.rows == full.n + novel.n) return &ds;
    int nh = hb, nl = lb;
    if (ds.valid && std::max(hb, ds.hi_bits) + std::max(lb, ds.lo_bits) <= dense_max_bits(rs, head)) {
        nh = std::max(hb, ds.hi_bits);
        nl = std::max(lb, ds.lo_bits);
    }
    ops_dense_state_build(c, ds, nh, nl, real_full(c, rs, head), novel);  // (`full` may be a view: its list is read here)
    return &ds;
}

// Replicated mode: the fixed domain of a head (every column holds values of at most vb bits).
static void repl_bits(const RunState& rs, uint32_t arity, int* hb, int* lb) {
    *lb = rs.repl.vb;
    *hb = arity == 2 ? rs.repl.vb : 0;
}

// Replicated mode: the candidate bitmap of `head` for the running iteration (created on first use),
// with the head's own bitmap attached so that marking skips what the head holds.
static DenseSet& repl_cand(xlb_ctx* c, RunState& rs, const std::string& head, const Keys& full, const Keys& novel) {
    int hb, lb;
    repl_bits(rs, rs.head_schema[head].arity, &hb, &lb);
    DenseState* state = dense_state(c, rs, head, hb, lb, full, novel);
    auto it = rs.repl.cand.find(head);
    if (it == rs.repl.cand.end()) {
        DenseSet d = ops_dense_begin(c, state->hi_bits, state->lo_bits);
        d.shared = true;
        it = rs.repl.cand.emplace(head, d).first;
    }
    it->second.visited = state->visited->as<unsigned int>();
    return it->second;
}

// Replicated mode, once per head and iteration: OR the ranks' candidate bitmaps, then count, emit
// and record what the head lacks.  Every rank ends up with the same new tuples, so the emptiness
// of an iteration needs no vote.
static Keys repl_finish(xlb_ctx* c, RunState& rs, const std::string& head, const Keys& full) {
    Keys none;
    DenseSet& d = repl_cand(c, rs, head, full, none);
    {
        PhaseTimer t(c, &rs.st.ms_exchange);
        comm_or_bitmaps(c, d.bitmap->as<unsigned int>(), d.words);
        rs.st.exchange_bytes += d.words * 4 * (uint64_t)(rs.repl.world - 1);
    }
    // what other ranks marked is not in this rank's OR bound: the domain's is
    d.bound = (((1ull << d.hi_bits) - 1) << 32) | ((1ull << d.lo_bits) - 1);
    PhaseTimer t(c, &rs.st.ms_setops);
    Keys fresh = ops_dense_finish(c, d, full);
    rs.dense[head].rows += fresh.n;
    rs.st.candidate_tuples += d.marked;
    rs.repl.cand.erase(head);
    return fresh;
}

static void dense_sink_begin(xlb_ctx* c, RunState& rs, DenseSink* sink, int hb, int lb) {
    if (rs.repl.on) {
        DenseSet& shared = repl_cand(c, rs, sink->head, *sink->full, *sink->novel);
        sink->state = &rs.dense[sink->head];
        sink->set = shared;  // shares the bitmap and the count words
        sink->used = true;
        return;
    }
    sink->state = dense_state(c, rs, sink->head, hb, lb, *sink->full, *sink->novel);
    sink->set = ops_dense_begin_state(c, *sink->state);
    sink->used = true;
}

// `out_part`: which half of the returned head tuples decides the rank they already sit on
// (SRC_HI / SRC_LO), or -1 when they are placed by nothing the head keeps.
static Keys run_pipeline(xlb_ctx* c, FlatRule fr /*by value: filter flags*/, size_t start, const Keys& start_rows, bool start_is_set, int start_part_half, uint64_t limit,
                         RunState& rs, DenseSink* sink = nullptr, int* out_part = nullptr) {
    std::vector<bool> done(fr.atoms.size(), false);
    if (out_part) *out_part = -1;
    Bag bag;
    const Atom& sa = fr.atoms[start];
    // every key of the bag occurs once: rows of a one-column set (a join output may repeat keys)
    bool bag_keys_unique = start_is_set && sa.arity == 1;
    bag.k = start_rows;
    if (sa.arity == 2) { bag.hi = sa.var[0]; bag.lo = sa.var[1]; }
    else bag.lo = sa.var[0];
    if (start_part_half == SRC_HI) bag.part = bag.hi;
    else if (start_part_half == SRC_LO) bag.part = bag.lo;
    done[start] = true;
    if (sa.arity == 2 && sa.var[0] == sa.var[1]) {  // p(X, X)
        bag.k = ops_filter(c, bag.k, XLB_EQ, SRC_HI, false, SRC_LO);
        bag.hi = -1;
    }
    {
        PhaseTimer t(c, &rs.st.ms_join);
        apply_ready_filters(c, fr, bag, rs);
    }
    size_t remaining = fr.atoms.size() - 1;
    while (remaining) {
        // atoms with both columns bound are membership tests on the bag: apply them first
        bool filtered = false;
        for (size_t i = 0; i < fr.atoms.size(); ++i) {
            const Atom& a = fr.atoms[i];
            if (done[i] || a.arity != 2 || a.var[0] == a.var[1]) continue;
            bool b0 = a.var[0] == bag.hi || a.var[0] == bag.lo, b1 = a.var[1] == bag.hi || a.var[1] == bag.lo;
            if (!b0 || !b1) continue;
            const Index& ix = get_index(c, a.rel, ROW_INDEX, rs);
            Keys probe = bag.k;
            if (c->world > 1 && bag.part != a.var[0] && !rs.replicated.count(a.rel)) {  // the row index is partitioned by its first column
                PhaseTimer t(c, &rs.st.ms_exchange);
                probe = comm_repartition(c, probe, src_of(bag, a.var[0]), false, rs.st);
                bag.part = a.var[0];
            }
            PhaseTimer t(c, &rs.st.ms_join);
            Keys rowkeys = (a.var[0] == bag.hi) ? probe : ops_remap(c, probe, SRC_LO, SRC_HI);  // the atom's (col0, col1) order
            bag.k = ops_semi_filter(c, probe, SRC_HI, ix, false, rowkeys.ptr());
            done[i] = true;
            remaining--;
            filtered = true;
        }
        if (filtered) {
            apply_ready_filters(c, fr, bag, rs);
            continue;
        }
        // next atom: exactly one of its columns is bound by the bag, and what must stay live fits two columns
        int pick = -1, kc = -1;
        std::set<int> keep;
        pick_next_atom(fr, done, bag.hi, bag.lo, &pick, &kc, &keep);
        if (pick < 0)
            xlb_fail(XLB_ERR_UNSUPPORTED, "rule for %s: no join order keeps at most two live columns with single-column keys", fr.head.c_str());
        const Atom& a = fr.atoms[pick];
        done[pick] = true;
        remaining--;
        int keyvar = a.var[kc];
        int othervar = a.arity == 2 ? a.var[1 - kc] : -1;
        // output layout: the head's layout when this is the last step and nothing is pending
        bool last = remaining == 0;
        bool pending = false;
        for (auto& f : fr.filters)
            if (!f.applied) pending = true;
        for (auto& k : fr.checks)
            if (!k.applied) pending = true;
        int out_hi = -1, out_lo = -1;
        if (last && !pending) {
            if (fr.head_vars.size() == 2) { out_hi = fr.head_vars[0]; out_lo = fr.head_vars[1]; }
            else out_lo = fr.head_vars[0];
        } else {
            std::vector<int> kv(keep.begin(), keep.end());
            if (kv.size() == 2) { out_hi = kv[0]; out_lo = kv[1]; }
            else if (kv.size() == 1) out_lo = kv[0];
        }
        auto sel = [&](int var) -> int {
            if (var < 0) return SRC_ZERO;
            if (var == bag.hi) return SRC_HI;
            if (var == bag.lo) return SRC_LO;
            if (var == othervar) return SRC_OTHER;
            xlb_fail(XLB_ERR_INVALID, "internal: variable %d is not available at this join step", var);
        };
        int hs = sel(out_hi), ls = sel(out_lo);
        Bag nb;
        Keys probe = bag.k;
        int keysel = src_of(bag, keyvar);
        // a relation every rank holds in full is joined where the bag's rows are; any other sits on
        // the owners of its join keys, and the bag goes there first
        const bool rel_everywhere = c->world > 1 && rs.replicated.count(a.rel);
        int part_after = keyvar;
        if (rel_everywhere) part_after = bag.part;
        else if (c->world > 1 && bag.part != keyvar) {
            PhaseTimer t(c, &rs.st.ms_exchange);
            probe = comm_repartition(c, probe, keysel, false, rs.st);
        }
        // Sides swapped: when the bag gives nothing but the join key and the relation has no index
        // yet, stream over the relation instead of building one.  An index costs about a dozen
        // such scans (three when the relation is already in key order), so scan that often, then
        // build it: at most twice the cost of the better choice, whatever the number of iterations.
        auto rel_src = [&](int src) { return src == keysel ? 0 : src == SRC_OTHER ? 1 : src == SRC_ZERO ? 2 : -1; };
        // (a bag that repeats keys would yield every row once per repeat through an index: keep to
        // bags without repeats so that both routes count the same candidates)
        if (c->world == 1 && bag_keys_unique && !(c->flags & XLB_FLAG_NO_DENSE) && a.arity == 2 && rel_src(hs) >= 0 && rel_src(ls) >= 0 && probe.bound != ~0ull) {
            xlb_rel* r = store_get(c, a.rel);
            const uint64_t kb = keysel == SRC_HI ? probe.bound >> 32 : probe.bound & 0xFFFFFFFFull;
            int key_bits = 0;
            while (key_bits < 32 && (kb >> key_bits)) ++key_bits;
            const bool indexed = index_ready(c, a.rel, kc, rs);
            int& scans = rs.scans[{a.rel, kc}];
            if (r && !indexed && key_bits <= 27 && scans < (r->canonical && kc == 0 ? 3 : 12)) {
                ++scans;
                PhaseTimer t(c, &rs.st.ms_join);
                Keys rows = ops_rel_packed(c, r);
                const int rel_keysel = kc == 0 ? SRC_HI : SRC_LO;
                int hb = 0, lb = 0;
                Keys shape;
                shape.n = 1;
                shape.bound = ops_scan_join_bound(probe, keysel, rows, rel_keysel, rel_src(hs), rel_src(ls));
                if (sink && last && !pending && (rs.repl.on || ops_dense_bits(shape, sink->known(), &hb, &lb, dense_max_bits(rs, sink->head)))) {
                    dense_sink_begin(c, rs, sink, hb, lb);
                    ops_scan_join_mark(c, probe, keysel, key_bits, rows, rel_keysel, rel_src(hs), rel_src(ls), sink->set);
                    Keys marked;  // no rows and no count: both are in the sink
                    marked.bound = shape.bound;
                    return marked;
                }
                nb.k = ops_scan_join(c, probe, keysel, key_bits, rows, rel_keysel, rel_src(hs), rel_src(ls));
                nb.part = part_after;
                if (limit && nb.k.n > limit && start_rows.n > 1) throw ChunkTooBig{};
                nb.hi = out_hi;
                nb.lo = out_lo;
                if (nb.part != nb.hi && nb.part != nb.lo) nb.part = -1;  // the step dropped the variable the rows were placed by
                bag = nb;
                bag_keys_unique = false;
                apply_ready_filters(c, fr, bag, rs);
                continue;
            }
        }
        const Index& ix = get_index(c, a.rel, kc, rs);
        {
            PhaseTimer t(c, &rs.st.ms_join);
            int hb = 0, lb = 0;
            Keys shape;  // stands for the rows this step would produce: only their OR bound matters here
            shape.n = 1;
            shape.bound = ops_expand_bound(probe, ix, hs, ls);
            // (on hash partitions a rank marks into the bitmap of its own shard, which takes tuples
            // that are already where they belong: only a head that moved to wide bitmaps, and only
            // when this step leaves its rows placed by the head's owner column)
            const bool marks_own_shard = c->world == 1 || (sink && rs.wide_dense.count(sink->head) && sink->home_var >= 0 && part_after == sink->home_var);
            if (sink && last && !pending && marks_own_shard && !(c->flags & XLB_FLAG_NO_DENSE) && (rs.repl.on || ops_dense_bits(shape, sink->known(), &hb, &lb, dense_max_bits(rs, sink->head)))) {
                dense_sink_begin(c, rs, sink, hb, lb);
                ops_join_expand_mark(c, probe, keysel, ix, hs, ls, sink->set);
                Keys marked;  // no rows and no count: both are in the sink
                marked.bound = shape.bound;
                return marked;
            }
            nb.k = ops_join_expand(c, probe, keysel, nullptr, ix, hs, ls);
            nb.part = part_after;
            if (limit && nb.k.n > limit && start_rows.n > 1) throw ChunkTooBig{};
            nb.hi = out_hi;
            nb.lo = out_lo;
            if (nb.part != nb.hi && nb.part != nb.lo) nb.part = -1;  // the step dropped the variable the rows were placed by
            bag = nb;
            bag_keys_unique = false;
            apply_ready_filters(c, fr, bag, rs);
        }
    }
    // head layout
    int want_hi = fr.head_vars.size() == 2 ? fr.head_vars[0] : -1;
    int want_lo = fr.head_vars.size() == 2 ? fr.head_vars[1] : fr.head_vars[0];
    for (auto& f : fr.filters)
        if (!f.applied) xlb_fail(XLB_ERR_UNSUPPORTED, "rule for %s: a filter refers to a column that no atom binds", fr.head.c_str());
    for (auto& k : fr.checks)
        if (!k.applied) xlb_fail(XLB_ERR_UNSUPPORTED, "rule for %s: a semi / anti join key is not live where it could be applied", fr.head.c_str());
    if (bag.hi != want_hi || bag.lo != want_lo) {
        auto sel = [&](int var) -> int {
            if (var < 0) return SRC_ZERO;
            if (var == bag.hi) return SRC_HI;
            if (var == bag.lo) return SRC_LO;
            xlb_fail(XLB_ERR_UNSUPPORTED, "rule for %s: a head column is not bound by the body", fr.head.c_str());
        };
        PhaseTimer t(c, &rs.st.ms_join);
        bag.k = ops_remap(c, bag.k, sel(want_hi), sel(want_lo));
    }
    if (out_part) *out_part = bag.part < 0 ? -1 : bag.part == want_hi ? SRC_HI : bag.part == want_lo ? SRC_LO : -1;
    return bag.k;
}

// Candidates of one rule variant -> sorted unique tuples not in `full`, merged into `novel`.
// The start rows are processed in chunks so no join output exceeds the configured bound.
static void eval_variant(xlb_ctx* c, const FlatRule& fr_in, size_t start, const Keys& start_rows_in, bool start_is_stored, int start_part_half,
                         const Keys& full, int home_sel, Keys& novel, RunState& rs) {
    FlatRule fr = fr_in;
    Keys start_rows = start_rows_in;
    if (start_is_stored) {
        // `atom(.., c, ..)` with a constant: fetch the matching rows through the atom's join index
        // instead of filtering the whole relation
        const Atom& sa = fr.atoms[start];
        for (auto& f : fr.filters) {
            if (f.applied || f.cmp != XLB_EQ || !f.rhs_const || f.rhs > 0xFFFFFFFFull) continue;
            int kc = -1;
            for (uint32_t j = 0; j < sa.arity; ++j)
                if (sa.var[j] == f.lhs) kc = (int)j;
            if (kc < 0 || (sa.arity == 2 && sa.var[0] == sa.var[1])) continue;
            // one filtering pass over the relation costs far less than building its index
            if (c->world == 1 && !index_ready(c, sa.rel, kc, rs)) continue;
            const Index& ix = get_index(c, sa.rel, kc, rs);
            uint64_t key = f.rhs;
            Keys probe = ops_from_host(c, &key, 1);
            int hs = SRC_ZERO, ls = SRC_LO;
            if (sa.arity == 2) {
                hs = kc == 0 ? SRC_LO : SRC_OTHER;
                ls = kc == 1 ? SRC_LO : SRC_OTHER;
            }
            PhaseTimer t(c, &rs.st.ms_join);
            start_rows = ops_join_expand(c, probe, SRC_LO, nullptr, ix, hs, ls);
            start_part_half = sa.arity == 2 ? (kc == 0 ? SRC_HI : SRC_LO) : SRC_LO;
            f.applied = true;
            break;
        }
    }
    // Several ranks, start rows that every rank holds in full (a replicated relation; in replicated
    // mode also a delta): each rank takes its slice of them, unless the rule joins a relation of
    // which every rank holds only its own rows, which splits the work already.
    {
        const std::string& srel = fr.atoms[start].rel;
        const bool everywhere = c->comm_world > 1 && (rs.repl.on ? !rs.repl.sliced.count(srel) : (start_is_stored && rs.replicated.count(srel) > 0));
        bool split_by_rule = false;
        if (rs.repl.on)
            for (auto& a : fr.atoms) split_by_rule |= rs.repl.sliced.count(a.rel) > 0;
        if (everywhere && !split_by_rule) {
            const uint64_t n = start_rows.n, lo = n * c->comm_rank / c->comm_world, hi = n * (c->comm_rank + 1) / c->comm_world;
            if (lo != 0 || hi != n) start_rows = ops_slice(c, start_rows, lo, hi);
            start_part_half = -1;  // a slice by position: its rows are placed by no column
        }
    }
    if (start_rows.n == 0 && c->world == 1) return;
    bool start_is_set = true;  // a delta is; a stored relation when it is certified sorted and unique
    if (start_is_stored) {
        xlb_rel* sr = store_get(c, fr.atoms[start].rel);
        start_is_set = sr && sr->canonical;
    }
    uint64_t limit = c->join_chunk;
    if (!limit) {
        uint64_t room = c->budget > c->allocated ? c->budget - c->allocated : 0;
        limit = std::max<uint64_t>(room / (8 * 8), 1u << 20);  // a chunk is held, sorted and merged: ~8 copies
    }
    // With several ranks on hash partitions every rank runs the same sequence of exchanges, so the
    // number of chunks is the one all ranks agreed on with the last vote, and no chunk is split.
    const bool fixed_chunks = c->world > 1;
    uint64_t chunk = std::max<uint64_t>(start_rows.n, 1), at = 0;
    uint64_t rounds_left = 1;
    if (fixed_chunks) {
        rounds_left = std::max<uint64_t>(rs.agreed_chunks, 1);
        chunk = std::max<uint64_t>((start_rows.n + rounds_left - 1) / rounds_left, 1);
        limit = 0;
    }
    while (fixed_chunks ? rounds_left > 0 : at < start_rows.n) {
        if (fixed_chunks) --rounds_left;
        uint64_t hi = std::min(start_rows.n, at + chunk);
        Keys part = (at == 0 && hi == start_rows.n) ? start_rows : ops_slice(c, start_rows, at, hi);
        Keys cand;
        DenseSink sink;
        sink.head = fr.head;
        sink.full = &full;
        sink.novel = &novel;
        if (c->world > 1 && !fr.head_vars.empty()) sink.home_var = home_sel == SRC_HI && fr.head_vars.size() == 2 ? fr.head_vars[0] : fr.head_vars.back();
        int placed = -1;
        try {
            cand = run_pipeline(c, fr, start, part, start_is_set, start_part_half, limit, rs, &sink, &placed);
        } catch (const ChunkTooBig&) {
            chunk = std::max<uint64_t>((hi - at) / 2, 1);
            continue;
        }
        at = hi;
        if (sink.used && rs.repl.on) {
            // marked into the head's shared candidate bitmap: counted and emitted once per iteration
            rs.repl.cand[fr.head].bound |= sink.set.bound;
            continue;
        }
        if (sink.used) {
            // the last join marked its tuples in the bitmap already (single rank only); how many
            // there were comes back with the count of the new ones
            if (rs.wide_dense.count(fr.head)) rs.tset.erase(fr.head);  // the hash set this head started with: gigabytes, not kept up to date from here on
            if (rs.bag_novel.erase(fr.head) && novel.n) {  // an earlier variant (hash-set route) left a bag: order it before the merge below
                PhaseTimer t(c, &rs.st.ms_sort);
                ops_sort(c, novel, /*keep_input=*/true);
            }
            PhaseTimer t(c, &rs.st.ms_setops);
            Keys fresh = ops_dense_finish(c, sink.set, full);
            sink.state->rows += fresh.n;
            rs.st.candidate_tuples += sink.set.marked;
            novel = novel.n ? ops_union(c, novel, fresh) : fresh;
            continue;
        }
        rs.st.candidate_tuples += cand.n;
        rs.max_cand_local = std::max(rs.max_cand_local, cand.n);
        if (rs.repl.on) {
            PhaseTimer t(c, &rs.st.ms_setops);
            ops_dense_mark_into(c, repl_cand(c, rs, fr.head, full, novel), cand);
            continue;
        }
        if (c->world > 1 && placed != home_sel) {
            PhaseTimer t(c, &rs.st.ms_exchange);
            cand = comm_repartition(c, cand, home_sel, false, rs.st);
        }
        if (cand.n == 0) continue;
        Keys fresh;
        int hb = 0, lb = 0;
        if (!(c->flags & XLB_FLAG_NO_DENSE) && ops_dense_bits(cand, sink.known(), &hb, &lb, dense_max_bits(rs, fr.head))) {
            // small dense domain: sort + dedup + difference on a bitmap
            PhaseTimer t(c, &rs.st.ms_setops);
            DenseState* ds = dense_state(c, rs, fr.head, hb, lb, full, novel);
            fresh = ops_dense_novel(c, cand, full, ds->hi_bits, ds->lo_bits, ds->visited->as<unsigned int>());
            ds->rows += fresh.n;
        } else if (!(c->flags & XLB_FLAG_NO_TUPLE_SET)) {
            // the head as a hash set: a candidate is new when its insertion takes an empty slot, and
            // only the new tuples are sorted
            rs.dense[fr.head].valid = false;
            TupleSet& ts = rs.tset[fr.head];
            {
                PhaseTimer t(c, &rs.st.ms_setops);
                if (!ts.valid || ts.rows != full.n + novel.n) ops_tuple_set_build(c, ts, real_full(c, rs, fr.head), novel, cand.n);
                fresh = ops_tuple_set_novel(c, ts, cand);
            }
            // A domain of 28 to 32 bits: once one variant brings more candidates than a 256th of
            // the domain, passes over bitmaps of the whole domain cost less than hashing every
            // candidate, the last join can mark its output without writing it, and the new tuples
            // come out in order.  From the next variant on this head takes the bitmap route (its
            // bitmap is built from the rows then; the hash set is dropped at the end of the iteration).
            const bool own_shard = c->world == 1 || (placed == home_sel && !(c->flags & XLB_FLAG_SHUFFLE_ONLY));  // several ranks: only tuples that need no exchange
            if (own_shard && !(c->flags & XLB_FLAG_NO_DENSE) && !rs.wide_dense.count(fr.head) && !getenv("XLB_NO_WIDE_DENSE") &&
                ops_dense_bits(cand, sink.known(), &hb, &lb, WIDE_DENSE_BITS) && cand.n >= ((1ull << (hb + lb)) / 256) / c->comm_world) {  // (a rank touches its share of the domain only)
                const uint64_t bitmaps = 4 * ((1ull << (hb + lb)) / 8);  // head, candidates, and room for a rebuild
                if (!c->budget || c->allocated + bitmaps <= c->budget) rs.wide_dense.insert(fr.head);
            }
            if (!rs.ordered_heads.count(fr.head)) {
                // unique, disjoint from everything found before: joining the bags is their union
                novel = novel.n ? ops_concat(c, {novel, fresh}) : fresh;
                rs.bag_novel.insert(fr.head);
                continue;
            }
            PhaseTimer t(c, &rs.st.ms_sort);
            ops_sort(c, fresh);
        } else {
            rs.dense[fr.head].valid = false;  // this route does not keep the bitmap: rebuilt when next wanted
            rs.tset[fr.head].valid = false;
            {
                PhaseTimer t(c, &rs.st.ms_sort);
                ops_sort(c, cand, /*keep_input=*/cand.buf == start_rows.buf);  // a single-atom body hands over a stored relation
            }
            PhaseTimer t(c, &rs.st.ms_setops);
            fresh = ops_dedup_diff(c, cand, real_full(c, rs, fr.head));  // duplicates dropped and `full` subtracted in one merge pass
        }
        if (rs.bag_novel.erase(fr.head) && novel.n) {  // an earlier variant left a bag: order it before the merge below
            PhaseTimer t(c, &rs.st.ms_sort);
            ops_sort(c, novel, /*keep_input=*/true);
        }
        PhaseTimer t2(c, &rs.st.ms_setops);
        novel = novel.n ? ops_union(c, novel, fresh) : fresh;
    }
}

// Orders the new tuples of `head` if they are still a bag (a merge into a sorted list is next).
static void order_novel(xlb_ctx* c, RunState& rs, const std::string& head, Keys& d) {
    if (!rs.bag_novel.erase(head) || d.n < 2) return;
    PhaseTimer t(c, &rs.st.ms_sort);
    ops_sort(c, d, /*keep_input=*/true);  // (a stored delta may share the buffer)
}

// The constant filter of a single-atom rule over `atom` (`rel(c, Y)`): column and value, or false.
static bool single_atom_filter(const FlatRule& fr, int* col, uint64_t* value, size_t* which) {
    if (fr.atoms.size() != 1 || fr.atoms[0].arity != 2 || fr.atoms[0].var[0] == fr.atoms[0].var[1]) return false;
    for (size_t i = 0; i < fr.filters.size(); ++i) {
        const FilterC& f = fr.filters[i];
        if (f.applied || f.cmp != XLB_EQ || !f.rhs_const || f.rhs > 0xFFFFFFFFull) continue;
        for (int j = 0; j < 2; ++j)
            if (fr.atoms[0].var[j] == f.lhs) {
                *col = j;
                *value = f.rhs;
                *which = i;
                return true;
            }
    }
    return false;
}

// Relation `name` before its first use by a rule (it may have come as columns).  When a
// single-atom rule filters it by a constant, the matching rows are collected in the pass over the
// columns that packs it.  A relation in rs.keep_cols is not packed at all: that pass only reads it
// (bound of its values, filtered rows), and the returned keys carry no rows unless need_rows.
static Keys packed_for_rules(xlb_ctx* c, const std::string& name, const std::vector<FlatRule>& rules, RunState& rs, bool need_rows = true) {
    xlb_rel* r = store_get(c, name);
    const bool keep = rs.keep_cols.count(name) != 0;
    if (!r->packed && (!keep || r->or_bound == ~0ull)) {
        bool done = false;
        for (auto& fr : rules) {
            int col;
            uint64_t value;
            size_t which;
            if (fr.atoms.size() != 1 || fr.atoms[0].rel != name || !single_atom_filter(fr, &col, &value, &which)) continue;
            Keys rows;
            if (keep ? ops_rel_bound_filtered(c, r, col, (uint32_t)value, &rows) : ops_rel_packed_filtered(c, r, col, (uint32_t)value, &rows)) {
                rs.prefiltered[std::make_tuple(name, col, value)] = rows;
                done = true;
            }
            break;
        }
        if (keep && !done) ops_rel_bound_filtered(c, r, -1, 0, nullptr);
    }
    if (keep && !need_rows && !r->packed && r->or_bound != ~0ull) {
        Keys k;
        k.n = r->rows;
        k.bound = r->or_bound;
        return k;
    }
    return ops_rel_packed(c, r);
}

static xlb_rel* empty_rel(xlb_ctx* c, const xlb_schema& s) {
    Keys k;
    k.buf = make_buf(c, 0);
    return ops_rel_from_keys(c, s, k, true);
}

static Keys canonical_keys(xlb_ctx* c, const xlb_rel* r, RunState& rs) {
    Keys k = ops_rel_packed(c, r);
    if (r->canonical) return k;
    {
        PhaseTimer t(c, &rs.st.ms_sort);
        ops_sort(c, k, /*keep_input=*/true);
    }
    PhaseTimer t(c, &rs.st.ms_setops);
    ops_dedup_sorted(c, k);
    return k;
}

// Which half of a head tuple decides its owner rank: the column its delta is probed by first.
static int home_half(const std::vector<FlatRule>& rules, const std::string& pred, const std::set<std::string>& rec, uint32_t arity) {
    if (arity == 1) return SRC_LO;
    int votes[2] = {0, 0};
    for (auto& fr : rules)
        for (size_t i = 0; i < fr.atoms.size(); ++i) {
            const Atom& a = fr.atoms[i];
            if (a.rel != pred || !rec.count(a.rel)) continue;
            for (size_t j = 0; j < fr.atoms.size(); ++j) {
                if (j == i) continue;
                for (uint32_t q = 0; q < fr.atoms[j].arity; ++q)
                    for (uint32_t p = 0; p < a.arity; ++p)
                        if (fr.atoms[j].var[q] == a.var[p]) votes[p]++;
            }
        }
    return votes[1] > votes[0] ? SRC_LO : SRC_HI;
}

// Start atom of a rule evaluated on full relations: the smallest one probes, the others build.
static size_t pick_seed_start(xlb_ctx* c, const FlatRule& fr) {
    if (c->world > 1) return 0;  // every rank must walk the same pipeline: shard sizes differ, so no size rule
    size_t best = 0;
    uint64_t rows = ~0ull;
    for (size_t i = 0; i < fr.atoms.size(); ++i) {
        if (i < fr.start_ok.size() && !fr.start_ok[i]) continue;  // no pipeline from there keeps two columns
        xlb_rel* r = store_get(c, fr.atoms[i].rel);
        uint64_t n = r ? r->rows : 0;
        if (n < rows) { rows = n; best = i; }
    }
    return best;
}

static void install_full(xlb_ctx* c, const std::string& pred, const xlb_schema& hs, const Keys& full_new, const Keys* delta, RunState& rs) {
    xlb_rel* nr = ops_rel_from_keys(c, hs, full_new, true);
    if (delta) indexes_on_merge(c, pred, nr, *delta, c->versions[pred] + 1, rs);
    store_put(c, pred, nr);
}

// Rules evaluated once on full relations; per head one union (recursive.rs:308-438 for a
// non-recursive SCC, :516-609 for the seeding pass of a recursive one).
static void seed_pass(xlb_ctx* c, const std::vector<FlatRule>& rules, const std::vector<std::string>& preds, const std::set<std::string>& rec,
                      std::map<std::string, xlb_schema>& schema, std::map<std::string, int>& home, bool make_delta, RunState& rs) {
    std::map<std::string, Keys> novel;
    for (auto& fr : rules) {
        bool any_empty = false;
        for (auto& a : fr.atoms) {
            xlb_rel* r = store_get(c, a.rel);
            if (!r || (r->rows == 0 && c->world == 1)) any_empty = true;
        }
        if (any_empty) continue;
        size_t start = pick_seed_start(c, fr);
        Keys rows = packed_for_rules(c, fr.atoms[start].rel, rules, rs, /*need_rows=*/false);
        FlatRule use = fr;
        {
            int col;
            uint64_t value;
            size_t which;
            if (single_atom_filter(fr, &col, &value, &which)) {
                auto hit = rs.prefiltered.find(std::make_tuple(fr.atoms[0].rel, col, value));
                if (hit != rs.prefiltered.end()) {  // collected in the first pass over the relation
                    rows = hit->second;
                    use.filters[which].applied = true;
                }
            }
        }
        if (!rows.buf) rows = ops_rel_packed(c, store_get(c, fr.atoms[start].rel));
        Keys full_old = canonical_keys(c, store_get(c, fr.head), rs);
        eval_variant(c, use, start, rows, true, rec.count(fr.atoms[start].rel) ? home[fr.atoms[start].rel] : -1, full_old, home[fr.head], novel[fr.head], rs);
    }
    for (auto& p : preds) {
        Keys full_old = canonical_keys(c, store_get(c, p), rs);
        if (rs.repl.on) novel[p] = repl_finish(c, rs, p, full_old);
        Keys& d = novel[p];
        if (!d.buf) d.buf = make_buf(c, 0);
        order_novel(c, rs, p, d);
        Keys full_new;
        {
            PhaseTimer t(c, &rs.st.ms_setops);
            full_new = d.n == 0 ? full_old : (full_old.n == 0 ? d : ops_merge_disjoint(c, full_old, d));
        }
        if (make_delta) store_put(c, "__delta_" + p, ops_rel_from_keys(c, schema[p], d, true));
        install_full(c, p, schema[p], full_new, nullptr, rs);
    }
}

// ------------------------------------------------------------------------------ several ranks
// rows: a smaller stored relation is copied to every rank rather than joined slice by slice
// (XLB_REPL_SLICE_MIN overrides it, so that a test can run the sliced route on a small input)
static uint64_t repl_slice_min() {
    const char* v = getenv("XLB_REPL_SLICE_MIN");
    return v ? strtoull(v, nullptr, 10) : (1ull << 20);
}
constexpr uint64_t REPL_COPY_MAX = 1ull << 27;         // rows: the largest relation replicated mode copies to every rank (1 GiB)
constexpr uint64_t BROADCAST_MAX = 1ull << 25;         // rows: the largest stored relation a partitioned component copies to every rank

static int bit_len(uint64_t v) { return v ? 64 - __builtin_clzll(v) : 0; }

static uint64_t chunk_limit(xlb_ctx* c) {
    if (c->join_chunk) return c->join_chunk;
    uint64_t room = c->budget > c->allocated ? c->budget - c->allocated : 0;
    return std::max<uint64_t>(room / (8 * 8), 1u << 20);  // a chunk is held, sorted and merged: ~8 copies
}

// Restores the context's planning view when a component that ran on replicated relations is done.
struct PlanAsOneRank {
    xlb_ctx* c = nullptr;
    uint32_t world = 1;
    bool on = false;
    void begin(xlb_ctx* ctx) {
        c = ctx;
        world = c->world;
        c->world = 1;
        on = true;
    }
    void end() {
        if (on) c->world = world;
        on = false;
    }
    ~PlanAsOneRank() { end(); }
};

// Several ranks: agree (one small all-gather) on how the component runs, and give every rank a full
// copy of the stored relations that are cheaper to copy than to join partition by partition.
//   replicated mode (rs.repl.on): every head fits a dense domain of at most 2^27 tuples; heads and
//     deltas live on every rank, at most one large stored relation per rule stays in slices;
//   partitioned mode: heads are hash-partitioned; small stored relations are copied everywhere, so
//     a join with one needs no exchange and keeps the placement of the rows.
// Every decision depends only on the plan, the flags and the gathered numbers, so all ranks agree.
static void setup_ranks(xlb_ctx* c, const xlb_scc& scc, std::vector<FlatRule>& rules, const std::vector<std::string>& preds, const std::set<std::string>& rec,
                        std::map<std::string, xlb_schema>& schema, RunState& rs) {
    if (c->world <= 1 || (c->flags & XLB_FLAG_SHUFFLE_ONLY)) return;
    std::set<std::string> stored, checked;
    for (auto& fr : rules) {
        for (auto& a : fr.atoms)
            if (!rec.count(a.rel)) stored.insert(a.rel);
        for (auto& k : fr.checks) {
            if (!rec.count(k.rel)) stored.insert(k.rel);
            checked.insert(k.rel);
        }
    }
    std::vector<std::string> names(stored.begin(), stored.end());
    if (names.size() + preds.size() + 2 > COMM_WORDS_MAX) return;  // no agreement vector that long: plain partitioned evaluation
    bool resume = scc.is_recursive != 0;
    for (auto& p : preds) resume = resume && store_get(c, "__delta_" + p) != nullptr;
    // this rank's numbers: rows per relation, the widest value it holds, whether it would resume
    std::vector<uint64_t> mine;
    uint64_t values = 0;
    bool unknown = false;
    auto look = [&](const std::string& name) {
        xlb_rel* r = store_get(c, name);
        mine.push_back(r ? r->rows : 0);
        if (!r || !r->rows) return;
        Keys k = packed_for_rules(c, name, rules, rs, /*need_rows=*/false);
        if (k.bound == ~0ull) unknown = true;
        else values |= (k.bound >> 32) | (k.bound & 0xFFFFFFFFull);
    };
    for (auto& n : names) look(n);
    for (auto& p : preds) look(p);
    mine.push_back(unknown ? 64 : (uint64_t)bit_len(values));
    mine.push_back(resume ? 1 : 0);
    const uint32_t K = (uint32_t)mine.size(), W = c->comm_world;
    std::vector<uint64_t> all((size_t)W * K);
    {
        PhaseTimer t(c, &rs.st.ms_exchange);
        comm_allgather_words(c, mine.data(), K, all.data());
    }
    std::map<std::string, uint64_t> rows;
    uint64_t head_rows = 0, vb = 1, any_resume = 0;
    for (uint32_t r = 0; r < W; ++r) {
        for (size_t i = 0; i < names.size(); ++i) rows[names[i]] += all[(size_t)r * K + i];
        for (size_t i = 0; i < preds.size(); ++i) head_rows += all[(size_t)r * K + names.size() + i];
        vb = std::max(vb, all[(size_t)r * K + K - 2]);
        any_resume |= all[(size_t)r * K + K - 1];
    }
    bool repl = scc.is_recursive && !any_resume && !(c->flags & (XLB_FLAG_NO_DENSE | XLB_FLAG_KEEP_DELTAS));
    for (auto& p : preds) repl = repl && schema[p].arity * vb <= 27;
    std::set<std::string> sliced, copy;
    if (repl) {
        // the largest stored relations stay in slices where no rule would then join two sliced atoms
        std::vector<std::string> by_size(names);
        std::sort(by_size.begin(), by_size.end(), [&](const std::string& a, const std::string& b) { return rows[a] != rows[b] ? rows[a] > rows[b] : a < b; });
        for (auto& n : by_size) {
            if (rows[n] < repl_slice_min() || checked.count(n)) continue;
            bool ok = true;
            for (auto& fr : rules) {
                int mine_n = 0, others = 0;
                for (auto& a : fr.atoms) {
                    mine_n += a.rel == n;
                    others += sliced.count(a.rel) > 0;
                }
                if (mine_n > 1 || (mine_n == 1 && others > 0)) ok = false;
            }
            if (ok) sliced.insert(n);
        }
        for (auto& n : names)
            if (!sliced.count(n)) {
                copy.insert(n);
                if (rows[n] > REPL_COPY_MAX) repl = false;
            }
    }
    if (!repl) {
        sliced.clear();
        copy.clear();
        for (auto& n : names)
            if (rows[n] <= BROADCAST_MAX) copy.insert(n);
    }
    // the copies: all ranks' rows of the relation, under an alias the rules are pointed to
    for (auto& n : copy) {
        xlb_rel* r = store_get(c, n);
        const std::string alias = "__all_" + n;
        Keys everything;
        {
            PhaseTimer t(c, &rs.st.ms_exchange);
            Keys local = ops_rel_packed(c, r);
            everything = comm_allgather_keys(c, local);
            rs.st.exchange_bytes += local.n * 8 * (uint64_t)(W - 1);
        }
        store_put(c, alias, ops_rel_from_keys(c, r->schema, everything, false));
        rs.aliases.push_back(alias);
        rs.replicated.insert(alias);
        for (auto& fr : rules) {
            for (auto& a : fr.atoms)
                if (a.rel == n) a.rel = alias;
            for (auto& k : fr.checks)
                if (k.rel == n) k.rel = alias;
        }
    }
    if (!repl) return;
    rs.repl.on = true;
    rs.repl.rank = c->comm_rank;
    rs.repl.world = W;
    rs.repl.vb = (int)vb;
    rs.repl.sliced = sliced;
    for (auto& p : preds) {
        rs.replicated.insert(p);
        if (!head_rows) continue;
        // a head that holds rows already: every rank gets all of them, sorted and unique
        Keys everything;
        {
            PhaseTimer t(c, &rs.st.ms_exchange);
            everything = comm_allgather_keys(c, ops_rel_packed(c, store_get(c, p)));
        }
        {
            PhaseTimer t(c, &rs.st.ms_sort);
            ops_sort(c, everything);
        }
        PhaseTimer t(c, &rs.st.ms_setops);
        ops_dedup_sorted(c, everything);
        store_put(c, p, ops_rel_from_keys(c, schema[p], everything, true));
    }
}

// Removes the full copies made for a component (and the indexes built over them).
static void drop_aliases(xlb_ctx* c, RunState& rs) {
    for (auto& alias : rs.aliases) {
        auto it = c->store.find(alias);
        if (it != c->store.end()) {
            delete it->second;
            c->store.erase(it);
            c->versions[alias]++;
        }
        for (int kc = 0; kc <= ROW_INDEX; ++kc) cache(c).m.erase({alias, kc});
        rs.replicated.erase(alias);
    }
    rs.aliases.clear();
}

// Partitioned mode, one head whose recursive rules all carry one of its columns over unchanged
// from their one recursive atom while every other atom is a relation all ranks hold in full: with
// the head placed by that column a rank derives only tuples it owns, and no tuple is exchanged.
static int carried_home(const std::vector<FlatRule>& rules, const std::string& pred, const std::set<std::string>& rec, uint32_t arity, const RunState& rs) {
    if (arity != 2 || rec.size() != 1) return -1;
    for (int q = 0; q < 2; ++q) {
        bool ok = true, any = false;
        for (auto& fr : rules) {
            if (fr.head != pred) continue;
            int nrec = 0, at = -1;
            for (size_t i = 0; i < fr.atoms.size(); ++i) {
                if (rec.count(fr.atoms[i].rel)) { ++nrec; at = (int)i; }
                else if (!rs.replicated.count(fr.atoms[i].rel)) ok = false;
            }
            for (auto& k : fr.checks)
                if (!rs.replicated.count(k.rel)) ok = false;
            if (nrec == 0) continue;  // a seeding rule: its tuples are sent home once
            any = true;
            if (nrec != 1 || fr.atoms[at].arity != 2 || fr.head_vars.size() != 2 || fr.atoms[at].var[q] != fr.head_vars[q]) ok = false;
        }
        if (ok && any) return q == 0 ? SRC_HI : SRC_LO;
    }
    return -1;
}

// ------------------------------------------------------------------------------ frontier loop
// A component of the shape  p(Z) :- p(Y), e(Y, Z)  — one head of one column, one recursive rule
// that joins the frontier with one stored relation, evaluated by streaming over the relation
// against a bitmap of the frontier, new tuples found on the head's bitmap — needs nothing from
// the host between iterations but the decision to stop.  So iteration k + 1 is enqueued before
// the row count of iteration k has come back: its frontier's length is read from device memory
// and its buffers are sized by what the domain still has room for.  The host reads the counts one
// iteration behind; the iteration that was enqueued on top of an empty frontier marks nothing
// and is dropped.  Every rank of a replicated component sees the same counts, so all ranks stop
// after the same number of exchanges.
struct FrontierPlan {
    const FlatRule* fr = nullptr;
    size_t ei = 0;   // the stored atom
    int kc = 0;      // its join column
    int rel_lo = 0;  // what the head's column takes from a row of it: 0 the key, 1 the other column
};

// The static part: one recursive rule, `head(V) :- head(K), rel(..)` with rel a stored two-column
// relation joined on K and V one of its columns, and a head of one column.
static bool frontier_rule_shape(const std::vector<FlatRule>& rules, const std::vector<std::string>& preds, const std::set<std::string>& rec,
                                const std::map<std::string, xlb_schema>& schema, FrontierPlan* fp) {
    if (preds.size() != 1 || schema.at(preds[0]).arity != 1) return false;
    const FlatRule* only = nullptr;
    for (auto& fr : rules) {
        int nrec = 0;
        for (auto& a : fr.atoms) nrec += rec.count(a.rel) ? 1 : 0;
        if (!nrec) continue;
        if (only) return false;
        only = &fr;
    }
    if (!only || only->atoms.size() != 2 || !only->filters.empty() || !only->checks.empty() || only->head_vars.size() != 1) return false;
    const size_t ai = rec.count(only->atoms[0].rel) ? 0 : 1, ei = 1 - ai;
    const Atom& pa = only->atoms[ai];
    const Atom& ea = only->atoms[ei];
    if (rec.count(ea.rel) || pa.arity != 1 || ea.arity != 2 || ea.var[0] == ea.var[1]) return false;
    int kc = ea.var[0] == pa.var[0] ? 0 : ea.var[1] == pa.var[0] ? 1 : -1;
    if (kc < 0) return false;
    const int hv = only->head_vars[0];
    if (hv != ea.var[0] && hv != ea.var[1]) return false;
    fp->fr = only;
    fp->ei = ei;
    fp->kc = kc;
    fp->rel_lo = hv == ea.var[kc] ? 0 : 1;
    return true;
}

static bool frontier_flags_ok(xlb_ctx* c) { return !(c->flags & (XLB_FLAG_NO_DENSE | XLB_FLAG_KEEP_DELTAS)) && !getenv("XLB_NO_FRONTIER_LOOP"); }

static bool frontier_shape(xlb_ctx* c, const std::vector<FlatRule>& rules, const std::vector<std::string>& preds, const std::set<std::string>& rec,
                           const std::map<std::string, xlb_schema>& schema, RunState& rs, FrontierPlan* fp) {
    if (c->world != 1 || !frontier_flags_ok(c)) return false;
    if (!frontier_rule_shape(rules, preds, rec, schema, fp)) return false;
    if (index_ready(c, fp->fr->atoms[fp->ei].rel, fp->kc, rs)) return false;  // an index exists: probing it beats streaming
    return true;
}

// Wait until a kernel has left three counts tagged with launch number `seq` in pinned memory
// (work enqueued behind that kernel keeps running: no event, no copy), and return them.  After
// 20 ms the full wait on the stream takes over, which knows how to give up on a late peer.
static void wait_published(xlb_ctx* c, const unsigned long long* words, unsigned long long seq, uint64_t out[3]) {
    const double tr0 = c->trace_on ? trace_now() : 0;
    auto t0 = std::chrono::steady_clock::now();
    const volatile unsigned long long* w = words;
    const unsigned long long tag = seq & PUBLISH_TAG_MASK;
    auto all_here = [&] { return (w[0] >> PUBLISH_COUNT_BITS) == tag && (w[1] >> PUBLISH_COUNT_BITS) == tag && (w[2] >> PUBLISH_COUNT_BITS) == tag; };
    for (uint64_t polls = 0; !all_here(); ++polls) {
        if ((polls & 255) == 255 && std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() > 20.0) {
            stream_wait(c);  // everything enqueued has run when this returns
            if (!all_here()) xlb_fail(XLB_ERR_CUDA, "internal: a frontier step finished without leaving its counts");
            break;
        }
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    for (int i = 0; i < 3; ++i) out[i] = w[i] & ((1ull << PUBLISH_COUNT_BITS) - 1);
    c->ms_sync_wait += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    c->syncs++;
    trace_note(c, "wait (counts in pinned memory)", tr0);
}

// Runs iterations from the state the seeding pass left (the head's list and "__delta_<head>" in the
// store).  `it` counts finished iterations; `fix` is set when one of them found nothing.  Returns
// with fix unset when the relation has been streamed over as often as building its index would
// have cost (or the iteration limit is near): the general loop carries on from the stored state.
// Inside, the head and the frontier exist as bitmaps only: an iteration is one stream over the
// relation (candidates marked unless the head has them) and one pass over the bitmaps (what is new
// becomes the next frontier and joins the head); on several ranks an all-gather of the candidate
// bitmaps sits between the two.  The sorted list is read off the head's bitmap once, at the end.
static void frontier_loop(xlb_ctx* c, const FrontierPlan& fp, const std::string& p, const xlb_schema& hs, RunState& rs, uint64_t& it, bool& fix) {
    const Atom& ea = fp.fr->atoms[fp.ei];
    xlb_rel* er = store_get(c, ea.rel);
    xlb_rel* d0 = store_get(c, "__delta_" + p);
    if (!er || !d0 || d0->rows == 0) return;
    // a relation that came as two columns and has not been packed is streamed over as it is: one
    // pass for the bound of its values instead of a pass that also writes the packed copy
    bool from_cols = !er->packed && er->schema.arity == 2 && rel_packable(er->schema) && er->cols[0] && er->cols[1];
    if (from_cols && er->or_bound == ~0ull) ops_rel_bound_filtered(c, er, -1, 0, nullptr);
    Keys rows;
    if (from_cols && er->or_bound != ~0ull) {
        rows.n = er->rows;
        rows.bound = er->or_bound;
    } else {
        from_cols = false;
        rows = ops_rel_packed(c, er);
    }
    Keys delta = ops_rel_packed(c, d0);
    Keys full = full_view(c, rs, p);
    if (rows.bound == ~0ull || delta.bound == ~0ull || (full.n && full.bound == ~0ull)) return;
    int hb = 0, lb = 0;
    if (rs.repl.on) repl_bits(rs, 1, &hb, &lb);
    else {
        const uint64_t taken = fp.rel_lo == 0 ? (fp.kc == 0 ? rows.bound >> 32 : rows.bound & 0xFFFFFFFFull) : (fp.kc == 0 ? rows.bound & 0xFFFFFFFFull : rows.bound >> 32);
        const uint64_t all = taken | delta.bound | (full.n ? full.bound : 0);
        if (all >> 32) return;
        lb = std::max(bit_len(all), 1);
    }
    if (lb > 27) return;
    int& scans = rs.scans[{ea.rel, fp.kc}];
    const int scan_limit = er->canonical && fp.kc == 0 ? 3 : 12;
    if (scans >= scan_limit || it + 1 > c->max_iterations) return;
    Keys none;
    DenseState* ds = dense_state(c, rs, p, hb, lb, full, none);
    if (ds->hi_bits != 0) return;
    lb = ds->lo_bits;
    const uint64_t domain = 1ull << lb, words = ds->words;
    const int rel_keysel = fp.kc == 0 ? SRC_HI : SRC_LO;
    uint64_t row_lo = 0, row_hi = rows.n;
    if (rs.repl.on && !rs.repl.sliced.count(ea.rel)) {
        // every rank holds all rows of this relation: each streams over its share of them (shares
        // start at multiples of four rows, so that 16-byte loads stay aligned)
        const uint64_t n = rows.n;
        row_lo = (n * c->comm_rank / c->comm_world) & ~3ull;
        row_hi = c->comm_rank + 1 == c->comm_world ? n : (n * (c->comm_rank + 1) / c->comm_world) & ~3ull;
    }
    ScanRows src;  // what the next scan streams over
    src.n_max = row_hi - row_lo;
    if (from_cols) {
        src.kcol = er->cols[fp.kc]->as<uint32_t>() + row_lo;
        src.ocol = er->cols[1 - fp.kc]->as<uint32_t>() + row_lo;
        if (((uintptr_t)src.kcol | (uintptr_t)src.ocol) & 15) return;
    } else {
        src.packed = rows.ptr() + row_lo;
        if ((uintptr_t)src.packed & 15) return;
    }
    const uint64_t share = src.n_max;

    // frontier bitmaps (two, used in turn), this rank's marks (the head plus the candidates of the
    // iteration under way: it starts as a copy of the head and every step leaves it so), and per launch four
    // counters: new tuples, rows of the relation with a key in the frontier, rows written to the
    // list of rows that can still match, (unused)
    const uint64_t bitmap_bytes = std::max<uint64_t>(words * 4, 16);
    const int max_launches = scan_limit + 1;
    // whether a row whose key the head holds must have it in the frontier: true of the relation
    // when the head holds nothing but the frontier, and of a list written by the scan just before
    bool visited_means_frontier = full.n == delta.n;
    // (the first scan then never looks at the first frontier bitmap: it need not be filled)
    Buf frontier[2] = {visited_means_frontier ? make_buf(c, bitmap_bytes) : ops_keyset(c, delta, SRC_LO, lb), make_buf(c, bitmap_bytes)};
    Buf cand = make_buf(c, bitmap_bytes);
    Buf counts = make_buf(c, (uint64_t)max_launches * 32 + 16);  // and, behind the counters, the step kernel's count of finished blocks
    unsigned int* visited = ds->visited->as<unsigned int>();
    CUDA_OK(cudaMemcpyAsync(cand->p, visited, words * 4, cudaMemcpyDeviceToDevice, c->stream));
    CUDA_OK(cudaMemsetAsync(counts->p, 0, (uint64_t)max_launches * 32 + 16, c->stream));
    unsigned int* ticket = reinterpret_cast<unsigned int*>(counts->as<unsigned long long>() + 4 * max_launches);
    struct Flight {
        unsigned long long seq = 0;  // the number the step kernel writes beside the counts it leaves in pinned memory
        unsigned slot = 0;
        int index = 0;
        unsigned long long* count = nullptr;  // device: [0] new tuples, [1] rows whose key was in the frontier, [2] rows kept for later scans
    };
    // A key enters the frontier once, so a row whose key the head holds is of no use to a later
    // scan: a scan that expects to lose a good part of its rows writes the others to a list, and
    // the next scan streams over that list.  The lists live in two buffers used in turn; their
    // lengths stay on the device (the next scan is enqueued before the host has read them).
    struct Launch {
        int producer;   // the launch that wrote the list this one streamed over; -1: the relation itself
        bool compacts;  // wrote a list of its own
        uint64_t kept;  // rows in that list, once read
    };
    std::vector<Launch> log;
    Buf live[2];
    int src_buf = -1, producer = -1;
    int launched = 0, cur_frontier = 0;
    auto launch = [&](const unsigned long long* keys_in_frontier, bool compact) {
        Flight f;
        f.index = launched;
        f.count = counts->as<unsigned long long>() + 4 * launched;
        f.slot = 20 + 4 * (launched & 3);  // (at most two launches are in flight)
        if ((++c->publish_seq & PUBLISH_TAG_MASK) == 0) ++c->publish_seq;  // tag 0 is what untouched words carry
        f.seq = c->publish_seq;
        uint64_t* out = nullptr;
        int dst = -1;
        if (compact) {
            dst = src_buf == 0 ? 1 : 0;
            if (!live[dst] || live[dst]->bytes < src.n_max * 8) live[dst] = make_buf(c, src.n_max * 8);
            out = live[dst]->as<uint64_t>();
        }
        {
            PhaseTimer t(c, &rs.st.ms_join);
            ops_frontier_scan(c, src, rel_keysel, lb, visited_means_frontier ? nullptr : frontier[cur_frontier]->as<unsigned int>(), fp.rel_lo, cand->as<unsigned int>(), visited,
                              f.count + 1, keys_in_frontier, out, f.count + 2);
        }
        log.push_back({producer, compact, 0});
        visited_means_frontier = compact;  // the list written now holds no row whose key the head held
        if (compact) {
            ScanRows next;
            next.packed = out;
            next.n_max = src.n_max;
            next.n_dev = f.count + 2;
            src = next;
            src_buf = dst;
            producer = launched;
        }
        Buf gathered;
        if (rs.repl.on) {
            PhaseTimer t(c, &rs.st.ms_exchange);
            gathered = comm_gather_bitmaps(c, cand->as<unsigned int>(), words);
            rs.st.exchange_bytes += words * 4 * (uint64_t)(rs.repl.world - 1);
        }
        {
            PhaseTimer t(c, &rs.st.ms_setops);
            ops_frontier_step(c, gathered ? gathered->as<unsigned int>() : cand->as<unsigned int>(), gathered ? rs.repl.world : 1, words, cand->as<unsigned int>(), visited,
                              frontier[1 - cur_frontier]->as<unsigned int>(), f.count, ticket, c->h_scalar_dev + f.slot, f.seq);
        }
        cur_frontier = 1 - cur_frontier;
        ++launched;
        ++scans;
        return f;
    };
    // whether launch number k should write a list: the first two do (nothing is known yet); later
    // ones if the last scan the host has the counts of lost at least an eighth of its rows
    uint64_t seen_rows = 0, seen_matched = 0;
    auto wants_list = [&](int k) { return k < 2 || seen_matched * 8 >= seen_rows; };
    uint64_t last_new = delta.n;
    int last_frontier = 0;  // which bitmap holds the tuples of the last finished iteration
    Flight cur = launch(nullptr, wants_list(0));
    for (;;) {
        // `cur` is the iteration in flight whose counts the host has not seen: the next one is
        // enqueued on top of it (it does nothing if cur finds nothing new)
        const bool more = scans < scan_limit && launched < max_launches && it + 2 <= c->max_iterations;
        const int cur_out = cur_frontier;
        Flight next;
        if (more) next = launch(cur.count, wants_list(launched));
        uint64_t got[3];
        wait_published(c, &c->h_scalar[cur.slot], cur.seq, got);
        const uint64_t tot = got[0], marked = got[1], kept = got[2];
        Launch& done = log[cur.index];
        done.kept = kept;
        const uint64_t streamed = done.producer < 0 ? share : log[done.producer].kept;
        seen_rows = streamed;
        seen_matched = marked;
        if (done.compacts && producer == cur.index) src.n_max = std::min(src.n_max, std::max<uint64_t>(kept, 1));  // the next launches size their grids by it
        prof_add_bytes(c, "scan_join_mark", (streamed + (done.compacts ? kept : 0)) * 8ull);
        ++it;
        rs.st.iterations++;
        rs.st.candidate_tuples += marked;
        ds->rows += tot;
        last_new = tot;
        last_frontier = cur_out;
        if (tot == 0) {
            fix = true;
            break;
        }
        if (!more) break;
        cur = next;
    }
    // back to lists: the head in order off its bitmap, and the last iteration's tuples as the delta
    {
        PhaseTimer t(c, &rs.st.ms_setops);
        if (ds->rows != full.n) install_full(c, p, hs, ops_dense_state_rows(c, *ds, domain - 1), nullptr, rs);
        Keys d;
        d.buf = make_buf(c, 0);
        if (last_new) {
            DenseState last;
            last.visited = frontier[last_frontier];
            last.words = words;
            last.hi_bits = 0;
            last.lo_bits = lb;
            last.rows = last_new;
            last.valid = true;
            d = ops_dense_state_rows(c, last, domain - 1);
        }
        store_put(c, "__delta_" + p, ops_rel_from_keys(c, hs, d, true));
    }
}

static void run_scc(xlb_ctx* c, const xlb_scc& scc, RunState& rs) {
    if (!scc.rules && scc.n_rules) xlb_fail(XLB_ERR_INVALID, "SCC %u has no rule array", scc.id);
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
    std::set<std::string> rec(preds.begin(), preds.end());
    for (auto& p : preds)
        if (!store_get(c, p)) store_put(c, p, empty_rel(c, schema[p]));  // recursive.rs:471-486
    // A rule the packed pipelines do not take (more than two live columns, relations of three and
    // more columns, two-column join keys that are not a membership test, a Union below the top of a
    // body) sends the whole component to the general, node-by-node evaluator.
    std::vector<FlatRule> rules;
    bool packed = !(c->flags & XLB_FLAG_GENERAL_ONLY);
    try {
        for (uint32_t i = 0; packed && i < scc.n_rules; ++i) {
            // a Union at the top of a body is one rule per input (RirNode::Union concatenates its inputs)
            std::vector<const xlb_node*> bodies{scc.rules[i].body};
            for (size_t q = 0; q < bodies.size();) {
                const xlb_node* b = bodies[q];
                if (b->kind == XLB_NODE_UNION) {
                    if (!b->inputs && b->n_inputs) xlb_fail(XLB_ERR_INVALID, "Union node without inputs");
                    bodies.erase(bodies.begin() + q);
                    for (uint32_t u = 0; u < b->n_inputs; ++u) bodies.push_back(b->inputs[u]);
                } else ++q;
            }
            for (const xlb_node* b : bodies) {
                xlb_rule r = scc.rules[i];
                r.body = b;
                rules.push_back(Flattener{c, {}, {}}.run(r));
            }
        }
    } catch (const XlbError& e) {
        if (e.st != XLB_ERR_UNSUPPORTED) throw;
        packed = false;
    }
    for (auto& fr : rules) {
        if (!packed) break;
        bool any = false;
        fr.start_ok.assign(fr.atoms.size(), 0);
        for (size_t a = 0; a < fr.atoms.size(); ++a) {
            fr.start_ok[a] = pipeline_feasible(fr, a) ? 1 : 0;
            any |= fr.start_ok[a] != 0;
            if (!fr.start_ok[a] && rec.count(fr.atoms[a].rel)) packed = false;  // its delta variant would have to start there
        }
        if (!any || (c->world > 1 && !fr.start_ok[0])) packed = false;
    }
    if (!packed) {
        run_scc_tree(c, scc, rs.st);
        return;
    }
    for (auto& p : preds) rs.head_schema[p] = schema[p];
    struct Cleanup {  // the full copies go when the component is done, however it ends
        xlb_ctx* c;
        RunState& rs;
        const std::vector<std::string>& preds;
        ~Cleanup() {
            for (auto& p : preds) rs.tset.erase(p);  // the hash sets can be gigabytes: they go with the component
            drop_aliases(c, rs);
            rs.wide_dense.clear();
            rs.repl = RunState::Repl();
            rs.replicated.clear();
        }
    } cleanup{c, rs, preds};
    // The relation a frontier loop would stream over stays as columns while its other uses are
    // single-atom rules (a constant filter reads the columns too); anything else packs it on demand.
    rs.keep_cols.clear();
    if (scc.is_recursive && frontier_flags_ok(c)) {
        FrontierPlan probe;
        if (frontier_rule_shape(rules, preds, rec, schema, &probe)) {
            const std::string& rel = probe.fr->atoms[probe.ei].rel;
            bool only_scans = true;
            for (auto& fr : rules) {
                if (&fr == probe.fr) continue;
                for (auto& a : fr.atoms)
                    if (a.rel == rel && fr.atoms.size() != 1) only_scans = false;
                for (auto& k : fr.checks)
                    if (k.rel == rel) only_scans = false;
            }
            if (only_scans) rs.keep_cols.insert(rel);
        }
    }
    PlanAsOneRank one_rank;
    setup_ranks(c, scc, rules, preds, rec, schema, rs);
    std::map<std::string, int> home;
    for (auto& p : preds) {
        home[p] = home_half(rules, p, rec, schema[p].arity);
        const int carried = c->world > 1 && !rs.repl.on && scc.is_recursive ? carried_home(rules, p, rec, schema[p].arity, rs) : -1;
        if (carried >= 0) home[p] = carried;
    }
    if (rs.repl.on) one_rank.begin(c);  // from here to the sharding of the result the component plans as a single rank
    // Heads whose sorted list some rule reads during the loop: the other recursive atoms of a rule
    // with several (a variant reads their full relations), and relations tested by a semi / anti
    // join.  For every other head the merge of an iteration's delta can wait.
    std::set<std::string> list_read;
    for (auto& fr : rules) {
        int nrec = 0;
        for (auto& a : fr.atoms) nrec += rec.count(a.rel) ? 1 : 0;
        for (auto& a : fr.atoms)
            if (nrec >= 2 && rec.count(a.rel)) list_read.insert(a.rel);
        for (auto& k : fr.checks) list_read.insert(k.rel);
    }
    rs.ordered_heads = list_read;
    rs.bag_novel.clear();
    if (c->world > 1) {
        // a head relation that already holds rows is re-homed so that equal tuples meet on one rank
        for (auto& p : preds) {
            xlb_rel* r = store_get(c, p);
            Keys k = canonical_keys(c, r, rs);
            if (k.buf == r->packed) k = ops_copy(c, k);
            k = comm_repartition(c, k, home[p], true, rs.st);
            store_put(c, p, ops_rel_from_keys(c, schema[p], k, true));
        }
    }

    // Resume: the caller restored (full, delta) of every head of this SCC, as left behind by a run
    // that stopped at the iteration limit with XLB_FLAG_KEEP_DELTAS.  The seed pass is then
    // skipped: its tuples are in `full` already, and the deltas say where the loop stood.
    bool resume = scc.is_recursive != 0;
    for (auto& p : preds) {
        xlb_rel* d = store_get(c, "__delta_" + p);
        if (!d || !rel_packable(d->schema) || d->schema.arity != schema[p].arity) resume = false;
    }
    if (resume) {
        for (auto& p : preds) {
            // both are handed to the loop as it keeps them: sorted and unique
            for (const std::string& name : {p, "__delta_" + p}) {
                xlb_rel* r = store_get(c, name);
                if (r->canonical) continue;
                Keys k = canonical_keys(c, r, rs);
                store_put(c, name, ops_rel_from_keys(c, schema[p], k, true));
            }
        }
    } else {
        seed_pass(c, rules, preds, rec, schema, home, scc.is_recursive != 0, rs);
    }
    if (!scc.is_recursive) return;

    bool fix = false;
    // A failure inside the loop (memory budget, a device status) must not leave deltas behind: a
    // later call would take them for a saved state and resume from them, over a full relation
    // that may lack merges still put off.  Without them the next call seeds again from the stored
    // relations, which are a valid earlier state.
    struct DropDeltasOnFailure {
        xlb_ctx* c;
        RunState& rs;
        const std::vector<std::string>& preds;
        bool armed = true;
        ~DropDeltasOnFailure() {
            if (!armed) return;
            rs.pending.clear();
            for (auto& p : preds) {
                auto it = c->store.find("__delta_" + p);
                if (it == c->store.end()) continue;
                delete it->second;
                c->store.erase(it);
                c->versions["__delta_" + p]++;
            }
        }
    } guard{c, rs, preds};
    uint64_t it = 0;
    {
        FrontierPlan fp;
        if (frontier_shape(c, rules, preds, rec, schema, rs, &fp)) frontier_loop(c, fp, preds[0], schema[preds[0]], rs, it, fix);
    }
    for (; !fix && it < c->max_iterations; ++it) {  // recursive.rs:619-937
        rs.st.iterations++;
        rs.bag_novel.clear();
        std::map<std::string, Keys> novel;
        for (auto& fr : rules) {
            for (size_t i = 0; i < fr.atoms.size(); ++i) {  // one variant per recursive occurrence (:636-664)
                if (!rec.count(fr.atoms[i].rel)) continue;
                xlb_rel* d = store_get(c, "__delta_" + fr.atoms[i].rel);
                if (!d) continue;
                if (d->rows == 0 && c->world == 1) continue;
                bool any_empty = false;
                for (size_t j = 0; j < fr.atoms.size(); ++j)
                    if (j != i && store_get(c, fr.atoms[j].rel)->rows == 0 && c->world == 1) any_empty = true;
                if (any_empty) continue;
                Keys full = full_view(c, rs, fr.head);
                eval_variant(c, fr, i, ops_rel_packed(c, d), false, home[fr.atoms[i].rel], full, home[fr.head], novel[fr.head], rs);
            }
        }
        if (rs.repl.on)
            for (auto& p : preds) novel[p] = repl_finish(c, rs, p, full_view(c, rs, p));  // the same tuples on every rank: no vote
        uint64_t changed = 0;
        for (auto& p : preds) changed += novel[p].n;
        if (c->world > 1) {
            // the emptiness vote; with it the ranks agree on the join chunks of the next iteration
            // (candidates of one chunk, doubled for growth, within the tightest rank's bound)
            PhaseTimer t(c, &rs.st.ms_exchange);
            const uint64_t lim = chunk_limit(c);
            uint64_t mine[2] = {changed, std::min<uint64_t>((2 * rs.max_cand_local * std::max<uint64_t>(rs.agreed_chunks, 1) + lim - 1) / lim, 4096)};
            std::vector<uint64_t> all((size_t)c->comm_world * 2);
            comm_allgather_words(c, mine, 2, all.data());
            changed = 0;
            rs.agreed_chunks = 1;
            for (uint32_t r = 0; r < c->comm_world; ++r) {
                changed += all[2 * r];
                rs.agreed_chunks = std::max(rs.agreed_chunks, all[2 * r + 1]);
            }
            rs.max_cand_local = 0;
        }
        for (auto& p : preds) {  // :735-858
            Keys& d = novel[p];
            if (!d.buf) d.buf = make_buf(c, 0);
            if (c->flags & XLB_FLAG_KEEP_DELTAS) order_novel(c, rs, p, d);  // a delta that may be saved is a sorted list
            store_put(c, "__delta_" + p, ops_rel_from_keys(c, schema[p], d, !rs.bag_novel.count(p)));
        }
        if (changed == 0) { fix = true; break; }  // :861-865
        for (auto& p : preds) {                    // :868-937
            Keys& d = novel[p];
            if (d.n == 0 && c->world == 1) continue;
            {
                // nobody reads the list and the bitmap is in step with full + delta: put the merge off
                const DenseState& ds = rs.dense[p];
                const TupleSet& ts = rs.tset[p];
                const Keys view = full_view(c, rs, p);
                const bool on_bitmap = c->world == 1 && !(c->flags & XLB_FLAG_NO_DENSE) && ds.valid && ds.rows == view.n + d.n;
                const bool in_set = ts.valid && ts.rows == view.n + d.n;  // (holds on every rank or none: the route is chosen from agreed bounds)
                if (!list_read.count(p) && (on_bitmap || in_set)) {
                    RunState::Pending& pd = rs.pending[p];
                    pd.deltas.push_back(d);
                    pd.rows += d.n;
                    pd.bound |= d.bound;
                    pd.bags |= rs.bag_novel.erase(p) > 0;
                    continue;
                }
            }
            order_novel(c, rs, p, d);
            materialize_full(c, rs, p);
            Keys full = ops_rel_packed(c, store_get(c, p));
            Keys merged;
            {
                PhaseTimer t(c, &rs.st.ms_setops);
                merged = full.n ? ops_merge_disjoint(c, full, d) : ops_copy(c, d);
            }
            install_full(c, p, schema[p], merged, &d, rs);
        }
    }
    for (auto& p : preds) {
        rs.tset.erase(p);  // gigabytes, and the lists are about to be written out
        materialize_full(c, rs, p);
    }
    if (rs.repl.on) {
        // every rank holds the whole result: each keeps the tuples it owns, as the partitioned
        // evaluation would have left them (sorted, unique, disjoint between ranks)
        one_rank.end();
        for (auto& p : preds) {
            PhaseTimer t(c, &rs.st.ms_setops);
            Keys mine = ops_filter_owner(c, ops_rel_packed(c, store_get(c, p)), home[p], c->comm_world, c->comm_rank);
            store_put(c, p, ops_rel_from_keys(c, schema[p], mine, true));
        }
    }
    guard.armed = false;  // the loop ended by itself: what follows decides about the deltas
    for (auto& p : preds) {  // :940-945
        if (!fix && (c->flags & XLB_FLAG_KEEP_DELTAS)) break;  // left for a checkpoint
        auto it = c->store.find("__delta_" + p);
        if (it != c->store.end()) {
            delete it->second;
            c->store.erase(it);
        }
    }
    if (!fix) xlb_fail(XLB_ERR_ITER_LIMIT, "Recursive SCC iteration limit (%llu) exceeded", (unsigned long long)c->max_iterations);
}

// ---- plans over wide or typed columns ------------------------------------------------------------
// The pipelines carry two 32-bit columns per tuple.  Relations with u64, signed or floating columns
// (the reference runs them on its general path, e.g. the u64 closure of
// crates/xlog-integration/tests/test_factorized_delta_e2e.rs:385-411) are therefore run as relations
// of dictionary ranks: one sorted dictionary over the order-preserving images of all values of all
// relations the plan touches, every column replaced by 32-bit ranks, the same engine, and the heads
// decoded at the end.  Ranks order and compare as the values do, so joins, comparisons between
// columns and the sorted result are unchanged; constants of filters are translated to rank bounds.
static bool rank32(uint8_t t) { return t == XLB_U32 || t == XLB_SYMBOL; }

struct EncodedRun {
    xlb_ctx* c = nullptr;
    Keys dict;
    std::deque<xlb_node> nodes;
    std::deque<std::vector<const xlb_node*>> lists;
    std::deque<std::vector<xlb_rule>> rules;
    std::vector<xlb_scc> sccs;
    xlb_plan plan{};
    std::map<std::string, xlb_rel*> originals;      // taken out of the store while the ranks stand in
    std::map<std::string, xlb_schema> head_types;   // as the plan declares them
    std::vector<const xlb_node*> const_filters;
    std::vector<uint64_t> below, not_above;
    bool active = false;

    static void walk(xlb_ctx* c, const xlb_node* n, std::set<std::string>& scanned, std::vector<const xlb_node*>& consts) {
        if (!n) return;
        if (n->kind == XLB_NODE_SCAN) {
            auto nm = c->rel_names.find(n->rel_id);
            if (nm != c->rel_names.end()) scanned.insert(nm->second);
        }
        if (n->kind == XLB_NODE_FILTER && n->cmp_rhs_is_const) consts.push_back(n);
        walk(c, n->input, scanned, consts);
        walk(c, n->left, scanned, consts);
        walk(c, n->right, scanned, consts);
        if (n->kind == XLB_NODE_UNION && n->inputs)
            for (uint32_t i = 0; i < n->n_inputs; ++i) walk(c, n->inputs[i], scanned, consts);
    }

    const xlb_node* clone(const xlb_node* n) {
        if (!n) return nullptr;
        nodes.push_back(*n);
        xlb_node& m = nodes.back();  // a deque keeps this reference through the pushes below
        m.input = clone(n->input);
        m.left = clone(n->left);
        m.right = clone(n->right);
        if (n->kind == XLB_NODE_UNION && n->inputs) {
            std::vector<const xlb_node*> list;
            for (uint32_t i = 0; i < n->n_inputs; ++i) list.push_back(clone(n->inputs[i]));
            lists.push_back(std::move(list));
            m.inputs = lists.back().data();
        }
        if (n->kind == XLB_NODE_FILTER && n->cmp_rhs_is_const) {
            size_t k = std::find(const_filters.begin(), const_filters.end(), n) - const_filters.begin();
            const uint64_t lo = below[k], hi = not_above[k];  // ranks of values below c; of values not above c
            switch (n->cmp) {
                case XLB_EQ: case XLB_NE: m.cmp_rhs = hi > lo ? lo : 0xFFFFFFFFull; break;  // absent: a rank no value has
                case XLB_LT: case XLB_GE: m.cmp_rhs = lo; break;                             // x < c  <=>  rank(x) < lo
                case XLB_LE: m.cmp = XLB_LT; m.cmp_rhs = hi; break;                          // x <= c <=>  rank(x) < hi
                default: m.cmp = XLB_GE; m.cmp_rhs = hi; break;                              // x > c  <=>  rank(x) >= hi
            }
        }
        return &m;
    }

    // Decide, and if the plan needs it swap the ranks in.  Returns the plan to run.
    const xlb_plan* begin(xlb_ctx* ctx, const xlb_plan* in) {
        c = ctx;
        std::set<std::string> names;
        bool wide = false;
        for (uint32_t s = 0; s < in->n_sccs; ++s) {
            const xlb_scc& scc = in->sccs[s];
            if (!scc.rules) continue;
            for (uint32_t i = 0; i < scc.n_rules; ++i) {
                const xlb_rule& r = scc.rules[i];
                if (!r.head || !r.body) continue;
                walk(c, r.body, names, const_filters);
                names.insert(r.head);
                if (!head_types.count(r.head)) head_types[r.head] = r.head_schema;
                for (uint32_t k = 0; k < r.head_schema.arity && k < XLB_MAX_ARITY; ++k) wide |= !rank32(r.head_schema.types[k]);
            }
        }
        std::vector<const xlb_rel*> rels;
        for (auto& n : names) {
            xlb_rel* r = store_get(c, n);
            if (!r) continue;
            rels.push_back(r);
            for (uint32_t k = 0; k < r->schema.arity; ++k) wide |= !rank32(r->schema.types[k]);
        }
        if (!wide) return in;
        if (c->world > 1) xlb_fail(XLB_ERR_UNSUPPORTED, "plans over u64, signed or floating columns run on one GPU");
        if (c->flags & XLB_FLAG_KEEP_DELTAS) xlb_fail(XLB_ERR_UNSUPPORTED, "XLB_FLAG_KEEP_DELTAS with u64, signed or floating columns is not built");
        for (const xlb_rel* r : rels) {
            if (r->schema.arity < 1) xlb_fail(XLB_ERR_UNSUPPORTED, "plans take relations of at least one column");
            for (uint32_t k = 0; k < r->schema.arity; ++k)
                if (!type_built(r->schema.types[k])) xlb_fail(XLB_ERR_INVALID, "unknown column type");
        }
        for (auto& h : head_types) {
            if (h.second.arity < 1 || h.second.arity > XLB_MAX_ARITY) xlb_fail(XLB_ERR_UNSUPPORTED, "head %s: derived relations of 1 to %u columns are built", h.first.c_str(), XLB_MAX_ARITY);
            for (uint32_t k = 0; k < h.second.arity; ++k)
                if (!type_built(h.second.types[k])) xlb_fail(XLB_ERR_INVALID, "unknown column type");
            if (store_get(c, "__delta_" + h.first)) xlb_fail(XLB_ERR_UNSUPPORTED, "resuming a fixpoint over u64, signed or floating columns is not built");
        }
        if (!const_filters.empty()) {
            // a filter constant is an unsigned value: its place among signed or floating values is not defined here
            auto ordered = [](uint8_t t) { return t == XLB_I32 || t == XLB_I64 || t == XLB_F32 || t == XLB_F64; };
            bool typed = false;
            for (const xlb_rel* r : rels)
                for (uint32_t k = 0; k < r->schema.arity; ++k) typed |= ordered(r->schema.types[k]);
            for (auto& h : head_types)
                for (uint32_t k = 0; k < h.second.arity; ++k) typed |= ordered(h.second.types[k]);
            if (typed) xlb_fail(XLB_ERR_UNSUPPORTED, "filters with constants over signed or floating columns are not built");
        }
        dict = ops_dict_build(c, rels);
        std::vector<uint64_t> consts;
        for (const xlb_node* f : const_filters) consts.push_back(f->cmp_rhs);
        ops_dict_bounds(c, dict, consts, below, not_above);
        // the plan, with rank constants and 32-bit heads
        for (uint32_t s = 0; s < in->n_sccs; ++s) {
            xlb_scc scc = in->sccs[s];
            std::vector<xlb_rule> rr;
            for (uint32_t i = 0; scc.rules && i < scc.n_rules; ++i) {
                xlb_rule r = scc.rules[i];
                r.body = clone(r.body);
                for (uint32_t k = 0; k < r.head_schema.arity && k < XLB_MAX_ARITY; ++k) r.head_schema.types[k] = XLB_U32;
                rr.push_back(r);
            }
            rules.push_back(std::move(rr));
            scc.rules = rules.back().data();
            sccs.push_back(scc);
        }
        plan.sccs = sccs.data();
        plan.n_sccs = (uint32_t)sccs.size();
        // the ranks stand in for the relations
        active = true;
        for (auto& n : names) {
            auto it = c->store.find(n);
            if (it == c->store.end()) continue;
            xlb_rel* enc = ops_dict_encode(c, it->second, dict);
            originals[n] = it->second;
            it->second = enc;
            c->versions[n]++;
        }
        return &plan;
    }

    // After a successful run: decode the heads, put the inputs back.
    void finish() {
        if (!active) return;
        for (auto& h : head_types) {
            xlb_rel* ranks = store_get(c, h.first);
            if (!ranks) continue;
            xlb_rel* decoded = ops_dict_decode(c, ranks, h.second, dict);
            store_put(c, h.first, decoded);  // frees the rank relation
            auto o = originals.find(h.first);
            if (o != originals.end()) {      // a head that held rows before: superseded by the result
                delete o->second;
                originals.erase(o);
            }
        }
        restore_inputs();
        active = false;
    }

    // After a failure: nothing in rank space may stay behind.
    void rollback() {
        if (!active) return;
        for (auto& h : head_types) {
            if (originals.count(h.first)) continue;  // put back below
            auto it = c->store.find(h.first);
            if (it == c->store.end()) continue;
            delete it->second;
            c->store.erase(it);
            c->versions[h.first]++;
        }
        restore_inputs();
        active = false;
    }

    void restore_inputs() {
        for (auto& o : originals) {
            auto it = c->store.find(o.first);
            if (it != c->store.end()) delete it->second;
            c->store[o.first] = o.second;
            c->versions[o.first]++;
        }
        originals.clear();
    }
};

extern "C" xlb_status xlb_execute_plan(xlb_ctx* c, const xlb_plan* plan, xlb_run_stats* stats) {
    if (!c || !plan) return XLB_ERR_INVALID;
    RunState rs;
    EncodedRun enc;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    uint64_t launches0 = c->launches, syncs0 = c->syncs;
    double wait0 = c->ms_sync_wait, alloc0 = c->ms_alloc;
    auto host_t0 = std::chrono::steady_clock::now();
    c->trace_on = getenv("XLB_TRACE_HOST") != nullptr;
    c->trace.clear();
    const double trace_t0 = trace_now();
    c->peak = c->allocated;
    xlb_status result = XLB_OK;
    try {
        CUDA_OK(cudaSetDevice(c->device));
        CUDA_OK(cudaEventCreate(&e0));
        CUDA_OK(cudaEventCreate(&e1));
        CUDA_OK(cudaEventRecord(e0, c->stream));
        if (!plan->sccs && plan->n_sccs) xlb_fail(XLB_ERR_INVALID, "plan has no SCC array");
        std::set<std::string> heads;
        const xlb_plan* run = enc.begin(c, plan);
        for (uint32_t s = 0; s < run->n_sccs; ++s) {
            run_scc(c, run->sccs[s], rs);
            for (uint32_t i = 0; i < run->sccs[s].n_rules; ++i) heads.insert(run->sccs[s].rules[i].head);
        }
        enc.finish();
        check_dev_status(c);
        CUDA_OK(cudaEventRecord(e1, c->stream));
        CUDA_OK(cudaStreamSynchronize(c->stream));  // executor/mod.rs:1463
        float ms = 0;
        CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
        rs.st.ms_total = ms;
        uint64_t derived = 0;
        for (auto& h : heads) derived += store_get(c, h)->rows;
        if (c->world > 1) derived = comm_allreduce_sum(c, derived);
        rs.st.derived_tuples = derived;
        if (c->world > 1) rs.st.candidate_tuples = comm_allreduce_sum(c, rs.st.candidate_tuples);
    } catch (const XlbError& e) {
        c->last_error = e.msg;
        result = e.st;
        cudaStreamSynchronize(c->stream);
    } catch (const std::bad_alloc&) {
        c->last_error = "host allocation failed";
        result = XLB_ERR_RESOURCE_EXHAUSTED;
    }
    if (result != XLB_OK) {
        try {
            enc.rollback();
        } catch (...) {
            // the error already being reported is the one the caller sees
        }
    }
    xlb_resolve_phase_timers(c);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    rs.st.kernel_launches = c->launches - launches0;
    rs.st.host_syncs = c->syncs - syncs0;
    rs.st.ms_host_wait = c->ms_sync_wait - wait0;
    rs.st.ms_host_alloc = c->ms_alloc - alloc0;
    rs.st.ms_host_total = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - host_t0).count();
    rs.st.peak_bytes = c->peak;
    if (c->trace_on) {
        fprintf(stderr, "[xlb %u] plan: %.1f us on the host, %.1f us on the device\n", c->comm_rank, rs.st.ms_host_total * 1e3, rs.st.ms_total * 1e3);
        for (auto& n : c->trace) fprintf(stderr, "[xlb %u] %9.1f %8.1f  %s\n", c->comm_rank, n.t0 - trace_t0, n.t1 - n.t0, n.what);
        c->trace_on = false;
    }
    if (stats && result == XLB_OK) *stats = rs.st;
    return result;
}
