// xlog_oracle.cpp — CPU restatement of the reference's semi-naive fixpoint data plane.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA path is compared
// against; nothing in the product library links, loads or calls it.
//
// It restates, on the host and in plain C++, the operator semantics of the reference's
// `CudaKernelProvider` (crates/xlog-cuda/src/provider/relational.rs) and the loop of
// `Executor::execute_recursive_scc` (crates/xlog-runtime/src/executor/recursive.rs:447-957).
// The reference is Rust + CUDA and cannot be compiled where this file is built, so parity
// is pinned on the reference's own known-answer tests, transcribed as fixtures and checked
// by the CPU test suite (parity pinned by golden vectors, not by running the reference).
//
// Relations are row-major arrays of unsigned cells of one width class (all 32-bit or all
// 64-bit columns), the same restriction the reference's multiway route states
// (crates/xlog-runtime/src/executor/wcoj_dispatch.rs:1804-2061).
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../include/xlb.h"

namespace {

struct Rel {
    uint32_t arity = 0;
    uint32_t width = 4;           // bytes per cell: 4 or 8
    std::vector<uint64_t> cells;  // row-major, one cell per u64 (simple and exact for both widths)
    bool canonical = false;       // sorted by all columns + unique (memory.rs:1771-1773)
    uint64_t rows() const { return arity ? cells.size() / arity : 0; }
};

// Arity <= 2 with 32-bit cells is the hot shape: such relations are also kept as packed
// u64 keys (c0 << 32 | c1) so set operations are single-key problems whose ascending
// order equals the reference's lexicographic column order (relational.rs:1972-2217).
struct Packed {
    std::vector<uint64_t> k;
};

int g_threads = 1;

template <class F>
void parallel_for(size_t n, F f) {
    int t = std::max(1, std::min<int>(g_threads, (int)n));
    if (t == 1) {
        for (size_t i = 0; i < n; ++i) f(i);
        return;
    }
    std::atomic<size_t> next{0};
    std::vector<std::thread> th;
    for (int w = 0; w < t; ++w)
        th.emplace_back([&] {
            for (;;) {
                size_t i = next.fetch_add(1);
                if (i >= n) break;
                f(i);
            }
        });
    for (auto& x : th) x.join();
}

// Sort u64 keys: bucket by the top bits, then std::sort every bucket on its own thread.
void sort_u64(std::vector<uint64_t>& v) {
    size_t n = v.size();
    if (g_threads <= 1 || n < (1u << 16)) {
        std::sort(v.begin(), v.end());
        return;
    }
    uint64_t mx = 0;
    for (uint64_t x : v) mx |= x;
    int bits = 64 - __builtin_clzll(mx | 1);
    int shift = std::max(0, bits - 10);
    size_t nb = (size_t)(mx >> shift) + 1;
    std::vector<size_t> cnt(nb + 1, 0);
    for (uint64_t x : v) cnt[(x >> shift) + 1]++;
    for (size_t b = 0; b < nb; ++b) cnt[b + 1] += cnt[b];
    std::vector<uint64_t> out(n);
    std::vector<size_t> pos(cnt.begin(), cnt.end() - 1);
    for (uint64_t x : v) out[pos[x >> shift]++] = x;
    parallel_for(nb, [&](size_t b) { std::sort(out.begin() + cnt[b], out.begin() + cnt[b + 1]); });
    v.swap(out);
}

bool packable(const Rel& r) { return r.width == 4 && r.arity >= 1 && r.arity <= 2; }

std::vector<uint64_t> pack(const Rel& r) {
    std::vector<uint64_t> k(r.rows());
    if (r.arity == 1) {
        for (size_t i = 0; i < k.size(); ++i) k[i] = r.cells[i];
    } else {
        for (size_t i = 0; i < k.size(); ++i) k[i] = (r.cells[2 * i] << 32) | r.cells[2 * i + 1];
    }
    return k;
}

Rel unpack(const std::vector<uint64_t>& k, uint32_t arity, bool canonical) {
    Rel r;
    r.arity = arity;
    r.width = 4;
    r.canonical = canonical;
    r.cells.resize(k.size() * arity);
    if (arity == 1) {
        for (size_t i = 0; i < k.size(); ++i) r.cells[i] = k[i];
    } else {
        for (size_t i = 0; i < k.size(); ++i) {
            r.cells[2 * i] = k[i] >> 32;
            r.cells[2 * i + 1] = k[i] & 0xFFFFFFFFull;
        }
    }
    return r;
}

struct RowLess {
    const Rel* r;
    const uint32_t* keys;
    uint32_t nk;
    bool operator()(uint64_t a, uint64_t b) const {
        for (uint32_t i = 0; i < nk; ++i) {
            uint64_t x = r->cells[a * r->arity + keys[i]], y = r->cells[b * r->arity + keys[i]];
            if (x != y) return x < y;
        }
        return false;
    }
};

Rel gather_rows(const Rel& in, const std::vector<uint64_t>& idx) {
    Rel out;
    out.arity = in.arity;
    out.width = in.width;
    out.cells.resize(idx.size() * in.arity);
    for (size_t i = 0; i < idx.size(); ++i)
        std::memcpy(&out.cells[i * in.arity], &in.cells[idx[i] * in.arity], in.arity * 8);
    return out;
}

// sort (relational.rs:1881): stable, lexicographic, first key most significant.
Rel op_sort(const Rel& in, const uint32_t* keys, uint32_t nk) {
    std::vector<uint64_t> idx(in.rows());
    for (size_t i = 0; i < idx.size(); ++i) idx[i] = i;
    std::stable_sort(idx.begin(), idx.end(), RowLess{&in, keys, nk});
    return gather_rows(in, idx);
}

// dedup_full_row_deterministic (relational.rs:1558-1677): sort by all columns, keep the
// first of every run of equal rows; the result is certified canonical.
Rel op_dedup_full(const Rel& in) {
    if (in.canonical) return in;
    if (packable(in)) {
        auto k = pack(in);
        sort_u64(k);
        k.erase(std::unique(k.begin(), k.end()), k.end());
        return unpack(k, in.arity, true);
    }
    std::vector<uint32_t> all(in.arity);
    for (uint32_t i = 0; i < in.arity; ++i) all[i] = i;
    Rel s = op_sort(in, all.data(), in.arity);
    Rel out;
    out.arity = in.arity;
    out.width = in.width;
    out.canonical = true;
    uint64_t n = s.rows();
    for (uint64_t i = 0; i < n; ++i) {
        if (i && std::memcmp(&s.cells[i * s.arity], &s.cells[(i - 1) * s.arity], s.arity * 8) == 0) continue;
        out.cells.insert(out.cells.end(), s.cells.begin() + i * s.arity, s.cells.begin() + (i + 1) * s.arity);
    }
    return out;
}

// dedup with a proper key subset (relational.rs:238-275): stable sort by the key columns,
// keep the first row of every key group.
Rel op_dedup_keys(const Rel& in, const uint32_t* keys, uint32_t nk) {
    Rel s = op_sort(in, keys, nk);
    Rel out;
    out.arity = in.arity;
    out.width = in.width;
    uint64_t n = s.rows();
    for (uint64_t i = 0; i < n; ++i) {
        bool same = i > 0;
        for (uint32_t j = 0; same && j < nk; ++j)
            same = s.cells[i * s.arity + keys[j]] == s.cells[(i - 1) * s.arity + keys[j]];
        if (same) continue;
        out.cells.insert(out.cells.end(), s.cells.begin() + i * s.arity, s.cells.begin() + (i + 1) * s.arity);
    }
    return out;
}

bool compatible(const Rel& a, const Rel& b) { return a.arity == b.arity && a.width == b.width; }

// union_many_gpu (relational.rs:859-971): concatenate, then full-row dedup.  Two canonical
// inputs are merged instead of re-sorted; the resulting set is the same.
Rel op_union(const std::vector<const Rel*>& ins) {
    if (ins.size() == 1) return op_dedup_full(*ins[0]);
    if (ins.size() == 2 && ins[0]->canonical && ins[1]->canonical && packable(*ins[0])) {
        auto a = pack(*ins[0]), b = pack(*ins[1]);
        std::vector<uint64_t> o(a.size() + b.size());
        o.erase(std::set_union(a.begin(), a.end(), b.begin(), b.end(), o.begin()), o.end());
        return unpack(o, ins[0]->arity, true);
    }
    Rel cat;
    cat.arity = ins[0]->arity;
    cat.width = ins[0]->width;
    for (auto* r : ins) cat.cells.insert(cat.cells.end(), r->cells.begin(), r->cells.end());
    return op_dedup_full(cat);
}

// diff_via_deterministic_set (relational.rs:1311-1428): dedup a, dedup b, keep the rows of
// a that a search in sorted b does not find.
Rel op_diff(const Rel& a, const Rel& b) {
    Rel da = op_dedup_full(a), db = op_dedup_full(b);
    if (packable(da)) {
        auto ka = pack(da), kb = pack(db);
        std::vector<uint64_t> o(ka.size());
        o.erase(std::set_difference(ka.begin(), ka.end(), kb.begin(), kb.end(), o.begin()), o.end());
        return unpack(o, a.arity, true);
    }
    Rel out;
    out.arity = a.arity;
    out.width = a.width;
    out.canonical = true;
    uint64_t na = da.rows(), nb = db.rows(), j = 0;
    auto cmp = [&](uint64_t i, uint64_t jj) {
        for (uint32_t c = 0; c < a.arity; ++c) {
            uint64_t x = da.cells[i * a.arity + c], y = db.cells[jj * a.arity + c];
            if (x != y) return x < y ? -1 : 1;
        }
        return 0;
    };
    for (uint64_t i = 0; i < na; ++i) {
        while (j < nb && cmp(i, j) > 0) ++j;
        if (j < nb && cmp(i, j) == 0) continue;
        out.cells.insert(out.cells.end(), da.cells.begin() + i * a.arity, da.cells.begin() + (i + 1) * a.arity);
    }
    return out;
}

inline uint64_t mix64(uint64_t x) {
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdull;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ull;
    x ^= x >> 33;
    return x;
}

// hash_join_inner_v2 (relational.rs:4417-4625): build a table on the right side, probe with
// the left side, compare the actual keys (not only hashes), emit every matching pair.
// Output rows are ordered by left row, then by right row; the reference's order is
// unspecified (atomic append), so callers compare as multisets.
Rel op_join(const Rel& l, const Rel& r, const uint32_t* lk, const uint32_t* rk, uint32_t nk, int type) {
    Rel out;
    out.width = l.width;
    out.arity = type == XLB_JOIN_INNER ? l.arity + r.arity : l.arity;
    uint64_t nl = l.rows(), nr = r.rows();
    if (nl == 0 || (nr == 0 && type != XLB_JOIN_ANTI)) return out;
    size_t cap = 16;
    while (cap < 2 * nr) cap <<= 1;
    std::vector<int64_t> head(cap, -1), next(nr, -1);
    auto hkey = [&](const Rel& x, uint64_t row, const uint32_t* ks) {
        uint64_t h = 0x9E3779B97F4A7C15ull;
        for (uint32_t i = 0; i < nk; ++i) h = mix64(h ^ x.cells[row * x.arity + ks[i]]);
        return h & (cap - 1);
    };
    for (int64_t j = (int64_t)nr - 1; j >= 0; --j) {
        size_t b = hkey(r, j, rk);
        next[j] = head[b];
        head[b] = j;
    }
    int T = std::max(1, std::min<int>(g_threads, (int)((nl + 65535) / 65536)));
    std::vector<std::vector<uint64_t>> parts(T);
    parallel_for(T, [&](size_t t) {
        uint64_t lo = nl * t / T, hi = nl * (t + 1) / T;
        auto& o = parts[t];
        for (uint64_t i = lo; i < hi; ++i) {
            bool any = false;
            for (int64_t j = head[hkey(l, i, lk)]; j >= 0; j = next[j]) {
                bool eq = true;
                for (uint32_t q = 0; eq && q < nk; ++q)
                    eq = l.cells[i * l.arity + lk[q]] == r.cells[j * r.arity + rk[q]];
                if (!eq) continue;
                any = true;
                if (type != XLB_JOIN_INNER) break;
                o.insert(o.end(), l.cells.begin() + i * l.arity, l.cells.begin() + (i + 1) * l.arity);
                o.insert(o.end(), r.cells.begin() + j * r.arity, r.cells.begin() + (j + 1) * r.arity);
            }
            if ((type == XLB_JOIN_SEMI && any) || (type == XLB_JOIN_ANTI && !any))
                o.insert(o.end(), l.cells.begin() + i * l.arity, l.cells.begin() + (i + 1) * l.arity);
        }
    });
    size_t tot = 0;
    for (auto& p : parts) tot += p.size();
    out.cells.reserve(tot);
    for (auto& p : parts) out.cells.insert(out.cells.end(), p.begin(), p.end());
    return out;
}

// execute_project with pass-through columns (executor/expression.rs:779-836).
Rel op_project(const Rel& in, const uint32_t* cols, uint32_t n) {
    Rel out;
    out.arity = n;
    out.width = in.width;
    uint64_t rows = in.rows();
    out.cells.resize(rows * n);
    for (uint64_t i = 0; i < rows; ++i)
        for (uint32_t c = 0; c < n; ++c) out.cells[i * n + c] = in.cells[i * in.arity + cols[c]];
    return out;
}

bool cmp_eval(uint32_t op, uint64_t a, uint64_t b) {
    switch (op) {
        case XLB_EQ: return a == b;
        case XLB_NE: return a != b;
        case XLB_LT: return a < b;
        case XLB_LE: return a <= b;
        case XLB_GT: return a > b;
        default: return a >= b;
    }
}

// filter_compare_* + mask compaction (kernels/filter.cu; provider/filter.rs:1792-1938).
Rel op_filter(const Rel& in, const xlb_node* n) {
    Rel out;
    out.arity = in.arity;
    out.width = in.width;
    uint64_t rows = in.rows();
    for (uint64_t i = 0; i < rows; ++i) {
        uint64_t a = in.cells[i * in.arity + n->cmp_lhs_col];
        uint64_t b = n->cmp_rhs_is_const ? n->cmp_rhs : in.cells[i * in.arity + n->cmp_rhs];
        if (cmp_eval(n->cmp, a, b))
            out.cells.insert(out.cells.end(), in.cells.begin() + i * in.arity, in.cells.begin() + (i + 1) * in.arity);
    }
    return out;
}

struct Exec {
    uint64_t max_iterations = 1000000;
    std::map<uint32_t, std::string> rel_names;  // register_relation
    std::map<std::string, Rel> store;           // RelationStore (relation.rs:45-140)
    std::string error;
    uint64_t iterations = 0, candidates = 0;
};

struct Fail {
    xlb_status st;
    std::string msg;
};

// execute_node arms Scan/Filter/Project/Join/Union (executor/node_dispatch.rs:98-319).
// `subst` maps a rel_id to a relation name for one delta variant (rewrite_scan_nth).
Rel eval(Exec& ex, const xlb_node* n, const std::map<const xlb_node*, std::string>& subst) {
    switch (n->kind) {
        case XLB_NODE_SCAN: {
            std::string name;
            auto s = subst.find(n);
            if (s != subst.end()) name = s->second;
            else {
                auto it = ex.rel_names.find(n->rel_id);
                if (it == ex.rel_names.end()) throw Fail{XLB_ERR_INVALID, "scan of unregistered relation id"};
                name = it->second;
            }
            auto r = ex.store.find(name);
            if (r == ex.store.end()) throw Fail{XLB_ERR_NOT_FOUND, "Missing relation: " + name};
            return r->second;  // the reference deep-copies every scan (node_dispatch.rs:68-83)
        }
        case XLB_NODE_FILTER: return op_filter(eval(ex, n->input, subst), n);
        case XLB_NODE_PROJECT: {
            Rel in = eval(ex, n->input, subst);
            for (uint32_t c = 0; c < n->n_cols; ++c)
                if (n->cols[c] >= in.arity) throw Fail{XLB_ERR_INVALID, "projection column out of range"};
            return op_project(in, n->cols, n->n_cols);
        }
        case XLB_NODE_JOIN: {
            Rel l = eval(ex, n->left, subst), r = eval(ex, n->right, subst);
            if (l.width != r.width) throw Fail{XLB_ERR_TYPE, "join key type mismatch"};
            Rel o = op_join(l, r, n->left_keys, n->right_keys, n->n_keys, (int)n->join_type);
            o.arity = n->join_type == XLB_JOIN_INNER ? l.arity + r.arity : l.arity;
            return o;
        }
        case XLB_NODE_UNION: {
            Rel cat;
            for (uint32_t i = 0; i < n->n_inputs; ++i) {
                Rel x = eval(ex, n->inputs[i], subst);
                if (i == 0) { cat.arity = x.arity; cat.width = x.width; }
                cat.cells.insert(cat.cells.end(), x.cells.begin(), x.cells.end());
            }
            return cat;
        }
        case XLB_NODE_DIFF: {  // execute_diff (executor/node_dispatch.rs:264)
            Rel l = eval(ex, n->left, subst), r = eval(ex, n->right, subst);
            if (!compatible(l, r)) throw Fail{XLB_ERR_TYPE, "difference of incompatible schemas"};
            return op_diff(l, r);
        }
        case XLB_NODE_DISTINCT: {  // execute_distinct -> dedup (relational.rs:238)
            Rel in = eval(ex, n->input, subst);
            for (uint32_t c = 0; c < n->n_cols; ++c)
                if (n->cols[c] >= in.arity) throw Fail{XLB_ERR_INVALID, "dedup key column out of range"};
            return (n->n_cols == 0 || n->n_cols >= in.arity) ? op_dedup_full(in) : op_dedup_keys(in, n->cols, n->n_cols);
        }
    }
    throw Fail{XLB_ERR_INVALID, "unknown plan node kind"};
}

void collect_scans(const xlb_node* n, std::vector<const xlb_node*>& out) {
    switch (n->kind) {
        case XLB_NODE_SCAN: out.push_back(n); break;
        case XLB_NODE_FILTER:
        case XLB_NODE_DISTINCT:
        case XLB_NODE_PROJECT: collect_scans(n->input, out); break;
        case XLB_NODE_DIFF:
        case XLB_NODE_JOIN: collect_scans(n->left, out); collect_scans(n->right, out); break;
        case XLB_NODE_UNION: for (uint32_t i = 0; i < n->n_inputs; ++i) collect_scans(n->inputs[i], out); break;
    }
}

Rel empty_like(const xlb_schema& s) {
    Rel r;
    r.arity = s.arity;
    r.width = (s.arity && (s.types[0] == XLB_U64 || s.types[0] == XLB_I64 || s.types[0] == XLB_F64)) ? 8 : 4;
    r.canonical = true;
    return r;
}

// Non-recursive SCC: every rule once, one multiway union per head
// (executor/recursive.rs:308-438, install_dispatched_head_batch).
void run_stable_scc(Exec& ex, const xlb_scc& scc) {
    std::map<std::string, std::vector<Rel>> by_head;
    for (uint32_t i = 0; i < scc.n_rules; ++i) {
        Rel r = eval(ex, scc.rules[i].body, {});
        ex.candidates += r.rows();
        by_head[scc.rules[i].head].push_back(std::move(r));
    }
    for (auto& kv : by_head) {
        std::vector<const Rel*> ins;
        auto old = ex.store.find(kv.first);
        if (old != ex.store.end()) ins.push_back(&old->second);
        for (auto& r : kv.second) ins.push_back(&r);
        Rel u = op_union(ins);
        ex.store[kv.first] = std::move(u);
    }
}

// execute_recursive_scc (executor/recursive.rs:447-957).
void run_recursive_scc(Exec& ex, const xlb_scc& scc) {
    std::vector<std::string> preds;
    std::map<std::string, xlb_schema> schema;
    for (uint32_t i = 0; i < scc.n_rules; ++i) {
        std::string h = scc.rules[i].head;
        if (!schema.count(h)) { preds.push_back(h); schema[h] = scc.rules[i].head_schema; }
    }
    std::sort(preds.begin(), preds.end());  // BTreeSet order (recursive.rs:456-467)
    for (auto& p : preds)
        if (!ex.store.count(p)) ex.store[p] = empty_like(schema[p]);  // :471-486
    auto delta_name = [](const std::string& p) { return "__delta_" + p; };

    // seed: all rules once against the current store (:516-523)
    std::map<std::string, std::vector<Rel>> seeded;
    for (uint32_t i = 0; i < scc.n_rules; ++i) {
        Rel r = eval(ex, scc.rules[i].body, {});
        ex.candidates += r.rows();
        seeded[scc.rules[i].head].push_back(std::move(r));
    }
    for (auto& p : preds) {  // :530-609
        Rel& full_old = ex.store[p];
        std::vector<const Rel*> ins{&full_old};
        for (auto& r : seeded[p]) ins.push_back(&r);
        Rel full_new = op_union(ins);
        Rel d0;
        if (full_new.rows() == 0) d0 = empty_like(schema[p]);
        else if (full_old.rows() == 0) d0 = full_new;
        else d0 = op_diff(full_new, full_old);
        ex.store[delta_name(p)] = std::move(d0);
        ex.store[p] = std::move(full_new);
    }

    bool fix = false;
    for (uint64_t it = 0; it < ex.max_iterations; ++it) {  // :619-937
        ex.iterations++;
        std::map<std::string, std::vector<Rel>> raw;
        for (uint32_t i = 0; i < scc.n_rules; ++i) {
            const xlb_rule& rule = scc.rules[i];
            std::vector<const xlb_node*> scans;
            collect_scans(rule.body, scans);
            for (const xlb_node* s : scans) {  // one variant per recursive scan occurrence (:636-664)
                auto nm = ex.rel_names.find(s->rel_id);
                if (nm == ex.rel_names.end()) continue;
                if (!schema.count(nm->second)) continue;
                const Rel& d = ex.store[delta_name(nm->second)];
                if (d.rows() == 0) continue;
                std::map<const xlb_node*, std::string> subst{{s, delta_name(nm->second)}};
                Rel out = eval(ex, rule.body, subst);  // :709
                ex.candidates += out.rows();
                raw[rule.head].push_back(std::move(out));
            }
        }
        bool changed = false;
        for (auto& p : preds) {  // :735-858
            auto& bufs = raw[p];
            Rel dn;
            if (bufs.empty()) dn = empty_like(schema[p]);
            else {
                std::vector<const Rel*> ins;
                for (auto& r : bufs) ins.push_back(&r);
                Rel draw = bufs.size() == 1 ? std::move(bufs[0]) : op_union(ins);
                dn = draw.rows() == 0 ? empty_like(schema[p]) : op_diff(draw, ex.store[p]);  // :790
            }
            if (dn.rows()) changed = true;
            ex.store[delta_name(p)] = std::move(dn);
        }
        if (!changed) { fix = true; break; }  // :861-865
        for (auto& p : preds) {               // :868-937
            Rel& d = ex.store[delta_name(p)];
            if (d.rows() == 0) continue;
            std::vector<const Rel*> ins{&ex.store[p], &d};
            Rel m = op_union(ins);
            ex.store[p] = std::move(m);
        }
    }
    for (auto& p : preds) ex.store.erase(delta_name(p));  // :940-945
    if (!fix) throw Fail{XLB_ERR_ITER_LIMIT, "Recursive SCC iteration limit (" + std::to_string(ex.max_iterations) + ") exceeded"};
}

}  // namespace

extern "C" {

struct xo_rel { Rel r; };
struct xo_exec { Exec e; };

void xo_set_threads(int t) { g_threads = t < 1 ? 1 : t; }

xo_rel* xo_rel_from_cols(uint32_t arity, uint32_t width, const void* const* cols, uint64_t rows) {
    auto* x = new xo_rel;
    x->r.arity = arity;
    x->r.width = width;
    x->r.cells.resize(rows * arity);
    for (uint32_t c = 0; c < arity; ++c)
        for (uint64_t i = 0; i < rows; ++i)
            x->r.cells[i * arity + c] = width == 4 ? ((const uint32_t*)cols[c])[i] : ((const uint64_t*)cols[c])[i];
    return x;
}
uint64_t xo_rel_rows(const xo_rel* r) { return r->r.rows(); }
uint32_t xo_rel_arity(const xo_rel* r) { return r->r.arity; }
uint32_t xo_rel_width(const xo_rel* r) { return r->r.width; }
int xo_rel_canonical(const xo_rel* r) { return r->r.canonical; }
void xo_rel_to_cols(const xo_rel* r, void* const* cols) {
    uint64_t rows = r->r.rows();
    for (uint32_t c = 0; c < r->r.arity; ++c)
        for (uint64_t i = 0; i < rows; ++i) {
            uint64_t v = r->r.cells[i * r->r.arity + c];
            if (r->r.width == 4) ((uint32_t*)cols[c])[i] = (uint32_t)v;
            else ((uint64_t*)cols[c])[i] = v;
        }
}
void xo_rel_free(xo_rel* r) { delete r; }

xo_rel* xo_sort(const xo_rel* in, const uint32_t* keys, uint32_t nk) { return new xo_rel{op_sort(in->r, keys, nk)}; }
xo_rel* xo_dedup(const xo_rel* in, const uint32_t* keys, uint32_t nk) {
    bool full = nk == 0 || nk >= in->r.arity;
    return new xo_rel{full ? op_dedup_full(in->r) : op_dedup_keys(in->r, keys, nk)};
}
xo_rel* xo_union(const xo_rel* const* ins, uint32_t n) {
    if (n == 0) return nullptr;  // union_many_gpu of no inputs is an error (set_ops_tests.rs:922)
    std::vector<const Rel*> v;
    for (uint32_t i = 0; i < n; ++i) {
        if (!compatible(ins[0]->r, ins[i]->r)) return nullptr;  // set_ops_tests.rs:952
        v.push_back(&ins[i]->r);
    }
    return new xo_rel{op_union(v)};
}
xo_rel* xo_diff(const xo_rel* a, const xo_rel* b) {
    if (!compatible(a->r, b->r)) return nullptr;
    return new xo_rel{op_diff(a->r, b->r)};
}
xo_rel* xo_hash_join(const xo_rel* l, const xo_rel* r, const uint32_t* lk, const uint32_t* rk, uint32_t nk, int type) {
    if (l->r.width != r->r.width) return nullptr;
    return new xo_rel{op_join(l->r, r->r, lk, rk, nk, type)};
}

xo_exec* xo_exec_new(uint64_t max_iterations) {
    auto* e = new xo_exec;
    if (max_iterations) e->e.max_iterations = max_iterations;
    return e;
}
void xo_exec_free(xo_exec* e) { delete e; }
void xo_register(xo_exec* e, uint32_t id, const char* name) { e->e.rel_names[id] = name; }
void xo_put(xo_exec* e, const char* name, const xo_rel* rel) { e->e.store[name] = rel->r; }
xo_rel* xo_get(xo_exec* e, const char* name) {
    auto it = e->e.store.find(name);
    return it == e->e.store.end() ? nullptr : new xo_rel{it->second};
}
const char* xo_error(const xo_exec* e) { return e->e.error.c_str(); }
uint64_t xo_iterations(const xo_exec* e) { return e->e.iterations; }
uint64_t xo_candidates(const xo_exec* e) { return e->e.candidates; }

// Executor::execute_plan (executor/mod.rs:1404-1469).
int xo_execute_plan(xo_exec* e, const xlb_plan* plan) {
    try {
        for (uint32_t s = 0; s < plan->n_sccs; ++s) {
            if (plan->sccs[s].is_recursive) run_recursive_scc(e->e, plan->sccs[s]);
            else run_stable_scc(e->e, plan->sccs[s]);
        }
    } catch (const Fail& f) {
        e->e.error = f.msg;
        return f.st;
    }
    return XLB_OK;
}

}  // extern "C"
