/* The C ABI from plain C (C99): transitive closure of {(1,2),(2,3),(3,4)}, the reference's first
 * end-to-end example (crates/xlog-integration/tests/e2e_integration_tests.rs:256-315), then a
 * group-by over the result.  Exit code 0 only if every row matches.
 *
 *   cc -std=c99 -Iinclude tests/abi_example.c -Lxlog_b200 -lxlb -o abi_example
 */
#include <stdio.h>
#include <string.h>

#include "xlb.h"

#define CHECK(call)                                                                   \
    do {                                                                              \
        xlb_status st_ = (call);                                                      \
        if (st_ != XLB_OK) {                                                          \
            fprintf(stderr, "%s -> %d: %s\n", #call, (int)st_, xlb_last_error(ctx)); /* NULL: the message of a failed xlb_ctx_create */ \
            return 10;                                                                \
        }                                                                             \
    } while (0)

int main(void) {
    xlb_ctx* ctx = NULL;
    xlb_config cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.device = 0;
    CHECK(xlb_ctx_create(&cfg, &ctx));

    /* edge(u32, u32) from two host columns */
    const uint32_t src[3] = {1, 2, 3}, dst[3] = {2, 3, 4};
    const void* cols[2] = {src, dst};
    xlb_schema pair;
    memset(&pair, 0, sizeof pair);
    pair.arity = 2;
    pair.types[0] = XLB_U32;
    pair.types[1] = XLB_U32;
    xlb_rel* edge = NULL;
    CHECK(xlb_rel_from_host(ctx, &pair, cols, 3, &edge));
    CHECK(xlb_register_relation(ctx, 0, "edge"));
    CHECK(xlb_register_relation(ctx, 1, "reach"));
    CHECK(xlb_store_put(ctx, "edge", edge)); /* the store owns it now */

    /* reach(X,Y) :- edge(X,Y).   reach(X,Z) :- reach(X,Y), edge(Y,Z). */
    xlb_node scan_edge, scan_reach, join, project;
    memset(&scan_edge, 0, sizeof scan_edge);
    scan_edge.kind = XLB_NODE_SCAN;
    scan_edge.rel_id = 0;
    scan_reach = scan_edge;
    scan_reach.rel_id = 1;
    memset(&join, 0, sizeof join);
    join.kind = XLB_NODE_JOIN;
    join.left = &scan_reach;
    join.right = &scan_edge;
    join.n_keys = 1;
    join.left_keys[0] = 1;
    join.right_keys[0] = 0;
    join.join_type = XLB_JOIN_INNER;
    memset(&project, 0, sizeof project);
    project.kind = XLB_NODE_PROJECT;
    project.input = &join;
    project.n_cols = 2;
    project.cols[0] = 0;
    project.cols[1] = 3;
    xlb_rule rules[2];
    rules[0].head = "reach";
    rules[0].body = &scan_edge;
    rules[0].head_schema = pair;
    rules[1].head = "reach";
    rules[1].body = &project;
    rules[1].head_schema = pair;
    xlb_scc scc;
    scc.id = 0;
    scc.is_recursive = 1;
    scc.rules = rules;
    scc.n_rules = 2;
    xlb_plan plan;
    plan.sccs = &scc;
    plan.n_sccs = 1;
    xlb_run_stats stats;
    CHECK(xlb_execute_plan(ctx, &plan, &stats));

    const xlb_rel* reach = NULL;
    CHECK(xlb_store_get(ctx, "reach", &reach));
    uint32_t x[8], y[8];
    void* out[2] = {x, y};
    uint64_t rows = 0;
    CHECK(xlb_rel_to_host(ctx, reach, out, 8, &rows));
    const uint32_t wx[6] = {1, 1, 1, 2, 2, 3}, wy[6] = {2, 3, 4, 3, 4, 4};
    int bad = rows != 6;
    for (uint64_t i = 0; i < rows && i < 6; ++i) bad |= x[i] != wx[i] || y[i] != wy[i];
    printf("reach: %llu rows, %llu iterations, %llu kernel launches\n", (unsigned long long)rows,
           (unsigned long long)stats.iterations, (unsigned long long)stats.kernel_launches);

    /* how many nodes each node reaches: group by column 0, count */
    const uint32_t key = 0, val = 1, op = XLB_AGG_COUNT;
    xlb_rel* counts = NULL;
    CHECK(xlb_groupby(ctx, reach, &key, 1, &val, &op, 1, &counts));
    uint32_t node[4];
    uint64_t n_reached[4];
    void* gout[2] = {node, n_reached};
    uint64_t groups = 0;
    CHECK(xlb_rel_to_host(ctx, counts, gout, 4, &groups));
    const uint64_t want_counts[3] = {3, 2, 1};
    bad |= groups != 3;
    for (uint64_t i = 0; i < groups && i < 3; ++i) bad |= node[i] != i + 1 || n_reached[i] != want_counts[i];
    xlb_rel_free(counts);
    xlb_ctx_destroy(ctx);
    printf(bad ? "MISMATCH\n" : "ok\n");
    return bad ? 1 : 0;
}
