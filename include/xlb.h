/*
 * xlb.h — C ABI of the B200-native semi-naive Datalog fixpoint data plane.
 *
 * Every entry point is what a foreign-function binding for the reference's
 * relational operator surface would bind.  The reference has no FFI seam of its
 * own (its executor calls inherent methods of `CudaKernelProvider`), so each
 * declaration cites the reference method or type whose contract it keeps, by
 * path inside the reference project.
 *
 * Conventions
 *   - every function returns an xlb_status and never aborts or traps;
 *   - out-parameters are written only on XLB_OK;
 *   - operators never mutate their inputs and return fresh relations
 *     (the reference's convention: crates/xlog-cuda/src/provider/relational.rs);
 *   - a relation handed back to the caller is caller-owned (xlb_rel_free);
 *     xlb_store_put transfers ownership to the context's store;
 *   - a context may be used from one thread at a time
 *     (crates/xlog-runtime/src/relation.rs:20-23 states the same for the reference);
 *   - all device work of a call has completed when the call returns;
 *   - there is no CPU fallback: without a CUDA device xlb_ctx_create fails.
 *
 * Relations are device-resident, column-major, with 32-bit or 64-bit unsigned
 * columns (crates/xlog-cuda/src/memory.rs:1429-1433,1758-1774).
 */
#ifndef XLB_H
#define XLB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XLB_MAX_ARITY 8u
#define XLB_MAX_KEYS 2u
#define XLB_UNIQUE_ID_BYTES 128u

typedef struct xlb_ctx xlb_ctx;
typedef struct xlb_rel xlb_rel;

/* Error classes of the reference's XlogError (crates/xlog-core/src/error.rs:8-100). */
typedef enum xlb_status {
    XLB_OK = 0,
    XLB_ERR_INVALID = 1,            /* bad argument / malformed plan   (XlogError::Execution)         */
    XLB_ERR_TYPE = 2,               /* schema or key type mismatch     (XlogError::Kernel)            */
    XLB_ERR_RESOURCE_EXHAUSTED = 3, /* device memory budget refused    (XlogError::ResourceExhausted) */
    XLB_ERR_CAPACITY = 4,           /* an output exceeded its capacity (device overflow flag)         */
    XLB_ERR_ITER_LIMIT = 5,         /* recursive SCC iteration limit   (executor/recursive.rs:947-954)*/
    XLB_ERR_CUDA = 6,
    XLB_ERR_NCCL = 7,
    XLB_ERR_TIMEOUT = 8,            /* a bounded device-side wait ran out */
    XLB_ERR_UNSUPPORTED = 9,        /* valid request outside the built scope */
    XLB_ERR_NOT_FOUND = 10          /* store lookup miss */
} xlb_status;

/* Column types: the reference's kernel type codes (crates/xlog-core/src/types.rs:33-62).
 * Built here: U32, U64 and SYMBOL (an interned u32 id, ordered as u32). */
typedef enum xlb_type {
    XLB_U32 = 0,
    XLB_U64 = 1,
    XLB_I32 = 2,
    XLB_I64 = 3,
    XLB_F32 = 4,
    XLB_F64 = 5,
    XLB_BOOL = 6,
    XLB_SYMBOL = 7
} xlb_type;

/* Schema: arity + column types (names are ignored by every operator, as in the
 * reference's type-compatibility check, relational.rs:859-971). */
typedef struct xlb_schema {
    uint32_t arity;
    uint8_t types[XLB_MAX_ARITY];
} xlb_schema;

/* RuntimeConfig subset (crates/xlog-core/src/config.rs:57-200). */
typedef struct xlb_config {
    int32_t device;               /* CUDA device ordinal; -1 = current device                     */
    uint64_t memory_budget_bytes; /* 0 = 90 % of the device's free memory (MemoryBudget)          */
    uint64_t max_iterations;      /* 0 = 1,000,000, the reference default (config.rs:164)         */
    uint64_t join_chunk_tuples;   /* upper bound on join candidates materialised at once; 0 = auto */
    uint32_t flags;               /* XLB_FLAG_*                                                    */
} xlb_config;

#define XLB_FLAG_PROFILE 1u        /* time every phase with CUDA events (RuntimeConfig.profile)     */
#define XLB_FLAG_NO_DENSE 2u       /* never take the bitmap route for small dense domains (the kill
                                      switch the reference gives its factorized routes,
                                      XLOG_DISABLE_FACTORIZED_DELTA)                                 */
#define XLB_FLAG_KEEP_DELTAS 4u    /* when a recursive SCC stops at the iteration limit, leave its
                                      delta relations in the store under "__delta_<head>" so that
                                      the state (full, delta) can be saved; a later
                                      xlb_execute_plan that finds the delta of every head of an SCC
                                      in the store resumes that SCC from them instead of seeding it */
#define XLB_FLAG_NO_TUPLE_SET 16u  /* never keep a derived relation as a hash set: candidates of a head
                                      too wide for a bitmap are then always sorted, deduplicated and
                                      subtracted by merging (the counterpart of the reference's
                                      XLOG_DISABLE_FACTORIZED_DELTA for its sparse route)            */
#define XLB_FLAG_GENERAL_ONLY 32u  /* evaluate every rule body node by node on column-major relations
                                      (the general evaluator that otherwise only takes rules with
                                      more than two live columns): the reference's own evaluation
                                      order, for comparing the two engines                           */
#define XLB_FLAG_SHUFFLE_ONLY 8u   /* several ranks: never give every rank a full copy of a relation
                                      (no replicated evaluation of small-domain components, no
                                      broadcast of small stored relations): every join runs on hash
                                      partitions with an all-to-all exchange                          */

/* ---- context ------------------------------------------------------------------------------ */

/* Replaces provider construction: CudaKernelProvider::with_runtime +
 * GpuMemoryManager::with_runtime (crates/xlog-cli/src/main.rs:1151-1186). */
xlb_status xlb_ctx_create(const xlb_config* cfg, xlb_ctx** out);
void xlb_ctx_destroy(xlb_ctx* ctx);

/* Message of the last failing call on this context (XlogError's Display text). */
const char* xlb_last_error(const xlb_ctx* ctx);

/* GpuMemoryManager::allocated_bytes / peak_bytes (crates/xlog-cuda/src/memory.rs:1096-1126). */
xlb_status xlb_memory_stats(const xlb_ctx* ctx, uint64_t* allocated_bytes, uint64_t* peak_bytes);

/* ---- relations ---------------------------------------------------------------------------- */

/* create_buffer_from_slices (crates/xlog-cuda/src/provider/io.rs:75): one host array per
 * column, `rows` elements each, of the width the schema gives.  Host -> device copy. */
xlb_status xlb_rel_from_host(xlb_ctx* ctx, const xlb_schema* schema, const void* const* cols,
                             uint64_t rows, xlb_rel** out);
/* create_empty_buffer(schema). */
xlb_status xlb_rel_empty(xlb_ctx* ctx, const xlb_schema* schema, xlb_rel** out);
/* device_row_count (crates/xlog-cuda/src/provider/mod.rs:2823): the logical row count. */
xlb_status xlb_rel_rows(const xlb_rel* rel, uint64_t* rows);
xlb_status xlb_rel_schema(const xlb_rel* rel, xlb_schema* schema);
/* canonical_full_row_set_certified (memory.rs:1771-1773): sorted by all columns and unique. */
xlb_status xlb_rel_is_canonical(const xlb_rel* rel, int* canonical);
/* download_column::<T> for every column (crates/xlog-cuda/src/provider/transfer.rs:22).
 * Copies min(rows, cap_rows) rows into the host arrays and reports the logical row count. */
xlb_status xlb_rel_to_host(xlb_ctx* ctx, const xlb_rel* rel, void* const* cols, uint64_t cap_rows,
                           uint64_t* rows);
/* clone_buffer (relational.rs:6113). */
xlb_status xlb_rel_clone(xlb_ctx* ctx, const xlb_rel* rel, xlb_rel** out);
void xlb_rel_free(xlb_rel* rel);
/* No counterpart in the reference (its tests download and compare).  An order-independent digest of
 * a relation's rows, computed on the device: every row is folded into one 64-bit word — for one or
 * two 32-bit columns the packed row (c0, or c0 << 32 | c1), for anything else h = 0, then for each
 * column h = mix(h ^ value) with mix the 64-bit finaliser xlb_owner_of uses — and mixed once more;
 * digest[0] = row count, digest[1] = XOR of the mixed words, digest[2] = sum of their low 32 bits
 * (mod 2^64).  Digests of disjoint shards combine by adding [0] and [2] and XOR-ing [1], so a
 * result spread over several ranks can be compared with the same result held by one. */
xlb_status xlb_rel_checksum(xlb_ctx* ctx, const xlb_rel* rel, uint64_t digest[3]);

/* ---- relational operators ----------------------------------------------------------------- */

/* JoinType (crates/xlog-ir/src/rir.rs). Built here: INNER, SEMI, ANTI. */
typedef enum xlb_join_type { XLB_JOIN_INNER = 0, XLB_JOIN_SEMI = 1, XLB_JOIN_ANTI = 2 } xlb_join_type;

/* hash_join_v2 (relational.rs:2926): equi-join on up to XLB_MAX_KEYS key columns.
 * INNER: output columns = all left columns then all right columns, bag semantics (every
 * matching pair once), rows ordered by left row then by right row.  SEMI / ANTI: the left rows
 * that have / lack a match, left columns only, in left order.  Key column types must match
 * pairwise (XLB_ERR_TYPE).  An empty side yields an empty relation of the output schema. */
xlb_status xlb_hash_join(xlb_ctx* ctx, const xlb_rel* left, const xlb_rel* right,
                         const uint32_t* left_keys, const uint32_t* right_keys, uint32_t n_keys,
                         xlb_join_type join_type, xlb_rel** out);

/* sort (relational.rs:1881): stable, lexicographic over key_cols, first key most significant,
 * unsigned order; all columns are carried. */
xlb_status xlb_sort(xlb_ctx* ctx, const xlb_rel* in, const uint32_t* key_cols, uint32_t n_keys,
                    xlb_rel** out);

/* dedup (relational.rs:238).  key_cols covering every column (or n_keys == 0) is the full-row
 * form: the result is sorted by all columns, unique, and certified canonical.  A proper subset
 * keeps, for every distinct key, the first row in stable key order. */
xlb_status xlb_dedup(xlb_ctx* ctx, const xlb_rel* in, const uint32_t* key_cols, uint32_t n_keys,
                     xlb_rel** out);

/* union_gpu / union_many_gpu (relational.rs:822,859): set union of n >= 1 type-compatible
 * relations; the result is sorted, unique and certified.  n == 0 is XLB_ERR_INVALID. */
xlb_status xlb_union(xlb_ctx* ctx, const xlb_rel* const* ins, uint32_t n, xlb_rel** out);

/* diff_gpu (relational.rs:1102): a \ b with set semantics on full rows; sorted, unique. */
xlb_status xlb_diff(xlb_ctx* ctx, const xlb_rel* a, const xlb_rel* b, xlb_rel** out);

/* AggOp (crates/xlog-ir/src/rir.rs).  Built here: count, sum, min, max. */
typedef enum xlb_agg_op { XLB_AGG_COUNT = 0, XLB_AGG_SUM = 1, XLB_AGG_MIN = 2, XLB_AGG_MAX = 3 } xlb_agg_op;

/* groupby_multi_agg (crates/xlog-cuda/src/provider/groupby.rs:66): one row per distinct value of
 * the key columns (u32, symbol or u64; ascending), the key columns first, then one column per
 * (agg_cols[i], agg_ops[i]) in the order given.  Count and sum columns are u64; min and max keep
 * the width of their value column (u32 or u64 values).  An empty input gives an empty relation of
 * the output schema; no key column or no aggregation is XLB_ERR_INVALID. */
xlb_status xlb_groupby(xlb_ctx* ctx, const xlb_rel* in, const uint32_t* key_cols, uint32_t n_keys,
                       const uint32_t* agg_cols, const uint32_t* agg_ops, uint32_t n_aggs, xlb_rel** out);

/* ---- plans: the subset of RirNode the fixpoint path uses (crates/xlog-ir/src/rir.rs:339-541) - */

typedef enum xlb_node_kind {
    XLB_NODE_SCAN = 1,    /* RirNode::Scan { rel }                                              */
    XLB_NODE_FILTER = 2,  /* RirNode::Filter { input, predicate } with a column comparison      */
    XLB_NODE_PROJECT = 3, /* RirNode::Project { input, columns } with pass-through columns      */
    XLB_NODE_JOIN = 4,    /* RirNode::Join { left, right, left_keys, right_keys, join_type }    */
    XLB_NODE_UNION = 5,   /* RirNode::Union { inputs }                                          */
    XLB_NODE_DIFF = 6,    /* RirNode::Diff { left, right } (rir.rs:429-434): set difference,
                             sorted and unique, as diff_gpu (executor/node_dispatch.rs:264)     */
    XLB_NODE_DISTINCT = 7 /* RirNode::Distinct { input, key_cols } (rir.rs:421-426): `cols` holds
                             the key columns; all columns or none = full-row, as xlb_dedup      */
} xlb_node_kind;

/* CompareOp (rir.rs:296-310). */
typedef enum xlb_cmp { XLB_EQ = 0, XLB_NE = 1, XLB_LT = 2, XLB_LE = 3, XLB_GT = 4, XLB_GE = 5 } xlb_cmp;

/* A promoted node (ChainJoin, MultiWayJoin) is passed as its `fallback` tree, which the
 * reference guarantees to be row-set equivalent (rir.rs:386-404, 449-457). */
typedef struct xlb_node {
    uint32_t kind;
    uint32_t rel_id;                      /* SCAN                                             */
    const struct xlb_node* input;         /* FILTER, PROJECT, DISTINCT                        */
    const struct xlb_node* left;          /* JOIN, DIFF                                       */
    const struct xlb_node* right;         /* JOIN, DIFF                                       */
    uint32_t n_keys;                      /* JOIN                                             */
    uint32_t left_keys[XLB_MAX_KEYS];     /* JOIN: column indices of the left input           */
    uint32_t right_keys[XLB_MAX_KEYS];    /* JOIN: column indices of the right input          */
    uint32_t n_cols;                      /* PROJECT, DISTINCT                                */
    uint32_t cols[XLB_MAX_ARITY];         /* PROJECT: input column per output column; DISTINCT: key columns */
    uint32_t cmp;                         /* FILTER: xlb_cmp                                  */
    uint32_t cmp_lhs_col;                 /* FILTER: left operand column                      */
    uint32_t cmp_rhs_is_const;            /* FILTER: 0 = column, 1 = constant                 */
    uint64_t cmp_rhs;                     /* FILTER: column index or constant                 */
    const struct xlb_node* const* inputs; /* UNION                                            */
    uint32_t n_inputs;                    /* UNION                                            */
    uint32_t join_type;                   /* JOIN: xlb_join_type (0 = inner).  SEMI / ANTI keep the
                                             left columns; their right input must be a Scan     */
} xlb_node;

/* CompiledRule { head, body } (crates/xlog-ir/src/plan.rs:28-36). */
typedef struct xlb_rule {
    const char* head;
    const xlb_node* body;
    xlb_schema head_schema; /* CompiledRule.meta.schema */
} xlb_rule;

/* Scc + its rules (plan.rs:8-16, ExecutionPlan.rules_by_scc). */
typedef struct xlb_scc {
    uint32_t id;
    uint32_t is_recursive;
    const xlb_rule* rules;
    uint32_t n_rules;
} xlb_scc;

/* ExecutionPlan with strata flattened into evaluation order (plan.rs:52-70):
 * sccs[0..n_sccs) are executed in order. */
typedef struct xlb_plan {
    const xlb_scc* sccs;
    uint32_t n_sccs;
} xlb_plan;

/* ExecutionStats subset (crates/xlog-runtime/src/profiler.rs:172-233) + data-plane counters. */
typedef struct xlb_run_stats {
    uint64_t iterations;       /* semi-naive iterations over all recursive SCCs                */
    uint64_t derived_tuples;   /* sum over heads of the final row count (all ranks' shards)    */
    uint64_t candidate_tuples; /* join outputs before dedup (bag), all ranks                   */
    uint64_t kernel_launches;  /* kernels this library launched during the call                */
    uint64_t peak_bytes;       /* allocator high-water mark during the call                    */
    double ms_total;           /* device time of the whole call (CUDA events)                  */
    double ms_join;            /* index build + probe + expand                                 */
    double ms_sort;            /* radix sort of candidates                                     */
    double ms_setops;          /* dedup + difference + union                                   */
    double ms_exchange;        /* partition + all-to-all + termination vote (multi-rank)       */
    uint64_t exchange_bytes;   /* bytes this rank sent to other ranks                          */
    uint64_t host_syncs;       /* times the host waited for the stream (row-count read-backs)  */
    double ms_host_wait;       /* host wall time inside those waits                            */
    double ms_host_total;      /* host wall time of the whole call                             */
    double ms_host_alloc;      /* host wall time inside the device allocator                   */
} xlb_run_stats;

/* ---- executor: Executor::{register_relation, put_relation, store().get, execute_plan} ----- */

/* register_relation(RelId, &str) (crates/xlog-runtime/src/executor/mod.rs:1242). */
xlb_status xlb_register_relation(xlb_ctx* ctx, uint32_t rel_id, const char* name);
/* put_relation(&str, CudaBuffer) (executor/mod.rs:587): the store takes ownership of `rel`.
 * With several ranks each rank puts its own slice of the relation; the relation is the union. */
xlb_status xlb_store_put(xlb_ctx* ctx, const char* name, xlb_rel* rel);
/* store().get(&str) (executor/mod.rs:562): borrowed handle, valid until the next put of that
 * name, the next xlb_execute_plan or the context's destruction.  With several ranks it is this
 * rank's shard (sorted, unique); the relation is the disjoint union of the shards. */
xlb_status xlb_store_get(xlb_ctx* ctx, const char* name, const xlb_rel** rel);
xlb_status xlb_store_remove(xlb_ctx* ctx, const char* name);
/* execute_plan(&ExecutionPlan) (executor/mod.rs:1404-1469); recursive SCCs run the semi-naive
 * loop of execute_recursive_scc (executor/recursive.rs:447-957).  `stats` may be NULL.
 * Relations of one or two columns.  u32 / symbol columns run as they are; when a relation or a
 * declared head has u64, signed or floating columns, the plan runs on 32-bit ranks of one sorted
 * dictionary of all values and the heads are decoded into their declared types (one GPU; at most
 * 2^32 - 1 distinct values; no constant filters over signed or floating columns). */
xlb_status xlb_execute_plan(xlb_ctx* ctx, const xlb_plan* plan, xlb_run_stats* stats);

/* ---- allocation-free entry point ---------------------------------------------------------- */
/* No counterpart in the reference.  For callers that may not allocate device memory when they
 * call in (a host runtime that owns the whole GPU through its own arena and forbids cudaMalloc
 * in plug-ins; a section where an allocation could stall the device; a caller with no allocator
 * to hand down): removes duplicates from `n` ascending keys at `d_sorted` (device memory),
 * writing the distinct keys, ascending, to `d_unique` (room for n keys) and their number to
 * `*d_count` (device memory), on `cuda_stream` (a cudaStream_t; NULL = the default stream).  Same
 * result as the full-row xlb_dedup of a sorted single-column u64 relation.
 *   - needs no context and calls no cudaMalloc/cudaFree or any allocating routine: its scratch
 *     (tile counts, tile offsets, scan partials) is a fixed array of about 385 KiB inside the
 *     library image, held by every GPU that loads the library until the process exits;
 *   - n above xlb_dedup_sorted_u64_static_max() (2^26 keys) is refused with XLB_ERR_CAPACITY;
 *   - `d_unique` must not overlap `d_sorted` (blocks write output while others still read
 *     input): overlapping ranges are refused with XLB_ERR_INVALID before anything is launched;
 *     so is a call made while an earlier CUDA error of the caller is still pending
 *     (XLB_ERR_CUDA; the pending error is left for the caller to read);
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call before starting any stream capture.  Every
 *     call waits for the stream before it returns;
 *   - every call shares the one array: calls that may overlap on the GPU (different streams,
 *     different host threads) race on it and must be serialised by the caller.  The array
 *     keeps the last call's contents; each call overwrites every word it later reads;
 *   - xlb_static_last_error() gives the message of the calling thread's last failing call. */
xlb_status xlb_dedup_sorted_u64_static(const uint64_t* d_sorted, uint64_t n, uint64_t* d_unique,
                                       uint64_t* d_count, void* cuda_stream);
uint64_t xlb_dedup_sorted_u64_static_max(void);
const char* xlb_static_last_error(void);

/* ---- per-kernel timing -------------------------------------------------------------------- */
/* Counterpart of the reference's feature-gated per-phase CUDA-event timing
 * (crates/xlog-runtime/src/profiler.rs:355-640, feature `wcoj-phase-timing`): brackets every
 * launch of the named kernels (names separated by commas; "*" = every kernel, NULL = off) with CUDA events on the launching
 * stream.  xlb_profile_read waits for the stream, then reports per kernel its launches, device
 * time and algorithmic bytes since xlb_profile_enable. */
typedef struct xlb_kernel_profile {
    char name[32];
    uint64_t launches;
    uint64_t bytes;
    double ms;
} xlb_kernel_profile;
xlb_status xlb_profile_enable(xlb_ctx* ctx, const char* kernel);
xlb_status xlb_profile_read(xlb_ctx* ctx, xlb_kernel_profile* out, uint32_t cap, uint32_t* n);

/* ---- several GPUs: one process and one context per GPU ------------------------------------ */
/* No counterpart in the reference (docs/architecture/multi-gpu.mdx:45-54 marks distributed
 * joins as not implemented).  Rank 0 obtains an id, the host program broadcasts its
 * XLB_UNIQUE_ID_BYTES bytes to every rank by its own means, and every rank then joins.  Derived
 * relations are hash-partitioned; joins exchange tuples with an NCCL all-to-all and the fixpoint
 * ends on an all-reduced emptiness vote. */
xlb_status xlb_comm_unique_id(uint8_t id[XLB_UNIQUE_ID_BYTES]);
xlb_status xlb_comm_init(xlb_ctx* ctx, const uint8_t id[XLB_UNIQUE_ID_BYTES], uint32_t rank,
                         uint32_t world);
/* Owner rank of a join-key value: identical on host and device. */
uint32_t xlb_owner_of(uint64_t key, uint32_t world);
/* Test support, no counterpart in the reference: puts the context into the state that an exchange
 * which timed out or failed leaves behind (communicator aborted), without any device work.  Every
 * later call that needs the other ranks then fails at once with XLB_ERR_NCCL.  On a context that
 * never joined a communicator it first records a world of two ranks. */
xlb_status xlb_comm_mark_aborted_for_test(xlb_ctx* ctx);
/* Test support, no counterpart in the reference.  Every wait inside a kernel is bounded: a tile of
 * the one-sweep radix sort polls at most `spin_limit` times (0 = the default, 2^22) for the tiles
 * before it, then reports XLB_ERR_TIMEOUT through the device status word and returns.  With
 * `first_tile` = 1 the tiles take their numbers from 1, so tile 0 never runs and never publishes
 * its counts: every other tile's wait runs out, which is how a test sees the limit work without
 * hanging the device (0 = normal numbering).  The result of such a sort is garbage, the call fails
 * with XLB_ERR_TIMEOUT, and the context stays usable. */
xlb_status xlb_test_set_lookback(xlb_ctx* ctx, uint32_t spin_limit, uint32_t first_tile);

#ifdef __cplusplus
}
#endif
#endif /* XLB_H */
