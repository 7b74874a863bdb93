// Host-level operations on device key arrays: the vocabulary the executor is written in.
// Implemented in xlb_ops.cu on top of the kernels of xlb_kernels.cuh.
#pragma once
#include "xlb_common.cuh"

// A bag or set of rows of at most two 32-bit columns, one u64 per row:
// arity 2 -> (c0 << 32) | c1, arity 1 -> c0 in the low half.
struct Keys {
    Buf buf;
    uint64_t n = 0;
    uint64_t bound = ~0ull;  // host-known upper bound of the OR of all rows (~0: unknown)
    const uint64_t* ptr() const { return buf ? buf->as<uint64_t>() : nullptr; }
};

// Column source selectors for remap / expand: which 32-bit value lands in an output half.
enum Src { SRC_HI = 0, SRC_LO = 1, SRC_OTHER = 2, SRC_ZERO = 3 };

// Join index over a relation sorted by its join key: distinct keys live in an open-addressing
// table whose slots carry (start, length) of the key's run in `S`.
struct Index {
    Buf S;             // sorted u64 words; join key = S[i] >> key_shift
    Buf pay;           // optional 32-bit payload per row; when absent the payload is the low half of S
    uint64_t n = 0;    // rows
    int key_shift = 32;
    Buf table;         // ulonglong2 slots
    uint64_t mask = 0; // capacity - 1
    uint64_t nkeys = 0;
    uint64_t bound = ~0ull;  // OR bound of the rows of S
    // Direct form (ops_index_build_direct): no S and no table; cursor[k] = end of key k's group in
    // `pay` for every key below `domain`.
    Buf cursor;
    uint64_t domain = 0;
    uint64_t pay_bound = 0xFFFFFFFFull;  // OR bound of the payload column
    bool built() const { return S || cursor; }
};

Keys ops_rel_packed(xlb_ctx* c, const xlb_rel* r);             // packed view (cached on the relation)
// The same for a two-column relation that is not packed yet, with the rows whose column fcol equals
// fval collected in the same pass (`filtered`, a bag).  False (nothing done): already packed.
bool ops_rel_packed_filtered(xlb_ctx* c, const xlb_rel* r, int fcol, uint32_t fval, Keys* filtered);
// One pass over the columns of such a relation without packing it: its OR bound becomes known (and
// the filtered rows are collected, fcol >= 0).  False (nothing done): already packed, or not two
// 32-bit columns.
bool ops_rel_bound_filtered(xlb_ctx* c, const xlb_rel* r, int fcol, uint32_t fval, Keys* filtered);
void ops_rel_columns(xlb_ctx* c, const xlb_rel* r);            // materialise column view (cached)
xlb_rel* ops_rel_from_keys(xlb_ctx* c, const xlb_schema& s, Keys k, bool canonical);

Keys ops_copy(xlb_ctx* c, const Keys& in);
Keys ops_from_host(xlb_ctx* c, const uint64_t* rows, uint64_t n);  // small host arrays only (n <= 16)
Keys ops_concat(xlb_ctx* c, const std::vector<Keys>& parts);
Keys ops_slice(xlb_ctx* c, const Keys& in, uint64_t lo, uint64_t hi);  // copy of rows [lo, hi)
// Sorts replace k.buf by a buffer holding the result.  With keep_input the buffer k.buf named on
// entry is not written (it may be a stored relation's); without it, it is used as scratch.
void ops_sort(xlb_ctx* c, Keys& k, bool keep_input = false);                 // ascending
void ops_sort_by_high_half(xlb_ctx* c, Keys& k, bool keep_input = false);    // stable, by bits 32..63 only (groups rows by join key)
void ops_dedup_sorted(xlb_ctx* c, Keys& k);                      // sorted -> sorted unique
Keys ops_diff(xlb_ctx* c, const Keys& a, const Keys& b);         // sorted unique a \ sorted unique b
Keys ops_dedup_diff(xlb_ctx* c, const Keys& a, const Keys& b);   // distinct rows of sorted a that are not in sorted unique b
// The same result through a bitmap over a dense domain; `ops_dense_bits` says whether the rows of
// both arrays fit one (returns false otherwise) and how many low-half bits to keep.
bool ops_dense_bits(const Keys& a, const Keys& b, int* hi_bits, int* lo_bits, int max_bits = 27);
Keys ops_dense_novel(xlb_ctx* c, const Keys& cand, const Keys& full, int hi_bits, int lo_bits, unsigned int* visited = nullptr);
// The same in pieces, so that a join can mark its output tuples straight into the bitmap:
struct DenseSet {
    Buf bitmap;
    uint64_t words = 0;
    int hi_bits = 0, lo_bits = 0;
    uint64_t bound = 0;  // OR bound of what was marked
    // three words behind the bitmap: [0] rows ops_dense_finish emits, [1] sum of the tuple counts of
    // the marking joins, which stay on the device until ops_dense_finish reads both at once,
    // [2] the ticket of the fused count-and-scan kernel
    uint64_t* counts = nullptr;
    uint64_t marked = 0;  // host copy of counts[1], valid after ops_dense_finish
    // Optional bitmap (same domain) of the tuples known already: marking skips them, and
    // ops_dense_finish emits only what it lacks and adds that to it.
    unsigned int* visited = nullptr;
    // Several marking steps share the set (every rule variant of an iteration, on ranks that hold
    // replicated relations): a marking join then adds its tuple count to counts[1] instead of
    // leaving it there.
    bool shared = false;
    // The bitmap started as a copy of `visited` (ops_dense_begin_from): one look-up then tells a
    // marking kernel both "known already" and "marked already", and it skips the look-up in
    // `visited`.  ops_dense_finish takes `bitmap & ~visited` either way.
    bool seeded = false;
    // A set over the persistent marks of a DenseState (ops_dense_begin_state): the count words live
    // in a buffer of their own, and `touched` has one byte per group of 256 bitmap words that a
    // marking kernel sets when it sets a bit there, so that counting and emitting skip the rest.
    Buf counts_buf;
    unsigned char* touched = nullptr;
};
// The tuples of one relation as a bitmap that lives across the iterations of a fixpoint, so that
// no iteration has to subtract the whole relation from its candidates again.
struct DenseState {
    Buf visited;
    // Bitmaps of 2^20 words and more also keep `marks`: the head plus whatever has been marked,
    // never cleared (what an iteration marks is added to `visited` when it is emitted, so the two
    // are equal again between iterations and no bitmap is copied or cleared per iteration), and
    // `touched`, one byte per 256 words, cleared per use.
    Buf marks, touched;
    uint64_t words = 0;
    int hi_bits = 0, lo_bits = 0;
    uint64_t rows = 0;  // tuples marked (the relation's rows plus what the running iteration found)
    bool valid = false;
};
// The tuples of one relation as a hash set that lives across the iterations of a fixpoint (heads
// too wide for a bitmap).
struct TupleSet {
    Buf table;          // slots of mix64(tuple); then one 32-bit flag: the word that equals the empty mark is stored
    uint64_t cap = 0;   // slots, a power of two; at most half of them are ever used
    int log2cap = 0;
    uint64_t rows = 0;  // tuples stored
    bool valid = false;
};
// (Re)build the set from the sorted lists `full` and `novel`, with room for `extra` more tuples.
void ops_tuple_set_build(xlb_ctx* c, TupleSet& s, const Keys& full, const Keys& novel, uint64_t extra);
// Insert the candidates; returns those that were new (a bag: once each, in no particular order).
// The set grows first when it could pass half full.
Keys ops_tuple_set_novel(xlb_ctx* c, TupleSet& s, const Keys& cand);
void ops_dense_state_build(xlb_ctx* c, DenseState& s, int hi_bits, int lo_bits, const Keys& full, const Keys& novel);
Keys ops_dense_state_rows(xlb_ctx* c, const DenseState& s, uint64_t bound);  // all its tuples, in order
// A set whose bitmap starts as a copy of `visited` (same domain) instead of empty.
DenseSet ops_dense_begin_from(xlb_ctx* c, int hi_bits, int lo_bits, unsigned int* visited);
// The candidate set of one use of a head's bitmap state: its persistent marks when it keeps them, else a copy of the head.
DenseSet ops_dense_begin_state(xlb_ctx* c, DenseState& s);
DenseSet ops_dense_begin(xlb_ctx* c, int hi_bits, int lo_bits);
// Emit, in order, the marked tuples that are new: with d.visited those it lacks (which it then
// gains; `full` is not read), else those not in `full` (cleared from the bitmap first).
Keys ops_dense_finish(xlb_ctx* c, DenseSet& d, const Keys& full);
// OR bound of the rows ops_join_expand would produce
uint64_t ops_expand_bound(const Keys& bag, const Index& ix, int hi_src, int lo_src);
// ops_join_expand that marks instead of materialising.  No count comes back to the host here:
// the number of tuples marked is d.marked after ops_dense_finish.
void ops_join_expand_mark(xlb_ctx* c, const Keys& bag, int keysel, const Index& ix, int hi_src, int lo_src, DenseSet& d);
// mark the rows of `cand` in d (skipping what d.visited holds)
void ops_dense_mark_into(xlb_ctx* c, DenseSet& d, const Keys& cand);
// rows whose half `keysel` belongs to `rank` of `world` (owner = mix64(key) mod world), in input order
Keys ops_filter_owner(xlb_ctx* c, const Keys& in, int keysel, uint32_t world, uint32_t rank);
Keys ops_merge_disjoint(xlb_ctx* c, const Keys& a, const Keys& b);
Keys ops_union(xlb_ctx* c, const Keys& a, const Keys& b);        // sorted unique a U b
Keys ops_remap(xlb_ctx* c, const Keys& in, int hi_src, int lo_src);
// rows where half(lhs_src) <cmp> (rhs_is_const ? rhs : half(rhs))
Keys ops_filter(xlb_ctx* c, const Keys& in, uint32_t cmp, int lhs_src, bool rhs_is_const, uint64_t rhs);

Index ops_index_build(xlb_ctx* c, Buf S, uint64_t n, int key_shift, Buf pay);
// Counting build for keys of at most key_bits bits: rows = packed two-column rows in any order,
// key = the half named by keysel (SRC_HI / SRC_LO), payload = the other half.
Index ops_index_build_direct(xlb_ctx* c, const Keys& rows, int keysel, int key_bits);
// Probe `bag` (key = the half named by keysel, or pkeys[i] when given) and expand every match:
// out row = (pick(hi_src) << 32) | pick(lo_src) with SRC_OTHER = the build row's payload.
Keys ops_join_expand(xlb_ctx* c, const Keys& bag, int keysel, const uint64_t* pkeys, const Index& ix, int hi_src, int lo_src);
// Scan join: the join of `bag` (key = its half keysel) with the stored rows `rel` (key = its half
// rel_keysel), run from the relation's side.  Only for outputs that take nothing from the bag but
// the key: rel_hi / rel_lo say what lands in each output half (0 key, 1 the relation's other
// column, 2 zero).  key_bits = bit length of the bag's keys (at most 27).  Every relation row
// with a key in the bag is produced once, however often the bag repeats the key.
uint64_t ops_scan_join_bound(const Keys& bag, int keysel, const Keys& rel, int rel_keysel, int rel_hi, int rel_lo);
Keys ops_scan_join(xlb_ctx* c, const Keys& bag, int keysel, int key_bits, const Keys& rel, int rel_keysel, int rel_hi, int rel_lo);
// the same, marking into d (one marking step per DenseSet; count in d.marked after ops_dense_finish)
void ops_scan_join_mark(xlb_ctx* c, const Keys& bag, int keysel, int key_bits, const Keys& rel, int rel_keysel, int rel_hi, int rel_lo, DenseSet& d);
// The key set of a scan join: a bitmap over 2^key_bits keys with the bits of the bag's keys set
// (whole 16-byte words).
Buf ops_keyset(xlb_ctx* c, const Keys& bag, int keysel, int key_bits);
// Frontier loop on bitmaps over one domain of 2^bits values (a head of one column).
//   scan: every row whose key is in `frontier` marks its head value in `marks`, a bitmap that
//         holds `visited` plus what the iteration has marked so far; *count_marked += the rows
//         with a key in the frontier.  `frontier` is a subset of `visited`, and null when every
//         row whose key `visited` holds has it in the frontier.  With keys_in_frontier (device)
//         the launch does nothing when that count is zero.  With live_out the rows whose key
//         `visited` lacks are appended to it, packed (*live_count += their number): a key enters
//         the frontier once, so no other row can match in a later scan.
//   step: what the marks (OR of `parts` bitmaps back to back) hold beyond `visited` becomes
//         `next_frontier` and joins `visited`; counts[0] += their number; `own` (this rank's
//         marks) is left equal to the new `visited`.  The block that finishes last (`ticket`, a
//         zeroed device word that is left zero) copies counts[0..2] to publish_to[0..2], each with
//         the low 24 bits of `seq` in its top 24 bits: publish_to is pinned host memory as the
//         device sees it, so the host can watch for the three tags instead of enqueuing a copy
//         and an event (counts stay below 2^40).
struct ScanRows {  // what a scan streams over: packed rows, or the join column and the other column of a relation
    const uint64_t* packed = nullptr;
    const uint32_t* kcol = nullptr;
    const uint32_t* ocol = nullptr;
    uint64_t n_max = 0;                         // rows (an upper bound when n_dev is set)
    const unsigned long long* n_dev = nullptr;  // device word with the row count, for a list whose length the host has not read
};
void ops_frontier_scan(xlb_ctx* c, const ScanRows& src, int rel_keysel, int bits, const unsigned int* frontier, int rel_lo, unsigned int* marks, const unsigned int* visited,
                       unsigned long long* count_marked, const unsigned long long* keys_in_frontier, uint64_t* live_out, unsigned long long* live_count);
void ops_frontier_step(xlb_ctx* c, const unsigned int* mark_parts, uint32_t parts, uint64_t words, unsigned int* own, unsigned int* visited, unsigned int* next_frontier,
                       unsigned long long* counts, unsigned int* ticket, unsigned long long* publish_to, unsigned long long seq);
// rows of `bag` whose key has (semi) or lacks (anti) a match in the index, in bag order
// (pkeys, when given, holds the key word of every bag row instead of a half named by keysel)
Keys ops_semi_filter(xlb_ctx* c, const Keys& bag, int keysel, const Index& ix, bool anti, const uint64_t* pkeys = nullptr);
// match[i] != 0 flags for semi / anti joins (device array of bag.n words)
Buf ops_probe_match(xlb_ctx* c, const Keys& bag, int keysel, const uint64_t* pkeys, const Index& ix);

// Dictionary encoding for the executor: relations whose columns are not all 32-bit unsigned
// (u64, signed, floating) run through the fixpoint as relations of dense 32-bit ranks.  The
// dictionary holds the order-preserving unsigned images (widened to 64 bits) of every value of
// every column, sorted and unique, so ranks compare as the values do and results come out in the
// values' order.
Keys ops_dict_build(xlb_ctx* c, const std::vector<const xlb_rel*>& rels);
xlb_rel* ops_dict_encode(xlb_ctx* c, const xlb_rel* r, const Keys& dict);                            // same arity, u32 rank columns
xlb_rel* ops_dict_decode(xlb_ctx* c, const xlb_rel* ranks, const xlb_schema& types, const Keys& dict);  // ranks back to values
// For every constant (as an unsigned value): the number of dictionary entries below it and the
// number not above it (equal: the constant is absent).
void ops_dict_bounds(xlb_ctx* c, const Keys& dict, const std::vector<uint64_t>& consts, std::vector<uint64_t>& below, std::vector<uint64_t>& not_above);

// owner rank of every row by the half `keysel`; stable partition into `world` runs, whose lengths
// are left in device memory at `counts_dev` (no read-back); returns the partitioned copy.
Keys ops_partition_by_owner_dev(xlb_ctx* c, const Keys& in, int keysel, uint32_t world, unsigned long long* counts_dev);

// Per-phase event timing (XLB_FLAG_PROFILE): bracket with phase_begin / phase_end.
struct PhaseTimer {
    xlb_ctx* c;
    double* acc;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    PhaseTimer(xlb_ctx* ctx, double* into);
    ~PhaseTimer();
};

// Relation-level operators on column-major relations of any arity: what the C ABI's operator
// entry points run, and what the general evaluator of rule bodies (xlb_tree.cu) is written in.
// Every function returns a fresh, caller-owned relation; inputs are never modified.
xlb_rel* rel_empty(xlb_ctx* c, const xlb_schema& s);
xlb_rel* rel_view(xlb_ctx* c, const xlb_rel* r);                                  // another handle on the same buffers
xlb_rel* rel_project(xlb_ctx* c, const xlb_rel* in, const uint32_t* cols, uint32_t n);  // columns shared, not copied
// rows where column lhs <cmp> (rhs_is_const ? rhs : column rhs), in input order; unsigned comparison
xlb_rel* rel_filter(xlb_ctx* c, const xlb_rel* in, uint32_t cmp, uint32_t lhs, bool rhs_is_const, uint64_t rhs);
xlb_rel* rel_concat(xlb_ctx* c, const xlb_rel* const* ins, uint32_t n);
xlb_rel* rel_canonical(xlb_ctx* c, const xlb_rel* in);                             // sorted by all columns, unique
xlb_rel* rel_distinct(xlb_ctx* c, const xlb_rel* in, const uint32_t* key_cols, uint32_t nk);  // dedup: full rows or by key columns
xlb_rel* rel_union_many(xlb_ctx* c, const xlb_rel* const* ins, uint32_t n);
xlb_rel* rel_difference(xlb_ctx* c, const xlb_rel* a, const xlb_rel* b);
xlb_rel* rel_join(xlb_ctx* c, const xlb_rel* l, const xlb_rel* r, const uint32_t* lk, const uint32_t* rk, uint32_t nk, xlb_join_type type);
