// Device kernels of the fixpoint data plane (sm_100a) and their launch wrappers.
//
//   radix sort     LSD over u64 keys (optionally with a u32 payload), 8-bit digits, shared-memory
//                  digit counters, warp match/ballot ranking, shared-memory reorder before the
//                  global scatter.  Replaces kernels/sort.cu:28-286 of the reference
//                  (4-bit digits, one thread per row, host-driven per-digit scans).
//   scan           reduce -> spine -> apply exclusive prefix sums; replaces kernels/scan.cu:133-270.
//   select         predicate count -> scan -> compaction; replaces kernels/filter.cu:902-940 and
//                  the mask kernels of kernels/dedup.cu:306-345.
//   merge path     set difference and disjoint union of sorted unique key arrays; replaces the
//                  per-row binary search of kernels/dedup.cu:515-565 and the concat + re-sort of
//                  kernels/set_ops.cu:46-116.
//   hash index     open-addressing table over the distinct join keys of a key-sorted relation;
//                  probe -> compact -> scan -> load-balanced expand.  Replaces kernels/join.cu:131-252
//                  and kernels/pack.cu:144-214.
//
// All arithmetic is integer; nothing here is a contraction, so no tensor-core path exists.
#pragma once
#include "xlb_common.cuh"

namespace xk {

constexpr int BLOCK = 256;
constexpr unsigned FULL = 0xFFFFFFFFu;

__device__ __forceinline__ unsigned lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// Lanes of the warp whose 8-bit value equals this lane's: eight ballots.  (The match.any
// instruction does the same but its cost grows with the number of distinct values in the warp,
// and radix digits are close to all-distinct.)
__device__ __forceinline__ unsigned match_digit(unsigned d) {
#ifdef XLB_RANK_MATCH
    return __match_any_sync(FULL, d);
#else
    unsigned peers = FULL;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
        bool bit = (d >> b) & 1u;
        unsigned vote = __ballot_sync(FULL, bit);
        peers &= bit ? vote : ~vote;
    }
    return peers;
#endif
}

__device__ __forceinline__ void set_status(DevStatus* st, unsigned code, unsigned where, unsigned long long detail) {
    if (atomicCAS(&st->code, 0u, code) == 0u) {
        st->where = where;
        st->detail = detail;
    }
}

// Block-wide exclusive scan of one value per thread (BLOCK threads); returns the exclusive
// prefix and writes the block total to `total`.
template <class T>
__device__ __forceinline__ T block_exclusive_scan(T v, T* total, T* smem /* >= 33 entries */) {
    unsigned lane = lane_id(), warp = threadIdx.x >> 5;
    T incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        T o = __shfl_up_sync(FULL, incl, d);
        if (lane >= (unsigned)d) incl += o;
    }
    if (lane == 31) smem[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int nw = blockDim.x >> 5;
        T w = lane < (unsigned)nw ? smem[lane] : T(0);
        T wi = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            T o = __shfl_up_sync(FULL, wi, d);
            if (lane >= (unsigned)d) wi += o;
        }
        if (lane < (unsigned)nw) smem[lane] = wi - w;
        if (lane == (unsigned)(nw - 1)) smem[32] = wi;
    }
    __syncthreads();
    T res = smem[warp] + incl - v;
    *total = smem[32];
    __syncthreads();
    return res;
}

// ------------------------------------------------------------------------------------ scan
constexpr int SCAN_IPT = 8;
constexpr int SCAN_TILE = BLOCK * SCAN_IPT;

template <class Load, class Tout>
static __global__ void __launch_bounds__(BLOCK) scan_reduce_k(Load load, uint64_t n, Tout* tile_sums) {
    __shared__ Tout sm[33];
    uint64_t base = (uint64_t)blockIdx.x * SCAN_TILE;
    Tout s = 0;
#pragma unroll
    for (int k = 0; k < SCAN_IPT; ++k) {
        uint64_t i = base + (uint64_t)k * BLOCK + threadIdx.x;
        if (i < n) s += (Tout)load(i);
    }
    Tout tot;
    block_exclusive_scan<Tout>(s, &tot, sm);
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = tot;
}

// One block walks the tile sums in chunks of blockDim.x, turning them into exclusive offsets in
// place; the grand total goes to *total.
template <class Tout>
static __global__ void __launch_bounds__(1024) scan_spine_k(Tout* tile_sums, uint64_t ntiles, Tout* total) {
    __shared__ Tout sm[33];
    __shared__ Tout carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (uint64_t base = 0; base < ntiles; base += blockDim.x) {
        uint64_t i = base + threadIdx.x;
        Tout v = i < ntiles ? tile_sums[i] : Tout(0);
        Tout tot;
        Tout ex = block_exclusive_scan<Tout>(v, &tot, sm);
        Tout carry = carry_s;
        if (i < ntiles) tile_sums[i] = carry + ex;
        __syncthreads();
        if (threadIdx.x == 0) carry_s = carry + tot;
        __syncthreads();
    }
    if (threadIdx.x == 0) *total = carry_s;
}

// out[i] = exclusive prefix.  tile_offsets may be null for a single tile; `total` (may be null)
// then receives the sum.  out has n entries; out_end (may be null) receives the grand total too.
template <class Load, class Tout>
static __global__ void __launch_bounds__(BLOCK) scan_apply_k(Load load, uint64_t n, const Tout* tile_offsets, Tout* out, Tout* total) {
    __shared__ Tout sm[33];
    uint64_t base = (uint64_t)blockIdx.x * SCAN_TILE + (uint64_t)threadIdx.x * SCAN_IPT;
    Tout v[SCAN_IPT];
    Tout s = 0;
#pragma unroll
    for (int k = 0; k < SCAN_IPT; ++k) {
        uint64_t i = base + k;
        v[k] = i < n ? (Tout)load(i) : Tout(0);
        s += v[k];
    }
    Tout tot;
    Tout ex = block_exclusive_scan<Tout>(s, &tot, sm);
    Tout run = ex + (tile_offsets ? tile_offsets[blockIdx.x] : Tout(0));
#pragma unroll
    for (int k = 0; k < SCAN_IPT; ++k) {
        uint64_t i = base + k;
        if (i < n) out[i] = run;
        run += v[k];
    }
    if (!tile_offsets && total && threadIdx.x == 0) *total = tot;
}

// scan_apply_k without the spine pass, for up to SCAN_SUMS_MAX tiles: every block adds up the sums
// of the tiles before it by itself (a few KB out of the L2), the last one also writes the total.
constexpr int SCAN_SUMS_MAX = 1024;
template <class Load, class Tout>
static __global__ void __launch_bounds__(BLOCK) scan_apply_sums_k(Load load, uint64_t n, const Tout* __restrict__ tile_sums, Tout* out, Tout* total) {
    __shared__ Tout sm[33];
    Tout part = 0;
    for (unsigned t = threadIdx.x; t < blockIdx.x; t += BLOCK) part += tile_sums[t];
    Tout offset;
    block_exclusive_scan<Tout>(part, &offset, sm);
    uint64_t base = (uint64_t)blockIdx.x * SCAN_TILE + (uint64_t)threadIdx.x * SCAN_IPT;
    Tout v[SCAN_IPT];
    Tout s = 0;
#pragma unroll
    for (int k = 0; k < SCAN_IPT; ++k) {
        uint64_t i = base + k;
        v[k] = i < n ? (Tout)load(i) : Tout(0);
        s += v[k];
    }
    Tout tot;
    Tout run = block_exclusive_scan<Tout>(s, &tot, sm) + offset;
#pragma unroll
    for (int k = 0; k < SCAN_IPT; ++k) {
        uint64_t i = base + k;
        if (i < n) out[i] = run;
        run += v[k];
    }
    if (total && blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) *total = offset + tot;
}

// The same for one block of 1024 threads: up to 8192 entries in one launch instead of three.
constexpr int SCAN_BLOCK_MAX = 1024 * SCAN_IPT;
template <class Load, class Tout>
static __global__ void __launch_bounds__(1024) scan_block_k(Load load, uint64_t n, Tout* out, Tout* total) {
    __shared__ Tout sm[33];
    uint64_t base = (uint64_t)threadIdx.x * SCAN_IPT;
    Tout v[SCAN_IPT];
    Tout s = 0;
#pragma unroll
    for (int k = 0; k < SCAN_IPT; ++k) {
        uint64_t i = base + k;
        v[k] = i < n ? (Tout)load(i) : Tout(0);
        s += v[k];
    }
    Tout tot;
    Tout run = block_exclusive_scan<Tout>(s, &tot, sm);
#pragma unroll
    for (int k = 0; k < SCAN_IPT; ++k) {
        uint64_t i = base + k;
        if (i < n) out[i] = run;
        run += v[k];
    }
    if (total && threadIdx.x == 0) *total = tot;
}

struct LoadU32 {
    const uint32_t* p;
    __device__ __forceinline__ uint32_t operator()(uint64_t i) const { return p[i]; }
};
struct LoadLow32 {  // low half of a u64 word (the match length of a probe result)
    const uint64_t* p;
    __device__ __forceinline__ uint32_t operator()(uint64_t i) const { return (uint32_t)p[i]; }
};

// Exclusive scan; `d_total` (device, one Tout) receives the sum.
template <class Load, class Tout>
void exclusive_scan(xlb_ctx* c, Load load, uint64_t n, Tout* out, Tout* d_total) {
    if (n == 0) {
        CUDA_OK(cudaMemsetAsync(d_total, 0, sizeof(Tout), c->stream));
        return;
    }
    uint64_t ntiles = (n + SCAN_TILE - 1) / SCAN_TILE;
    if (ntiles == 1) {
        prof_begin(c, "scan_apply", 0);
        scan_apply_k<Load, Tout><<<1, BLOCK, 0, c->stream>>>(load, n, nullptr, out, d_total);
        check_launch(c, "scan_apply");
        return;
    }
    if (n <= (uint64_t)SCAN_BLOCK_MAX) {
        prof_begin(c, "scan_block", 0);
        scan_block_k<Load, Tout><<<1, 1024, 0, c->stream>>>(load, n, out, d_total);
        check_launch(c, "scan_block");
        return;
    }
    Buf sums = make_buf(c, ntiles * sizeof(Tout));
    prof_begin(c, "scan_reduce", 0);
    scan_reduce_k<Load, Tout><<<(unsigned)ntiles, BLOCK, 0, c->stream>>>(load, n, sums->as<Tout>());
    check_launch(c, "scan_reduce");
    if (ntiles <= (uint64_t)SCAN_SUMS_MAX) {
        prof_begin(c, "scan_apply", 0);
        scan_apply_sums_k<Load, Tout><<<(unsigned)ntiles, BLOCK, 0, c->stream>>>(load, n, sums->as<Tout>(), out, d_total);
        check_launch(c, "scan_apply");
        return;
    }
    prof_begin(c, "scan_spine", 0);
    scan_spine_k<Tout><<<1, 1024, 0, c->stream>>>(sums->as<Tout>(), ntiles, d_total);
    check_launch(c, "scan_spine");
    prof_begin(c, "scan_apply", 0);
    scan_apply_k<Load, Tout><<<(unsigned)ntiles, BLOCK, 0, c->stream>>>(load, n, sums->as<Tout>(), out, nullptr);
    check_launch(c, "scan_apply");
}

// ---------------------------------------------------------------------------------- select
// Stable compaction: Pred(i) -> keep?, Emit(i, pos) stores row i at output position pos.
template <class Pred>
static __global__ void __launch_bounds__(BLOCK) select_count_k(Pred pred, uint64_t n, uint32_t* tile_counts) {
    __shared__ uint32_t sm[33];
    uint64_t base = (uint64_t)blockIdx.x * SCAN_TILE;
    uint32_t s = 0;
#pragma unroll
    for (int k = 0; k < SCAN_IPT; ++k) {
        uint64_t i = base + (uint64_t)k * BLOCK + threadIdx.x;
        if (i < n && pred(i)) s++;
    }
    uint32_t tot;
    block_exclusive_scan<uint32_t>(s, &tot, sm);
    if (threadIdx.x == 0) tile_counts[blockIdx.x] = tot;
}

// Each warp owns 256 consecutive rows and walks them 32 at a time, so reads are coalesced and
// the predicate runs once per row; ballots give the stable position inside the warp.
template <class Pred, class Emit>
static __global__ void __launch_bounds__(BLOCK) select_write_k(Pred pred, Emit emit, uint64_t n, const uint64_t* tile_offsets, uint64_t* total) {
    __shared__ uint32_t sm[33];
    constexpr int ROUNDS = SCAN_TILE / BLOCK;  // 8 rounds of 32 rows per warp
    const unsigned lane = lane_id(), warp = threadIdx.x >> 5;
    const uint64_t wbase = (uint64_t)blockIdx.x * SCAN_TILE + (uint64_t)warp * (32 * ROUNDS);
    unsigned flags[ROUNDS];
    uint32_t cnt = 0;
    bool f[ROUNDS];
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {  // all predicates first: their loads are in flight together
        uint64_t i = wbase + r * 32 + lane;
        f[r] = i < n && pred(i);
    }
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        flags[r] = __ballot_sync(FULL, f[r]);
        cnt += __popc(flags[r]);
    }
    // every lane of a warp holds the warp's count: scan one value per warp
    uint32_t tot;
    uint32_t ex = block_exclusive_scan<uint32_t>(lane == 0 ? cnt : 0u, &tot, sm);
    ex = __shfl_sync(FULL, ex, 0);
    uint64_t pos = (tile_offsets ? tile_offsets[blockIdx.x] : 0ull) + ex;
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        unsigned b = flags[r];
        if ((b >> lane) & 1u) emit(wbase + r * 32 + lane, pos + __popc(b & lanemask_lt()));
        pos += __popc(b);
    }
    if (!tile_offsets && threadIdx.x == 0) *total = tot;
}

// Returns the number of selected rows (one host read-back).
template <class Pred, class Emit>
uint64_t select(xlb_ctx* c, Pred pred, Emit emit, uint64_t n) {
    if (n == 0) return 0;
    uint64_t ntiles = (n + SCAN_TILE - 1) / SCAN_TILE;
    Buf total = make_buf(c, 8);
    unsigned long long h;
    if (ntiles == 1) {
        prof_begin(c, "select_write", 0);
        select_write_k<Pred, Emit><<<1, BLOCK, 0, c->stream>>>(pred, emit, n, nullptr, total->as<uint64_t>());
        check_launch(c, "select_write");
        read_words(c, total->p, 1, &h);
        return h;
    }
    Buf counts = make_buf(c, ntiles * 4);
    Buf offs = make_buf(c, ntiles * 8);
    prof_begin(c, "select_count", 0);
    select_count_k<Pred><<<(unsigned)ntiles, BLOCK, 0, c->stream>>>(pred, n, counts->as<uint32_t>());
    check_launch(c, "select_count");
    exclusive_scan<LoadU32, uint64_t>(c, LoadU32{counts->as<uint32_t>()}, ntiles, offs->as<uint64_t>(), total->as<uint64_t>());
    prof_begin(c, "select_write", 0);
    select_write_k<Pred, Emit><<<(unsigned)ntiles, BLOCK, 0, c->stream>>>(pred, emit, n, offs->as<uint64_t>(), nullptr);
    check_launch(c, "select_write");
    read_words(c, total->p, 1, &h);
    return h;
}

// The same selection in one pass for callers that do not need the input order kept (a bag of
// tuples): every block reserves its place with one atomic add on the running total, so blocks
// land in the order they finish; rows keep their order inside a block.  Atomics on one address
// are served one after the other, several nanoseconds each, so blocks are as large as they get
// (1024 threads, 8192 rows): a 16 M-row filter with a match in every tile then queues 2 K of
// them instead of 8 K.  (Counting eight tiles, reserving once and reading them again to write
// was slower: 94 us against 59.)
constexpr int SA_BLOCK = 1024, SA_ROUNDS = 8, SA_TILE = SA_BLOCK * SA_ROUNDS;
template <class Pred, class Emit>
static __global__ void __launch_bounds__(SA_BLOCK) select_append_k(Pred pred, Emit emit, uint64_t n, unsigned long long* total) {
    __shared__ uint32_t sm[33];
    __shared__ unsigned long long base_s;
    const unsigned lane = lane_id(), warp = threadIdx.x >> 5;
    const uint64_t wbase = (uint64_t)blockIdx.x * SA_TILE + (uint64_t)warp * (32 * SA_ROUNDS);
    unsigned flags[SA_ROUNDS];
    uint32_t cnt = 0;
    bool f[SA_ROUNDS];
#pragma unroll
    for (int r = 0; r < SA_ROUNDS; ++r) {  // all predicates first: their loads are in flight together
        uint64_t i = wbase + r * 32 + lane;
        f[r] = i < n && pred(i);
    }
#pragma unroll
    for (int r = 0; r < SA_ROUNDS; ++r) {
        flags[r] = __ballot_sync(FULL, f[r]);
        cnt += __popc(flags[r]);
    }
    uint32_t tot;
    uint32_t ex = block_exclusive_scan<uint32_t>(lane == 0 ? cnt : 0u, &tot, sm);
    ex = __shfl_sync(FULL, ex, 0);
    if (threadIdx.x == 0) base_s = tot ? atomicAdd(total, (unsigned long long)tot) : 0ull;
    __syncthreads();
    uint64_t pos = base_s + ex;
#pragma unroll
    for (int r = 0; r < SA_ROUNDS; ++r) {
        unsigned b = flags[r];
        if ((b >> lane) & 1u) emit(wbase + r * 32 + lane, pos + __popc(b & lanemask_lt()));
        pos += __popc(b);
    }
}

// Returns the number of selected rows (one host read-back); output order unspecified.
template <class Pred, class Emit>
uint64_t select_unordered(xlb_ctx* c, Pred pred, Emit emit, uint64_t n, const char* name = "select_append", uint64_t bytes = 0) {
    if (n == 0) return 0;
    uint64_t ntiles = (n + SA_TILE - 1) / SA_TILE;
    Buf total = make_buf(c, 8);
    CUDA_OK(cudaMemsetAsync(total->p, 0, 8, c->stream));
    prof_begin(c, name, bytes);
    select_append_k<Pred, Emit><<<(unsigned)ntiles, SA_BLOCK, 0, c->stream>>>(pred, emit, n, total->as<unsigned long long>());
    check_launch(c, name);
    unsigned long long h;
    read_words(c, total->p, 1, &h);
    return h;
}

// -------------------------------------------------------------------------------- pack/unpack
// pack kernels also reduce the OR of the packed rows into *or_out (may be null)
// (`vec`: all three arrays are 16-byte aligned, so whole groups of four rows move as 16-byte words)
// Without `out` nothing is packed: the sweep only reduces the OR (and filters).
// With `fcol` >= 0 the rows whose column fcol equals fval are also appended, packed, to `fout` in
// no particular order (*fcount += their number): a rule that reads `rel(c, Y)` from a relation that
// is packed for the first time gets its rows without a second pass over the relation.
static __global__ void pack2_k(const uint32_t* __restrict__ c0, const uint32_t* __restrict__ c1, uint64_t* __restrict__ out, uint64_t n, unsigned long long* or_out,
                               bool vec, int fcol = -1, uint32_t fval = 0, uint64_t* __restrict__ fout = nullptr, unsigned long long* fcount = nullptr) {
    uint64_t acc = 0;
    const uint64_t n4 = vec ? n / 4 : 0;
    const uint4* a4 = reinterpret_cast<const uint4*>(c0);
    const uint4* b4 = reinterpret_cast<const uint4*>(c1);
    ulonglong2* o2 = reinterpret_cast<ulonglong2*>(out);
    auto keep = [&](uint32_t a, uint32_t b) {
        if (fcol >= 0 && (fcol == 0 ? a : b) == fval) fout[atomicAdd(fcount, 1ull)] = ((uint64_t)a << 32) | b;  // a few rows out of millions
    };
    for (uint64_t q = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; q < n4; q += (uint64_t)gridDim.x * blockDim.x) {
        uint4 a = a4[q], b = b4[q];
        ulonglong2 lo, hi;
        lo.x = ((uint64_t)a.x << 32) | b.x;
        lo.y = ((uint64_t)a.y << 32) | b.y;
        hi.x = ((uint64_t)a.z << 32) | b.z;
        hi.y = ((uint64_t)a.w << 32) | b.w;
        if (out) {
            o2[2 * q] = lo;
            o2[2 * q + 1] = hi;
        }
        acc |= lo.x | lo.y | hi.x | hi.y;
        if (fcol >= 0) {  // one test for the four rows: a match is rare
            const uint4 f = fcol == 0 ? a : b;
            if (f.x == fval || f.y == fval || f.z == fval || f.w == fval) {
                keep(a.x, b.x);
                keep(a.y, b.y);
                keep(a.z, b.z);
                keep(a.w, b.w);
            }
        }
    }
    for (uint64_t i = n4 * 4 + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t k = ((uint64_t)c0[i] << 32) | c1[i];
        if (out) out[i] = k;
        acc |= k;
        keep(c0[i], c1[i]);
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) acc |= __shfl_xor_sync(FULL, acc, d);
    if (or_out && lane_id() == 0 && acc) atomicOr(or_out, (unsigned long long)acc);
}
// The read-only sweep of a two-column relation that is not packed: OR of the packed rows into
// *or_out, and with fcol >= 0 the rows whose column fcol equals fval appended, packed, to `fout`
// (*fcount += their number; a match is rare).  Sixteen rows per thread and step: eight 16-byte
// loads in flight (the columns are 16-byte aligned; the host checks).
static __global__ void __launch_bounds__(BLOCK) cols_or_filter_k(const uint32_t* __restrict__ c0, const uint32_t* __restrict__ c1, uint64_t n, unsigned long long* or_out, int fcol,
                                                            uint32_t fval, uint64_t* __restrict__ fout, unsigned long long* fcount) {
    uint32_t acc0 = 0, acc1 = 0;
    auto keep = [&](uint32_t a, uint32_t b) {
        if ((fcol == 0 ? a : b) == fval) fout[atomicAdd(fcount, 1ull)] = ((uint64_t)a << 32) | b;
    };
    constexpr int V = 4;  // 16-byte words per column, thread and step
    const uint64_t per_step = (uint64_t)BLOCK * V * 4;
    const uint64_t steps = n / per_step;
    const uint4* a4 = reinterpret_cast<const uint4*>(c0);
    const uint4* b4 = reinterpret_cast<const uint4*>(c1);
    for (uint64_t s = blockIdx.x; s < steps; s += gridDim.x) {
        uint4 a[V], b[V];
#pragma unroll
        for (int q = 0; q < V; ++q) {
            a[q] = a4[s * (BLOCK * V) + q * BLOCK + threadIdx.x];
            b[q] = b4[s * (BLOCK * V) + q * BLOCK + threadIdx.x];
        }
#pragma unroll
        for (int q = 0; q < V; ++q) {
            acc0 |= a[q].x | a[q].y | a[q].z | a[q].w;
            acc1 |= b[q].x | b[q].y | b[q].z | b[q].w;
            if (fcol >= 0) {
                const uint4 f = fcol == 0 ? a[q] : b[q];
                if (f.x == fval || f.y == fval || f.z == fval || f.w == fval) {
                    keep(a[q].x, b[q].x);
                    keep(a[q].y, b[q].y);
                    keep(a[q].z, b[q].z);
                    keep(a[q].w, b[q].w);
                }
            }
        }
    }
    for (uint64_t i = steps * per_step + (uint64_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += (uint64_t)gridDim.x * BLOCK) {
        const uint32_t a = c0[i], b = c1[i];
        acc0 |= a;
        acc1 |= b;
        if (fcol >= 0) keep(a, b);
    }
    uint64_t acc = ((uint64_t)acc0 << 32) | acc1;
#pragma unroll
    for (int d = 16; d; d >>= 1) acc |= __shfl_xor_sync(FULL, acc, d);
    if (lane_id() == 0 && acc) atomicOr(or_out, (unsigned long long)acc);
}
static __global__ void pack1_k(const uint32_t* __restrict__ c0, uint64_t* __restrict__ out, uint64_t n, unsigned long long* or_out) {
    uint64_t acc = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        out[i] = c0[i];
        acc |= c0[i];
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) acc |= __shfl_xor_sync(FULL, acc, d);
    if (or_out && lane_id() == 0 && acc) atomicOr(or_out, (unsigned long long)acc);
}
static __global__ void unpack2_k(const uint64_t* __restrict__ in, uint32_t* __restrict__ c0, uint32_t* __restrict__ c1, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t k = in[i];
        c0[i] = (uint32_t)(k >> 32);
        c1[i] = (uint32_t)k;
    }
}
static __global__ void unpack1_k(const uint64_t* __restrict__ in, uint32_t* __restrict__ c0, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        c0[i] = (uint32_t)in[i];
}
// out[i] = (sel(in[i], hi_src) << 32) | sel(in[i], lo_src); src: 0 = high half, 1 = low half, 2 = zero.
static __global__ void remap_k(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, uint64_t n, int hi_src, int lo_src) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t k = in[i];
        uint32_t h = (uint32_t)(k >> 32), l = (uint32_t)k;
        uint32_t oh = hi_src == 0 ? h : hi_src == 1 ? l : 0u;
        uint32_t ol = lo_src == 0 ? h : lo_src == 1 ? l : 0u;
        out[i] = ((uint64_t)oh << 32) | ol;
    }
}

inline unsigned grid_for(xlb_ctx* c, uint64_t n, int per_block = BLOCK) {
    uint64_t g = (n + per_block - 1) / per_block;
    uint64_t cap = (uint64_t)c->sm_count * 16;  // grid-stride kernels: a multiple of the SM count
    return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
}

// ------------------------------------------------------------------------------ radix sort
#ifndef XLB_SORT_THREADS
#define XLB_SORT_THREADS 256
#endif
#ifndef XLB_SORT_IPT
#define XLB_SORT_IPT 16
#endif
constexpr int SORT_THREADS = XLB_SORT_THREADS;
constexpr int SORT_IPT = XLB_SORT_IPT;
constexpr int SORT_TILE = SORT_THREADS * SORT_IPT;  // keys per tile
constexpr int SORT_WARPS = SORT_THREADS / 32;

// OR and AND of all keys in one read: a digit whose bits never vary needs no pass.
static __global__ void __launch_bounds__(BLOCK) radix_bits_k(const uint64_t* __restrict__ keys, uint64_t n, unsigned long long* __restrict__ or_and /* [2] */) {
    uint64_t o = 0, a = ~0ull;
    for (uint64_t i = (uint64_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += (uint64_t)gridDim.x * BLOCK) {
        uint64_t k = keys[i];
        o |= k;
        a &= k;
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) {
        o |= __shfl_xor_sync(FULL, o, d);
        a &= __shfl_xor_sync(FULL, a, d);
    }
    if (lane_id() == 0) {
        atomicOr(&or_and[0], (unsigned long long)o);
        atomicAnd(&or_and[1], (unsigned long long)a);
    }
}

// Histograms of all eight digits in one read of the keys.  A digit on which a whole warp agrees
// (constant high bytes are the common case) costs one shared-memory add per warp.
// `digits`: bit d set = digit d is wanted (the others are known constant or take no part).
static __global__ void __launch_bounds__(BLOCK) radix_upfront_k(const uint64_t* __restrict__ keys, uint64_t n, unsigned int* __restrict__ ghist /* 8*256 */, unsigned digits) {
    __shared__ unsigned int sh[8 * 256];
    for (int i = threadIdx.x; i < 8 * 256; i += BLOCK) sh[i] = 0;
    __syncthreads();
    const unsigned lane = lane_id();
    const uint64_t stride = (uint64_t)gridDim.x * BLOCK;
    for (uint64_t base = (uint64_t)blockIdx.x * BLOCK + (threadIdx.x & ~31u); base < n; base += stride) {
        uint64_t i = base + lane;
        bool ok = i < n;
        uint64_t k = ok ? keys[i] : 0;
        unsigned live = __ballot_sync(FULL, ok);
        unsigned first_lane = __ffs(live) - 1;
#pragma unroll
        for (int d = 0; d < 8; ++d) {
            if (!((digits >> d) & 1u)) continue;
            unsigned dig = (unsigned)((k >> (8 * d)) & 255);
            unsigned first = __shfl_sync(FULL, dig, first_lane);
            bool uni = __all_sync(FULL, !ok || dig == first);
            if (uni) {
                if (lane == first_lane) atomicAdd(&sh[d * 256 + first], (unsigned)__popc(live));
            } else if (ok) {
                atomicAdd(&sh[d * 256 + dig], 1u);
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 8 * 256; i += BLOCK)
        if (sh[i]) atomicAdd(&ghist[i], sh[i]);
}

// Exclusive scan of each digit histogram (the digit bases of the sweep) and, per digit, whether
// more than one bin is occupied.
static __global__ void __launch_bounds__(BLOCK) radix_bases_k(const unsigned int* __restrict__ ghist, unsigned long long n, unsigned int* __restrict__ bases, unsigned long long* __restrict__ varies) {
    __shared__ unsigned int sm[33];
    for (int d = 0; d < 8; ++d) {
        unsigned v = ghist[d * 256 + threadIdx.x];
        unsigned tot;
        unsigned ex = block_exclusive_scan<unsigned>(v, &tot, sm);
        bases[d * 256 + threadIdx.x] = ex;
        int constant = __syncthreads_or(v == n);
        if (threadIdx.x == 0) varies[d] = constant ? 0ull : 1ull;
    }
}

// Per-tile histogram of one digit: hist[d * ntiles + tile].
static __global__ void __launch_bounds__(BLOCK) radix_tile_hist_k(const uint64_t* __restrict__ keys, uint64_t n, int shift, uint32_t* __restrict__ hist, uint32_t ntiles) {
    __shared__ unsigned int sh[BLOCK / 32][256];
    for (int i = threadIdx.x; i < (BLOCK / 32) * 256; i += BLOCK) (&sh[0][0])[i] = 0;
    __syncthreads();
    uint64_t base = (uint64_t)blockIdx.x * SORT_TILE;
    unsigned warp = threadIdx.x >> 5, lane = lane_id();
#pragma unroll
    for (int k = 0; k < SORT_TILE / BLOCK; ++k) {
        uint64_t i = base + (uint64_t)k * BLOCK + threadIdx.x;
        // keys past the end count as digit 256 (none): match on 9 bits so they group apart
        unsigned d = i < n ? (unsigned)((keys[i] >> shift) & 255) : 256u;
        unsigned peers = __match_any_sync(FULL, d);
        if (d < 256u && lane == (unsigned)(__ffs(peers) - 1)) sh[warp][d] += __popc(peers);
        __syncwarp();
    }
    __syncthreads();
    unsigned s = 0;
#pragma unroll
    for (int w = 0; w < BLOCK / 32; ++w) s += sh[w][threadIdx.x];
    hist[(uint64_t)threadIdx.x * ntiles + blockIdx.x] = s;
}

// Stable scatter of one tile by one digit.  `offs` is the exclusive scan of the per-tile
// histograms in (digit-major, tile-minor) order, i.e. the global position of the first key of
// digit d of this tile.
//
// LOOKBACK = false: `offs` is the exclusive scan of the per-tile histograms in (digit-major,
// tile-minor) order, i.e. the global position of the first key of digit d of this tile.
// LOOKBACK = true ("one sweep"): `offs` holds the 256 global digit bases; tiles take their
// number from an atomic counter, publish their digit counts in `status` and obtain the sum over
// all earlier tiles by a decoupled look-back, so the pass reads and writes every key once.
// A tile only waits for tiles that took an earlier number, which are running already; every
// wait is bounded and reports XLB_ERR_TIMEOUT through `dst` instead of spinning for ever.
constexpr unsigned LB_FLAG_AGG = 1u << 30, LB_FLAG_INC = 2u << 30, LB_MASK = (1u << 30) - 1;

#ifndef XLB_SORT_MINB
#define XLB_SORT_MINB 4
#endif
template <bool HAS_VALUES, bool LOOKBACK>
static __global__ void __launch_bounds__(SORT_THREADS, XLB_SORT_MINB) radix_scatter_k(const uint64_t* __restrict__ keys_in, uint64_t* __restrict__ keys_out,
                                                          const uint32_t* __restrict__ vals_in, uint32_t* __restrict__ vals_out,
                                                          uint64_t n, int shift, const uint32_t* __restrict__ offs, uint32_t ntiles,
                                                          unsigned int* __restrict__ tile_counter, volatile unsigned int* status, DevStatus* dst,
                                                          unsigned spin_limit) {
    extern __shared__ __align__(16) unsigned char sort_smem[];
    uint64_t* skeys = reinterpret_cast<uint64_t*>(sort_smem);
    unsigned int (*whist)[256] = reinterpret_cast<unsigned int (*)[256]>(sort_smem + SORT_TILE * 8);
    unsigned int* tile_start = reinterpret_cast<unsigned int*>(sort_smem + SORT_TILE * 8 + SORT_WARPS * 1024);
    unsigned int* glob_off = tile_start + 256;
    unsigned int* scan_sm = glob_off + 256;

    __shared__ unsigned int tile_s;
    const unsigned lane = lane_id(), warp = threadIdx.x >> 5;
    unsigned tile = blockIdx.x;
    if (LOOKBACK) {
        if (threadIdx.x == 0) tile_s = atomicAdd(tile_counter, 1u);
        __syncthreads();
        tile = tile_s;
        if (tile >= ntiles) return;  // only when the counter did not start at zero (the bounded-wait test)
    }
    const uint64_t tile_base = (uint64_t)tile * SORT_TILE;
    const uint64_t rem = n - tile_base;
    const unsigned valid = rem < (uint64_t)SORT_TILE ? (unsigned)rem : (unsigned)SORT_TILE;

    for (int i = threadIdx.x; i < SORT_WARPS * 256; i += SORT_THREADS) (&whist[0][0])[i] = 0;
    if (!LOOKBACK && threadIdx.x < 256) glob_off[threadIdx.x] = offs[(uint64_t)threadIdx.x * ntiles + tile];

    // warp-striped load: key j of lane l sits at warp*512 + j*32 + l (memory order = (j, l))
    uint64_t key[SORT_IPT];
    unsigned short rank[SORT_IPT];
    const unsigned wbase = warp * (32 * SORT_IPT);
#pragma unroll
    for (int j = 0; j < SORT_IPT; ++j) {
        unsigned t = wbase + j * 32 + lane;
        key[j] = t < valid ? keys_in[tile_base + t] : ~0ull;
    }
    __syncthreads();

    // rank every key among the keys of its warp with the same digit, in memory order
#pragma unroll
    for (int j = 0; j < SORT_IPT; ++j) {
        unsigned t = wbase + j * 32 + lane;
        unsigned d = t < valid ? (unsigned)((key[j] >> shift) & 255) : 255u;
        unsigned peers = match_digit(d);
        unsigned leader = __ffs(peers) - 1;
        unsigned before = 0;
        if (lane == leader) {
            before = whist[warp][d];
            whist[warp][d] = before + __popc(peers);
        }
        before = __shfl_sync(FULL, before, leader);
        rank[j] = (unsigned short)(before + __popc(peers & lanemask_lt()));
        __syncwarp();
    }
    __syncthreads();

    // per digit: exclusive prefix over warps, then exclusive prefix over digits
    {
        const bool dig = threadIdx.x < 256;
        unsigned d = threadIdx.x & 255, run = 0;
        if (dig) {
#pragma unroll
            for (int w = 0; w < SORT_WARPS; ++w) {
                unsigned v = whist[w][d];
                whist[w][d] = run;
                run += v;
            }
        }
        if (LOOKBACK && dig) {
            // keys past the end were counted under digit 255: take them out of the published count
            unsigned cnt = run - (d == 255 ? (unsigned)SORT_TILE - valid : 0u);
            volatile unsigned int* mine = status + (uint64_t)tile * 256 + d;
            unsigned excl = 0;
            if (tile == 0) {
                *mine = cnt | LB_FLAG_INC;
            } else {
                *mine = cnt | LB_FLAG_AGG;
                int64_t t = (int64_t)tile - 1;
                unsigned spins = 0;
                while (t >= 0) {
                    unsigned v = status[(uint64_t)t * 256 + d];
                    unsigned f = v & ~LB_MASK;
                    if (f == 0) {
                        if (++spins > spin_limit) {
                            set_status(dst, XLB_ERR_TIMEOUT, 2, tile);
                            break;
                        }
                        __nanosleep(20);
                        continue;
                    }
                    excl += v & LB_MASK;
                    if (f == LB_FLAG_INC) break;
                    --t;
                }
                *mine = (excl + cnt) | LB_FLAG_INC;
            }
            glob_off[d] = offs[d] + excl;
        }
        unsigned tot;
        unsigned ex = block_exclusive_scan<unsigned>(run, &tot, scan_sm);
        if (dig) tile_start[d] = ex;
    }
    __syncthreads();

    unsigned short pos[SORT_IPT];
#pragma unroll
    for (int j = 0; j < SORT_IPT; ++j) {
        unsigned t = wbase + j * 32 + lane;
        unsigned d = t < valid ? (unsigned)((key[j] >> shift) & 255) : 255u;
        unsigned p = tile_start[d] + whist[warp][d] + rank[j];
        pos[j] = (unsigned short)p;
        skeys[p] = key[j];
    }
    __syncthreads();
    // coalesced runs: consecutive shared-memory slots of one digit go to consecutive addresses
    for (unsigned i = threadIdx.x; i < valid; i += SORT_THREADS) {
        uint64_t k = skeys[i];
        unsigned d = (unsigned)((k >> shift) & 255);
        keys_out[(uint64_t)glob_off[d] + (i - tile_start[d])] = k;
    }
    if (HAS_VALUES) {
        // Payloads take the same route through the (now free) shared key array: slot p gets the
        // payload and the digit of the key that went to slot p.
        __syncthreads();
        uint32_t* sv = reinterpret_cast<uint32_t*>(skeys);                 // 16 KB of payloads
        uint8_t* sd = reinterpret_cast<uint8_t*>(skeys) + SORT_TILE * 4;   // 4 KB of digits
#pragma unroll
        for (int j = 0; j < SORT_IPT; ++j) {
            unsigned t = wbase + j * 32 + lane;
            if (t < valid) {
                sv[pos[j]] = vals_in[tile_base + t];
                sd[pos[j]] = (uint8_t)((key[j] >> shift) & 255);
            }
        }
        __syncthreads();
        for (unsigned i = threadIdx.x; i < valid; i += SORT_THREADS) {
            unsigned d = sd[i];
            vals_out[(uint64_t)glob_off[d] + (i - tile_start[d])] = sv[i];
        }
    }
}

constexpr size_t SORT_SMEM = (size_t)SORT_TILE * 8 + SORT_WARPS * 1024 + 256 * 4 * 2 + 64 * 4;

// The scatter kernel takes more than the 48 KB a launch gets by default: opt in once per context
// (the attribute belongs to the device that is current when it is set).
inline void radix_sort_setup(xlb_ctx* c) {
    bool& done = c->sort_attr_set;
    if (done) return;
    cudaFuncSetAttribute(radix_scatter_k<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SORT_SMEM);
    cudaFuncSetAttribute(radix_scatter_k<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SORT_SMEM);
    cudaFuncSetAttribute(radix_scatter_k<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SORT_SMEM);
    cudaFuncSetAttribute(radix_scatter_k<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SORT_SMEM);
    done = true;
}

struct SortPlan {
    int npasses = 0;
    int shifts[8];
};

// Which 8-bit digits vary over the keys (one read of the keys + one read-back).
inline SortPlan plan_sort(xlb_ctx* c, const uint64_t* keys, uint64_t n) {
    SortPlan p;
    Buf oa = make_buf(c, 16);
    CUDA_OK(cudaMemsetAsync(oa->p, 0, 8, c->stream));
    CUDA_OK(cudaMemsetAsync((char*)oa->p + 8, 0xFF, 8, c->stream));
    prof_begin(c, "radix_bits", n * 8ull);
    radix_bits_k<<<grid_for(c, n, BLOCK * 8), BLOCK, 0, c->stream>>>(keys, n, oa->as<unsigned long long>());
    check_launch(c, "radix_bits");
    unsigned long long h[2];
    read_words(c, oa->p, 2, h);
    uint64_t varying = h[0] & ~h[1];
    for (int d = 0; d < 8; ++d)
        if ((varying >> (8 * d)) & 255) p.shifts[p.npasses++] = 8 * d;
    return p;
}

// Sorts `n` keys ascending (stable).  keys/vals are replaced by buffers holding the result;
// vals may be empty.  n must be below 2^32.
// `digit_mask` bit d set = digit d (bits 8d..8d+7) takes part in the order; a join index only
// needs its rows grouped by the key half, i.e. digits 4..7.
// `known_bound` != ~0: an upper bound of the OR of all keys that the host already holds; digits
// outside it are constant, so the digit plan needs no read-back.
// `keep_input`: the buffer `keys` names on entry is left untouched (it may belong to a stored
// relation); the first pass reads it and later passes ping-pong between two fresh buffers.
inline void radix_sort(xlb_ctx* c, Buf& keys, Buf* vals, uint64_t n, unsigned digit_mask = 0xFFu, uint64_t known_bound = ~0ull, bool keep_input = false) {
    if (n <= 1) return;
    if (n >= (1ull << 32)) xlb_fail(XLB_ERR_CAPACITY, "sort of %llu keys exceeds the 2^32 limit of one sort", (unsigned long long)n);
    radix_sort_setup(c);
    uint32_t ntiles = (uint32_t)((n + SORT_TILE - 1) / SORT_TILE);
    Buf tmpk = make_buf(c, n * 8);
    Buf tmpv = vals ? make_buf(c, n * 4) : Buf();
    if (n < (1ull << 30)) {
        // one sweep: a histogram read, then one read + one write of the keys per varying digit
        Buf gh = make_buf(c, 8 * 256 * 4 * 2 + 64);  // histograms | bases | varies
        unsigned int* ghist = gh->as<unsigned int>();
        unsigned int* bases = ghist + 8 * 256;
        unsigned long long* varies = (unsigned long long*)(bases + 8 * 256);
        CUDA_OK(cudaMemsetAsync(ghist, 0, 8 * 256 * 4, c->stream));
        unsigned want = digit_mask & 0xFFu;
        if (known_bound != ~0ull)
            for (int d = 0; d < 8; ++d)
                if (!((known_bound >> (8 * d)) & 255)) want &= ~(1u << d);
        if (want == 0) return;
        prof_begin(c, "radix_upfront", n * 8ull);
        radix_upfront_k<<<grid_for(c, n, BLOCK * 8), BLOCK, 0, c->stream>>>(keys->as<uint64_t>(), n, ghist, want);
        check_launch(c, "radix_upfront");
        prof_begin(c, "radix_bases", 0);
        radix_bases_k<<<1, BLOCK, 0, c->stream>>>(ghist, n, bases, varies);
        check_launch(c, "radix_bases");
        unsigned long long v[8];
        if (known_bound != ~0ull) {
            for (int d = 0; d < 8; ++d) v[d] = (known_bound >> (8 * d)) & 255 ? 1 : 0;
        } else {
            read_words(c, varies, 8, v);
        }
        int np = 0, digits[8];
        for (int d = 0; d < 8; ++d)
            if (v[d] && ((digit_mask >> d) & 1u)) digits[np++] = d;
        if (np == 0) return;
        uint64_t status_words = (uint64_t)ntiles * 256;
        Buf status = make_buf(c, (status_words * np + 8) * 4);  // per pass: tile status; then 8 tile counters
        CUDA_OK(cudaMemsetAsync(status->p, 0, (status_words * np + 8) * 4, c->stream));
        unsigned int* counters = status->as<unsigned int>() + status_words * np;
        if (c->lb_first_tile) {  // test knob: tiles take their numbers from here on, so tile 0 never publishes
            for (int q = 0; q < 8; ++q) ((unsigned int*)&c->h_scalar[56])[q] = c->lb_first_tile;
            CUDA_OK(cudaMemcpyAsync(counters, &c->h_scalar[56], 8 * 4, cudaMemcpyHostToDevice, c->stream));
        }
        for (int q = 0; q < np; ++q) {
            int d = digits[q];
            unsigned int* st = status->as<unsigned int>() + status_words * q;
            prof_begin(c, "radix_scatter", n * (vals ? 24ull : 16ull));
            if (vals)
                radix_scatter_k<true, true><<<ntiles, SORT_THREADS, SORT_SMEM, c->stream>>>(keys->as<uint64_t>(), tmpk->as<uint64_t>(), (*vals)->as<uint32_t>(), tmpv->as<uint32_t>(), n, 8 * d, bases + d * 256, ntiles, counters + q, st, c->d_status, c->lb_spin_limit);
            else
                radix_scatter_k<false, true><<<ntiles, SORT_THREADS, SORT_SMEM, c->stream>>>(keys->as<uint64_t>(), tmpk->as<uint64_t>(), nullptr, nullptr, n, 8 * d, bases + d * 256, ntiles, counters + q, st, c->d_status, c->lb_spin_limit);
            check_launch(c, "radix_scatter");
            if (keep_input && q == 0) {
                keys = tmpk;
                tmpk = np > 1 ? make_buf(c, n * 8) : Buf();
            } else std::swap(keys, tmpk);
            if (vals) std::swap(*vals, tmpv);
        }
        return;
    }
    // 2^30 keys and more: per-tile histograms, a scan, then the scatter (counts exceed the
    // 30 bits of a look-back status word)
    SortPlan p0 = plan_sort(c, keys->as<uint64_t>(), n), p;
    for (int q = 0; q < p0.npasses; ++q)
        if ((digit_mask >> (p0.shifts[q] / 8)) & 1u) p.shifts[p.npasses++] = p0.shifts[q];
    if (p.npasses == 0) return;
    Buf hist = make_buf(c, (uint64_t)256 * ntiles * 4);
    Buf offs = make_buf(c, (uint64_t)256 * ntiles * 4);
    Buf total = make_buf(c, 4);
    for (int q = 0; q < p.npasses; ++q) {
        int shift = p.shifts[q];
        prof_begin(c, "radix_tile_hist", n * 8ull);
        radix_tile_hist_k<<<ntiles, BLOCK, 0, c->stream>>>(keys->as<uint64_t>(), n, shift, hist->as<uint32_t>(), ntiles);
        check_launch(c, "radix_tile_hist");
        exclusive_scan<LoadU32, uint32_t>(c, LoadU32{hist->as<uint32_t>()}, (uint64_t)256 * ntiles, offs->as<uint32_t>(), total->as<uint32_t>());
        prof_begin(c, "radix_scatter", n * (vals ? 24ull : 16ull));
        if (vals)
            radix_scatter_k<true, false><<<ntiles, SORT_THREADS, SORT_SMEM, c->stream>>>(keys->as<uint64_t>(), tmpk->as<uint64_t>(), (*vals)->as<uint32_t>(), tmpv->as<uint32_t>(), n, shift, offs->as<uint32_t>(), ntiles, nullptr, nullptr, c->d_status, 0u);
        else
            radix_scatter_k<false, false><<<ntiles, SORT_THREADS, SORT_SMEM, c->stream>>>(keys->as<uint64_t>(), tmpk->as<uint64_t>(), nullptr, nullptr, n, shift, offs->as<uint32_t>(), ntiles, nullptr, nullptr, c->d_status, 0u);
        check_launch(c, "radix_scatter");
        if (keep_input && q == 0) {
            keys = tmpk;
            tmpk = p.npasses > 1 ? make_buf(c, n * 8) : Buf();
        } else std::swap(keys, tmpk);
        if (vals) std::swap(*vals, tmpv);
    }
}

// ------------------------------------------------------------------------------ warp searches
// A tile kernel finds its own slice of the input with a 32-way search run by one warp: a few
// dependent rounds of loads instead of one per halving step, and no separate partition launch.
// Number of leading indices in [0, n) for which pred holds (pred is true on a prefix).
template <class Pred>
__device__ __forceinline__ uint64_t warp_partition_point(uint64_t n, Pred pred) {
    const unsigned lane = lane_id();
    uint64_t lo = 0, hi = n;
    while (hi - lo > 32) {
        uint64_t step = (hi - lo + 31) / 32;
        uint64_t idx = lo + (uint64_t)(lane + 1) * step - 1;  // last index of this lane's chunk
        bool whole = idx < hi && pred(idx);
        unsigned k = __popc(__ballot_sync(FULL, whole));
        lo = lo + (uint64_t)k * step;
        if (lo > hi) lo = hi;
        hi = lo + step < hi ? lo + step : hi;
    }
    bool t = lo + lane < hi && pred(lo + lane);
    return lo + __popc(__ballot_sync(FULL, t));
}

// ------------------------------------------------------------------------------ merge path
constexpr int MP_IPT = 8;
constexpr int MP_TILE = BLOCK * MP_IPT;  // 2048 merged elements per tile

// Number of A elements among the first `diag` merged elements (A first on ties).
__device__ __forceinline__ uint64_t merge_path(const uint64_t* A, uint64_t na, const uint64_t* B, uint64_t nb, uint64_t diag) {
    uint64_t lo = diag > nb ? diag - nb : 0, hi = diag < na ? diag : na;
    while (lo < hi) {
        uint64_t mid = (lo + hi) >> 1;
        if (A[mid] <= B[diag - 1 - mid]) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

// MODE 0: keep[i] = 1 iff A[i] is not in B (A, B sorted unique).
// MODE 1: out = merge of A and B (disjoint), out has na + nb entries.
template <int MODE>
static __global__ void __launch_bounds__(BLOCK) mp_tile_k(const uint64_t* __restrict__ A, uint64_t na, const uint64_t* __restrict__ B, uint64_t nb,
                                                    uint8_t* __restrict__ keep, uint64_t* __restrict__ out) {
    __shared__ uint64_t sA[MP_TILE + 1];
    __shared__ uint64_t sB[MP_TILE + 2];
    __shared__ uint64_t split_s[2];
    uint64_t t = blockIdx.x;
    uint64_t d0 = t * MP_TILE, d1 = d0 + MP_TILE;
    if (d1 > na + nb) d1 = na + nb;
    if (threadIdx.x < 64) {  // warp 0 finds the split of diagonal d0, warp 1 that of d1 (A first on ties)
        uint64_t diag = threadIdx.x < 32 ? d0 : d1;
        uint64_t lo = diag > nb ? diag - nb : 0, hi = diag < na ? diag : na;
        uint64_t k = warp_partition_point(hi - lo, [&](uint64_t i) { return A[lo + i] <= B[diag - 1 - (lo + i)]; });
        if (lane_id() == 0) split_s[threadIdx.x >> 5] = lo + k;
    }
    __syncthreads();
    uint64_t a0 = split_s[0], a1 = split_s[1];
    uint64_t b0 = d0 - a0, b1 = d1 - a1;
    unsigned la = (unsigned)(a1 - a0), lb = (unsigned)(b1 - b0);
    unsigned lbx = lb + ((b1 < nb) ? 1u : 0u);  // one look-ahead element of B for a match across the tile edge
    for (unsigned i = threadIdx.x; i < la; i += BLOCK) sA[i] = A[a0 + i];
    for (unsigned i = threadIdx.x; i < lbx; i += BLOCK) sB[i] = B[b0 + i];
    __syncthreads();
    unsigned diag = threadIdx.x * MP_IPT;
    unsigned total = la + lb;
    if (diag > total) diag = total;
    // local merge path (A first on ties)
    unsigned lo = diag > lb ? diag - lb : 0, hi = diag < la ? diag : la;
    while (lo < hi) {
        unsigned mid = (lo + hi) >> 1;
        if (sA[mid] <= sB[diag - 1 - mid]) lo = mid + 1;
        else hi = mid;
    }
    unsigned ai = lo, bi = diag - lo;
    uint64_t res[MP_IPT];
#pragma unroll
    for (int k = 0; k < MP_IPT; ++k) {
        unsigned o = diag + k;
        res[k] = 0;
        if (o >= total) continue;
        bool takeA = ai < la && (bi >= lb || sA[ai] <= sB[bi]);
        if (takeA) {
            uint64_t a = sA[ai];
            if (MODE == 0) keep[a0 + ai] = (bi < lbx && sB[bi] == a) ? 0 : 1;
            res[k] = a;
            ai++;
        } else {
            res[k] = sB[bi];
            bi++;
        }
    }
    if (MODE == 1) {
        // stage the merged run through shared memory (the inputs are consumed) for coalesced stores
        __syncthreads();
#pragma unroll
        for (int k = 0; k < MP_IPT; ++k)
            if (diag + k < total) sA[diag + k] = res[k];
        __syncthreads();
        for (unsigned i = threadIdx.x; i < total; i += BLOCK) out[d0 + i] = sA[i];
    }
}

struct PredKeep {
    const uint8_t* keep;
    __device__ __forceinline__ bool operator()(uint64_t i) const { return keep[i] != 0; }
};
struct PredKeepHead {  // first of a run of equal keys, and not found in the other set
    const uint8_t* keep;
    const uint64_t* k;
    __device__ __forceinline__ bool operator()(uint64_t i) const { return keep[i] != 0 && (i == 0 || k[i] != k[i - 1]); }
};
struct EmitKey {
    const uint64_t* in;
    uint64_t* out;
    __device__ __forceinline__ void operator()(uint64_t i, uint64_t pos) const { out[pos] = in[i]; }
};
struct PredHead {  // first element of every run of equal keys
    const uint64_t* k;
    __device__ __forceinline__ bool operator()(uint64_t i) const { return i == 0 || k[i] != k[i - 1]; }
};

// Sorted keys -> sorted unique keys.  Returns the unique count; `out` has room for n keys.
inline uint64_t dedup_sorted(xlb_ctx* c, const uint64_t* in, uint64_t n, uint64_t* out) {
    return select(c, PredHead{in}, EmitKey{in, out}, n);
}

// A \ B for a sorted array A (duplicates allowed when `a_has_dups`: they are dropped in the same
// pass) and a sorted unique array B.  Returns the result and its length.
inline Buf set_difference(xlb_ctx* c, const uint64_t* A, uint64_t na, const uint64_t* B, uint64_t nb, uint64_t* n_out, bool a_has_dups = false) {
    if (na == 0) { *n_out = 0; return make_buf(c, 0); }
    if (nb == 0) {
        Buf o = make_buf(c, na * 8);
        if (a_has_dups) *n_out = dedup_sorted(c, A, na, o->as<uint64_t>());
        else {
            CUDA_OK(cudaMemcpyAsync(o->p, A, na * 8, cudaMemcpyDeviceToDevice, c->stream));
            *n_out = na;
        }
        return o;
    }
    uint64_t ntiles = (na + nb + MP_TILE - 1) / MP_TILE;
    Buf keep = make_buf(c, na);
    prof_begin(c, "mp_diff", (na + nb) * 8ull + na);
    mp_tile_k<0><<<(unsigned)ntiles, BLOCK, 0, c->stream>>>(A, na, B, nb, keep->as<uint8_t>(), nullptr);
    check_launch(c, "mp_diff");
    Buf tmp = make_buf(c, na * 8);
    uint64_t m = a_has_dups ? select(c, PredKeepHead{keep->as<uint8_t>(), A}, EmitKey{A, tmp->as<uint64_t>()}, na)
                            : select(c, PredKeep{keep->as<uint8_t>()}, EmitKey{A, tmp->as<uint64_t>()}, na);
    *n_out = m;
    return tmp;
}

// Merge of two sorted arrays with no common element.
inline Buf merge_disjoint(xlb_ctx* c, const uint64_t* A, uint64_t na, const uint64_t* B, uint64_t nb) {
    Buf o = make_buf(c, (na + nb) * 8);
    if (na == 0 || nb == 0) {
        if (na + nb) CUDA_OK(cudaMemcpyAsync(o->p, na ? A : B, (na + nb) * 8, cudaMemcpyDeviceToDevice, c->stream));
        return o;
    }
    uint64_t ntiles = (na + nb + MP_TILE - 1) / MP_TILE;
    prof_begin(c, "mp_union", (na + nb) * 16ull);
    mp_tile_k<1><<<(unsigned)ntiles, BLOCK, 0, c->stream>>>(A, na, B, nb, nullptr, o->as<uint64_t>());
    check_launch(c, "mp_union");
    return o;
}

// ------------------------------------------------------------------------------ dense sets
// When the tuples of a relation fit a small dense domain (hi_bits + lo_bits <= 27 after dropping
// the bits that are zero in every tuple), "sort, dedup, subtract the full relation" is done on a
// bitmap instead: mark the candidates, clear the tuples of the full relation, then emit the
// surviving bits in ascending order, which is the relation's lexicographic order.  The reference's
// default route for small domains works the same way (fj_delta_mark / subtract / popcount / emit,
// kernels/wcoj.cu:3811-3935), on a domain x domain bitmap.
__device__ __forceinline__ uint32_t dense_index(uint64_t k, int lo_bits) {
    return (uint32_t)(((k >> 32) << lo_bits) | (k & 0xFFFFFFFFull));
}
// A marking kernel that sets a bit in a bitmap with a `touched` summary also sets the byte of the
// bit's group of 256 words (8192 bits): counting and emitting then skip the groups nobody touched.
constexpr int DENSE_TOUCH_SHIFT = 13;
template <bool SET>
static __global__ void __launch_bounds__(BLOCK) dense_mark_k(const uint64_t* __restrict__ keys, uint64_t n, int lo_bits, unsigned int* __restrict__ bitmap,
                                                           uint64_t words, DevStatus* st, const unsigned int* __restrict__ visited = nullptr,
                                                           unsigned char* __restrict__ touched = nullptr) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t k = keys[i];
        uint32_t x = dense_index(k, lo_bits);
        // a tuple outside the domain the host derived would mean a wrong bound: report, never write
        if ((k & 0xFFFFFFFFull) >> lo_bits || (uint64_t)(x >> 5) >= words) {
            set_status(st, XLB_ERR_CAPACITY, 3, k);
            continue;
        }
        unsigned bit = 1u << (x & 31);
        if (SET && visited && (__ldg(&visited[x >> 5]) & bit)) continue;  // known already (read-only here: cacheable)
        unsigned cur = bitmap[x >> 5];  // most candidates repeat a tuple already seen: skip the atomic then
        if (SET) {
            if (!(cur & bit)) {
                atomicOr(&bitmap[x >> 5], bit);
                if (touched) touched[x >> DENSE_TOUCH_SHIFT] = 1;
            }
        } else if (cur & bit) atomicAnd(&bitmap[x >> 5], ~bit);
    }
}
// The bitmap is counted and emitted in groups of 32 words (1024 tuples): one warp per group, so the
// prefix sum that places the output runs over domain / 1024 entries only.
// (with `visited`, bits set there do not count and are not emitted; the emit pass adds what it emits)
static __global__ void __launch_bounds__(BLOCK) dense_count_k(const unsigned int* __restrict__ bitmap, uint64_t words, uint32_t* __restrict__ group_counts, uint64_t groups,
                                                            const unsigned int* __restrict__ visited) {
    uint64_t g = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (g >= groups) return;
    uint64_t w = g * 32 + lane_id();
    unsigned cnt = w < words ? __popc(bitmap[w] & ~(visited ? visited[w] : 0u)) : 0;
#pragma unroll
    for (int d = 16; d; d >>= 1) cnt += __shfl_xor_sync(FULL, cnt, d);
    if (lane_id() == 0) group_counts[g] = cnt;
}
// dense_count_k and the prefix sum over its group counts in one launch, for up to
// DENSE_FUSED_GROUPS groups: the block that finishes last (an atomic ticket after a fence, the
// pattern of a single-pass reduction) scans the counts.  `ticket` must be zero on entry and is
// zero again on exit.
constexpr int DENSE_FUSED_GROUPS = 8192;
static __global__ void __launch_bounds__(BLOCK) dense_count_scan_k(const unsigned int* __restrict__ bitmap, uint64_t words, uint32_t* group_counts, uint64_t groups,
                                                              const unsigned int* __restrict__ visited, uint64_t* __restrict__ group_offs, uint64_t* total,
                                                              unsigned int* ticket) {
    __shared__ uint64_t sm[33];
    __shared__ bool last_s;
    uint64_t g = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (g < groups) {
        uint64_t w = g * 32 + lane_id();
        unsigned cnt = w < words ? __popc(bitmap[w] & ~(visited ? visited[w] : 0u)) : 0;
#pragma unroll
        for (int d = 16; d; d >>= 1) cnt += __shfl_xor_sync(FULL, cnt, d);
        if (lane_id() == 0) group_counts[g] = cnt;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last_s = atomicAdd(ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    const uint64_t per = (groups + BLOCK - 1) / BLOCK;  // at most 32
    const uint64_t lo = (uint64_t)threadIdx.x * per, hi = lo + per < groups ? lo + per : groups;
    uint64_t s = 0;
    for (uint64_t i = lo; i < hi; ++i) s += __ldcg(&group_counts[i]);
    uint64_t tot;
    uint64_t run = block_exclusive_scan<uint64_t>(s, &tot, sm);
    for (uint64_t i = lo; i < hi; ++i) {
        group_offs[i] = run;
        run += __ldcg(&group_counts[i]);
    }
    if (threadIdx.x == 0) {
        *total = tot;
        *ticket = 0;
    }
}
static __global__ void __launch_bounds__(BLOCK) dense_emit_k(const unsigned int* __restrict__ bitmap, uint64_t words, const uint64_t* __restrict__ group_offs,
                                                           uint64_t groups, int lo_bits, uint64_t* __restrict__ out, unsigned int* __restrict__ visited,
                                                           uint64_t cap, DevStatus* st) {
    uint64_t g = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (g >= groups) return;
    const unsigned lane = lane_id();
    const uint64_t lo_mask = (1ull << lo_bits) - 1;
    uint64_t w = g * 32 + lane;
    unsigned m = w < words ? bitmap[w] : 0;
    if (visited && w < words) {
        unsigned v = visited[w];
        m &= ~v;
        if (m) visited[w] = v | m;  // one thread per word
    }
    unsigned cnt = __popc(m), incl = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        unsigned o = __shfl_up_sync(FULL, incl, d);
        if (lane >= (unsigned)d) incl += o;
    }
    uint64_t pos = group_offs[g] + (incl - cnt);
    while (m) {
        unsigned b = __ffs(m) - 1;
        m &= m - 1;
        uint64_t x = (w << 5) | b;
        if (pos >= cap) {  // more bits than the rows the host sized the output for: report, never write past it
            set_status(st, XLB_ERR_CAPACITY, 8, pos);
            break;
        }
        out[pos++] = ((x >> lo_bits) << 32) | (x & lo_mask);
    }
}

// The same two passes for bitmaps of a million words and more (domains of 2^25 bits and up): a
// lane takes DW_WPL consecutive words with 16-byte loads, a warp 32 * DW_WPL words (one group), so
// there are eight times fewer groups to scan and every thread has 64 bytes of loads in flight.
// `words` is a multiple of 32 * DW_WPL (the host checks).  Most words of such a bitmap are empty:
// a lane whose words hold nothing new touches nothing else.
constexpr int DW_WPL = 8;
static __global__ void __launch_bounds__(BLOCK) dense_count_wide_k(const unsigned int* __restrict__ bitmap, uint32_t* __restrict__ group_counts, uint64_t groups,
                                                              const unsigned int* __restrict__ visited, const unsigned char* __restrict__ touched) {
    const uint64_t g = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (g >= groups) return;
    if (touched && !touched[g]) {  // nothing was marked in this group
        if (lane_id() == 0) group_counts[g] = 0;
        return;
    }
    const uint64_t w0 = (g * 32 + lane_id()) * DW_WPL;
    const uint4* b4 = reinterpret_cast<const uint4*>(bitmap + w0);
    uint4 a = b4[0], b = b4[1];
    if (visited && (a.x | a.y | a.z | a.w | b.x | b.y | b.z | b.w)) {
        const uint4* v4 = reinterpret_cast<const uint4*>(visited + w0);
        const uint4 va = v4[0], vb = v4[1];
        a.x &= ~va.x, a.y &= ~va.y, a.z &= ~va.z, a.w &= ~va.w;
        b.x &= ~vb.x, b.y &= ~vb.y, b.z &= ~vb.z, b.w &= ~vb.w;
    }
    unsigned cnt = __popc(a.x) + __popc(a.y) + __popc(a.z) + __popc(a.w) + __popc(b.x) + __popc(b.y) + __popc(b.z) + __popc(b.w);
#pragma unroll
    for (int d = 16; d; d >>= 1) cnt += __shfl_xor_sync(FULL, cnt, d);
    if (lane_id() == 0) group_counts[g] = cnt;
}
static __global__ void __launch_bounds__(BLOCK) dense_emit_wide_k(const unsigned int* __restrict__ bitmap, const uint64_t* __restrict__ group_offs, uint64_t groups, int lo_bits,
                                                             uint64_t* __restrict__ out, unsigned int* __restrict__ visited, uint64_t cap, DevStatus* st,
                                                             const unsigned char* __restrict__ touched) {
    const uint64_t g = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (g >= groups) return;
    if (touched && !touched[g]) return;
    const unsigned lane = lane_id();
    const uint64_t lo_mask = (1ull << lo_bits) - 1;
    const uint64_t w0 = (g * 32 + lane) * DW_WPL;
    const uint4* b4 = reinterpret_cast<const uint4*>(bitmap + w0);
    const uint4 a = b4[0], b = b4[1];
    unsigned m[DW_WPL] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    unsigned any = a.x | a.y | a.z | a.w | b.x | b.y | b.z | b.w;
    if (visited && any) {
        uint4* v4 = reinterpret_cast<uint4*>(visited + w0);
        uint4 va = v4[0], vb = v4[1];
        const unsigned v[DW_WPL] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
        any = 0;
#pragma unroll
        for (int i = 0; i < DW_WPL; ++i) {
            m[i] &= ~v[i];
            any |= m[i];
        }
        if (any) {  // one thread per word: what comes out joins the head
            va.x |= m[0], va.y |= m[1], va.z |= m[2], va.w |= m[3];
            vb.x |= m[4], vb.y |= m[5], vb.z |= m[6], vb.w |= m[7];
            v4[0] = va;
            v4[1] = vb;
        }
    }
    unsigned cnt = 0;
#pragma unroll
    for (int i = 0; i < DW_WPL; ++i) cnt += __popc(m[i]);
    unsigned incl = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        unsigned o = __shfl_up_sync(FULL, incl, d);
        if (lane >= (unsigned)d) incl += o;
    }
    const unsigned group_total = __shfl_sync(FULL, incl, 31);
    if (!group_total) return;
    if (__reduce_max_sync(FULL, cnt) >= 32) {
        // A dense group: the warp walks its 256 words in order and lane b writes bit b of the word
        // at hand, so the tuples of a word go out side by side (one lane writing its own 256 bits
        // one after the other would scatter 8-byte stores over 32 places per step).
        uint64_t base = group_offs[g];
        if (base + group_total > cap) {
            if (lane == 0) set_status(st, XLB_ERR_CAPACITY, 8, base + group_total);
            return;
        }
        const unsigned below = (1u << lane) - 1;
        for (int owner = 0; owner < 32; ++owner) {
#pragma unroll
            for (int i = 0; i < DW_WPL; ++i) {
                const unsigned word = __shfl_sync(FULL, m[i], owner);
                if (!word) continue;
                if ((word >> lane) & 1u) {
                    const uint64_t x = ((((g * 32 + owner) * DW_WPL) + i) << 5) | lane;
                    out[base + __popc(word & below)] = ((x >> lo_bits) << 32) | (x & lo_mask);
                }
                base += __popc(word);
            }
        }
        return;
    }
    if (!cnt) return;
    uint64_t pos = group_offs[g] + (incl - cnt);
#pragma unroll
    for (int i = 0; i < DW_WPL; ++i) {
        unsigned mm = m[i];
        while (mm) {
            const unsigned bit = __ffs(mm) - 1;
            mm &= mm - 1;
            const uint64_t x = ((w0 + i) << 5) | bit;
            if (pos >= cap) {  // more bits than the rows the host sized the output for: report, never write past it
                set_status(st, XLB_ERR_CAPACITY, 8, pos);
                return;
            }
            out[pos++] = ((x >> lo_bits) << 32) | (x & lo_mask);
        }
    }
}

// One step of a frontier loop on bitmaps over one domain: what the marks (the OR of `parts` bitmaps
// laid out back to back, each the head plus one rank's candidates) hold beyond the head becomes the
// next frontier and joins the head; their number is added to *count_new.  `own` (this rank's marks)
// is left equal to the new head, which is what the next scan starts from.
// (`own` may be `mark_parts` itself: neither is declared restrict)
static __global__ void __launch_bounds__(BLOCK) frontier_step_k(const unsigned int* mark_parts, uint32_t parts, uint64_t words, unsigned int* own,
                                                           unsigned int* __restrict__ visited, unsigned int* __restrict__ next_frontier,
                                                           unsigned long long* counts, unsigned int* ticket, unsigned long long* publish_to, unsigned long long seq) {
    unsigned mine = 0;
    for (uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (uint64_t)gridDim.x * blockDim.x) {
        unsigned all = 0;
        for (uint32_t p = 0; p < parts; ++p) all |= mark_parts[(uint64_t)p * words + w];
        const unsigned vis = visited[w];
        const unsigned fresh = all & ~vis;
        if (fresh) {
            visited[w] = vis | fresh;
            own[w] = vis | fresh;
        }
        next_frontier[w] = fresh;
        mine += __popc(fresh);
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) mine += __shfl_down_sync(FULL, mine, d);
    if (lane_id() == 0 && mine) atomicAdd(counts, (unsigned long long)mine);
    if (!publish_to) return;
    // The block that finishes last leaves the iteration's counts where the host is watching.  Each
    // of the three words carries the launch's number in its top 24 bits, so the host knows a word
    // is of this launch whichever order the three writes arrive in: no fence towards the host (a
    // round trip over the bus) is needed between them.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
            __threadfence();
            volatile unsigned long long* in = counts;
            volatile unsigned long long* out = publish_to;
            const unsigned long long tag = (seq & PUBLISH_TAG_MASK) << PUBLISH_COUNT_BITS;
            const unsigned long long a = in[0], b = in[1], k = in[2];
            out[0] = tag | a;
            out[1] = tag | b;
            out[2] = tag | k;
            *ticket = 0;
        }
    }
}

// ------------------------------------------------------------------------------ hash index
// 64-bit finaliser (the mixer family the reference hashes join keys with, kernels/join.cu:18-25).
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t x) {
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdull;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ull;
    x ^= x >> 33;
    return x;
}

// Slot: x = key, y = (start << 32) | len of the key's run in the key-sorted relation; y == 0 is
// an empty slot (a run has at least one row).
struct PredRunHead {  // S sorted by (key << 32 | other): a run starts where the high half changes
    const uint64_t* s;
    __device__ __forceinline__ bool operator()(uint64_t i) const { return i == 0 || (s[i] >> 32) != (s[i - 1] >> 32); }
};
struct EmitRunHead {
    uint32_t* starts;
    __device__ __forceinline__ void operator()(uint64_t i, uint64_t pos) const { starts[pos] = (uint32_t)i; }
};

static __global__ void hash_insert_k(const uint64_t* __restrict__ S, uint64_t n, int key_shift, const uint32_t* __restrict__ starts, uint64_t nu,
                              ulonglong2* __restrict__ table, uint64_t mask, DevStatus* st) {
    for (uint64_t u = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; u < nu; u += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t s = starts[u];
        uint64_t e = u + 1 < nu ? starts[u + 1] : n;
        uint64_t key = S[s] >> key_shift;
        unsigned long long val = (s << 32) | (e - s);
        uint64_t h = mix64(key) & mask;
        bool done = false;
        for (uint64_t probe = 0; probe <= mask; ++probe) {  // bounded by the table size
            unsigned long long* vp = &table[h].y;
            if (atomicCAS(vp, 0ull, val) == 0ull) {
                table[h].x = key;
                done = true;
                break;
            }
            h = (h + 1) & mask;
        }
        if (!done) set_status(st, XLB_ERR_CAPACITY, 1, key);
    }
}

struct LoadKeyHalf {  // join key = one half of the probe tuple (sel 0: high, 1: low)
    const uint64_t* bag;
    int sel;
    __device__ __forceinline__ uint64_t operator()(uint64_t i) const {
        uint64_t t = bag[i];
        return sel == 0 ? (t >> 32) : (t & 0xFFFFFFFFull);
    }
};
struct LoadKey64 {  // join key from a separate array of key words
    const uint64_t* keys;
    __device__ __forceinline__ uint64_t operator()(uint64_t i) const { return keys[i]; }
};

// match[i] = (start << 32) | len, or 0 when the key is absent.  Keys are compared, not only
// their hashes (the reference pins this in crates/xlog-cuda/tests/join_collision_test.rs:19-53).
template <class LoadKey>
static __global__ void __launch_bounds__(BLOCK) hash_probe_k(LoadKey load_key, uint64_t n, const ulonglong2* __restrict__ table, uint64_t mask, uint64_t* __restrict__ match) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t key = load_key(i);
        uint64_t h = mix64(key) & mask;
        uint64_t m = 0;
        for (uint64_t probe = 0; probe <= mask; ++probe) {  // bounded by the table size
            ulonglong2 s = __ldg(&table[h]);
            if (s.y == 0) break;
            if (s.x == key) { m = s.y; break; }
            h = (h + 1) & mask;
        }
        match[i] = m;
    }
}

// ------------------------------------------------------------------------------ tuple hash set
// The tuples of one relation as an open-addressing set of 64-bit words (linear probing, at most
// half full, empty = all ones), kept across the iterations of a fixpoint: a candidate is new
// exactly when its insertion takes an empty slot, so "sort the candidates, drop duplicates,
// subtract the relation" becomes one table access per candidate and only the new tuples are
// ever sorted.  The reference has the same route for heads too wide for a bitmap
// (fj_delta_sparse_novel, kernels/wcoj.cu:4008-4121).
//
// Random accesses to a table of gigabytes run at a fraction of the memory's streaming rate
// (measured: 17 G insertions/s into an 8 GB table).  So the set stores mix64(tuple) — a bijection,
// inverted when tuples leave the set — and a slot's index is the TOP bits of that word: one pass of
// the radix sort over the top byte then groups the candidates into 256 runs that each fall into
// one 256th of the table, a window the L2 holds, and the insertions of a run are L2 accesses.
constexpr unsigned long long HSET_EMPTY = ~0ull;

// Inverse of mix64: x ^= x >> 33 undoes itself (33 >= 32), the multipliers are inverted mod 2^64.
__host__ __device__ __forceinline__ uint64_t unmix64(uint64_t x) {
    x ^= x >> 33;
    x *= 0x9cb4b2f8129337dbull;  // inverse of 0xc4ceb9fe1a85ec53
    x ^= x >> 33;
    x *= 0x4f74430c22a54005ull;  // inverse of 0xff51afd7ed558ccd
    x ^= x >> 33;
    return x;
}
static __global__ void mix_k(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, uint64_t n, int inverse) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) out[i] = inverse ? unmix64(in[i]) : mix64(in[i]);
}

// mix_k that also counts the top byte of every mixed word (the digit the grouping pass sorts by),
// so the pass needs no histogram read of its own.
static __global__ void __launch_bounds__(BLOCK) mix_hist_k(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, uint64_t n, unsigned int* __restrict__ ghist /* 256 */) {
    __shared__ unsigned int sh[256];
    sh[threadIdx.x] = 0;
    __syncthreads();
    for (uint64_t i = (uint64_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += (uint64_t)gridDim.x * BLOCK) {
        const uint64_t w = mix64(in[i]);
        out[i] = w;
        atomicAdd(&sh[w >> 56], 1u);
    }
    __syncthreads();
    if (sh[threadIdx.x]) atomicAdd(&ghist[threadIdx.x], sh[threadIdx.x]);
}

// Mixed copies of `n` words, grouped by their top byte (stable): mix + histogram in one pass, then
// one scatter pass of the radix sort.  n < 2^30.
inline Buf mix_and_group(xlb_ctx* c, const uint64_t* in, uint64_t n) {
    radix_sort_setup(c);
    const uint32_t ntiles = (uint32_t)((n + SORT_TILE - 1) / SORT_TILE);
    Buf words = make_buf(c, n * 8), out = make_buf(c, n * 8);
    Buf gh = make_buf(c, 8 * 256 * 4 * 2 + 64);  // histograms | bases | varies, laid out as the sort's
    unsigned int* ghist = gh->as<unsigned int>();
    unsigned int* bases = ghist + 8 * 256;
    unsigned long long* varies = (unsigned long long*)(bases + 8 * 256);
    CUDA_OK(cudaMemsetAsync(ghist, 0, 8 * 256 * 4, c->stream));
    prof_begin(c, "mix", n * 16ull);
    mix_hist_k<<<grid_for(c, n, BLOCK * 8), BLOCK, 0, c->stream>>>(in, words->as<uint64_t>(), n, ghist + 7 * 256);
    check_launch(c, "mix");
    prof_begin(c, "radix_bases", 0);
    radix_bases_k<<<1, BLOCK, 0, c->stream>>>(ghist, n, bases, varies);
    check_launch(c, "radix_bases");
    const uint64_t status_words = (uint64_t)ntiles * 256;
    Buf status = make_buf(c, (status_words + 8) * 4);
    CUDA_OK(cudaMemsetAsync(status->p, 0, (status_words + 8) * 4, c->stream));
    unsigned int* counters = status->as<unsigned int>() + status_words;
    if (c->lb_first_tile) {
        for (int q = 0; q < 8; ++q) ((unsigned int*)&c->h_scalar[56])[q] = c->lb_first_tile;
        CUDA_OK(cudaMemcpyAsync(counters, &c->h_scalar[56], 8 * 4, cudaMemcpyHostToDevice, c->stream));
    }
    prof_begin(c, "radix_scatter", n * 16ull);
    radix_scatter_k<false, true><<<ntiles, SORT_THREADS, SORT_SMEM, c->stream>>>(words->as<uint64_t>(), out->as<uint64_t>(), nullptr, nullptr, n, 56, bases + 7 * 256, ntiles, counters,
                                                                               status->as<unsigned int>(), c->d_status, c->lb_spin_limit);
    check_launch(c, "radix_scatter");
    return out;
}

// true: the (mixed) word was not in the set and is now.  Bounded by the table size.
// The one word that equals the empty mark is kept in a flag of its own.
__device__ __forceinline__ bool hset_insert(unsigned long long* __restrict__ table, int index_shift, uint64_t mask, uint64_t word, unsigned int* __restrict__ has_empty_word,
                                            DevStatus* st) {
    if (word == HSET_EMPTY) return atomicExch(has_empty_word, 1u) == 0u;
    uint64_t h = word >> index_shift;
    for (uint64_t probe = 0; probe <= mask; ++probe) {
        unsigned long long cur = table[h];
        if (cur == word) return false;
        if (cur == HSET_EMPTY) {
            unsigned long long old = atomicCAS(&table[h], HSET_EMPTY, (unsigned long long)word);
            if (old == HSET_EMPTY) return true;
            if (old == word) return false;  // another thread stored the same tuple first
        }
        h = (h + 1) & mask;
    }
    set_status(st, XLB_ERR_CAPACITY, 12, word);
    return false;
}

// Insert every word (already mixed) without reporting which were new: filling the set from a
// relation, or from an older table, whose empty slots are skipped.
static __global__ void __launch_bounds__(BLOCK) hset_fill_k(const uint64_t* __restrict__ words, uint64_t n, unsigned long long* __restrict__ table, int index_shift, uint64_t mask,
                                                       unsigned int* __restrict__ has_empty_word, bool skip_empty, DevStatus* st) {
    for (uint64_t i = (uint64_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += (uint64_t)gridDim.x * BLOCK) {
        const uint64_t w = words[i];
        if (!(skip_empty && w == HSET_EMPTY)) hset_insert(table, index_shift, mask, w, has_empty_word, st);
    }
}
// Insertion as the predicate of a one-pass compaction (select_append_k): the words that were new
// come out as a bag, and a block of 8192 candidates costs one atomic add on the output counter
// (a warp-level append was measured at 26 G insertions/s, all of it the queue on that one address).
struct PredInsert {
    const uint64_t* words;
    unsigned long long* table;
    int index_shift;
    uint64_t mask;
    unsigned int* has_empty_word;
    DevStatus* st;
    __device__ __forceinline__ bool operator()(uint64_t i) const { return hset_insert(table, index_shift, mask, words[i], has_empty_word, st); }
};

// The host sized an output from a count it kept itself: the device's own count must agree.
static __global__ void verify_count_k(const uint64_t* device_count, uint64_t host_count, DevStatus* st) {
    if (*device_count != host_count) set_status(st, XLB_ERR_CAPACITY, 9, *device_count);
}

// ------------------------------------------------------- direct (counting) join index
// For join keys from a small dense domain the build side needs no sort and no hash table: count
// the rows of every key, prefix-sum the counts, and drop every row's other column at its key's
// cursor.  After the fill pass cursor[k] is the end of key k's group (= the start of key k+1's),
// which is all a probe needs.  Rows of one key land in no particular order: the consumers are
// set-valued (their output is sorted or marked in a bitmap).
// Skewed inputs (a power-law graph's hub) put tens of thousands of rows on one key, and atomics on
// one address serialise in the L2 (measured: 16 M rows with a 69 K-row hub took 250 us per pass,
// the hub's own chain).  So every tile first combines its rows per key in a small shared-memory
// table (open addressing, a few probes; a row that finds no slot goes to global memory on its
// own) and touches global memory once per distinct key.
constexpr int DX_IPT = 8, DX_TILE = BLOCK * DX_IPT, DX_SLOTS = 2048, DX_PROBES = 4;
constexpr uint32_t DX_EMPTY = 0xFFFFFFFFu, DX_NONE = 0xFFFFFFFFu;

// slot of `key` in the tile's table, or DX_NONE
__device__ __forceinline__ uint32_t dx_slot(uint32_t* skey, uint32_t key) {
    uint32_t h = (key * 2654435761u) >> 21;  // 11 bits: DX_SLOTS
#pragma unroll
    for (int t = 0; t < DX_PROBES; ++t) {
        uint32_t old = atomicCAS(&skey[h], DX_EMPTY, key);
        if (old == DX_EMPTY || old == key) return h;
        h = (h + 1) & (DX_SLOTS - 1);
    }
    return DX_NONE;
}

static __global__ void __launch_bounds__(BLOCK) direct_count_k(const uint64_t* __restrict__ rows, uint64_t n, int keysel, unsigned int* __restrict__ cnt, uint64_t domain,
                                                          DevStatus* st) {
    __shared__ uint32_t skey[DX_SLOTS], scnt[DX_SLOTS];
    const uint64_t ntiles = (n + DX_TILE - 1) / DX_TILE;
    for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        for (int s = threadIdx.x; s < DX_SLOTS; s += BLOCK) {
            skey[s] = DX_EMPTY;
            scnt[s] = 0;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < DX_IPT; ++k) {
            uint64_t i = tile * DX_TILE + (uint64_t)k * BLOCK + threadIdx.x;
            if (i >= n) break;
            uint64_t t = rows[i];
            uint64_t key = keysel == 0 ? (t >> 32) : (t & 0xFFFFFFFFull);
            if (key >= domain) {
                set_status(st, XLB_ERR_CAPACITY, 5, key);
                continue;
            }
            uint32_t h = dx_slot(skey, (uint32_t)key);
            if (h != DX_NONE) atomicAdd(&scnt[h], 1u);
            else atomicAdd(&cnt[key], 1u);
        }
        __syncthreads();
        for (int s = threadIdx.x; s < DX_SLOTS; s += BLOCK)
            if (scnt[s]) atomicAdd(&cnt[skey[s]], scnt[s]);
        __syncthreads();
    }
}
static __global__ void __launch_bounds__(BLOCK) direct_fill_k(const uint64_t* __restrict__ rows, uint64_t n, int keysel, unsigned long long* __restrict__ cursor, uint64_t domain,
                                                         uint32_t* __restrict__ pay) {
    __shared__ uint32_t skey[DX_SLOTS], scnt[DX_SLOTS], sbase[DX_SLOTS];
    const uint64_t ntiles = (n + DX_TILE - 1) / DX_TILE;
    for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        for (int s = threadIdx.x; s < DX_SLOTS; s += BLOCK) {
            skey[s] = DX_EMPTY;
            scnt[s] = 0;
        }
        __syncthreads();
        uint32_t other[DX_IPT], where[DX_IPT];  // where = (slot << 16) | rank within the slot, or DX_NONE
#pragma unroll
        for (int k = 0; k < DX_IPT; ++k) {
            where[k] = DX_NONE;
            uint64_t i = tile * DX_TILE + (uint64_t)k * BLOCK + threadIdx.x;
            if (i >= n) continue;
            uint64_t t = rows[i];
            uint64_t key = keysel == 0 ? (t >> 32) : (t & 0xFFFFFFFFull);
            other[k] = keysel == 0 ? (uint32_t)t : (uint32_t)(t >> 32);
            if (key >= domain) continue;  // reported by the counting pass
            uint32_t h = dx_slot(skey, (uint32_t)key);
            if (h != DX_NONE) {
                where[k] = (h << 16) | atomicAdd(&scnt[h], 1u);  // rank < DX_TILE = 2^11
            } else {
                unsigned long long pos = atomicAdd(&cursor[key], 1ull);
                if (pos < n) pay[pos] = other[k];
            }
        }
        __syncthreads();
        for (int s = threadIdx.x; s < DX_SLOTS; s += BLOCK)
            if (scnt[s]) sbase[s] = (uint32_t)atomicAdd(&cursor[skey[s]], (unsigned long long)scnt[s]);  // positions stay below n < 2^32
        __syncthreads();
#pragma unroll
        for (int k = 0; k < DX_IPT; ++k) {
            if (where[k] == DX_NONE) continue;
            uint64_t pos = (uint64_t)sbase[where[k] >> 16] + (where[k] & 0xFFFFu);
            if (pos < n) pay[pos] = other[k];
        }
        __syncthreads();
    }
}
// match[i] = (start << 32) | len, or 0 when the key has no rows (same form as hash_probe_k)
template <class LoadKey>
static __global__ void __launch_bounds__(BLOCK) direct_probe_k(LoadKey load_key, uint64_t n, const unsigned long long* __restrict__ cursor, uint64_t domain,
                                                          uint64_t* __restrict__ match) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t key = load_key(i);
        uint64_t m = 0;
        if (key < domain) {
            uint64_t e = __ldg(&cursor[key]);
            uint64_t s = key ? __ldg(&cursor[key - 1]) : 0;
            if (e > s) m = (s << 32) | (e - s);
        }
        match[i] = m;
    }
}

// ------------------------------------------------------------------ scan join (sides swapped)
// When the probing bag contributes nothing but the join key to the output and its keys come from
// a small dense domain, the join can run from the other side without any index on the stored
// relation: mark the bag's keys in a bitmap, then stream over the relation's rows and keep those
// whose key is marked.  One sequential read of the relation per use, against a sort of it (or a
// counting build) for an index.
static __global__ void __launch_bounds__(BLOCK) keyset_mark_k(const uint64_t* __restrict__ rows, uint64_t n, int keysel, unsigned int* __restrict__ bitmap, uint64_t domain,
                                                         DevStatus* st) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t t = rows[i];
        uint64_t key = keysel == 0 ? (t >> 32) : (t & 0xFFFFFFFFull);
        if (key >= domain) {
            set_status(st, XLB_ERR_CAPACITY, 6, key);
            continue;
        }
        unsigned bit = 1u << (key & 31);
        if (!(bitmap[key >> 5] & bit)) atomicOr(&bitmap[key >> 5], bit);
    }
}
// output half from a relation row: 0 = its key column, 1 = its other column, 2 = zero
__device__ __forceinline__ uint32_t sj_pick(int src, uint32_t key, uint32_t other) { return src == 0 ? key : src == 1 ? other : 0u; }
// (Staging the key set in shared memory first — 128 KB for 2^20 keys, one block of 1024 threads
// per SM — was measured slower than these cached loads: 50 us against 46 per 16 M-row stream.)
__device__ __forceinline__ bool sj_in(const unsigned int* __restrict__ keyset, uint64_t domain, uint32_t key) {
    return key < domain && ((__ldg(&keyset[key >> 5]) >> (key & 31)) & 1u);
}
// Rows whose key is in the key set, marked in the head's bitmap; *count += their number.
// Memory-bound streaming: every thread keeps SJ_VEC 16-byte loads in flight per step (one 8-byte
// load per thread and step left the kernel at 1.9 TB/s, latency-bound).
constexpr int SJ_VEC = 4, SJ_TILE = BLOCK * SJ_VEC * 2;
__device__ __forceinline__ unsigned sj_mark_row(uint64_t t, int keysel, const unsigned int* __restrict__ keyset, uint64_t domain, int hi_src, int lo_src,
                                                unsigned int* __restrict__ bitmap, uint64_t words, int lo_bits, DevStatus* st,
                                                const unsigned int* __restrict__ visited, unsigned char* __restrict__ touched) {
    uint32_t key = keysel == 0 ? (uint32_t)(t >> 32) : (uint32_t)t;
    uint32_t other = keysel == 0 ? (uint32_t)t : (uint32_t)(t >> 32);
    if (!sj_in(keyset, domain, key)) return 0;
    uint64_t out = ((uint64_t)sj_pick(hi_src, key, other) << 32) | sj_pick(lo_src, key, other);
    uint32_t x = dense_index(out, lo_bits);
    if ((out & 0xFFFFFFFFull) >> lo_bits || (uint64_t)(x >> 5) >= words) {
        set_status(st, XLB_ERR_CAPACITY, 7, out);
        return 1;
    }
    unsigned bit = 1u << (x & 31);
    if (visited && (__ldg(&visited[x >> 5]) & bit)) return 1;  // known already: most of a hub's tuples
    // (a plain load, served by the L1: reading the hot words of a hub through to the L2 instead
    // made the kernel three times slower)
    if (!(bitmap[x >> 5] & bit)) {
        atomicOr(&bitmap[x >> 5], bit);
        if (touched) touched[x >> DENSE_TOUCH_SHIFT] = 1;
    }
    return 1;
}
static __global__ void __launch_bounds__(BLOCK) scan_join_mark_k(const uint64_t* __restrict__ rows, uint64_t n, int keysel, const unsigned int* __restrict__ keyset,
                                                            uint64_t domain, int hi_src, int lo_src, unsigned int* __restrict__ bitmap, uint64_t words, int lo_bits,
                                                            unsigned long long* __restrict__ count, DevStatus* st, const unsigned int* __restrict__ visited,
                                                            const unsigned long long* __restrict__ keys_in_set = nullptr, unsigned char* __restrict__ touched = nullptr) {
    // (keys_in_set: the number of keys in the key set when the host enqueued this launch without
    // knowing it; over an empty set there is nothing to find)
    if (keys_in_set && *keys_in_set == 0) return;
    unsigned long long mine = 0;
    const uint64_t ntiles = n / SJ_TILE;  // whole tiles, 16-byte loads (the row array is 16-byte aligned: checked by the host)
    const ulonglong2* rows2 = reinterpret_cast<const ulonglong2*>(rows);
    for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        ulonglong2 v[SJ_VEC];
#pragma unroll
        for (int k = 0; k < SJ_VEC; ++k) v[k] = rows2[tile * (SJ_TILE / 2) + (uint64_t)k * BLOCK + threadIdx.x];
#pragma unroll
        for (int k = 0; k < SJ_VEC; ++k) {
            mine += sj_mark_row(v[k].x, keysel, keyset, domain, hi_src, lo_src, bitmap, words, lo_bits, st, visited, touched);
            mine += sj_mark_row(v[k].y, keysel, keyset, domain, hi_src, lo_src, bitmap, words, lo_bits, st, visited, touched);
        }
    }
    for (uint64_t i = ntiles * SJ_TILE + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        mine += sj_mark_row(rows[i], keysel, keyset, domain, hi_src, lo_src, bitmap, words, lo_bits, st, visited, touched);
    for (int d = 16; d; d >>= 1) mine += __shfl_down_sync(0xFFFFFFFFu, mine, d);
    if (lane_id() == 0 && mine) atomicAdd(count, mine);
}
// The scan of a frontier loop: rows whose key is in the frontier mark their value in `marks`
// (*count_marked += their number), and — because a key enters the frontier of such a loop
// exactly once — a row whose key the head already holds can never match again.  `visited` is the
// head as the iteration found it; `marks` starts every iteration as a copy of it, so one look-up
// tells whether a value is known or marked already.  `frontier` may be null when every row whose
// key `visited` holds is known to have its key in the frontier (a list written by the scan before
// this one holds no other rows; nor does a relation when the head holds the frontier only).
// Random look-ups into the bitmaps, not the stream over the rows, are what a scan pays for (the
// L1 serves one line per cycle): one per row and one more per matching row.  With `live_out`
// the rows whose key the head does not hold yet are appended to it, packed (*live_count += their
// number): the next scan streams over those instead of over the whole relation.  The rows come
// either packed (`rows`) or as the relation's two columns (COLS: `kcol` the join column, `ocol` the
// other one), so that a relation given as columns need not be packed for the first scan.
// `n_ptr`, when set, holds the number of rows (a list written by an earlier launch whose length the
// host has not read yet).  Every thread keeps 64 bytes of loads in flight; a tile is FS_TILE rows.
#ifndef XLB_FS_MINBLOCKS
#define XLB_FS_MINBLOCKS 8
#endif
constexpr int FS_IPT = 8, FS_TILE = BLOCK * FS_IPT;
template <bool COLS>
__device__ __forceinline__ void frontier_scan_body(const uint64_t* __restrict__ rows, const uint32_t* __restrict__ kcol, const uint32_t* __restrict__ ocol, uint64_t n, int keysel,
                                                   const unsigned int* __restrict__ frontier, const unsigned int* __restrict__ visited, uint64_t domain, int value_is_key,
                                                   unsigned int* __restrict__ marks,
                                                   uint64_t words, int lo_bits, unsigned long long* count_marked, DevStatus* st, uint64_t* live_out,
                                                   unsigned long long* live_count, unsigned* warp_sum, unsigned long long& base_s) {
    const uint64_t ntiles = (n + FS_TILE - 1) / FS_TILE;
    unsigned long long mine = 0;
    for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const uint64_t t0 = tile * FS_TILE;
        uint32_t key[FS_IPT], other[FS_IPT];
        unsigned have = 0;  // bit j: row j of this thread exists
        if (t0 + FS_TILE <= n) {
            have = (1u << FS_IPT) - 1;
            if (COLS) {
                const uint4* k4 = reinterpret_cast<const uint4*>(kcol + t0);
                const uint4* o4 = reinterpret_cast<const uint4*>(ocol + t0);
                uint4 a[FS_IPT / 4], b[FS_IPT / 4];
#pragma unroll
                for (int q = 0; q < FS_IPT / 4; ++q) {
                    a[q] = k4[q * BLOCK + threadIdx.x];
                    b[q] = o4[q * BLOCK + threadIdx.x];
                }
#pragma unroll
                for (int q = 0; q < FS_IPT / 4; ++q) {
                    key[4 * q] = a[q].x, key[4 * q + 1] = a[q].y, key[4 * q + 2] = a[q].z, key[4 * q + 3] = a[q].w;
                    other[4 * q] = b[q].x, other[4 * q + 1] = b[q].y, other[4 * q + 2] = b[q].z, other[4 * q + 3] = b[q].w;
                }
            } else {
                const ulonglong2* r2 = reinterpret_cast<const ulonglong2*>(rows + t0);
                ulonglong2 v[FS_IPT / 2];
#pragma unroll
                for (int q = 0; q < FS_IPT / 2; ++q) v[q] = r2[q * BLOCK + threadIdx.x];
#pragma unroll
                for (int q = 0; q < FS_IPT / 2; ++q) {
                    const uint64_t x = v[q].x, y = v[q].y;
                    key[2 * q] = keysel == 0 ? (uint32_t)(x >> 32) : (uint32_t)x;
                    other[2 * q] = keysel == 0 ? (uint32_t)x : (uint32_t)(x >> 32);
                    key[2 * q + 1] = keysel == 0 ? (uint32_t)(y >> 32) : (uint32_t)y;
                    other[2 * q + 1] = keysel == 0 ? (uint32_t)y : (uint32_t)(y >> 32);
                }
            }
        } else {  // the last, partial tile
#pragma unroll
            for (int j = 0; j < FS_IPT; ++j) {
                const uint64_t i = t0 + (uint64_t)j * BLOCK + threadIdx.x;
                key[j] = other[j] = 0;
                if (i < n) {
                    have |= 1u << j;
                    if (COLS) {
                        key[j] = kcol[i];
                        other[j] = ocol[i];
                    } else {
                        const uint64_t x = rows[i];
                        key[j] = keysel == 0 ? (uint32_t)(x >> 32) : (uint32_t)x;
                        other[j] = keysel == 0 ? (uint32_t)x : (uint32_t)(x >> 32);
                    }
                }
            }
        }
        unsigned live = 0;  // bit j: the head does not hold row j's key yet
#pragma unroll
        for (int j = 0; j < FS_IPT; ++j) {
            if (!((have >> j) & 1u) || key[j] >= domain) continue;  // (a key outside the domain can never be derived)
            const unsigned bit = 1u << (key[j] & 31);
            if (!(__ldg(&visited[key[j] >> 5]) & bit)) {
                live |= 1u << j;
                continue;
            }
            if (frontier && !(__ldg(&frontier[key[j] >> 5]) & bit)) continue;  // was in an earlier frontier
            ++mine;
            const uint32_t x = value_is_key ? key[j] : other[j];
            if ((uint64_t)x >> lo_bits || (uint64_t)(x >> 5) >= words) {
                set_status(st, XLB_ERR_CAPACITY, 7, x);
                continue;
            }
            const unsigned xb = 1u << (x & 31);
            // (a plain load, served by the L1: known already or marked already is the common case;
            // a stale line only costs an atomic that changes nothing)
            if (!(marks[x >> 5] & xb)) atomicOr(&marks[x >> 5], xb);
        }
        if (live_out) {
            // The tile's live rows go out as one contiguous piece, without staging them in shared
            // memory (which would take the L1 space the bitmaps live in): one reservation per
            // block, and within a warp row j of every lane is written in round j, the lanes that
            // hold one at consecutive addresses.
            unsigned ballots[FS_IPT];
            unsigned warp_total = 0;
#pragma unroll
            for (int j = 0; j < FS_IPT; ++j) {
                ballots[j] = __ballot_sync(FULL, (live >> j) & 1u);
                warp_total += __popc(ballots[j]);
            }
            const int w = threadIdx.x >> 5;
            if (lane_id() == 0) warp_sum[w] = warp_total;
            __syncthreads();
            unsigned before = 0, total = 0;
#pragma unroll
            for (int q = 0; q < BLOCK / 32; ++q) {
                const unsigned ws = warp_sum[q];
                if (q < w) before += ws;
                total += ws;
            }
            if (threadIdx.x == 0 && total) base_s = atomicAdd(live_count, (unsigned long long)total);
            __syncthreads();  // (also: warp_sum is not rewritten before every warp has read it)
            unsigned long long at = base_s + before;
            const unsigned below = (1u << lane_id()) - 1;
#pragma unroll
            for (int j = 0; j < FS_IPT; ++j) {
                if ((live >> j) & 1u)
                    live_out[at + __popc(ballots[j] & below)] = keysel == 0 ? ((uint64_t)key[j] << 32) | other[j] : ((uint64_t)other[j] << 32) | key[j];
                at += __popc(ballots[j]);
            }
        }
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) mine += __shfl_down_sync(FULL, mine, d);
    if (lane_id() == 0 && mine) atomicAdd(count_marked, mine);
}

template <bool COLS>
static __global__ void __launch_bounds__(BLOCK, XLB_FS_MINBLOCKS) frontier_scan_k(const uint64_t* __restrict__ rows, const uint32_t* __restrict__ kcol, const uint32_t* __restrict__ ocol,
                                                           uint64_t n_max, const unsigned long long* __restrict__ n_ptr, int keysel, const unsigned int* frontier,
                                                           const unsigned int* visited, uint64_t domain, int value_is_key, unsigned int* marks, uint64_t words, int lo_bits,
                                                           unsigned long long* count_marked, DevStatus* st, const unsigned long long* __restrict__ keys_in_frontier,
                                                           uint64_t* live_out, unsigned long long* live_count) {
    if (keys_in_frontier && *keys_in_frontier == 0) return;  // enqueued on top of an iteration that found nothing
    __shared__ unsigned warp_sum[BLOCK / 32];
    __shared__ unsigned long long base_s;
    uint64_t n = n_ptr ? (uint64_t)*n_ptr : n_max;
    if (n > n_max) n = n_max;
    frontier_scan_body<COLS>(rows, kcol, ocol, n, keysel, frontier, visited, domain, value_is_key, marks, words, lo_bits, count_marked, st, live_out, live_count, warp_sum, base_s);
}

struct PredKeyIn {  // the row's key is in the key set
    const uint64_t* rows;
    int keysel;
    const unsigned int* keyset;
    uint64_t domain;
    __device__ __forceinline__ bool operator()(uint64_t i) const {
        uint64_t t = rows[i];
        return sj_in(keyset, domain, keysel == 0 ? (uint32_t)(t >> 32) : (uint32_t)t);
    }
};
struct EmitScanRow {  // the row in the output layout
    const uint64_t* rows;
    int keysel, hi_src, lo_src;
    uint64_t* out;
    __device__ __forceinline__ void operator()(uint64_t i, uint64_t pos) const {
        uint64_t t = rows[i];
        uint32_t key = keysel == 0 ? (uint32_t)(t >> 32) : (uint32_t)t;
        uint32_t other = keysel == 0 ? (uint32_t)t : (uint32_t)(t >> 32);
        out[pos] = ((uint64_t)sj_pick(hi_src, key, other) << 32) | sj_pick(lo_src, key, other);
    }
};

struct PredMatched {
    const uint64_t* match;
    __device__ __forceinline__ bool operator()(uint64_t i) const { return match[i] != 0; }
};
struct EmitMatched {
    const uint64_t* bag;
    const uint64_t* match;
    uint64_t* mbag;
    uint64_t* mmatch;
    __device__ __forceinline__ void operator()(uint64_t i, uint64_t pos) const {
        mbag[pos] = bag[i];
        mmatch[pos] = match[i];
    }
};

constexpr int EX_IPT = 8;
constexpr int EX_TILE = BLOCK * EX_IPT;

// Output column source: 0 = probe high half, 1 = probe low half, 2 = the build row's other
// column, 3 = zero (arity-1 output keeps the value in the low half).
__device__ __forceinline__ uint32_t ex_pick(int src, uint64_t probe, uint32_t other) {
    return src == 0 ? (uint32_t)(probe >> 32) : src == 1 ? (uint32_t)probe : src == 2 ? other : 0u;
}

// Load-balanced expansion: every matched probe row contributes len outputs; each tile of EX_TILE
// outputs finds its rows by a search over the row offsets held in shared memory, so writes are
// coalesced whatever the degree skew.  Output order: probe row order, then build order.
// MARK = true: instead of storing the output tuples, set their bits in a dense-domain bitmap (the
// candidates of a small-domain head never touch memory as a list).
template <bool MARK>
static __global__ void __launch_bounds__(BLOCK, 8) expand_k(const uint64_t* __restrict__ mbag, const uint64_t* __restrict__ mmatch, const uint64_t* __restrict__ off,
                                                   uint64_t nrows, uint64_t total, const uint64_t* __restrict__ S,
                                                   const uint32_t* __restrict__ pay, int hi_src, int lo_src, uint64_t* __restrict__ out,
                                                   unsigned int* __restrict__ bitmap, uint64_t words, int lo_bits, DevStatus* st,
                                                   const uint64_t* __restrict__ total_dev, const unsigned int* __restrict__ visited,
                                                   unsigned char* __restrict__ touched) {
    // Row offsets of the tile's span relative to the tile's first output, 32 bits each: rel[0] = 0
    // stands for the row that owns that output (its offset may lie before the tile; `skip0` says by
    // how much), every later row starts inside the tile or at EX_TILE (beyond it).  The search per
    // output then runs on 32-bit words.
    __shared__ unsigned rel[EX_TILE + 2];
    __shared__ uint64_t row_s[2];
    // With total_dev the output count is still on the device (the host launched a fixed grid
    // without reading it back): tiles are then walked grid-strided.
    if (total_dev) total = *total_dev;
  for (uint64_t tile = blockIdx.x; tile * EX_TILE < total; tile += gridDim.x) {
    uint64_t o0 = tile * EX_TILE;
    uint64_t o1 = o0 + EX_TILE < total ? o0 + EX_TILE : total;
    if (threadIdx.x < 64) {  // warp 0: the row that owns output o0; warp 1: the row that owns the next tile's first output
        uint64_t o = threadIdx.x < 32 ? o0 : o0 + EX_TILE;
        uint64_t ub = o < total ? warp_partition_point(nrows, [&](uint64_t i) { return off[i] <= o; }) : nrows + 1;
        if (lane_id() == 0) row_s[threadIdx.x >> 5] = ub - 1;  // last row with offset <= o
    }
    __syncthreads();
    uint64_t r0 = row_s[0], r1 = row_s[1];
    if (r1 >= nrows) r1 = nrows - 1;
    // Probe rows without a match stay in the arrays (equal consecutive offsets), so a tile may span
    // any number of rows; the usual span fits shared memory, a longer one is searched in place.
    const uint64_t span = r1 - r0 + 1;
    const bool in_smem = span <= (uint64_t)(EX_TILE + 2);
    if (in_smem)
        for (unsigned i = threadIdx.x; i < (unsigned)span; i += BLOCK) {
            const uint64_t at = off[r0 + i];
            rel[i] = at <= o0 ? 0u : (at - o0 < (uint64_t)EX_TILE ? (unsigned)(at - o0) : (unsigned)EX_TILE);
        }
    const uint64_t skip0 = o0 - off[r0];  // outputs of row r0 that earlier tiles wrote
    __syncthreads();
    const unsigned in_tile = (unsigned)(o1 - o0);
#pragma unroll
    for (int k = 0; k < EX_IPT; ++k) {
        const unsigned t = (unsigned)k * BLOCK + threadIdx.x;  // the output's place in the tile
        if (t >= in_tile) break;
        uint64_t r, j_in_row;
        if (in_smem) {
            unsigned lo = 0, hi = (unsigned)span;  // first row of the span that starts after t; the one before it owns t
            while (lo < hi) {
                const unsigned mid = (lo + hi) >> 1;
                if (rel[mid] <= t) lo = mid + 1;
                else hi = mid;
            }
            r = r0 + lo - 1;
            j_in_row = lo == 1 ? skip0 + t : (uint64_t)(t - rel[lo - 1]);
        } else {
            const uint64_t o = o0 + t;
            uint64_t lo = 0, hi = span;
            while (lo < hi) {
                uint64_t mid = (lo + hi) >> 1;
                if (off[r0 + mid] <= o) lo = mid + 1;
                else hi = mid;
            }
            r = r0 + lo - 1;
            j_in_row = o - off[r];
        }
        uint64_t probe = mbag[r];
        uint64_t start = mmatch[r] >> 32;
        uint64_t j = start + j_in_row;
        uint32_t other = pay ? pay[j] : (uint32_t)S[j];
        uint64_t key = ((uint64_t)ex_pick(hi_src, probe, other) << 32) | ex_pick(lo_src, probe, other);
        if (!MARK) {
            out[o0 + t] = key;
        } else {
            uint32_t x = dense_index(key, lo_bits);
            if ((key & 0xFFFFFFFFull) >> lo_bits || (uint64_t)(x >> 5) >= words) {
                set_status(st, XLB_ERR_CAPACITY, 4, key);
            } else {
                unsigned bit = 1u << (x & 31);
                if (!(visited && (__ldg(&visited[x >> 5]) & bit)) && !(bitmap[x >> 5] & bit)) {
                    atomicOr(&bitmap[x >> 5], bit);
                    if (touched) touched[x >> DENSE_TOUCH_SHIFT] = 1;
                }
            }
        }
    }
    __syncthreads();  // the next tile refills rel / row_s
  }
}

}  // namespace xk
