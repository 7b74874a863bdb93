// Context, relations and relational operators of the C ABI (include/xlb.h), plus the host-level
// key-array operations the executor uses.  Every device loop lives in xlb_kernels.cuh.
#include <algorithm>
#include <cstring>

#include "xlb_kernels.cuh"
#include "xlb_ops.h"

using namespace xk;

// ------------------------------------------------------------------------------ small kernels
namespace {

__global__ void iota_k(uint32_t* out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) out[i] = (uint32_t)i;
}
__global__ void iota64_k(uint64_t* out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) out[i] = i;
}
// key word of a row from up to two columns: (a << 32 | b) for two 32-bit columns, the value itself otherwise
__global__ void build_key_k(const void* c0, int w0, const void* c1, int w1, const uint32_t* idx, uint64_t* out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t r = idx ? idx[i] : i;
        uint64_t a = w0 == 4 ? ((const uint32_t*)c0)[r] : w0 == 8 ? ((const uint64_t*)c0)[r] : ((const uint8_t*)c0)[r];
        if (c1) {
            uint64_t b = ((const uint32_t*)c1)[r];
            a = (a << 32) | b;
        }
        out[i] = a;
    }
}
template <class T>
__global__ void gather_k(const T* __restrict__ in, const uint32_t* __restrict__ idx, T* __restrict__ out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) out[i] = in[idx[i]];
}
// gather by one half of a u64 pair array (hi: left row, lo: right row)
template <class T>
__global__ void gather_pair_k(const T* __restrict__ in, const uint64_t* __restrict__ pairs, int half, T* __restrict__ out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t p = pairs[i];
        out[i] = in[half == 0 ? (p >> 32) : (p & 0xFFFFFFFFull)];
    }
}

struct ColSet {  // columns of a gathered (sorted) relation for multi-column run detection
    const void* col[XLB_MAX_ARITY];
    int width[XLB_MAX_ARITY];
    int n;
};
__device__ __forceinline__ bool rows_equal(const ColSet& cs, uint64_t a, uint64_t b) {
    for (int c = 0; c < cs.n; ++c) {
        uint64_t x = cs.width[c] == 4 ? ((const uint32_t*)cs.col[c])[a] : cs.width[c] == 8 ? ((const uint64_t*)cs.col[c])[a] : ((const uint8_t*)cs.col[c])[a];
        uint64_t y = cs.width[c] == 4 ? ((const uint32_t*)cs.col[c])[b] : cs.width[c] == 8 ? ((const uint64_t*)cs.col[c])[b] : ((const uint8_t*)cs.col[c])[b];
        if (x != y) return false;
    }
    return true;
}
// Segmented reduction for group-by over rows sorted by key.  heads[g] = first row of group g.
// A thread walks GB_ITEMS consecutive rows and hands a group's partial result over with one atomic
// when the group changes, so a group of any size costs at most one atomic per GB_ITEMS of its
// rows.  vals: the value column in sorted order (null for a count); out: one u64 per group, set to
// the operator's identity beforehand.
constexpr int GB_ITEMS = 8;
template <class V>
__global__ void groupby_reduce_k(const V* __restrict__ vals, const uint32_t* __restrict__ heads, uint64_t m, uint64_t n, int op,
                                 unsigned long long* __restrict__ out) {
    const unsigned long long ident = op == XLB_AGG_MIN ? ~0ull : 0ull;
    auto flush = [&](uint64_t g, unsigned long long acc) {
        if (op == XLB_AGG_MIN) atomicMin(&out[g], acc);
        else if (op == XLB_AGG_MAX) atomicMax(&out[g], acc);
        else if (acc) atomicAdd(&out[g], acc);
    };
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t * GB_ITEMS < n; t += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t first = t * GB_ITEMS, last = first + GB_ITEMS < n ? first + GB_ITEMS : n;
        // group of the first row: the last head at or before it
        uint64_t lo = 0, hi = m;
        while (lo < hi) {
            uint64_t mid = (lo + hi) >> 1;
            if (heads[mid] <= first) lo = mid + 1;
            else hi = mid;
        }
        uint64_t g = lo - 1;
        uint64_t next = g + 1 < m ? heads[g + 1] : n;
        unsigned long long acc = ident;
        for (uint64_t i = first; i < last; ++i) {
            if (i == next) {
                flush(g, acc);
                acc = ident;
                ++g;
                next = g + 1 < m ? heads[g + 1] : n;
            }
            unsigned long long v = op == XLB_AGG_COUNT ? 1ull : (unsigned long long)vals[i];
            if (op == XLB_AGG_MIN) acc = v < acc ? v : acc;
            else if (op == XLB_AGG_MAX) acc = v > acc ? v : acc;
            else acc += v;
        }
        flush(g, acc);
    }
}
__global__ void fill_u64_k(unsigned long long* out, uint64_t n, unsigned long long v) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) out[i] = v;
}
__global__ void narrow_u64_k(const unsigned long long* in, uint32_t* out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) out[i] = (uint32_t)in[i];
}

struct PredRowHead {
    ColSet cs;
    __device__ __forceinline__ bool operator()(uint64_t i) const { return i == 0 || !rows_equal(cs, i, i - 1); }
};
// run head whose run does not start with a row of the excluded input (origin index < n_excl)
struct PredRowHeadNotExcluded {
    ColSet cs;
    const uint32_t* origin;
    uint32_t n_excl;
    __device__ __forceinline__ bool operator()(uint64_t i) const {
        if (i != 0 && rows_equal(cs, i, i - 1)) return false;
        return origin[i] >= n_excl;
    }
};
struct EmitIndex {
    uint32_t* out;
    __device__ __forceinline__ void operator()(uint64_t i, uint64_t pos) const { out[pos] = (uint32_t)i; }
};
struct PredCmp {
    const uint64_t* in;
    uint32_t cmp;
    int lhs;
    bool rhs_const;
    uint64_t rhs;
    __device__ __forceinline__ bool operator()(uint64_t i) const {
        uint64_t k = in[i];
        uint64_t a = lhs == SRC_HI ? (k >> 32) : (k & 0xFFFFFFFFull);
        uint64_t b = rhs_const ? rhs : (rhs == SRC_HI ? (k >> 32) : (k & 0xFFFFFFFFull));
        switch (cmp) {
            case XLB_EQ: return a == b;
            case XLB_NE: return a != b;
            case XLB_LT: return a < b;
            case XLB_LE: return a <= b;
            case XLB_GT: return a > b;
            default: return a >= b;
        }
    }
};
struct PredOwner {
    const uint64_t* in;
    int keysel;
    uint32_t world, rank;
    __device__ __forceinline__ bool operator()(uint64_t i) const {
        uint64_t w = in[i];
        uint64_t key = keysel == 0 ? (w >> 32) : (w & 0xFFFFFFFFull);
        return (uint32_t)(mix64(key) % world) == rank;
    }
};
__global__ void add_word_k(unsigned long long* dst, const unsigned long long* src) { *dst += *src; }
struct PredCmpCols {  // comparison between a column and a constant or another column (values widened to 64 bits)
    ColSet cs;
    uint32_t cmp, lhs;
    bool rhs_const;
    uint64_t rhs;
    __device__ __forceinline__ uint64_t at(uint32_t col, uint64_t i) const {
        return cs.width[col] == 4 ? ((const uint32_t*)cs.col[col])[i] : cs.width[col] == 8 ? ((const uint64_t*)cs.col[col])[i] : ((const uint8_t*)cs.col[col])[i];
    }
    __device__ __forceinline__ bool operator()(uint64_t i) const {
        const uint64_t a = at(lhs, i), b = rhs_const ? rhs : at((uint32_t)rhs, i);
        switch (cmp) {
            case XLB_EQ: return a == b;
            case XLB_NE: return a != b;
            case XLB_LT: return a < b;
            case XLB_LE: return a <= b;
            case XLB_GT: return a > b;
            default: return a >= b;
        }
    }
};
// Order-independent digest of rows: XOR and low-32-bit sum of one mixed word per row.
__global__ void digest_packed_k(const uint64_t* __restrict__ rows, uint64_t n, unsigned long long* out) {
    unsigned long long x = 0, lo = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t h = mix64(rows[i]);
        x ^= h;
        lo += h & 0xFFFFFFFFull;
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) {
        x ^= __shfl_xor_sync(FULL, x, d);
        lo += __shfl_xor_sync(FULL, lo, d);
    }
    if (lane_id() == 0) {
        atomicXor(&out[0], x);
        atomicAdd(&out[1], lo);
    }
}
__global__ void digest_cols_k(ColSet cs, uint64_t n, unsigned long long* out) {
    unsigned long long x = 0, lo = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t h = 0;
        for (int c = 0; c < cs.n; ++c) {
            const uint64_t v = cs.width[c] == 4 ? ((const uint32_t*)cs.col[c])[i] : cs.width[c] == 8 ? ((const uint64_t*)cs.col[c])[i] : ((const uint8_t*)cs.col[c])[i];
            h = mix64(h ^ v);
        }
        h = mix64(h);
        x ^= h;
        lo += h & 0xFFFFFFFFull;
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) {
        x ^= __shfl_xor_sync(FULL, x, d);
        lo += __shfl_xor_sync(FULL, lo, d);
    }
    if (lane_id() == 0) {
        atomicXor(&out[0], x);
        atomicAdd(&out[1], lo);
    }
}
struct PredFlag {
    const uint64_t* match;
    bool want;
    __device__ __forceinline__ bool operator()(uint64_t i) const { return (match[i] != 0) == want; }
};

// Partition by owner rank in two sweeps: count per destination, then scatter.  Counters are kept
// per block in shared memory; a block claims its slice of every destination's segment with one
// global atomic per destination, so the hot counters see one update per 2048 rows.  Rows keep no
// particular order inside a destination (they are sorted or re-indexed on arrival).
constexpr int OWN_IPT = 8;
__global__ void __launch_bounds__(BLOCK) owner_count_k(const uint64_t* __restrict__ in, uint64_t n, int keysel, uint32_t world, unsigned long long* __restrict__ counts) {
    __shared__ unsigned int sh[64];
    if (threadIdx.x < 64) sh[threadIdx.x] = 0;
    __syncthreads();
    uint64_t base = (uint64_t)blockIdx.x * (BLOCK * OWN_IPT);
#pragma unroll
    for (int k = 0; k < OWN_IPT; ++k) {
        uint64_t i = base + (uint64_t)k * BLOCK + threadIdx.x;
        if (i < n) {
            uint64_t w = in[i];
            uint64_t key = keysel == 0 ? (w >> 32) : (w & 0xFFFFFFFFull);
            atomicAdd(&sh[(uint32_t)(mix64(key) % world)], 1u);
        }
    }
    __syncthreads();
    if (threadIdx.x < world && sh[threadIdx.x]) atomicAdd(&counts[threadIdx.x], (unsigned long long)sh[threadIdx.x]);
}
// cursors[d] = start of destination d's segment (exclusive scan of the counts; world <= 64)
__global__ void owner_starts_k(const unsigned long long* __restrict__ counts, uint32_t world, unsigned long long* __restrict__ cursors) {
    if (threadIdx.x == 0) {
        unsigned long long run = 0;
        for (uint32_t d = 0; d < world; ++d) {
            cursors[d] = run;
            run += counts[d];
        }
    }
}
__global__ void __launch_bounds__(BLOCK) owner_scatter_k(const uint64_t* __restrict__ in, uint64_t n, int keysel, uint32_t world,
                                                         unsigned long long* __restrict__ cursors, uint64_t* __restrict__ out) {
    __shared__ unsigned int sh[64];
    __shared__ unsigned long long sbase[64];
    if (threadIdx.x < 64) sh[threadIdx.x] = 0;
    __syncthreads();
    uint64_t base = (uint64_t)blockIdx.x * (BLOCK * OWN_IPT);
    uint64_t row[OWN_IPT];
    unsigned dest[OWN_IPT], local[OWN_IPT];
#pragma unroll
    for (int k = 0; k < OWN_IPT; ++k) {
        uint64_t i = base + (uint64_t)k * BLOCK + threadIdx.x;
        dest[k] = 0xFFFFFFFFu;
        if (i < n) {
            row[k] = in[i];
            uint64_t key = keysel == 0 ? (row[k] >> 32) : (row[k] & 0xFFFFFFFFull);
            dest[k] = (uint32_t)(mix64(key) % world);
            local[k] = atomicAdd(&sh[dest[k]], 1u);
        }
    }
    __syncthreads();
    if (threadIdx.x < world) sbase[threadIdx.x] = sh[threadIdx.x] ? atomicAdd(&cursors[threadIdx.x], (unsigned long long)sh[threadIdx.x]) : 0ull;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < OWN_IPT; ++k)
        if (dest[k] != 0xFFFFFFFFu) out[sbase[dest[k]] + local[k]] = row[k];
}

}  // namespace

extern "C" uint32_t xlb_owner_of(uint64_t key, uint32_t world) { return world ? (uint32_t)(xk::mix64(key) % world) : 0; }

// ------------------------------------------------------------------------------ phase timing
struct PhaseRec {
    cudaEvent_t e0, e1;
    double* acc;
};
static thread_local std::vector<PhaseRec> g_phase_recs;

PhaseTimer::PhaseTimer(xlb_ctx* ctx, double* into) : c(ctx), acc(into) {
    if (!(c->flags & XLB_FLAG_PROFILE) || !into) return;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, c->stream);
}
PhaseTimer::~PhaseTimer() {
    if (!e0) return;
    cudaEventRecord(e1, c->stream);
    g_phase_recs.push_back({e0, e1, acc});
}
void xlb_resolve_phase_timers(xlb_ctx* c) {
    cudaStreamSynchronize(c->stream);
    for (auto& r : g_phase_recs) {
        float ms = 0;
        if (cudaEventElapsedTime(&ms, r.e0, r.e1) == cudaSuccess) *r.acc += ms;
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
    }
    g_phase_recs.clear();
    for (auto& kv : c->prof) {
        for (auto& e : kv.second.pending) {
            float ms = 0;
            if (cudaEventElapsedTime(&ms, e.first, e.second) == cudaSuccess) kv.second.ms += ms;
            cudaEventDestroy(e.first);
            cudaEventDestroy(e.second);
        }
        kv.second.pending.clear();
    }
}

extern "C" xlb_status xlb_profile_enable(xlb_ctx* c, const char* kernel) {
    if (!c) return XLB_ERR_INVALID;
    xlb_resolve_phase_timers(c);
    c->prof.clear();
    c->prof_filter = kernel ? kernel : "";
    return XLB_OK;
}

extern "C" xlb_status xlb_profile_read(xlb_ctx* c, xlb_kernel_profile* out, uint32_t cap, uint32_t* n) {
    if (!c || !n) return XLB_ERR_INVALID;
    xlb_resolve_phase_timers(c);
    uint32_t i = 0;
    for (auto& kv : c->prof) {
        if (out && i < cap) {
            memset(&out[i], 0, sizeof out[i]);
            strncpy(out[i].name, kv.first.c_str(), sizeof(out[i].name) - 1);
            out[i].launches = kv.second.launches;
            out[i].ms = kv.second.ms;
            out[i].bytes = kv.second.bytes;
        }
        ++i;
    }
    *n = i;
    return XLB_OK;
}

// ------------------------------------------------------------------------------ key-array ops
static Keys rel_packed(xlb_ctx* c, const xlb_rel* r, int fcol, uint32_t fval, Keys* filtered, bool materialize = true) {
    Keys k;
    k.n = r->rows;
    k.bound = r->or_bound;
    if (r->packed) { k.buf = r->packed; return k; }
    if (!rel_packable(r->schema)) xlb_fail(XLB_ERR_UNSUPPORTED, "relation is not a one- or two-column 32-bit relation");
    Buf b = make_buf(c, materialize ? r->rows * 8 : 0);
    if (r->rows) {
        // pack and, in the same sweep, reduce the OR of all rows: later sorts of anything derived
        // from this relation plan their digits from it without a read-back
        Buf oa = make_buf(c, 16);
        CUDA_OK(cudaMemsetAsync(oa->p, 0, 16, c->stream));
        prof_begin(c, "pack", r->rows * (materialize ? 16ull : 8ull));
        const bool fuse = filtered && r->schema.arity == 2 && fcol >= 0 && fcol < 2;
        if (fuse) filtered->buf = make_buf(c, r->rows * 8);  // at most every row; trimmed below
        if (r->schema.arity == 2 && !materialize && (((uintptr_t)r->cols[0]->p | (uintptr_t)r->cols[1]->p) & 15) == 0) {
            cols_or_filter_k<<<grid_for(c, r->rows, BLOCK * 16), BLOCK, 0, c->stream>>>(r->cols[0]->as<uint32_t>(), r->cols[1]->as<uint32_t>(), r->rows, oa->as<unsigned long long>(),
                                                                                         fuse ? fcol : -1, fval, fuse ? filtered->buf->as<uint64_t>() : nullptr,
                                                                                         oa->as<unsigned long long>() + 1);
        } else if (r->schema.arity == 2) {
            const bool vec = (((uintptr_t)r->cols[0]->p | (uintptr_t)r->cols[1]->p | (uintptr_t)b->p) & 15) == 0;
            pack2_k<<<grid_for(c, r->rows, BLOCK * 4), BLOCK, 0, c->stream>>>(r->cols[0]->as<uint32_t>(), r->cols[1]->as<uint32_t>(), materialize ? b->as<uint64_t>() : nullptr, r->rows,
                                                                              oa->as<unsigned long long>(), vec, fuse ? fcol : -1, fval,
                                                                              fuse ? filtered->buf->as<uint64_t>() : nullptr, oa->as<unsigned long long>() + 1);
        }
        else pack1_k<<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(r->cols[0]->as<uint32_t>(), b->as<uint64_t>(), r->rows, oa->as<unsigned long long>());
        check_launch(c, "pack");
        unsigned long long h[2];
        read_words(c, oa->p, 2, h);
        r->or_bound = h[0];
        if (fuse) {
            filtered->n = h[1];
            filtered->bound = h[0];
            if (filtered->n * 2 < r->rows) filtered->buf = ops_slice(c, *filtered, 0, filtered->n).buf;  // give the large buffer back
        }
    } else {
        r->or_bound = 0;
        if (filtered) filtered->buf = make_buf(c, 0);
    }
    if (materialize) r->packed = b;
    k.buf = b;
    k.bound = r->or_bound;
    return k;
}

Keys ops_rel_packed(xlb_ctx* c, const xlb_rel* r) { return rel_packed(c, r, -1, 0, nullptr); }

bool ops_rel_bound_filtered(xlb_ctx* c, const xlb_rel* r, int fcol, uint32_t fval, Keys* filtered) {
    if (r->packed || r->schema.arity != 2 || !rel_packable(r->schema)) return false;
    rel_packed(c, r, fcol, fval, filtered, /*materialize=*/false);
    return true;
}

bool ops_rel_packed_filtered(xlb_ctx* c, const xlb_rel* r, int fcol, uint32_t fval, Keys* filtered) {
    if (r->packed || r->schema.arity != 2 || !rel_packable(r->schema)) return false;
    rel_packed(c, r, fcol, fval, filtered);
    return true;
}

void ops_rel_columns(xlb_ctx* c, const xlb_rel* r) {
    if (r->schema.arity == 0 || r->cols[0]) return;
    for (uint32_t i = 0; i < r->schema.arity; ++i) r->cols[i] = make_buf(c, r->rows * 4);
    if (!r->rows) return;
    prof_begin(c, "unpack", 0);
    if (r->schema.arity == 2) unpack2_k<<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(r->packed->as<uint64_t>(), r->cols[0]->as<uint32_t>(), r->cols[1]->as<uint32_t>(), r->rows);
    else unpack1_k<<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(r->packed->as<uint64_t>(), r->cols[0]->as<uint32_t>(), r->rows);
    check_launch(c, "unpack");
}

xlb_rel* ops_rel_from_keys(xlb_ctx* c, const xlb_schema& s, Keys k, bool canonical) {
    auto* r = new xlb_rel;
    r->ctx = c;
    r->schema = s;
    r->rows = k.n;
    r->packed = k.buf ? k.buf : make_buf(c, 0);
    r->or_bound = k.n ? k.bound : 0;
    r->canonical = canonical;
    return r;
}

Keys ops_copy(xlb_ctx* c, const Keys& in) {
    Keys o;
    o.n = in.n;
    o.bound = in.bound;
    o.buf = make_buf(c, in.n * 8);
    if (in.n) CUDA_OK(cudaMemcpyAsync(o.buf->p, in.buf->p, in.n * 8, cudaMemcpyDeviceToDevice, c->stream));
    return o;
}

Keys ops_from_host(xlb_ctx* c, const uint64_t* rows, uint64_t n) {
    if (n > 16) xlb_fail(XLB_ERR_INVALID, "internal: ops_from_host is for a handful of rows");
    Keys o;
    o.n = n;
    o.bound = 0;
    for (uint64_t i = 0; i < n; ++i) o.bound |= rows[i];
    o.buf = make_buf(c, n * 8);
    for (uint64_t i = 0; i < n; ++i) c->h_scalar[40 + i] = rows[i];  // pinned staging words
    if (n) {
        CUDA_OK(cudaMemcpyAsync(o.buf->p, &c->h_scalar[40], n * 8, cudaMemcpyHostToDevice, c->stream));
        stream_wait(c);  // the staging words are reused by the next call
    }
    return o;
}

Keys ops_slice(xlb_ctx* c, const Keys& in, uint64_t lo, uint64_t hi) {
    Keys o;
    o.n = hi - lo;
    o.bound = in.bound;
    o.buf = make_buf(c, o.n * 8);
    if (o.n) CUDA_OK(cudaMemcpyAsync(o.buf->p, in.ptr() + lo, o.n * 8, cudaMemcpyDeviceToDevice, c->stream));
    return o;
}

Keys ops_concat(xlb_ctx* c, const std::vector<Keys>& parts) {
    Keys o;
    o.bound = 0;
    for (auto& p : parts) {
        o.n += p.n;
        if (p.n) o.bound |= p.bound;
    }
    o.buf = make_buf(c, o.n * 8);
    uint64_t at = 0;
    for (auto& p : parts) {
        if (p.n) CUDA_OK(cudaMemcpyAsync(o.buf->as<uint64_t>() + at, p.buf->p, p.n * 8, cudaMemcpyDeviceToDevice, c->stream));
        at += p.n;
    }
    return o;
}

void ops_sort(xlb_ctx* c, Keys& k, bool keep_input) { radix_sort(c, k.buf, nullptr, k.n, 0xFFu, k.bound, keep_input); }
void ops_sort_by_high_half(xlb_ctx* c, Keys& k, bool keep_input) { radix_sort(c, k.buf, nullptr, k.n, 0xF0u, k.bound, keep_input); }

void ops_dedup_sorted(xlb_ctx* c, Keys& k) {
    if (k.n <= 1) return;
    Buf out = make_buf(c, k.n * 8);
    k.n = dedup_sorted(c, k.ptr(), k.n, out->as<uint64_t>());
    k.buf = out;
}

Keys ops_diff(xlb_ctx* c, const Keys& a, const Keys& b) {
    Keys o;
    o.bound = a.bound;
    o.buf = set_difference(c, a.ptr(), a.n, b.ptr(), b.n, &o.n);
    return o;
}

Keys ops_dedup_diff(xlb_ctx* c, const Keys& a, const Keys& b) {
    Keys o;
    o.bound = a.bound;
    o.buf = set_difference(c, a.ptr(), a.n, b.ptr(), b.n, &o.n, true);
    return o;
}

static int bit_length(uint64_t v) { return v ? 64 - __builtin_clzll(v) : 0; }

bool ops_dense_bits(const Keys& a, const Keys& b, int* hi_bits, int* lo_bits, int max_bits) {
    uint64_t ba = a.n ? a.bound : 0, bb = b.n ? b.bound : 0;
    if (ba == ~0ull || bb == ~0ull) return false;  // bits unknown
    uint64_t all = ba | bb;
    *hi_bits = bit_length(all >> 32);
    *lo_bits = bit_length(all & 0xFFFFFFFFull);
    return *hi_bits + *lo_bits <= max_bits && *hi_bits + *lo_bits >= 1;
}

DenseSet ops_dense_begin(xlb_ctx* c, int hi_bits, int lo_bits) {
    DenseSet d;
    d.hi_bits = hi_bits;
    d.lo_bits = lo_bits;
    d.words = ((1ull << (hi_bits + lo_bits)) + 31) / 32;
    const uint64_t bitmap_bytes = (d.words * 4 + 7) & ~7ull;
    d.bitmap = make_buf(c, bitmap_bytes + 24);
    d.counts = (uint64_t*)((char*)d.bitmap->p + bitmap_bytes);
    CUDA_OK(cudaMemsetAsync(d.bitmap->p, 0, bitmap_bytes + 24, c->stream));
    return d;
}

DenseSet ops_dense_begin_from(xlb_ctx* c, int hi_bits, int lo_bits, unsigned int* visited) {
    DenseSet d;
    d.hi_bits = hi_bits;
    d.lo_bits = lo_bits;
    d.words = ((1ull << (hi_bits + lo_bits)) + 31) / 32;
    const uint64_t bitmap_bytes = (d.words * 4 + 7) & ~7ull;
    d.bitmap = make_buf(c, bitmap_bytes + 24);
    d.counts = (uint64_t*)((char*)d.bitmap->p + bitmap_bytes);
    CUDA_OK(cudaMemcpyAsync(d.bitmap->p, visited, d.words * 4, cudaMemcpyDeviceToDevice, c->stream));
    CUDA_OK(cudaMemsetAsync((char*)d.bitmap->p + d.words * 4, 0, bitmap_bytes + 24 - d.words * 4, c->stream));
    d.visited = visited;
    d.seeded = true;
    return d;
}

constexpr uint64_t DENSE_WIDE_WORDS = 1ull << 20;  // bitmaps from this size on are counted and emitted by the wide kernels

DenseSet ops_dense_begin_state(xlb_ctx* c, DenseState& s) {
    if (!s.marks) return ops_dense_begin_from(c, s.hi_bits, s.lo_bits, s.visited->as<unsigned int>());
    DenseSet d;
    d.hi_bits = s.hi_bits;
    d.lo_bits = s.lo_bits;
    d.words = s.words;
    d.bitmap = s.marks;
    d.counts_buf = make_buf(c, 24);
    d.counts = d.counts_buf->as<uint64_t>();
    CUDA_OK(cudaMemsetAsync(d.counts_buf->p, 0, 24, c->stream));
    CUDA_OK(cudaMemsetAsync(s.touched->p, 0, s.touched->bytes, c->stream));
    d.touched = s.touched->as<unsigned char>();
    d.visited = s.visited->as<unsigned int>();
    d.seeded = true;
    return d;
}

static Keys dense_finish(xlb_ctx* c, DenseSet& d, const Keys& full, const uint64_t* known_total);
Keys ops_dense_finish(xlb_ctx* c, DenseSet& d, const Keys& full) { return dense_finish(c, d, full, nullptr); }

// known_total: the number of rows that will come out, when the host knows it already (no read-back)
static Keys dense_finish(xlb_ctx* c, DenseSet& d, const Keys& full, const uint64_t* known_total) {
    Keys o;
    o.bound = d.bound;
    const uint64_t words = d.words;
    if (full.n && !d.visited) {
        prof_begin(c, "dense_clear", full.n * 8ull);
        dense_mark_k<false><<<grid_for(c, full.n), BLOCK, 0, c->stream>>>(full.ptr(), full.n, d.lo_bits, d.bitmap->as<unsigned int>(), words, c->d_status);
        check_launch(c, "dense_clear");
    }
    // a bitmap of a million words and more is counted and emitted in groups of 256 words per warp
    const bool wide = words >= DENSE_WIDE_WORDS && words % (32 * DW_WPL) == 0 && ((uintptr_t)d.bitmap->p & 15) == 0 && (!d.visited || ((uintptr_t)d.visited & 15) == 0);
    uint64_t groups = wide ? words / (32 * DW_WPL) : (words + 31) / 32;
    Buf gcnt = make_buf(c, groups * 4);
    Buf offs = make_buf(c, groups * 8);
    prof_begin(c, "dense_count", words * 4ull);
    if (wide) {
        dense_count_wide_k<<<(unsigned)((groups * 32 + BLOCK - 1) / BLOCK), BLOCK, 0, c->stream>>>(d.bitmap->as<unsigned int>(), gcnt->as<uint32_t>(), groups, d.visited, d.touched);
        check_launch(c, "dense_count");
        exclusive_scan<LoadU32, uint64_t>(c, LoadU32{gcnt->as<uint32_t>()}, groups, offs->as<uint64_t>(), d.counts);
    } else if (groups <= (uint64_t)DENSE_FUSED_GROUPS) {
        dense_count_scan_k<<<(unsigned)((groups * 32 + BLOCK - 1) / BLOCK), BLOCK, 0, c->stream>>>(d.bitmap->as<unsigned int>(), words, gcnt->as<uint32_t>(), groups, d.visited,
                                                                                                  offs->as<uint64_t>(), d.counts, (unsigned int*)(d.counts + 2));
        check_launch(c, "dense_count");
    } else {
        dense_count_k<<<(unsigned)((groups * 32 + BLOCK - 1) / BLOCK), BLOCK, 0, c->stream>>>(d.bitmap->as<unsigned int>(), words, gcnt->as<uint32_t>(), groups, d.visited);
        check_launch(c, "dense_count");
        exclusive_scan<LoadU32, uint64_t>(c, LoadU32{gcnt->as<uint32_t>()}, groups, offs->as<uint64_t>(), d.counts);
    }
    unsigned long long both[2] = {known_total ? *known_total : 0ull, 0ull};
    if (!known_total) read_words(c, d.counts, 2, both);
    else {
        verify_count_k<<<1, 1, 0, c->stream>>>(d.counts, *known_total, c->d_status);  // a mismatch surfaces as an error at the next status check
        check_launch(c, "verify_count");
    }
    const uint64_t tot = both[0];
    d.marked = both[1];
    prof_add_bytes(c, "expand_mark", d.marked * 4ull);
    o.n = tot;
    o.buf = make_buf(c, tot * 8);
    if (tot) {
        prof_begin(c, "dense_emit", words * 4ull + tot * 8ull);
        if (wide)
            dense_emit_wide_k<<<(unsigned)((groups * 32 + BLOCK - 1) / BLOCK), BLOCK, 0, c->stream>>>(d.bitmap->as<unsigned int>(), offs->as<uint64_t>(), groups, d.lo_bits, o.buf->as<uint64_t>(),
                                                                                                    d.visited, tot, c->d_status, d.touched);
        else
            dense_emit_k<<<(unsigned)((groups * 32 + BLOCK - 1) / BLOCK), BLOCK, 0, c->stream>>>(d.bitmap->as<unsigned int>(), words, offs->as<uint64_t>(), groups, d.lo_bits, o.buf->as<uint64_t>(), d.visited, tot, c->d_status);
        check_launch(c, "dense_emit");
    }
    return o;
}

void ops_dense_state_build(xlb_ctx* c, DenseState& s, int hi_bits, int lo_bits, const Keys& full, const Keys& novel) {
    s.hi_bits = hi_bits;
    s.lo_bits = lo_bits;
    s.words = ((1ull << (hi_bits + lo_bits)) + 31) / 32;
    s.visited = make_buf(c, s.words * 4);
    CUDA_OK(cudaMemsetAsync(s.visited->p, 0, s.words * 4, c->stream));
    for (const Keys* k : {&full, &novel}) {
        if (!k->n) continue;
        prof_begin(c, "dense_mark", k->n * 8ull);
        dense_mark_k<true><<<grid_for(c, k->n), BLOCK, 0, c->stream>>>(k->ptr(), k->n, lo_bits, s.visited->as<unsigned int>(), s.words, c->d_status);
        check_launch(c, "dense_mark");
    }
    s.marks = nullptr;
    s.touched = nullptr;
    if (s.words >= DENSE_WIDE_WORDS && s.words % (32 * DW_WPL) == 0) {
        s.marks = make_buf(c, s.words * 4);
        CUDA_OK(cudaMemcpyAsync(s.marks->p, s.visited->p, s.words * 4, cudaMemcpyDeviceToDevice, c->stream));
        s.touched = make_buf(c, s.words / (32 * DW_WPL));
    }
    s.rows = full.n + novel.n;
    s.valid = true;
}

Keys ops_dense_state_rows(xlb_ctx* c, const DenseState& s, uint64_t bound) {
    DenseSet d;
    d.hi_bits = s.hi_bits;
    d.lo_bits = s.lo_bits;
    d.words = s.words;
    d.bitmap = s.visited;
    d.bound = bound;
    Buf counts = make_buf(c, 24);
    CUDA_OK(cudaMemsetAsync(counts->p, 0, 24, c->stream));
    d.counts = counts->as<uint64_t>();
    Keys none;
    return dense_finish(c, d, none, &s.rows);  // nothing to subtract, no second bitmap: every set bit comes out, s.rows of them
}

static void tuple_set_alloc(xlb_ctx* c, TupleSet& s, uint64_t tuples) {
    s.log2cap = 10;
    while ((1ull << s.log2cap) < 2 * tuples) ++s.log2cap;
    s.cap = 1ull << s.log2cap;
    s.table = make_buf(c, s.cap * 8 + 8);
    CUDA_OK(cudaMemsetAsync(s.table->p, 0xFF, s.cap * 8, c->stream));
    CUDA_OK(cudaMemsetAsync((char*)s.table->p + s.cap * 8, 0, 8, c->stream));
}

static unsigned int* tuple_set_flag(const TupleSet& s) { return (unsigned int*)((char*)s.table->p + s.cap * 8); }

// mix64 of every key (or its inverse), into a fresh buffer
static Buf mixed_copy(xlb_ctx* c, const uint64_t* in, uint64_t n, bool inverse) {
    Buf out = make_buf(c, n * 8);
    if (n) {
        prof_begin(c, "mix", n * 16ull);
        mix_k<<<grid_for(c, n, BLOCK * 4), BLOCK, 0, c->stream>>>(in, out->as<uint64_t>(), n, inverse ? 1 : 0);
        check_launch(c, "mix");
    }
    return out;
}

// The candidates as mixed words, grouped by the top byte (= by the 256th of the table they fall into)
// when there are enough of them for the grouping pass to pay.
static Buf tuple_set_words(xlb_ctx* c, const TupleSet& s, const uint64_t* keys, uint64_t n) {
    const bool table_in_l2 = s.cap * 8 <= (48ull << 20);  // then any order of insertion is an L2 access
    if (!table_in_l2 && n >= (1ull << 20) && n < (1ull << 30)) return mix_and_group(c, keys, n);
    return mixed_copy(c, keys, n, false);
}

static void tuple_set_fill(xlb_ctx* c, TupleSet& s, const uint64_t* words, uint64_t n, bool skip_empty) {
    if (!n) return;
    prof_begin(c, "hset_fill", n * 16ull);
    hset_fill_k<<<grid_for(c, n), BLOCK, 0, c->stream>>>(words, n, s.table->as<unsigned long long>(), 64 - s.log2cap, s.cap - 1, tuple_set_flag(s), skip_empty, c->d_status);
    check_launch(c, "hset_fill");
}

void ops_tuple_set_build(xlb_ctx* c, TupleSet& s, const Keys& full, const Keys& novel, uint64_t extra) {
    s.table.reset();
    tuple_set_alloc(c, s, full.n + novel.n + extra);
    for (const Keys* k : {&full, &novel}) {
        if (!k->n) continue;
        Buf words = tuple_set_words(c, s, k->ptr(), k->n);
        tuple_set_fill(c, s, words->as<uint64_t>(), k->n, false);
    }
    s.rows = full.n + novel.n;
    s.valid = true;
}

Keys ops_tuple_set_novel(xlb_ctx* c, TupleSet& s, const Keys& cand) {
    Keys o;
    o.bound = cand.bound;
    if (cand.n == 0) {
        o.buf = make_buf(c, 0);
        return o;
    }
    if (2 * (s.rows + cand.n) > s.cap) {
        // every candidate could be new: grow (to twice what is needed, so that this is rare) and
        // move the stored words over, straight from the old table (in slot order, which is the new
        // table's order too: the insertions walk through it front to back)
        TupleSet old = s;
        const uint64_t need = s.rows + cand.n;
        tuple_set_alloc(c, s, need < (1ull << 27) ? 2 * need : need);  // (a table of gigabytes grows to what is needed only)
        tuple_set_fill(c, s, old.table->as<uint64_t>(), old.cap, true);
        CUDA_OK(cudaMemcpyAsync(tuple_set_flag(s), tuple_set_flag(old), 4, cudaMemcpyDeviceToDevice, c->stream));
    }
    Buf words = tuple_set_words(c, s, cand.ptr(), cand.n);
    Buf out = make_buf(c, cand.n * 8);
    o.n = select_unordered(c, PredInsert{words->as<uint64_t>(), s.table->as<unsigned long long>(), 64 - s.log2cap, s.cap - 1, tuple_set_flag(s), c->d_status},
                           EmitKey{words->as<uint64_t>(), out->as<uint64_t>()}, cand.n, "hset_insert", cand.n * 16ull);
    s.rows += o.n;
    words.reset();
    o.buf = mixed_copy(c, out->as<uint64_t>(), o.n, true);  // back to tuples, in a buffer of their own size
    return o;
}

Keys ops_dense_novel(xlb_ctx* c, const Keys& cand, const Keys& full, int hi_bits, int lo_bits, unsigned int* visited) {
    DenseSet d = ops_dense_begin(c, hi_bits, lo_bits);
    d.bound = cand.bound;
    d.visited = visited;
    if (cand.n) {
        prof_begin(c, "dense_mark", cand.n * 8ull);
        dense_mark_k<true><<<grid_for(c, cand.n), BLOCK, 0, c->stream>>>(cand.ptr(), cand.n, lo_bits, d.bitmap->as<unsigned int>(), d.words, c->d_status, visited);
        check_launch(c, "dense_mark");
    }
    Keys none;
    return ops_dense_finish(c, d, cand.n ? full : none);
}

void ops_dense_mark_into(xlb_ctx* c, DenseSet& d, const Keys& cand) {
    if (cand.n == 0) return;
    d.bound |= cand.bound;
    prof_begin(c, "dense_mark", cand.n * 8ull);
    dense_mark_k<true><<<grid_for(c, cand.n), BLOCK, 0, c->stream>>>(cand.ptr(), cand.n, d.lo_bits, d.bitmap->as<unsigned int>(), d.words, c->d_status, d.seeded ? nullptr : d.visited, d.touched);
    check_launch(c, "dense_mark");
}

Keys ops_filter_owner(xlb_ctx* c, const Keys& in, int keysel, uint32_t world, uint32_t rank) {
    Keys o;
    o.bound = in.bound;
    o.buf = make_buf(c, in.n * 8);
    o.n = select(c, PredOwner{in.ptr(), keysel == SRC_HI ? 0 : 1, world, rank}, EmitKey{in.ptr(), o.buf->as<uint64_t>()}, in.n);
    return o;
}

Keys ops_merge_disjoint(xlb_ctx* c, const Keys& a, const Keys& b) {
    Keys o;
    o.bound = (a.n ? a.bound : 0) | (b.n ? b.bound : 0);
    o.n = a.n + b.n;
    o.buf = merge_disjoint(c, a.ptr(), a.n, b.ptr(), b.n);
    return o;
}

Keys ops_union(xlb_ctx* c, const Keys& a, const Keys& b) {
    if (b.n == 0) return a;
    if (a.n == 0) return b;
    const Keys& small = a.n <= b.n ? a : b;
    const Keys& big = a.n <= b.n ? b : a;
    Keys extra = ops_diff(c, small, big);
    return ops_merge_disjoint(c, big, extra);
}

static uint64_t half_bound(uint64_t bound, int src, uint64_t other) {
    if (bound == ~0ull && src != SRC_OTHER && src != SRC_ZERO) return 0xFFFFFFFFull;
    return src == SRC_HI ? (bound >> 32) : src == SRC_LO ? (bound & 0xFFFFFFFFull) : src == SRC_OTHER ? other : 0;
}

Keys ops_remap(xlb_ctx* c, const Keys& in, int hi_src, int lo_src) {
    Keys o;
    o.n = in.n;
    o.bound = (half_bound(in.bound, hi_src, 0) << 32) | half_bound(in.bound, lo_src, 0);
    o.buf = make_buf(c, in.n * 8);
    if (in.n) {
        prof_begin(c, "remap", 0);
        remap_k<<<grid_for(c, in.n), BLOCK, 0, c->stream>>>(in.ptr(), o.buf->as<uint64_t>(), in.n, hi_src == SRC_ZERO ? 2 : hi_src, lo_src == SRC_ZERO ? 2 : lo_src);
        check_launch(c, "remap");
    }
    return o;
}

Keys ops_filter(xlb_ctx* c, const Keys& in, uint32_t cmp, int lhs_src, bool rhs_is_const, uint64_t rhs) {
    Keys o;
    o.bound = in.bound;
    o.buf = make_buf(c, in.n * 8);
    o.n = select_unordered(c, PredCmp{in.ptr(), cmp, lhs_src, rhs_is_const, rhs}, EmitKey{in.ptr(), o.buf->as<uint64_t>()}, in.n);  // a bag: any order
    return o;
}

Index ops_index_build(xlb_ctx* c, Buf S, uint64_t n, int key_shift, Buf pay) {
    Index ix;
    ix.S = S;
    ix.pay = pay;
    ix.n = n;
    ix.key_shift = key_shift;
    if (n >= 0xFFFFFFFFull) xlb_fail(XLB_ERR_CAPACITY, "join build side of %llu rows exceeds the 2^32 - 1 row limit", (unsigned long long)n);
    Buf starts = make_buf(c, (n + 1) * 4);
    uint64_t nu = 0;
    if (n) {
        if (key_shift == 32) nu = select(c, PredRunHead{S->as<uint64_t>()}, EmitRunHead{starts->as<uint32_t>()}, n);
        else nu = select(c, PredHead{S->as<uint64_t>()}, EmitRunHead{starts->as<uint32_t>()}, n);
    }
    ix.nkeys = nu;
    uint64_t cap = 1024;
    while (cap < 2 * nu) cap <<= 1;
    ix.mask = cap - 1;
    ix.table = make_buf(c, cap * 16);
    CUDA_OK(cudaMemsetAsync(ix.table->p, 0, cap * 16, c->stream));
    if (nu) {
        prof_begin(c, "hash_insert", 0);
        hash_insert_k<<<grid_for(c, nu), BLOCK, 0, c->stream>>>(S->as<uint64_t>(), n, key_shift, starts->as<uint32_t>(), nu, ix.table->as<ulonglong2>(), ix.mask, c->d_status);
        check_launch(c, "hash_insert");
    }
    return ix;
}

Index ops_index_build_direct(xlb_ctx* c, const Keys& rows, int keysel, int key_bits) {
    Index ix;
    ix.n = rows.n;
    if (rows.n >= 0xFFFFFFFFull) xlb_fail(XLB_ERR_CAPACITY, "join build side of %llu rows exceeds the 2^32 - 1 row limit", (unsigned long long)rows.n);
    ix.domain = 1ull << key_bits;
    ix.bound = rows.bound;
    const uint64_t other = keysel == SRC_HI ? (rows.bound & 0xFFFFFFFFull) : (rows.bound >> 32);
    ix.pay_bound = rows.bound == ~0ull ? 0xFFFFFFFFull : other;
    Buf cnt = make_buf(c, ix.domain * 4);
    CUDA_OK(cudaMemsetAsync(cnt->p, 0, ix.domain * 4, c->stream));
    ix.cursor = make_buf(c, ix.domain * 8);
    ix.pay = make_buf(c, rows.n * 4);
    Buf total = make_buf(c, 8);
    if (rows.n) {
        prof_begin(c, "direct_count", rows.n * 8ull);
        direct_count_k<<<grid_for(c, rows.n, DX_TILE), BLOCK, 0, c->stream>>>(rows.ptr(), rows.n, keysel, cnt->as<unsigned int>(), ix.domain, c->d_status);
        check_launch(c, "direct_count");
    }
    exclusive_scan<LoadU32, uint64_t>(c, LoadU32{cnt->as<uint32_t>()}, ix.domain, ix.cursor->as<uint64_t>(), total->as<uint64_t>());
    if (rows.n) {
        prof_begin(c, "direct_fill", rows.n * 12ull);
        direct_fill_k<<<grid_for(c, rows.n, DX_TILE), BLOCK, 0, c->stream>>>(rows.ptr(), rows.n, keysel, ix.cursor->as<unsigned long long>(), ix.domain, ix.pay->as<uint32_t>());
        check_launch(c, "direct_fill");
    }
    return ix;
}

Buf ops_probe_match(xlb_ctx* c, const Keys& bag, int keysel, const uint64_t* pkeys, const Index& ix) {
    Buf match = make_buf(c, bag.n * 8);
    if (bag.n && ix.cursor) {
        prof_begin(c, "direct_probe", bag.n * 32ull);
        if (pkeys) direct_probe_k<LoadKey64><<<grid_for(c, bag.n), BLOCK, 0, c->stream>>>(LoadKey64{pkeys}, bag.n, ix.cursor->as<unsigned long long>(), ix.domain, match->as<uint64_t>());
        else direct_probe_k<LoadKeyHalf><<<grid_for(c, bag.n), BLOCK, 0, c->stream>>>(LoadKeyHalf{bag.ptr(), keysel}, bag.n, ix.cursor->as<unsigned long long>(), ix.domain, match->as<uint64_t>());
        check_launch(c, "direct_probe");
    } else if (bag.n) {
        prof_begin(c, "hash_probe", bag.n * 32ull);
        if (pkeys) hash_probe_k<LoadKey64><<<grid_for(c, bag.n), BLOCK, 0, c->stream>>>(LoadKey64{pkeys}, bag.n, ix.table->as<ulonglong2>(), ix.mask, match->as<uint64_t>());
        else hash_probe_k<LoadKeyHalf><<<grid_for(c, bag.n), BLOCK, 0, c->stream>>>(LoadKeyHalf{bag.ptr(), keysel}, bag.n, ix.table->as<ulonglong2>(), ix.mask, match->as<uint64_t>());
        check_launch(c, "hash_probe");
    }
    return match;
}

uint64_t ops_scan_join_bound(const Keys& bag, int keysel, const Keys& rel, int rel_keysel, int rel_hi, int rel_lo) {
    const uint64_t kb = half_bound(bag.bound, keysel, 0) & half_bound(rel.bound, rel_keysel, 0);  // a produced key is in both
    const uint64_t ob = half_bound(rel.bound, rel_keysel == SRC_HI ? SRC_LO : SRC_HI, 0);
    auto pick = [&](int src) { return src == 0 ? kb : src == 1 ? ob : 0ull; };
    return (pick(rel_hi) << 32) | pick(rel_lo);
}

Buf ops_keyset(xlb_ctx* c, const Keys& bag, int keysel, int key_bits) {
    const uint64_t domain = 1ull << key_bits;
    const uint64_t bytes = std::max<uint64_t>(domain / 8, 16);  // whole 16-byte words: the streaming kernel copies it that way
    Buf keyset = make_buf(c, bytes);
    CUDA_OK(cudaMemsetAsync(keyset->p, 0, bytes, c->stream));
    if (bag.n) {
        prof_begin(c, "keyset_mark", bag.n * 8ull);
        keyset_mark_k<<<grid_for(c, bag.n), BLOCK, 0, c->stream>>>(bag.ptr(), bag.n, keysel, keyset->as<unsigned int>(), domain, c->d_status);
        check_launch(c, "keyset_mark");
    }
    return keyset;
}

Keys ops_scan_join(xlb_ctx* c, const Keys& bag, int keysel, int key_bits, const Keys& rel, int rel_keysel, int rel_hi, int rel_lo) {
    Keys o;
    o.bound = ops_scan_join_bound(bag, keysel, rel, rel_keysel, rel_hi, rel_lo);
    if (bag.n == 0 || rel.n == 0) {
        o.buf = make_buf(c, 0);
        return o;
    }
    Buf keyset = ops_keyset(c, bag, keysel, key_bits);
    // the output is at most the relation
    Buf out = make_buf(c, rel.n * 8);
    o.n = select_unordered(c, PredKeyIn{rel.ptr(), rel_keysel, keyset->as<unsigned int>(), 1ull << key_bits}, EmitScanRow{rel.ptr(), rel_keysel, rel_hi, rel_lo, out->as<uint64_t>()}, rel.n);
    if (o.n * 2 < rel.n) {  // give the large buffer back
        Keys full;
        full.buf = out;
        full.n = o.n;
        o.buf = ops_slice(c, full, 0, o.n).buf;
    } else o.buf = out;
    return o;
}

void ops_scan_join_mark(xlb_ctx* c, const Keys& bag, int keysel, int key_bits, const Keys& rel, int rel_keysel, int rel_hi, int rel_lo, DenseSet& d) {
    d.bound |= ops_scan_join_bound(bag, keysel, rel, rel_keysel, rel_hi, rel_lo);
    if (bag.n == 0 || rel.n == 0) return;
    Buf keyset = ops_keyset(c, bag, keysel, key_bits);
    prof_begin(c, "scan_join_mark", rel.n * 8ull);
    if ((uintptr_t)rel.ptr() & 15) xlb_fail(XLB_ERR_INVALID, "internal: scan join over a row array that is not 16-byte aligned");
    scan_join_mark_k<<<grid_for(c, rel.n, SJ_TILE), BLOCK, 0, c->stream>>>(rel.ptr(), rel.n, rel_keysel, keyset->as<unsigned int>(), 1ull << key_bits, rel_hi, rel_lo,
                                                                  d.bitmap->as<unsigned int>(), d.words, d.lo_bits, (unsigned long long*)(d.counts + 1), c->d_status, d.seeded ? nullptr : d.visited, nullptr, d.touched);
    check_launch(c, "scan_join_mark");
}

void ops_frontier_scan(xlb_ctx* c, const ScanRows& src, int rel_keysel, int bits, const unsigned int* frontier, int rel_lo, unsigned int* marks, const unsigned int* visited,
                       unsigned long long* count_marked, const unsigned long long* keys_in_frontier, uint64_t* live_out, unsigned long long* live_count) {
    if (src.n_max == 0) return;
    const bool cols = src.packed == nullptr;
    if (cols ? (((uintptr_t)src.kcol | (uintptr_t)src.ocol) & 15) != 0 : ((uintptr_t)src.packed & 15) != 0)
        xlb_fail(XLB_ERR_INVALID, "internal: frontier scan over rows that are not 16-byte aligned");
    const uint64_t domain = 1ull << bits, words = (domain + 31) / 32;
    // how many rows a launch streams over, and how many it writes back, is known only once its
    // counts have been read: the caller adds the bytes then
    prof_begin(c, "scan_join_mark", 0);
    const unsigned grid = grid_for(c, src.n_max, FS_TILE);
    if (cols)
        frontier_scan_k<true><<<grid, BLOCK, 0, c->stream>>>(nullptr, src.kcol, src.ocol, src.n_max, src.n_dev, rel_keysel, frontier, visited, domain, rel_lo == 0, marks, words, bits,
                                                             count_marked, c->d_status, keys_in_frontier, live_out, live_count);
    else
        frontier_scan_k<false><<<grid, BLOCK, 0, c->stream>>>(src.packed, nullptr, nullptr, src.n_max, src.n_dev, rel_keysel, frontier, visited, domain, rel_lo == 0, marks, words, bits,
                                                              count_marked, c->d_status, keys_in_frontier, live_out, live_count);
    check_launch(c, "scan_join_mark");
}

void ops_frontier_step(xlb_ctx* c, const unsigned int* mark_parts, uint32_t parts, uint64_t words, unsigned int* own, unsigned int* visited, unsigned int* next_frontier,
                       unsigned long long* counts, unsigned int* ticket, unsigned long long* publish_to, unsigned long long seq) {
    prof_begin(c, "frontier_step", words * 4ull * (parts + 3));
    frontier_step_k<<<grid_for(c, words), BLOCK, 0, c->stream>>>(mark_parts, parts, words, own, visited, next_frontier, counts, ticket, publish_to, seq);
    check_launch(c, "frontier_step");
}

Keys ops_semi_filter(xlb_ctx* c, const Keys& bag, int keysel, const Index& ix, bool anti, const uint64_t* pkeys) {
    Keys o;
    o.bound = bag.bound;
    o.buf = make_buf(c, bag.n * 8);
    if (bag.n == 0) return o;
    if (ix.n == 0) return anti ? ops_copy(c, bag) : o;
    Buf match = ops_probe_match(c, bag, keysel, pkeys, ix);
    o.n = select(c, PredFlag{match->as<uint64_t>(), !anti}, EmitKey{bag.ptr(), o.buf->as<uint64_t>()}, bag.n);
    return o;
}

uint64_t ops_expand_bound(const Keys& bag, const Index& ix, int hi_src, int lo_src) {
    uint64_t other_bound = ix.pay ? ix.pay_bound : (ix.bound == ~0ull ? 0xFFFFFFFFull : (ix.bound & 0xFFFFFFFFull));
    return (half_bound(bag.bound, hi_src, other_bound) << 32) | half_bound(bag.bound, lo_src, other_bound);
}

// Probe, prefix-sum the match lengths over all probe rows (rows without a match keep length 0),
// then a load-balanced expansion: one count read-back per join step.  With `dense` the output
// tuples are marked in its bitmap and no list is produced.
static Keys join_expand(xlb_ctx* c, const Keys& bag, int keysel, const uint64_t* pkeys, const Index& ix, int hi_src, int lo_src, DenseSet* dense) {
    Keys out;
    out.bound = ops_expand_bound(bag, ix, hi_src, lo_src);
    if (bag.n == 0 || ix.n == 0) { out.buf = make_buf(c, 0); return out; }
    Buf match = ops_probe_match(c, bag, keysel, pkeys, ix);
    Buf off = make_buf(c, bag.n * 8);
    const uint32_t* pay = ix.pay ? ix.pay->as<uint32_t>() : nullptr;
    if (dense) {
        // Nothing is allocated by the count, so it stays on the device: a fixed grid walks the
        // tiles and the host reads the count later, together with the bitmap's.
        // (one marking join per DenseSet: the scan leaves its total in the set's count word)
        Buf own_total = dense->shared ? make_buf(c, 8) : Buf();
        uint64_t* total_dev = dense->shared ? own_total->as<uint64_t>() : dense->counts + 1;
        exclusive_scan<LoadLow32, uint64_t>(c, LoadLow32{match->as<uint64_t>()}, bag.n, off->as<uint64_t>(), total_dev);
        const unsigned grid = (unsigned)c->sm_count * 8;
        prof_begin(c, "expand_mark", bag.n * 24ull);
        expand_k<true><<<grid, BLOCK, 0, c->stream>>>(bag.ptr(), match->as<uint64_t>(), off->as<uint64_t>(), bag.n, 0, ix.S ? ix.S->as<uint64_t>() : nullptr, pay, hi_src, lo_src,
                                                       nullptr, dense->bitmap->as<unsigned int>(), dense->words, dense->lo_bits, c->d_status, total_dev, dense->seeded ? nullptr : dense->visited, dense->touched);
        check_launch(c, "expand_mark");
        if (dense->shared) {
            add_word_k<<<1, 1, 0, c->stream>>>((unsigned long long*)(dense->counts + 1), (const unsigned long long*)total_dev);
            check_launch(c, "add_word");
        }
        dense->bound |= out.bound;
        return out;
    }
    Buf total = make_buf(c, 8);
    exclusive_scan<LoadLow32, uint64_t>(c, LoadLow32{match->as<uint64_t>()}, bag.n, off->as<uint64_t>(), total->as<uint64_t>());
    unsigned long long tot;
    read_words(c, total->p, 1, &tot);
    out.n = tot;
    out.buf = make_buf(c, tot * 8);
    if (tot == 0) return out;
    uint64_t ntiles = (tot + EX_TILE - 1) / EX_TILE;
    prof_begin(c, "expand", tot * 12ull + bag.n * 24ull);
    expand_k<false><<<(unsigned)ntiles, BLOCK, 0, c->stream>>>(bag.ptr(), match->as<uint64_t>(), off->as<uint64_t>(), bag.n, tot, ix.S ? ix.S->as<uint64_t>() : nullptr, pay, hi_src, lo_src,
                                                                out.buf->as<uint64_t>(), nullptr, 0, 0, c->d_status, nullptr, nullptr, nullptr);
    check_launch(c, "expand");
    return out;
}

Keys ops_join_expand(xlb_ctx* c, const Keys& bag, int keysel, const uint64_t* pkeys, const Index& ix, int hi_src, int lo_src) {
    return join_expand(c, bag, keysel, pkeys, ix, hi_src, lo_src, nullptr);
}

void ops_join_expand_mark(xlb_ctx* c, const Keys& bag, int keysel, const Index& ix, int hi_src, int lo_src, DenseSet& d) {
    join_expand(c, bag, keysel, nullptr, ix, hi_src, lo_src, &d);
}

Keys ops_partition_by_owner_dev(xlb_ctx* c, const Keys& in, int keysel, uint32_t world, unsigned long long* counts) {
    Keys out;
    out.bound = in.bound;
    out.n = in.n;
    out.buf = make_buf(c, in.n * 8);
    if (world > 64) xlb_fail(XLB_ERR_UNSUPPORTED, "at most 64 ranks");
    CUDA_OK(cudaMemsetAsync(counts, 0, (size_t)world * 8, c->stream));
    if (in.n == 0) return out;
    Buf cur = make_buf(c, 64 * 8);
    unsigned long long* cursors = cur->as<unsigned long long>();
    unsigned grid = (unsigned)((in.n + BLOCK * OWN_IPT - 1) / (BLOCK * OWN_IPT));
    prof_begin(c, "owner_count", in.n * 8ull);
    owner_count_k<<<grid, BLOCK, 0, c->stream>>>(in.ptr(), in.n, keysel, world, counts);
    check_launch(c, "owner_count");
    prof_begin(c, "owner_starts", 0);
    owner_starts_k<<<1, 32, 0, c->stream>>>(counts, world, cursors);
    check_launch(c, "owner_starts");
    prof_begin(c, "owner_scatter", in.n * 16ull);
    owner_scatter_k<<<grid, BLOCK, 0, c->stream>>>(in.ptr(), in.n, keysel, world, cursors, out.buf->as<uint64_t>());
    check_launch(c, "owner_scatter");
    return out;
}

// ------------------------------------------------------------------------------ C ABI: context
#define API_BEGIN(ctxp) \
    xlb_ctx* ctx__ = (ctxp); \
    try {                    \
        if (ctx__) CUDA_OK(cudaSetDevice(ctx__->device));
#define API_END()                                  \
    }                                              \
    catch (const XlbError& e) {                    \
        if (ctx__) ctx__->last_error = e.msg;      \
        return e.st;                               \
    }                                              \
    catch (const std::bad_alloc&) {                \
        if (ctx__) ctx__->last_error = "host allocation failed"; \
        return XLB_ERR_RESOURCE_EXHAUSTED;         \
    }                                              \
    return XLB_OK;

static thread_local std::string g_create_error;

extern "C" xlb_status xlb_ctx_create(const xlb_config* cfg, xlb_ctx** out) {
    if (!out) return XLB_ERR_INVALID;
    xlb_ctx* c = nullptr;
    try {
        int ndev = 0;
        cudaError_t e = cudaGetDeviceCount(&ndev);
        if (e != cudaSuccess || ndev == 0)
            xlb_fail(XLB_ERR_CUDA, "no CUDA device: %s (this library has no CPU path)", cudaGetErrorString(e));
        c = new xlb_ctx;
        int dev = cfg ? cfg->device : -1;
        if (dev < 0) CUDA_OK(cudaGetDevice(&dev));
        if (dev >= ndev) xlb_fail(XLB_ERR_INVALID, "device %d out of range (%d devices)", dev, ndev);
        c->device = dev;
        CUDA_OK(cudaSetDevice(dev));
        CUDA_OK(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        c->arena.device = dev;
        size_t fr = 0, tot = 0;
        CUDA_OK(cudaMemGetInfo(&fr, &tot));
        c->budget = cfg && cfg->memory_budget_bytes ? cfg->memory_budget_bytes : (uint64_t)(fr * 0.9);
        c->max_iterations = cfg && cfg->max_iterations ? cfg->max_iterations : 1000000ull;
        c->join_chunk = cfg ? cfg->join_chunk_tuples : 0;
        c->flags = cfg ? cfg->flags : 0;
        CUDA_OK(cudaHostAlloc((void**)&c->h_scalar, 64 * 8, cudaHostAllocMapped));
        CUDA_OK(cudaHostGetDevicePointer((void**)&c->h_scalar_dev, c->h_scalar, 0));
        memset(c->h_scalar, 0, 64 * 8);
        CUDA_OK(cudaMalloc(&c->d_status, sizeof(DevStatus)));
        CUDA_OK(cudaMemset(c->d_status, 0, sizeof(DevStatus)));
        cudaDeviceProp prop;
        CUDA_OK(cudaGetDeviceProperties(&prop, dev));
        c->sm_count = prop.multiProcessorCount;
        *out = c;
    } catch (const XlbError& e) {
        g_create_error = e.msg;
        delete c;
        return e.st;
    }
    return XLB_OK;
}

void xlb_exec_teardown(xlb_ctx* c);  // xlb_exec.cu: store, indexes, communicator

extern "C" void xlb_ctx_destroy(xlb_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    xlb_exec_teardown(c);
    cudaStreamSynchronize(c->stream);
    if (c->h_scalar) cudaFreeHost(c->h_scalar);
    if (c->d_status) cudaFree(c->d_status);
    c->arena.destroy();
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

// Test support: how long a sort tile polls for its predecessors before it gives up, and the number
// the first tile takes (see include/xlb.h).
extern "C" xlb_status xlb_test_set_lookback(xlb_ctx* c, uint32_t spin_limit, uint32_t first_tile) {
    if (!c) return XLB_ERR_INVALID;
    c->lb_spin_limit = spin_limit ? spin_limit : 1u << 22;
    c->lb_first_tile = first_tile;
    return XLB_OK;
}

extern "C" const char* xlb_last_error(const xlb_ctx* c) { return c ? c->last_error.c_str() : g_create_error.c_str(); }

extern "C" xlb_status xlb_memory_stats(const xlb_ctx* c, uint64_t* allocated, uint64_t* peak) {
    if (!c) return XLB_ERR_INVALID;
    if (allocated) *allocated = c->allocated;
    if (peak) *peak = c->peak;
    return XLB_OK;
}

// ------------------------------------------------------------------------------ C ABI: relations
static void check_schema(const xlb_schema* s) {
    if (!s || s->arity > XLB_MAX_ARITY) xlb_fail(XLB_ERR_INVALID, "schema missing or arity above %u", XLB_MAX_ARITY);
    for (uint32_t i = 0; i < s->arity; ++i)
        if (!type_built(s->types[i])) xlb_fail(XLB_ERR_UNSUPPORTED, "column %u: type code %u is not a column type", i, s->types[i]);
}

xlb_rel* rel_empty(xlb_ctx* c, const xlb_schema& s) {
    auto* r = new xlb_rel;
    r->ctx = c;
    r->schema = s;
    r->rows = 0;
    for (uint32_t i = 0; i < s.arity; ++i) r->cols[i] = make_buf(c, 0);
    r->canonical = true;
    return r;
}

extern "C" xlb_status xlb_rel_from_host(xlb_ctx* c, const xlb_schema* s, const void* const* cols, uint64_t rows, xlb_rel** out) {
    if (!c || !out) return XLB_ERR_INVALID;
    API_BEGIN(c)
    check_schema(s);
    if (rows && s->arity && !cols) xlb_fail(XLB_ERR_INVALID, "column pointers missing");
    std::unique_ptr<xlb_rel> r(new xlb_rel);
    r->ctx = c;
    r->schema = *s;
    r->rows = s->arity ? rows : std::min<uint64_t>(rows, 1);
    for (uint32_t i = 0; i < s->arity; ++i) {
        uint64_t bytes = rows * type_width(s->types[i]);
        r->cols[i] = make_buf(c, bytes);
        if (bytes) {
            if (!cols[i]) xlb_fail(XLB_ERR_INVALID, "column %u pointer is null", i);
            CUDA_OK(cudaMemcpyAsync(r->cols[i]->p, cols[i], bytes, cudaMemcpyHostToDevice, c->stream));
        }
    }
    CUDA_OK(cudaStreamSynchronize(c->stream));
    r->canonical = r->rows == 0;
    *out = r.release();
    API_END()
}

extern "C" xlb_status xlb_rel_empty(xlb_ctx* c, const xlb_schema* s, xlb_rel** out) {
    if (!c || !out) return XLB_ERR_INVALID;
    API_BEGIN(c)
    check_schema(s);
    *out = rel_empty(c, *s);
    API_END()
}

extern "C" xlb_status xlb_rel_rows(const xlb_rel* r, uint64_t* rows) {
    if (!r || !rows) return XLB_ERR_INVALID;
    *rows = r->rows;
    return XLB_OK;
}
extern "C" xlb_status xlb_rel_schema(const xlb_rel* r, xlb_schema* s) {
    if (!r || !s) return XLB_ERR_INVALID;
    *s = r->schema;
    return XLB_OK;
}
extern "C" xlb_status xlb_rel_is_canonical(const xlb_rel* r, int* canonical) {
    if (!r || !canonical) return XLB_ERR_INVALID;
    *canonical = r->canonical ? 1 : 0;
    return XLB_OK;
}

extern "C" xlb_status xlb_rel_to_host(xlb_ctx* c, const xlb_rel* r, void* const* cols, uint64_t cap_rows, uint64_t* rows) {
    if (!c || !r) return XLB_ERR_INVALID;
    API_BEGIN(c)
    uint64_t n = std::min(r->rows, cap_rows);
    if (n && r->schema.arity) {
        if (!cols) xlb_fail(XLB_ERR_INVALID, "column pointers missing");
        ops_rel_columns(c, r);
        for (uint32_t i = 0; i < r->schema.arity; ++i) {
            if (!cols[i]) xlb_fail(XLB_ERR_INVALID, "column %u pointer is null", i);
            CUDA_OK(cudaMemcpyAsync(cols[i], r->cols[i]->p, n * type_width(r->schema.types[i]), cudaMemcpyDeviceToHost, c->stream));
        }
    }
    CUDA_OK(cudaStreamSynchronize(c->stream));
    if (rows) *rows = r->rows;
    API_END()
}

static xlb_rel* rel_clone(xlb_ctx* c, const xlb_rel* r) {
    std::unique_ptr<xlb_rel> o(new xlb_rel);
    o->ctx = c;
    o->schema = r->schema;
    o->rows = r->rows;
    o->canonical = r->canonical;
    if (r->packed) {
        Keys k;
        k.buf = r->packed;
        k.n = r->rows;
        o->packed = ops_copy(c, k).buf;
    } else {
        for (uint32_t i = 0; i < r->schema.arity; ++i) {
            uint64_t bytes = r->rows * type_width(r->schema.types[i]);
            o->cols[i] = make_buf(c, bytes);
            if (bytes) CUDA_OK(cudaMemcpyAsync(o->cols[i]->p, r->cols[i]->p, bytes, cudaMemcpyDeviceToDevice, c->stream));
        }
    }
    return o.release();
}

extern "C" xlb_status xlb_rel_clone(xlb_ctx* c, const xlb_rel* r, xlb_rel** out) {
    if (!c || !r || !out) return XLB_ERR_INVALID;
    API_BEGIN(c)
    *out = rel_clone(c, r);
    CUDA_OK(cudaStreamSynchronize(c->stream));
    API_END()
}

static ColSet colset_of(const xlb_rel* r);

extern "C" xlb_status xlb_rel_checksum(xlb_ctx* c, const xlb_rel* r, uint64_t digest[3]) {
    if (!c || !r || !digest) return XLB_ERR_INVALID;
    API_BEGIN(c)
    Buf acc = make_buf(c, 16);
    CUDA_OK(cudaMemsetAsync(acc->p, 0, 16, c->stream));
    if (r->rows && r->schema.arity) {
        prof_begin(c, "digest", 0);
        if (rel_packable(r->schema)) {
            Keys k = ops_rel_packed(c, r);
            digest_packed_k<<<grid_for(c, k.n, BLOCK * 4), BLOCK, 0, c->stream>>>(k.ptr(), k.n, acc->as<unsigned long long>());
        } else {
            ops_rel_columns(c, r);
            digest_cols_k<<<grid_for(c, r->rows, BLOCK * 4), BLOCK, 0, c->stream>>>(colset_of(r), r->rows, acc->as<unsigned long long>());
        }
        check_launch(c, "digest");
    }
    unsigned long long h[2];
    read_words(c, acc->p, 2, h);
    digest[0] = r->rows;
    digest[1] = h[0];
    digest[2] = h[1];
    API_END()
}

extern "C" void xlb_rel_free(xlb_rel* r) {
    if (!r) return;
    cudaSetDevice(r->ctx->device);
    delete r;
}

// ------------------------------------------------------------------------------ operators
// An operator builds its result under this guard and hands it over only after the device status
// word has been read clean: a failure a kernel reported (a bounded wait that ran out, a capacity
// check) then fails the call that caused it, and the half-written relation is freed.
struct ResultGuard {
    xlb_rel* r = nullptr;
    ~ResultGuard() { delete r; }
    void deliver(xlb_ctx* c, xlb_rel** to) {
        check_dev_status(c);  // waits for the stream
        *to = r;
        r = nullptr;
    }
};

static bool schemas_compatible(const xlb_schema& a, const xlb_schema& b) {
    if (a.arity != b.arity) return false;
    for (uint32_t i = 0; i < a.arity; ++i) {
        uint8_t x = a.types[i] == XLB_SYMBOL ? XLB_U32 : a.types[i];
        uint8_t y = b.types[i] == XLB_SYMBOL ? XLB_U32 : b.types[i];
        if (x != y) return false;
    }
    return true;
}

// rows that fit one u64 word: (u32), (u32,u32) as packed keys, or a single u64 column as is
static bool single_word(const xlb_schema& s) { return rel_packable(s) || (s.arity == 1 && type_width(s.types[0]) == 8); }

static Keys rel_word_keys(xlb_ctx* c, const xlb_rel* r) {
    if (rel_packable(r->schema)) return ops_rel_packed(c, r);
    Keys k;
    k.buf = r->cols[0];
    k.n = r->rows;
    return k;
}
static xlb_rel* rel_from_word_keys(xlb_ctx* c, const xlb_schema& s, Keys k, bool canonical) {
    if (rel_packable(s)) return ops_rel_from_keys(c, s, k, canonical);
    auto* r = new xlb_rel;
    r->ctx = c;
    r->schema = s;
    r->rows = k.n;
    r->cols[0] = k.buf ? k.buf : make_buf(c, 0);
    r->canonical = canonical;
    return r;
}

static ColSet colset_of(const xlb_rel* r) {
    ColSet cs{};
    cs.n = (int)r->schema.arity;
    for (int i = 0; i < cs.n; ++i) {
        cs.col[i] = r->cols[i]->p;
        cs.width[i] = (int)type_width(r->schema.types[i]);
    }
    return cs;
}

// Stable sort permutation by key columns (first key most significant): LSD over the key
// columns, least significant first, each a stable (key word, row index) radix sort.
static Buf sort_permutation(xlb_ctx* c, const xlb_rel* r, const uint32_t* keys, uint32_t nk) {
    uint64_t n = r->rows;
    Buf idx = make_buf(c, n * 4);
    if (n == 0) return idx;
    if (n >= (1ull << 32)) xlb_fail(XLB_ERR_CAPACITY, "sort of %llu rows exceeds the 2^32 row limit", (unsigned long long)n);
    prof_begin(c, "iota", 0);
    iota_k<<<grid_for(c, n), BLOCK, 0, c->stream>>>(idx->as<uint32_t>(), n);
    check_launch(c, "iota");
    int k = (int)nk - 1;
    while (k >= 0) {
        // fuse two adjacent 32-bit key columns into one 64-bit key word
        int w1 = (int)type_width(r->schema.types[keys[k]]);
        const void* lo = nullptr;
        int hi_col = k;
        if (w1 == 4 && k >= 1 && type_width(r->schema.types[keys[k - 1]]) == 4) {
            lo = r->cols[keys[k]]->p;
            hi_col = k - 1;
        }
        Buf kw = make_buf(c, n * 8);
        const xlb_rel* rr = r;
        prof_begin(c, "build_key", 0);
        build_key_k<<<grid_for(c, n), BLOCK, 0, c->stream>>>(rr->cols[keys[hi_col]]->p, (int)type_width(r->schema.types[keys[hi_col]]), lo, 4, idx->as<uint32_t>(), kw->as<uint64_t>(), n);
        check_launch(c, "build_key");
        radix_sort(c, kw, &idx, n);
        k = hi_col - 1;
    }
    return idx;
}

static xlb_rel* gather_rel(xlb_ctx* c, const xlb_rel* r, const uint32_t* idx, uint64_t n) {
    std::unique_ptr<xlb_rel> o(new xlb_rel);
    o->ctx = c;
    o->schema = r->schema;
    o->rows = n;
    for (uint32_t i = 0; i < r->schema.arity; ++i) {
        uint32_t w = type_width(r->schema.types[i]);
        o->cols[i] = make_buf(c, n * w);
        if (!n) continue;
        prof_begin(c, "gather", 0);
        if (w == 4) gather_k<uint32_t><<<grid_for(c, n), BLOCK, 0, c->stream>>>(r->cols[i]->as<uint32_t>(), idx, o->cols[i]->as<uint32_t>(), n);
        else if (w == 8) gather_k<uint64_t><<<grid_for(c, n), BLOCK, 0, c->stream>>>(r->cols[i]->as<uint64_t>(), idx, o->cols[i]->as<uint64_t>(), n);
        else gather_k<uint8_t><<<grid_for(c, n), BLOCK, 0, c->stream>>>(r->cols[i]->as<uint8_t>(), idx, o->cols[i]->as<uint8_t>(), n);
        check_launch(c, "gather");
    }
    return o.release();
}

static xlb_status sort_unsigned(xlb_ctx* c, const xlb_rel* in, const uint32_t* key_cols, uint32_t nk, xlb_rel** out_final) {
    if (!c || !in || !out_final) return XLB_ERR_INVALID;
    API_BEGIN(c)
    ResultGuard guard;
    xlb_rel** out = &guard.r;
    for (uint32_t i = 0; i < nk; ++i)
        if (key_cols[i] >= in->schema.arity) xlb_fail(XLB_ERR_INVALID, "sort key column %u out of range", key_cols[i]);
    ops_rel_columns(c, in);
    Buf idx = sort_permutation(c, in, key_cols, nk);
    *out = gather_rel(c, in, idx->as<uint32_t>(), in->rows);
    guard.deliver(c, out_final);
    API_END()
}

xlb_rel* rel_view(xlb_ctx* c, const xlb_rel* r) {
    auto* o = new xlb_rel;
    o->ctx = c;
    o->schema = r->schema;
    o->rows = r->rows;
    for (uint32_t i = 0; i < r->schema.arity; ++i) o->cols[i] = r->cols[i];
    o->packed = r->packed;
    o->or_bound = r->or_bound;
    o->canonical = r->canonical;
    return o;
}

xlb_rel* rel_project(xlb_ctx* c, const xlb_rel* in, const uint32_t* cols, uint32_t n) {
    ops_rel_columns(c, in);
    auto* o = new xlb_rel;
    o->ctx = c;
    o->schema.arity = n;
    o->rows = n ? in->rows : std::min<uint64_t>(in->rows, 1);
    for (uint32_t i = 0; i < n; ++i) {
        o->schema.types[i] = in->schema.types[cols[i]];
        o->cols[i] = in->cols[cols[i]];
    }
    return o;
}

xlb_rel* rel_filter(xlb_ctx* c, const xlb_rel* in, uint32_t cmp, uint32_t lhs, bool rhs_is_const, uint64_t rhs) {
    if (in->rows == 0) return rel_view(c, in);
    if (in->rows >= (1ull << 32)) xlb_fail(XLB_ERR_CAPACITY, "filter input exceeds the 2^32 row limit");
    ops_rel_columns(c, in);
    Buf idx = make_buf(c, in->rows * 4);
    uint64_t m = select(c, PredCmpCols{colset_of(in), cmp, lhs, rhs_is_const, rhs}, EmitIndex{idx->as<uint32_t>()}, in->rows);
    xlb_rel* o = gather_rel(c, in, idx->as<uint32_t>(), m);
    o->canonical = in->canonical;  // a subsequence of a sorted unique list is one
    return o;
}

// Full-row canonicalisation of a wide relation (more than one 64-bit word per row).
static xlb_rel* wide_dedup(xlb_ctx* c, const xlb_rel* in, const uint32_t* origin_excl, uint32_t n_excl) {
    (void)origin_excl;
    uint32_t all[XLB_MAX_ARITY];
    for (uint32_t i = 0; i < in->schema.arity; ++i) all[i] = i;
    Buf idx = sort_permutation(c, in, all, in->schema.arity);
    std::unique_ptr<xlb_rel> sorted(gather_rel(c, in, idx->as<uint32_t>(), in->rows));
    Buf heads = make_buf(c, in->rows * 4);
    uint64_t m;
    if (n_excl) m = select(c, PredRowHeadNotExcluded{colset_of(sorted.get()), idx->as<uint32_t>(), n_excl}, EmitIndex{heads->as<uint32_t>()}, in->rows);
    else m = select(c, PredRowHead{colset_of(sorted.get())}, EmitIndex{heads->as<uint32_t>()}, in->rows);
    xlb_rel* o = gather_rel(c, sorted.get(), heads->as<uint32_t>(), m);
    o->canonical = true;
    return o;
}

xlb_rel* rel_concat(xlb_ctx* c, const xlb_rel* const* ins, uint32_t n) {
    std::unique_ptr<xlb_rel> o(new xlb_rel);
    o->ctx = c;
    o->schema = ins[0]->schema;
    uint64_t rows = 0;
    for (uint32_t i = 0; i < n; ++i) rows += ins[i]->rows;
    o->rows = rows;
    for (uint32_t col = 0; col < o->schema.arity; ++col) {
        uint32_t w = type_width(o->schema.types[col]);
        o->cols[col] = make_buf(c, rows * w);
        uint64_t at = 0;
        for (uint32_t i = 0; i < n; ++i) {
            if (ins[i]->rows) {
                ops_rel_columns(c, ins[i]);
                CUDA_OK(cudaMemcpyAsync((char*)o->cols[col]->p + at * w, ins[i]->cols[col]->p, ins[i]->rows * w, cudaMemcpyDeviceToDevice, c->stream));
            }
            at += ins[i]->rows;
        }
    }
    return o.release();
}

xlb_rel* rel_canonical(xlb_ctx* c, const xlb_rel* in) {
    if (in->schema.arity == 0) {  // the 0-arity relation is {} or {()} (set_ops_tests.rs:160-183)
        xlb_rel* o = rel_empty(c, in->schema);
        o->rows = in->rows ? 1 : 0;
        return o;
    }
    if (in->canonical) return rel_clone(c, in);
    if (single_word(in->schema)) {
        Keys k = ops_copy(c, rel_word_keys(c, in));
        ops_sort(c, k);
        ops_dedup_sorted(c, k);
        return rel_from_word_keys(c, in->schema, k, true);
    }
    ops_rel_columns(c, in);
    return wide_dedup(c, in, nullptr, 0);
}

// dedup (relational.rs:238): key columns covering every column (or none) = full-row form; a proper
// subset keeps, for every distinct key, the first row in stable key order.
xlb_rel* rel_distinct(xlb_ctx* c, const xlb_rel* in, const uint32_t* key_cols, uint32_t nk) {
    if (nk == 0 || nk >= in->schema.arity) return rel_canonical(c, in);
    for (uint32_t i = 0; i < nk; ++i)
        if (key_cols[i] >= in->schema.arity) xlb_fail(XLB_ERR_INVALID, "dedup key column %u out of range", key_cols[i]);
    ops_rel_columns(c, in);
    Buf idx = sort_permutation(c, in, key_cols, nk);
    std::unique_ptr<xlb_rel> sorted(gather_rel(c, in, idx->as<uint32_t>(), in->rows));
    ColSet cs{};
    cs.n = (int)nk;
    for (uint32_t i = 0; i < nk; ++i) {
        cs.col[i] = sorted->cols[key_cols[i]]->p;
        cs.width[i] = (int)type_width(in->schema.types[key_cols[i]]);
    }
    Buf heads = make_buf(c, in->rows * 4);
    uint64_t m = select(c, PredRowHead{cs}, EmitIndex{heads->as<uint32_t>()}, in->rows);
    return gather_rel(c, sorted.get(), heads->as<uint32_t>(), m);
}

static xlb_status dedup_unsigned(xlb_ctx* c, const xlb_rel* in, const uint32_t* key_cols, uint32_t nk, xlb_rel** out_final) {
    if (!c || !in || !out_final) return XLB_ERR_INVALID;
    API_BEGIN(c)
    ResultGuard guard;
    guard.r = rel_distinct(c, in, key_cols, nk);
    guard.deliver(c, out_final);
    API_END()
}

// Set union of n >= 1 type-compatible relations: sorted, unique, certified (union_many_gpu).
xlb_rel* rel_union_many(xlb_ctx* c, const xlb_rel* const* ins, uint32_t n) {
    if (n == 0 || !ins) xlb_fail(XLB_ERR_INVALID, "union of no inputs");
    for (uint32_t i = 0; i < n; ++i) {
        if (!ins[i]) xlb_fail(XLB_ERR_INVALID, "union input %u is null", i);
        if (!schemas_compatible(ins[0]->schema, ins[i]->schema)) xlb_fail(XLB_ERR_TYPE, "union input %u has an incompatible schema", i);
    }
    const xlb_schema& s = ins[0]->schema;
    if (s.arity == 0) {
        xlb_rel* o = rel_empty(c, s);
        for (uint32_t i = 0; i < n; ++i)
            if (ins[i]->rows) o->rows = 1;
        return o;
    }
    if (single_word(s)) {
        // canonical inputs are merged; the rest are concatenated, sorted and deduplicated once
        std::vector<Keys> loose;
        Keys acc;
        bool have_acc = false;
        for (uint32_t i = 0; i < n; ++i) {
            if (ins[i]->rows == 0) continue;
            Keys k = rel_word_keys(c, ins[i]);
            if (ins[i]->canonical) {
                acc = have_acc ? ops_union(c, acc, k) : k;
                have_acc = true;
            } else loose.push_back(k);
        }
        if (!loose.empty()) {
            Keys cat = ops_concat(c, loose);
            ops_sort(c, cat);
            ops_dedup_sorted(c, cat);
            acc = have_acc ? ops_union(c, acc, cat) : cat;
            have_acc = true;
        }
        if (!have_acc) return rel_empty(c, s);
        bool aliased = false;
        for (uint32_t i = 0; i < n; ++i) {
            if (!ins[i]->rows) continue;
            Keys k = rel_word_keys(c, ins[i]);
            if (k.buf == acc.buf) aliased = true;
        }
        if (aliased) acc = ops_copy(c, acc);
        return rel_from_word_keys(c, s, acc, true);
    }
    std::unique_ptr<xlb_rel> cat(rel_concat(c, ins, n));
    return wide_dedup(c, cat.get(), nullptr, 0);
}

static xlb_status union_unsigned(xlb_ctx* c, const xlb_rel* const* ins, uint32_t n, xlb_rel** out_final) {
    if (!c || !out_final) return XLB_ERR_INVALID;
    API_BEGIN(c)
    ResultGuard guard;
    guard.r = rel_union_many(c, ins, n);
    guard.deliver(c, out_final);
    API_END()
}

// a \ b with set semantics on full rows: sorted, unique, certified (diff_gpu).
xlb_rel* rel_difference(xlb_ctx* c, const xlb_rel* a, const xlb_rel* b) {
    if (!schemas_compatible(a->schema, b->schema)) xlb_fail(XLB_ERR_TYPE, "difference of incompatible schemas");
    const xlb_schema& s = a->schema;
    if (s.arity == 0) {
        xlb_rel* o = rel_empty(c, s);
        o->rows = (a->rows && !b->rows) ? 1 : 0;
        return o;
    }
    if (a->rows == 0) return rel_empty(c, s);
    if (single_word(s)) {
        std::unique_ptr<xlb_rel> ca(rel_canonical(c, a)), cb(rel_canonical(c, b));
        Keys d = ops_diff(c, rel_word_keys(c, ca.get()), rel_word_keys(c, cb.get()));
        return rel_from_word_keys(c, s, d, true);
    }
    // rows of b first: a run of equal rows that starts with a row of b is dropped whole
    const xlb_rel* both[2] = {b, a};
    std::unique_ptr<xlb_rel> cat(rel_concat(c, both, 2));
    if (b->rows >= (1ull << 32)) xlb_fail(XLB_ERR_CAPACITY, "difference input exceeds the 2^32 row limit");
    return wide_dedup(c, cat.get(), nullptr, (uint32_t)b->rows);
}

static xlb_status diff_unsigned(xlb_ctx* c, const xlb_rel* a, const xlb_rel* b, xlb_rel** out_final) {
    if (!c || !a || !b || !out_final) return XLB_ERR_INVALID;
    API_BEGIN(c)
    ResultGuard guard;
    guard.r = rel_difference(c, a, b);
    guard.deliver(c, out_final);
    API_END()
}

// ---- typed columns ---------------------------------------------------------------------------
// Signed and floating columns are ordered the way the reference orders them (sign flip for
// i32/i64; IEEE totalOrder for f32/f64: crates/xlog-cuda/kernels/sort.cu:296-448, totalorder.cuh)
// by mapping them to order-preserving unsigned words, running the unsigned operator and mapping
// the result back.  Equality stays bitwise (NaN payloads and signed zeros are distinct), as in
// crates/xlog-cuda/tests/test_full_row_set_algebra.rs:234-310.
namespace {
// a bool column (one byte per value, ordered false < true: kernels/sort.cu:331-345) as 32-bit words and back
__global__ void bool_widen_k(const uint8_t* __restrict__ in, uint32_t* __restrict__ out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) out[i] = in[i];
}
__global__ void bool_narrow_k(const uint32_t* __restrict__ in, uint8_t* __restrict__ out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) out[i] = (uint8_t)in[i];
}
// kind 1: signed; kind 2: float.  Forward then inverse is the identity.
template <class T>
__global__ void order_map_k(const T* __restrict__ in, T* __restrict__ out, uint64_t n, int kind, int inverse) {
    const T sign = T(1) << (sizeof(T) * 8 - 1);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        T x = in[i];
        if (kind == 1) x ^= sign;
        else if (!inverse) x = (x & sign) ? ~x : (x | sign);
        else x = (x & sign) ? (x ^ sign) : ~x;
        out[i] = x;
    }
}
}  // namespace

static int order_kind(uint8_t t) { return (t == XLB_I32 || t == XLB_I64) ? 1 : (t == XLB_F32 || t == XLB_F64) ? 2 : t == XLB_BOOL ? 3 : 0; }
static bool schema_typed(const xlb_schema& s) {
    for (uint32_t i = 0; i < s.arity; ++i)
        if (order_kind(s.types[i])) return true;
    return false;
}

// ---- dictionary encoding -----------------------------------------------------------------------
namespace {
// order-preserving unsigned image of one value, widened to 64 bits (kind as in order_map_k)
__device__ __forceinline__ uint64_t dict_image(const void* col, int width, int kind, uint64_t i) {
    if (width == 1) return ((const uint8_t*)col)[i];
    if (width == 4) {
        uint32_t x = ((const uint32_t*)col)[i];
        const uint32_t sign = 0x80000000u;
        if (kind == 1) x ^= sign;
        else if (kind == 2) x = (x & sign) ? ~x : (x | sign);
        return x;
    }
    uint64_t x = ((const uint64_t*)col)[i];
    const uint64_t sign = 1ull << 63;
    if (kind == 1) x ^= sign;
    else if (kind == 2) x = (x & sign) ? ~x : (x | sign);
    return x;
}
__global__ void dict_image_k(const void* col, int width, int kind, uint64_t* __restrict__ out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) out[i] = dict_image(col, width, kind, i);
}
// number of dictionary entries below v
__device__ __forceinline__ uint64_t dict_below(const uint64_t* __restrict__ dict, uint64_t m, uint64_t v) {
    uint64_t lo = 0, hi = m;
    while (lo < hi) {
        uint64_t mid = (lo + hi) >> 1;
        if (dict[mid] < v) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}
__global__ void dict_rank_k(const void* col, int width, int kind, const uint64_t* __restrict__ dict, uint64_t m, uint32_t* __restrict__ out, uint64_t n,
                            DevStatus* st) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t v = dict_image(col, width, kind, i);
        const uint64_t r = dict_below(dict, m, v);
        if (r >= m || dict[r] != v) {  // every value was put into the dictionary: a miss means it is not the right one
            set_status(st, XLB_ERR_CAPACITY, 10, v);
            out[i] = 0;
        } else out[i] = (uint32_t)r;
    }
}
__global__ void dict_decode_k(const uint32_t* __restrict__ ranks, const uint64_t* __restrict__ dict, uint64_t m, int width, int kind, void* out, uint64_t n,
                              DevStatus* st) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = ranks[i];
        if (r >= m) {
            set_status(st, XLB_ERR_CAPACITY, 11, r);
            continue;
        }
        uint64_t x = dict[r];
        if (width == 1) {
            ((uint8_t*)out)[i] = (uint8_t)x;
        } else if (width == 4) {
            uint32_t y = (uint32_t)x;
            const uint32_t sign = 0x80000000u;
            if (kind == 1) y ^= sign;
            else if (kind == 2) y = (y & sign) ? (y ^ sign) : ~y;
            ((uint32_t*)out)[i] = y;
        } else {
            const uint64_t sign = 1ull << 63;
            if (kind == 1) x ^= sign;
            else if (kind == 2) x = (x & sign) ? (x ^ sign) : ~x;
            ((uint64_t*)out)[i] = x;
        }
    }
}
__global__ void dict_bounds_k(const uint64_t* __restrict__ dict, uint64_t m, const uint64_t* __restrict__ consts, uint32_t k, uint64_t* __restrict__ out) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= k) return;
    const uint64_t v = consts[i];
    const uint64_t below = dict_below(dict, m, v);
    out[2 * i] = below;
    out[2 * i + 1] = below + ((below < m && dict[below] == v) ? 1 : 0);
}
}  // namespace

static int order_kind(uint8_t t);

Keys ops_dict_build(xlb_ctx* c, const std::vector<const xlb_rel*>& rels) {
    uint64_t total = 0;
    for (const xlb_rel* r : rels) total += r->rows * r->schema.arity;
    Keys k;
    k.n = total;
    k.buf = make_buf(c, total * 8);
    uint64_t at = 0;
    for (const xlb_rel* r : rels) {
        if (!r->rows) continue;
        ops_rel_columns(c, r);
        for (uint32_t i = 0; i < r->schema.arity; ++i) {
            prof_begin(c, "dict_image", r->rows * 12ull);
            dict_image_k<<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(r->cols[i]->p, (int)type_width(r->schema.types[i]), order_kind(r->schema.types[i]),
                                                                       k.buf->as<uint64_t>() + at, r->rows);
            check_launch(c, "dict_image");
            at += r->rows;
        }
    }
    ops_sort(c, k);
    ops_dedup_sorted(c, k);
    if (k.n >= 0xFFFFFFFFull) xlb_fail(XLB_ERR_CAPACITY, "%llu distinct values exceed the 2^32 - 1 a plan over wide columns can hold", (unsigned long long)k.n);
    return k;
}

xlb_rel* ops_dict_encode(xlb_ctx* c, const xlb_rel* r, const Keys& dict) {
    ops_rel_columns(c, r);
    std::unique_ptr<xlb_rel> o(new xlb_rel);
    o->ctx = c;
    o->rows = r->rows;
    o->schema.arity = r->schema.arity;
    o->canonical = r->canonical;  // ranks order as the values do
    for (uint32_t i = 0; i < r->schema.arity; ++i) {
        o->schema.types[i] = XLB_U32;
        o->cols[i] = make_buf(c, r->rows * 4);
        if (!r->rows) continue;
        prof_begin(c, "dict_rank", r->rows * 12ull);
        dict_rank_k<<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(r->cols[i]->p, (int)type_width(r->schema.types[i]), order_kind(r->schema.types[i]), dict.ptr(), dict.n,
                                                                  o->cols[i]->as<uint32_t>(), r->rows, c->d_status);
        check_launch(c, "dict_rank");
    }
    return o.release();
}

xlb_rel* ops_dict_decode(xlb_ctx* c, const xlb_rel* ranks, const xlb_schema& types, const Keys& dict) {
    if (ranks->schema.arity != types.arity) xlb_fail(XLB_ERR_INVALID, "internal: decoding %u columns into %u", ranks->schema.arity, types.arity);
    ops_rel_columns(c, ranks);
    std::unique_ptr<xlb_rel> o(new xlb_rel);
    o->ctx = c;
    o->rows = ranks->rows;
    o->schema = types;
    o->canonical = ranks->canonical;
    for (uint32_t i = 0; i < types.arity; ++i) {
        const uint32_t w = type_width(types.types[i]);
        o->cols[i] = make_buf(c, ranks->rows * w);
        if (!ranks->rows) continue;
        prof_begin(c, "dict_decode", ranks->rows * (4ull + w));
        dict_decode_k<<<grid_for(c, ranks->rows), BLOCK, 0, c->stream>>>(ranks->cols[i]->as<uint32_t>(), dict.ptr(), dict.n, (int)w, order_kind(types.types[i]), o->cols[i]->p,
                                                                        ranks->rows, c->d_status);
        check_launch(c, "dict_decode");
    }
    return o.release();
}

void ops_dict_bounds(xlb_ctx* c, const Keys& dict, const std::vector<uint64_t>& consts, std::vector<uint64_t>& below, std::vector<uint64_t>& not_above) {
    below.assign(consts.size(), 0);
    not_above.assign(consts.size(), 0);
    for (size_t base = 0; base < consts.size(); base += 8) {  // the pinned staging area holds a few words at a time
        const uint32_t k = (uint32_t)std::min<size_t>(8, consts.size() - base);
        Keys cs = ops_from_host(c, consts.data() + base, k);
        Buf out = make_buf(c, 2 * k * 8);
        dict_bounds_k<<<1, 32, 0, c->stream>>>(dict.ptr(), dict.n, cs.ptr(), k, out->as<uint64_t>());
        check_launch(c, "dict_bounds");
        unsigned long long h[16];
        read_words(c, out->p, 2 * (int)k, h);
        for (uint32_t i = 0; i < k; ++i) {
            below[base + i] = h[2 * i];
            not_above[base + i] = h[2 * i + 1];
        }
    }
}

// forward: a view of `r` whose typed columns are mapped to unsigned words (schema becomes
// unsigned); inverse: `r` is an unsigned result, `types` the schema to restore.
static xlb_rel* map_rel(xlb_ctx* c, const xlb_rel* r, const xlb_schema& types, bool inverse) {
    ops_rel_columns(c, r);
    std::unique_ptr<xlb_rel> o(new xlb_rel);
    o->ctx = c;
    o->rows = r->rows;
    o->canonical = r->canonical;
    o->schema = types;
    for (uint32_t i = 0; i < types.arity; ++i) {
        int kind = order_kind(types.types[i]);
        uint32_t w = type_width(types.types[i]);
        if (!inverse) o->schema.types[i] = kind ? (w == 8 ? XLB_U64 : XLB_U32) : types.types[i];
        if (!kind) { o->cols[i] = r->cols[i]; continue; }  // relations are immutable: share the column
        if (kind == 3) {  // bool: bytes <-> words
            o->cols[i] = make_buf(c, r->rows * (inverse ? 1 : 4));
            if (!r->rows) continue;
            prof_begin(c, "order_map", r->rows * 5ull);
            if (!inverse) bool_widen_k<<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(r->cols[i]->as<uint8_t>(), o->cols[i]->as<uint32_t>(), r->rows);
            else bool_narrow_k<<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(r->cols[i]->as<uint32_t>(), o->cols[i]->as<uint8_t>(), r->rows);
            check_launch(c, "order_map");
            continue;
        }
        o->cols[i] = make_buf(c, r->rows * w);
        if (!r->rows) continue;
        prof_begin(c, "order_map", r->rows * 2ull * w);
        if (w == 4) order_map_k<uint32_t><<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(r->cols[i]->as<uint32_t>(), o->cols[i]->as<uint32_t>(), r->rows, kind, inverse);
        else order_map_k<uint64_t><<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(r->cols[i]->as<uint64_t>(), o->cols[i]->as<uint64_t>(), r->rows, kind, inverse);
        check_launch(c, "order_map");
    }
    return o.release();
}

static bool schemas_compatible(const xlb_schema& a, const xlb_schema& b);

// Run `op` on unsigned views of the inputs and restore the first input's column types.
template <class Op>
static xlb_status with_typed(xlb_ctx* c, const xlb_rel* const* ins, uint32_t n, xlb_rel** out, Op op) {
    bool typed = false;
    for (uint32_t i = 0; i < n; ++i)
        if (ins[i] && schema_typed(ins[i]->schema)) typed = true;
    if (!typed) return op(ins, out);
    std::vector<std::unique_ptr<xlb_rel>> mapped;
    std::vector<const xlb_rel*> ptrs;
    try {
        for (uint32_t i = 0; i < n; ++i) {
            if (!schemas_compatible(ins[0]->schema, ins[i]->schema)) xlb_fail(XLB_ERR_TYPE, "input %u has an incompatible schema", i);
            mapped.emplace_back(map_rel(c, ins[i], ins[i]->schema, false));
            ptrs.push_back(mapped.back().get());
        }
    } catch (const XlbError& e) {
        c->last_error = e.msg;
        return e.st;
    }
    xlb_rel* u = nullptr;
    xlb_status st = op(ptrs.data(), &u);
    if (st != XLB_OK) return st;
    std::unique_ptr<xlb_rel> ur(u);
    try {
        ResultGuard guard;
        guard.r = map_rel(c, u, ins[0]->schema, true);
        guard.deliver(c, out);
    } catch (const XlbError& e) {
        c->last_error = e.msg;
        return e.st;
    }
    return XLB_OK;
}

extern "C" xlb_status xlb_sort(xlb_ctx* c, const xlb_rel* in, const uint32_t* key_cols, uint32_t nk, xlb_rel** out) {
    if (!c || !in || !out) return XLB_ERR_INVALID;
    return with_typed(c, &in, 1, out, [&](const xlb_rel* const* v, xlb_rel** o) { return sort_unsigned(c, v[0], key_cols, nk, o); });
}
extern "C" xlb_status xlb_dedup(xlb_ctx* c, const xlb_rel* in, const uint32_t* key_cols, uint32_t nk, xlb_rel** out) {
    if (!c || !in || !out) return XLB_ERR_INVALID;
    return with_typed(c, &in, 1, out, [&](const xlb_rel* const* v, xlb_rel** o) { return dedup_unsigned(c, v[0], key_cols, nk, o); });
}
extern "C" xlb_status xlb_union(xlb_ctx* c, const xlb_rel* const* ins, uint32_t n, xlb_rel** out) {
    if (!c || !out) return XLB_ERR_INVALID;
    if (n == 0 || !ins) { c->last_error = "union of no inputs"; return XLB_ERR_INVALID; }
    for (uint32_t i = 0; i < n; ++i)
        if (!ins[i]) { c->last_error = "union input is null"; return XLB_ERR_INVALID; }
    return with_typed(c, ins, n, out, [&](const xlb_rel* const* v, xlb_rel** o) { return union_unsigned(c, v, n, o); });
}
extern "C" xlb_status xlb_diff(xlb_ctx* c, const xlb_rel* a, const xlb_rel* b, xlb_rel** out) {
    if (!c || !a || !b || !out) return XLB_ERR_INVALID;
    const xlb_rel* both[2] = {a, b};
    return with_typed(c, both, 2, out, [&](const xlb_rel* const* v, xlb_rel** o) { return diff_unsigned(c, v[0], v[1], o); });
}

// groupby_multi_agg (crates/xlog-cuda/src/provider/groupby.rs:66-770): sort by the key columns,
// find the group boundaries, reduce every aggregate per group.  Output: key columns, then one
// column per aggregate in the order given; one row per group, ascending by key.
extern "C" xlb_status xlb_groupby(xlb_ctx* c, const xlb_rel* in, const uint32_t* key_cols, uint32_t nk, const uint32_t* agg_cols, const uint32_t* agg_ops,
                                  uint32_t na, xlb_rel** out_final) {
    if (!c || !in || !out_final) return XLB_ERR_INVALID;
    API_BEGIN(c)
    ResultGuard guard;
    xlb_rel** out = &guard.r;
    if (nk == 0 || !key_cols) xlb_fail(XLB_ERR_INVALID, "GroupBy requires at least one key column");
    if (na == 0 || !agg_cols || !agg_ops) xlb_fail(XLB_ERR_INVALID, "GroupBy requires at least one aggregation");
    if (nk + na > XLB_MAX_ARITY) xlb_fail(XLB_ERR_UNSUPPORTED, "GroupBy output arity above %u", XLB_MAX_ARITY);
    xlb_schema os{};
    for (uint32_t i = 0; i < nk; ++i) {
        if (key_cols[i] >= in->schema.arity) xlb_fail(XLB_ERR_INVALID, "Key column %u out of bounds (arity %u)", key_cols[i], in->schema.arity);
        uint8_t t = in->schema.types[key_cols[i]];
        if (!type_unsigned(t)) xlb_fail(XLB_ERR_TYPE, "GroupBy keys must be u32, symbol or u64 columns");
        os.types[os.arity++] = t;
    }
    for (uint32_t i = 0; i < na; ++i) {
        if (agg_cols[i] >= in->schema.arity) xlb_fail(XLB_ERR_INVALID, "Value column %u out of bounds (arity %u)", agg_cols[i], in->schema.arity);
        if (agg_ops[i] > XLB_AGG_MAX) xlb_fail(XLB_ERR_UNSUPPORTED, "aggregation %u is not built (count, sum, min, max are)", agg_ops[i]);
        uint8_t vt = in->schema.types[agg_cols[i]];
        if (agg_ops[i] != XLB_AGG_COUNT && vt != XLB_U32 && vt != XLB_U64)
            xlb_fail(XLB_ERR_TYPE, "%s currently requires U32 or U64 values", agg_ops[i] == XLB_AGG_SUM ? "Sum" : agg_ops[i] == XLB_AGG_MIN ? "Min" : "Max");
        // count and sum are u64; min and max keep the width of the value column (groupby.rs:799-811)
        os.types[os.arity++] = (agg_ops[i] == XLB_AGG_COUNT || agg_ops[i] == XLB_AGG_SUM) ? XLB_U64 : (vt == XLB_U64 ? XLB_U64 : XLB_U32);
    }
    if (in->rows == 0) {
        *out = rel_empty(c, os);
        (*out)->canonical = false;
    } else {
        if (in->rows > 0xFFFFFFFFull) xlb_fail(XLB_ERR_CAPACITY, "GroupBy supports at most %u rows, got %llu", 0xFFFFFFFFu, (unsigned long long)in->rows);
        ops_rel_columns(c, in);
        const uint64_t n = in->rows;
        Buf idx = sort_permutation(c, in, key_cols, nk);
        // the key columns in sorted order, then the first row of every group
        xlb_rel keys_only;
        keys_only.ctx = c;
        keys_only.rows = n;
        for (uint32_t i = 0; i < nk; ++i) {
            keys_only.schema.types[i] = in->schema.types[key_cols[i]];
            keys_only.cols[i] = in->cols[key_cols[i]];
        }
        keys_only.schema.arity = nk;
        std::unique_ptr<xlb_rel> ksorted(gather_rel(c, &keys_only, idx->as<uint32_t>(), n));
        Buf heads = make_buf(c, n * 4);
        const uint64_t m = select(c, PredRowHead{colset_of(ksorted.get())}, EmitIndex{heads->as<uint32_t>()}, n);
        std::unique_ptr<xlb_rel> o(gather_rel(c, ksorted.get(), heads->as<uint32_t>(), m));
        o->schema = os;
        for (uint32_t a = 0; a < na; ++a) {
            const uint32_t vc = agg_cols[a], op = agg_ops[a];
            const uint32_t vw = type_width(in->schema.types[vc]);
            Buf acc = make_buf(c, m * 8);
            fill_u64_k<<<grid_for(c, m), BLOCK, 0, c->stream>>>(acc->as<unsigned long long>(), m, op == XLB_AGG_MIN ? ~0ull : 0ull);
            check_launch(c, "groupby_fill");
            const unsigned grid = grid_for(c, (n + GB_ITEMS - 1) / GB_ITEMS);
            prof_begin(c, "groupby_reduce", n * (op == XLB_AGG_COUNT ? 0ull : vw) + m * 12ull);
            if (op == XLB_AGG_COUNT) {
                groupby_reduce_k<uint32_t><<<grid, BLOCK, 0, c->stream>>>(nullptr, heads->as<uint32_t>(), m, n, (int)op, acc->as<unsigned long long>());
            } else if (vw == 4) {
                Buf vs = make_buf(c, n * 4);
                gather_k<uint32_t><<<grid_for(c, n), BLOCK, 0, c->stream>>>(in->cols[vc]->as<uint32_t>(), idx->as<uint32_t>(), vs->as<uint32_t>(), n);
                groupby_reduce_k<uint32_t><<<grid, BLOCK, 0, c->stream>>>(vs->as<uint32_t>(), heads->as<uint32_t>(), m, n, (int)op, acc->as<unsigned long long>());
            } else {
                Buf vs = make_buf(c, n * 8);
                gather_k<uint64_t><<<grid_for(c, n), BLOCK, 0, c->stream>>>(in->cols[vc]->as<uint64_t>(), idx->as<uint32_t>(), vs->as<uint64_t>(), n);
                groupby_reduce_k<uint64_t><<<grid, BLOCK, 0, c->stream>>>(vs->as<uint64_t>(), heads->as<uint32_t>(), m, n, (int)op, acc->as<unsigned long long>());
            }
            check_launch(c, "groupby_reduce");
            if (os.types[nk + a] == XLB_U64) {
                o->cols[nk + a] = acc;
            } else {
                Buf narrow = make_buf(c, m * 4);
                narrow_u64_k<<<grid_for(c, m), BLOCK, 0, c->stream>>>(acc->as<unsigned long long>(), narrow->as<uint32_t>(), m);
                check_launch(c, "groupby_narrow");
                o->cols[nk + a] = narrow;
            }
        }
        o->canonical = false;
        *out = o.release();
    }
    guard.deliver(c, out_final);
    API_END()
}

// key word per row for a join side; two 32-bit key columns fuse into one word
static Buf join_keys(xlb_ctx* c, const xlb_rel* r, const uint32_t* keys, uint32_t nk) {
    Buf kw = make_buf(c, r->rows * 8);
    if (!r->rows) return kw;
    int w0 = (int)type_width(r->schema.types[keys[0]]);
    const void* c1 = nullptr;
    if (nk == 2) {
        if (w0 != 4 || type_width(r->schema.types[keys[1]]) != 4) xlb_fail(XLB_ERR_UNSUPPORTED, "two-column join keys must both be 32-bit");
        c1 = r->cols[keys[1]]->p;
    }
    prof_begin(c, "build_key", 0);
    build_key_k<<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(r->cols[keys[0]]->p, w0, c1, 4, nullptr, kw->as<uint64_t>(), r->rows);
    check_launch(c, "build_key");
    return kw;
}

// hash_join_v2: see include/xlb.h.  Returns a fresh relation.
xlb_rel* rel_join(xlb_ctx* c, const xlb_rel* l, const xlb_rel* r, const uint32_t* lk, const uint32_t* rk, uint32_t nk, xlb_join_type type) {
    if (nk < 1 || nk > XLB_MAX_KEYS || !lk || !rk) xlb_fail(XLB_ERR_INVALID, "join needs 1..%u key columns", XLB_MAX_KEYS);
    for (uint32_t i = 0; i < nk; ++i) {
        if (lk[i] >= l->schema.arity || rk[i] >= r->schema.arity) xlb_fail(XLB_ERR_INVALID, "join key column out of range");
        uint8_t a = l->schema.types[lk[i]] == XLB_SYMBOL ? XLB_U32 : l->schema.types[lk[i]];
        uint8_t b = r->schema.types[rk[i]] == XLB_SYMBOL ? XLB_U32 : r->schema.types[rk[i]];
        if (a != b) xlb_fail(XLB_ERR_TYPE, "join key %u: type mismatch", i);
        if (a == XLB_BOOL) xlb_fail(XLB_ERR_UNSUPPORTED, "join key %u: bool key columns are not built", i);
    }
    xlb_schema os = l->schema;
    if (type == XLB_JOIN_INNER) {
        if (l->schema.arity + r->schema.arity > XLB_MAX_ARITY) xlb_fail(XLB_ERR_UNSUPPORTED, "join output arity above %u", XLB_MAX_ARITY);
        for (uint32_t i = 0; i < r->schema.arity; ++i) os.types[os.arity++] = r->schema.types[i];
    }
    bool empty = l->rows == 0 || (r->rows == 0 && type != XLB_JOIN_ANTI);
    if (empty) {
        xlb_rel* o = rel_empty(c, os);
        o->canonical = false;
        return o;
    }
    if (l->rows >= (1ull << 32)) xlb_fail(XLB_ERR_CAPACITY, "join probe side exceeds the 2^32 row limit");
    ops_rel_columns(c, l);
    ops_rel_columns(c, r);
    // build side: rows ordered by key word (stable, so equal keys keep right-row order)
    Buf rkeys = join_keys(c, r, rk, nk);
    Buf ridx = make_buf(c, r->rows * 4);
    if (r->rows) {
        prof_begin(c, "iota", 0);
        iota_k<<<grid_for(c, r->rows), BLOCK, 0, c->stream>>>(ridx->as<uint32_t>(), r->rows);
        check_launch(c, "iota");
        radix_sort(c, rkeys, &ridx, r->rows);
    }
    Index ix = ops_index_build(c, rkeys, r->rows, 0, ridx);
    Buf lkeys = join_keys(c, l, lk, nk);
    Keys lrows;
    lrows.n = l->rows;
    lrows.buf = make_buf(c, l->rows * 8);
    prof_begin(c, "iota64", 0);
    iota64_k<<<grid_for(c, l->rows), BLOCK, 0, c->stream>>>(lrows.buf->as<uint64_t>(), l->rows);
    check_launch(c, "iota64");
    if (type == XLB_JOIN_INNER) {
        Keys pairs = ops_join_expand(c, lrows, SRC_LO, lkeys->as<uint64_t>(), ix, SRC_LO, SRC_OTHER);
        std::unique_ptr<xlb_rel> o(new xlb_rel);
        o->ctx = c;
        o->schema = os;
        o->rows = pairs.n;
        for (uint32_t i = 0; i < os.arity; ++i) {
            bool left = i < l->schema.arity;
            const xlb_rel* src = left ? l : r;
            uint32_t sc = left ? i : i - l->schema.arity;
            uint32_t w = type_width(os.types[i]);
            o->cols[i] = make_buf(c, pairs.n * w);
            if (!pairs.n) continue;
            prof_begin(c, "gather_pair", 0);
            if (w == 4) gather_pair_k<uint32_t><<<grid_for(c, pairs.n), BLOCK, 0, c->stream>>>(src->cols[sc]->as<uint32_t>(), pairs.ptr(), left ? 0 : 1, o->cols[i]->as<uint32_t>(), pairs.n);
            else if (w == 8) gather_pair_k<uint64_t><<<grid_for(c, pairs.n), BLOCK, 0, c->stream>>>(src->cols[sc]->as<uint64_t>(), pairs.ptr(), left ? 0 : 1, o->cols[i]->as<uint64_t>(), pairs.n);
            else gather_pair_k<uint8_t><<<grid_for(c, pairs.n), BLOCK, 0, c->stream>>>(src->cols[sc]->as<uint8_t>(), pairs.ptr(), left ? 0 : 1, o->cols[i]->as<uint8_t>(), pairs.n);
            check_launch(c, "gather_pair");
        }
        return o.release();
    }
    Buf match = ops_probe_match(c, lrows, SRC_LO, lkeys->as<uint64_t>(), ix);
    Buf sel = make_buf(c, l->rows * 4);
    uint64_t m = select(c, PredFlag{match->as<uint64_t>(), type == XLB_JOIN_SEMI}, EmitIndex{sel->as<uint32_t>()}, l->rows);
    return gather_rel(c, l, sel->as<uint32_t>(), m);
}

extern "C" xlb_status xlb_hash_join(xlb_ctx* c, const xlb_rel* l, const xlb_rel* r, const uint32_t* lk, const uint32_t* rk, uint32_t nk,
                                    xlb_join_type type, xlb_rel** out_final) {
    if (!c || !l || !r || !out_final) return XLB_ERR_INVALID;
    API_BEGIN(c)
    ResultGuard guard;
    guard.r = rel_join(c, l, r, lk, rk, nk, type);
    guard.deliver(c, out_final);
    API_END()
}
