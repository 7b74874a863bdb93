// Shared host-side plumbing: status handling, the context, the stream-ordered device arena.
#pragma once
#include <cuda_runtime.h>

#include <chrono>
#include <cstdarg>
#include <cstring>
#include <cstdint>
#include <cstdio>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/xlb.h"

struct XlbError {
    xlb_status st;
    std::string msg;
};

[[noreturn]] inline void xlb_fail(xlb_status st, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    throw XlbError{st, buf};
}

#define CUDA_OK(expr)                                                                            \
    do {                                                                                         \
        cudaError_t e__ = (expr);                                                                \
        if (e__ != cudaSuccess)                                                                  \
            xlb_fail(e__ == cudaErrorMemoryAllocation ? XLB_ERR_RESOURCE_EXHAUSTED : XLB_ERR_CUDA, \
                     "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
    } while (0)

struct Comm;  // NCCL exchange layer (xlb_comm.cu)

// Device-side status word, after the reference's ResidentTerminalStatus convention
// (crates/xlog-cuda/kernels/resident_relational.cu:22-31): kernels never trap; the first failure
// publishes (code, detail) and the host reads it at the next phase boundary.
struct DevStatus {
    unsigned int code;   // xlb_status
    unsigned int where;  // kernel-specific site id
    unsigned long long detail;
};

struct xlb_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaMemPool_t pool = nullptr;
    uint64_t budget = 0, allocated = 0, peak = 0;
    uint64_t max_iterations = 1000000;
    uint64_t join_chunk = 0;
    uint32_t flags = 0;
    uint64_t launches = 0;
    uint64_t syncs = 0;       // host waits on the stream (count read-backs)
    double ms_sync_wait = 0;  // wall time spent inside those waits
    std::string last_error;
    // pinned scratch for scalar read-backs
    unsigned long long* h_scalar = nullptr;  // 64 words
    DevStatus* d_status = nullptr;
    int sm_count = 148;
    // executor state
    std::map<uint32_t, std::string> rel_names;
    std::map<std::string, xlb_rel*> store;
    std::map<std::string, uint64_t> versions;
    struct IndexCache* indexes = nullptr;
    Comm* comm = nullptr;
    uint32_t rank = 0, world = 1;
    // per-kernel event timing (xlb_profile_enable)
    struct ProfEntry {
        uint64_t launches = 0, bytes = 0;
        double ms = 0;
        std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending;
    };
    std::map<std::string, ProfEntry> prof;
    std::string prof_filter;  // "" = off, "*" = every kernel, else one kernel name
    ProfEntry* prof_open = nullptr;
    cudaEvent_t prof_e0 = nullptr;
};

// Bracket one launch with CUDA events on the launching stream when its kernel is profiled.
inline void prof_begin(xlb_ctx* c, const char* name, uint64_t bytes) {
    if (c->prof_filter.empty()) return;
    if (c->prof_filter != "*" && c->prof_filter != name) return;
    auto& e = c->prof[name];
    e.launches++;
    e.bytes += bytes;
    cudaEventCreate(&c->prof_e0);
    cudaEventRecord(c->prof_e0, c->stream);
    c->prof_open = &e;
}

// A device allocation charged to the context's budget (GpuMemoryManager::alloc with a
// MemoryBudget, crates/xlog-cuda/src/memory.rs:57-1350).  Freed stream-ordered.
struct DevBuf {
    xlb_ctx* ctx;
    void* p = nullptr;
    uint64_t bytes = 0;
    DevBuf(xlb_ctx* c, uint64_t n) : ctx(c), bytes(n) {
        if (n == 0) return;
        if (c->budget && c->allocated + n > c->budget)
            xlb_fail(XLB_ERR_RESOURCE_EXHAUSTED, "device memory budget exceeded: %llu + %llu > %llu bytes",
                     (unsigned long long)c->allocated, (unsigned long long)n, (unsigned long long)c->budget);
        CUDA_OK(cudaMallocAsync(&p, n, c->pool, c->stream));
        c->allocated += n;
        if (c->allocated > c->peak) c->peak = c->allocated;
    }
    ~DevBuf() {
        if (p) {
            cudaFreeAsync(p, ctx->stream);
            ctx->allocated -= bytes;
        }
    }
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    template <class T>
    T* as() const { return (T*)p; }
};
using Buf = std::shared_ptr<DevBuf>;
inline Buf make_buf(xlb_ctx* c, uint64_t bytes) { return std::make_shared<DevBuf>(c, bytes); }

inline void check_launch(xlb_ctx* c, const char* what) {
    c->launches++;
    if (c->prof_open) {
        cudaEvent_t e1;
        cudaEventCreate(&e1);
        cudaEventRecord(e1, c->stream);
        c->prof_open->pending.emplace_back(c->prof_e0, e1);
        c->prof_open = nullptr;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) xlb_fail(XLB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
}

// Read `n` 64-bit words from device memory (one stream synchronisation).
inline void stream_wait(xlb_ctx* c) {
    auto t0 = std::chrono::steady_clock::now();
    CUDA_OK(cudaStreamSynchronize(c->stream));
    c->ms_sync_wait += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    c->syncs++;
}

inline void read_words(xlb_ctx* c, const void* dptr, int n, unsigned long long* out) {
    CUDA_OK(cudaMemcpyAsync(c->h_scalar, dptr, (size_t)n * 8, cudaMemcpyDeviceToHost, c->stream));
    stream_wait(c);
    for (int i = 0; i < n; ++i) out[i] = c->h_scalar[i];
}

inline void check_dev_status(xlb_ctx* c) {
    DevStatus s;
    CUDA_OK(cudaMemcpyAsync(c->h_scalar, c->d_status, sizeof s, cudaMemcpyDeviceToHost, c->stream));
    stream_wait(c);
    memcpy(&s, c->h_scalar, sizeof s);
    if (s.code != 0) {
        CUDA_OK(cudaMemsetAsync(c->d_status, 0, sizeof s, c->stream));
        xlb_fail((xlb_status)s.code, "device kernel reported status %u at site %u (detail %llu)", s.code, s.where, s.detail);
    }
}

// The relation handle.  Either representation may be present; both describe the same rows.
//   cols   : column-major, one allocation per column (the ABI's layout);
//   packed : arity <= 2 and 32-bit columns only: one u64 per row, (c0 << 32) | c1 for arity 2,
//            c0 for arity 1, so ascending u64 order is the lexicographic column order.
struct xlb_rel {
    xlb_ctx* ctx = nullptr;
    xlb_schema schema{};
    uint64_t rows = 0;
    mutable Buf cols[XLB_MAX_ARITY];
    mutable Buf packed;
    mutable uint64_t or_bound = ~0ull;  // host-known upper bound of the OR of the packed rows (~0: unknown)
    bool canonical = false;
};

inline uint32_t type_width(uint8_t t) {
    switch (t) {
        case XLB_U32: case XLB_I32: case XLB_F32: case XLB_SYMBOL: return 4;
        case XLB_U64: case XLB_I64: case XLB_F64: return 8;
        default: return 1;
    }
}
inline bool type_built(uint8_t t) { return t != XLB_BOOL && t <= XLB_SYMBOL; }
inline bool type_unsigned(uint8_t t) { return t == XLB_U32 || t == XLB_SYMBOL || t == XLB_U64; }
inline bool rel_packable(const xlb_schema& s) {
    if (s.arity < 1 || s.arity > 2) return false;
    for (uint32_t i = 0; i < s.arity; ++i)
        if (s.types[i] != XLB_U32 && s.types[i] != XLB_SYMBOL) return false;
    return true;
}
