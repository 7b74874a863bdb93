// Shared host-side plumbing: status handling, the context, the stream-ordered device arena.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include <chrono>
#include <algorithm>
#include <cstdarg>
#include <cstring>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
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

// Driver entry points of the virtual-memory API, looked up through the runtime so that the
// library does not link against the driver library (it must load on a machine without one).
struct VmmApi {
    PFN_cuMemAddressReserve reserve = nullptr;
    PFN_cuMemAddressFree addr_free = nullptr;
    PFN_cuMemCreate create = nullptr;
    PFN_cuMemRelease release = nullptr;
    PFN_cuMemMap map = nullptr;
    PFN_cuMemUnmap unmap = nullptr;
    PFN_cuMemSetAccess set_access = nullptr;
    PFN_cuMemGetAllocationGranularity granularity = nullptr;
    bool ok = false;
    static const VmmApi& get() {
        static const VmmApi api = load();
        return api;
    }
    static VmmApi load() {
        VmmApi a;
        auto sym = [](const char* name, void** fn) {
            cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
            return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess && *fn != nullptr;
        };
        a.ok = sym("cuMemAddressReserve", (void**)&a.reserve) && sym("cuMemAddressFree", (void**)&a.addr_free) && sym("cuMemCreate", (void**)&a.create) &&
               sym("cuMemRelease", (void**)&a.release) && sym("cuMemMap", (void**)&a.map) && sym("cuMemUnmap", (void**)&a.unmap) &&
               sym("cuMemSetAccess", (void**)&a.set_access) && sym("cuMemGetAllocationGranularity", (void**)&a.granularity);
        if (!a.ok) cudaGetLastError();
        return a;
    }
};

// Device memory arena.  Every buffer of a context is used on the context's one stream, so a block
// that the host has freed can be handed out again at once: the work that used it was enqueued
// earlier on the same stream.  That makes a plain host-side free list enough, and keeps the CUDA
// allocator off the hot path: a fixpoint allocates and frees a few hundred temporaries, and the
// driver's stream-ordered pool was measured to spend milliseconds remapping its reserve in one
// step out of three for the first twenty steps of a repeated workload.
//
// Backing store: one reserved virtual address range as large as the device's memory, with physical
// memory mapped at its front chunk by chunk (the driver's virtual-memory API).  The arena is then
// one contiguous block that grows at its end, free neighbours always coalesce, and a request that
// does not fit extends the last free block by the missing part only.  With separate cudaMalloc
// slabs instead, a repeated workload with 128 MB buffers was seen to need a new 1 GB slab (a 4 to
// 11 ms stall) in its eighth repetition with 380 MB free in six pieces.  Slabs remain as the
// fallback where the virtual-memory API is unavailable (or XLB_ARENA_SLABS is set).
struct Arena {
    struct Slab {
        char* base;
        uint64_t size;
    };
    struct Chunk {
        CUmemGenericAllocationHandle handle;
        uint64_t size;
    };
    std::vector<Slab> slabs;    // fallback backing
    std::vector<Chunk> chunks;  // virtual-memory backing: mapped back to back from va_base
    char* va_base = nullptr;
    uint64_t va_size = 0, mapped = 0, gran = 0;
    int device = 0;
    bool vmm = false, vmm_tried = false;
    std::map<char*, uint64_t> free_by_addr;
    std::multimap<uint64_t, char*> free_by_size;
    uint64_t reserved = 0;
    bool trace = getenv("XLB_ARENA_TRACE") != nullptr;  // report every time the arena has to grow
    static constexpr uint64_t ALIGN = 512, MIN_SLAB = 256ull << 20, MAX_GROW = 8ull << 30;
    static constexpr uint64_t VMM_MIN_STEP = 64ull << 20, VMM_MAX_STEP = 2ull << 30;

    static uint64_t round_up(uint64_t n) { return (n + ALIGN - 1) / ALIGN * ALIGN; }
    void insert_free(char* p, uint64_t n) {
        free_by_addr[p] = n;
        free_by_size.emplace(n, p);
    }
    void erase_free(char* p, uint64_t n) {
        free_by_addr.erase(p);
        auto r = free_by_size.equal_range(n);
        for (auto it = r.first; it != r.second; ++it)
            if (it->second == p) {
                free_by_size.erase(it);
                break;
            }
    }
    CUmemAllocationProp vmm_prop() const {
        CUmemAllocationProp prop;
        memset(&prop, 0, sizeof prop);
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = device;
        return prop;
    }
    // Reserve the address range (once).  False: use slabs.
    bool vmm_start() {
        if (vmm_tried) return vmm;
        vmm_tried = true;
        if (getenv("XLB_ARENA_SLABS")) return false;
        const VmmApi& api = VmmApi::get();
        int supported = 0;
        if (!api.ok || cudaDeviceGetAttribute(&supported, cudaDevAttrMemoryPoolsSupported, device) != cudaSuccess || !supported) {
            cudaGetLastError();
            return false;
        }
        CUmemAllocationProp prop = vmm_prop();
        size_t g = 0;
        if (api.granularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0) return false;
        size_t free_b = 0, total_b = 0;
        if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        gran = g;
        va_size = (total_b + gran - 1) / gran * gran;
        CUdeviceptr base = 0;
        if (api.reserve(&base, va_size, 0, 0, 0) != CUDA_SUCCESS) return false;
        va_base = (char*)base;
        vmm = true;
        return true;
    }
    // Map `step` more bytes at the end of the mapped part and hand them to the free list.
    bool vmm_map(uint64_t step) {
        const VmmApi& api = VmmApi::get();
        if (mapped + step > va_size) return false;
        CUmemAllocationProp prop = vmm_prop();
        CUmemGenericAllocationHandle h;
        if (api.create(&h, step, &prop, 0) != CUDA_SUCCESS) return false;
        CUdeviceptr at = (CUdeviceptr)(va_base + mapped);
        if (api.map(at, step, 0, h, 0) != CUDA_SUCCESS) {
            api.release(h);
            return false;
        }
        CUmemAccessDesc acc;
        memset(&acc, 0, sizeof acc);
        acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc.location.id = device;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        if (api.set_access(at, step, &acc, 1) != CUDA_SUCCESS) {
            api.unmap(at, step);
            api.release(h);
            return false;
        }
        chunks.push_back({h, step});
        char* p = va_base + mapped;
        mapped += step;
        reserved += step;
        release(p, step);  // coalesces with a free block that ended at the old end
        return true;
    }
    // size of the free block that ends where the mapped part ends (0: none)
    uint64_t vmm_tail_free() const {
        if (free_by_addr.empty()) return 0;
        auto last = std::prev(free_by_addr.end());
        return last->first + last->second == va_base + mapped ? last->second : 0;
    }
    bool vmm_grow(uint64_t n) {
        const uint64_t tail = vmm_tail_free();
        const uint64_t need = ((n > tail ? n - tail : 0) + gran - 1) / gran * gran;
        if (need == 0) return true;
        // grow by half of what is mapped, within [64 MB, 2 GB], or by the request if that is more
        uint64_t step = std::max<uint64_t>(need, std::min<uint64_t>(std::max<uint64_t>(mapped / 2, VMM_MIN_STEP), VMM_MAX_STEP));
        step = (step + gran - 1) / gran * gran;
        return vmm_map(step) || (step > need && vmm_map(need));
    }
    // Unmap whole chunks at the end that are entirely free (after the stream has drained).
    void vmm_trim() {
        const VmmApi& api = VmmApi::get();
        while (!chunks.empty()) {
            const uint64_t tail = vmm_tail_free(), sz = chunks.back().size;
            if (tail < sz) break;
            char* tail_at = va_base + mapped - tail;
            erase_free(tail_at, tail);
            if (tail > sz) insert_free(tail_at, tail - sz);
            api.unmap((CUdeviceptr)(va_base + mapped - sz), sz);
            api.release(chunks.back().handle);
            chunks.pop_back();
            mapped -= sz;
            reserved -= sz;
        }
    }
    bool add_slab(uint64_t size) {
        void* p = nullptr;
        if (cudaMalloc(&p, size) != cudaSuccess) {
            cudaGetLastError();  // clear the sticky-less allocation error
            return false;
        }
        slabs.push_back({(char*)p, size});
        reserved += size;
        insert_free((char*)p, size);
        return true;
    }
    // Give back every part of the backing store that is entirely free (after the stream has drained).
    void trim(cudaStream_t stream) {
        cudaStreamSynchronize(stream);
        if (vmm) {
            vmm_trim();
            return;
        }
        for (size_t i = 0; i < slabs.size();) {
            auto it = free_by_addr.find(slabs[i].base);
            if (it != free_by_addr.end() && it->second == slabs[i].size) {
                erase_free(slabs[i].base, slabs[i].size);
                cudaFree(slabs[i].base);
                reserved -= slabs[i].size;
                slabs.erase(slabs.begin() + i);
            } else ++i;
        }
    }
    void* alloc(uint64_t n, cudaStream_t stream) {
        n = round_up(n);
        for (int attempt = 0; attempt < 3; ++attempt) {
            auto it = free_by_size.lower_bound(n);  // best fit
            if (it != free_by_size.end()) {
                char* p = it->second;
                uint64_t have = it->first;
                erase_free(p, have);
                if (have > n) insert_free(p + n, have - n);
                return p;
            }
            if (trace) {
                uint64_t free_total = 0;
                for (auto& f : free_by_size) free_total += f.first;
                fprintf(stderr, "[xlb arena] attempt %d: no block of %llu bytes; reserved %llu in %zu pieces, free %llu in %zu blocks, largest %llu\n", attempt,
                        (unsigned long long)n, (unsigned long long)reserved, vmm ? chunks.size() : slabs.size(), (unsigned long long)free_total, free_by_size.size(),
                        (unsigned long long)(free_by_size.empty() ? 0 : free_by_size.rbegin()->first));
            }
            if (vmm_start()) {
                if (attempt == 0 && vmm_grow(n)) continue;
                return nullptr;  // the device (or the address range) is full: trimming this arena cannot help it
            }
            if (attempt == 0) {
                uint64_t grow = std::max<uint64_t>(MIN_SLAB, std::min<uint64_t>(reserved, MAX_GROW));
                if (add_slab(std::max(n, grow)) || (grow > n && add_slab(n))) continue;
            } else if (attempt == 1) {
                trim(stream);
                if (add_slab(n)) continue;
            }
        }
        return nullptr;
    }
    void release(void* ptr, uint64_t n) {
        char* p = (char*)ptr;
        n = round_up(n);
        auto next = free_by_addr.lower_bound(p);
        // coalesce with the free block after and before, unless a slab boundary lies between
        if (next != free_by_addr.end() && next->first == p + n && !is_slab_base(next->first)) {
            uint64_t m = next->second;
            erase_free(next->first, m);
            n += m;
        }
        auto prev = free_by_addr.lower_bound(p);
        if (prev != free_by_addr.begin()) {
            --prev;
            if (prev->first + prev->second == p && !is_slab_base(p)) {
                char* q = prev->first;
                uint64_t m = prev->second;
                erase_free(q, m);
                p = q;
                n += m;
            }
        }
        insert_free(p, n);
    }
    bool is_slab_base(char* p) const {
        for (auto& s : slabs)
            if (s.base == p) return true;
        return false;
    }
    void destroy() {
        for (auto& s : slabs) cudaFree(s.base);
        slabs.clear();
        if (vmm) {
            const VmmApi& api = VmmApi::get();
            uint64_t at = mapped;
            for (size_t i = chunks.size(); i-- > 0;) {
                at -= chunks[i].size;
                api.unmap((CUdeviceptr)(va_base + at), chunks[i].size);
                api.release(chunks[i].handle);
            }
            chunks.clear();
            api.addr_free((CUdeviceptr)va_base, va_size);
            va_base = nullptr;
            va_size = mapped = 0;
            vmm = vmm_tried = false;
        }
        free_by_addr.clear();
        free_by_size.clear();
        reserved = 0;
    }
};

struct xlb_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    Arena arena;
    uint64_t budget = 0, allocated = 0, peak = 0;
    uint64_t max_iterations = 1000000;
    uint64_t join_chunk = 0;
    uint32_t flags = 0;
    uint64_t launches = 0;
    uint64_t syncs = 0;       // host waits on the stream (count read-backs)
    double ms_sync_wait = 0;  // wall time spent inside those waits
    double ms_alloc = 0;      // wall time spent in the device allocator (allocate + free calls)
    std::string last_error;
    // pinned scratch for scalar read-backs
    unsigned long long* h_scalar = nullptr;  // 64 words
    unsigned long long* h_scalar_dev = nullptr;  // the same words as the device sees them (mapped): a kernel can leave counts there
    unsigned long long publish_seq = 0;          // number of the last set of counts a kernel was asked to leave there
    DevStatus* d_status = nullptr;
    int sm_count = 148;
    // executor state
    std::map<uint32_t, std::string> rel_names;
    std::map<std::string, xlb_rel*> store;
    std::map<std::string, uint64_t> versions;
    struct IndexCache* indexes = nullptr;
    Comm* comm = nullptr;
    // `world` / `rank` are what the executor plans by; while a strongly connected component runs
    // on replicated relations they read 1 / 0 although the communicator has comm_world ranks.
    uint32_t rank = 0, world = 1;
    uint32_t comm_rank = 0, comm_world = 1;
    void (*wait_hook)(xlb_ctx*) = nullptr;  // set with a communicator: host waits then watch it as well
    // bounded look-back of the one-sweep sort: polls before a tile gives up (XLB_ERR_TIMEOUT), and
    // the number the first tile takes (0; a test makes tile 0 never run so that the wait runs out)
    unsigned lb_spin_limit = 1u << 22, lb_first_tile = 0;
    bool sort_attr_set = false;  // the scatter kernels' shared-memory opt-in was made on this context's device
    // per-kernel event timing (xlb_profile_enable)
    struct ProfEntry {
        uint64_t launches = 0, bytes = 0;
        double ms = 0;
        std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending;
    };
    std::map<std::string, ProfEntry> prof;
    std::string prof_filter;  // "" = off, "*" = every kernel, else kernel names separated by commas
    ProfEntry* prof_open = nullptr;
    cudaEvent_t prof_e0 = nullptr;
    // host timeline of one plan execution (XLB_TRACE_HOST=1): every launch and every wait with its
    // wall-clock interval, printed to stderr when the plan is done
    struct TraceNote {
        double t0, t1;
        const char* what;
    };
    bool trace_on = false;
    std::vector<TraceNote> trace;
};

// Counts a kernel leaves in pinned memory for the host: low 40 bits the count, top 24 the number
// of the launch that wrote it.
constexpr int PUBLISH_COUNT_BITS = 40;
constexpr unsigned long long PUBLISH_TAG_MASK = 0xFFFFFFull;

inline double trace_now() { return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
inline void trace_note(xlb_ctx* c, const char* what, double t0) {
    if (c->trace_on) c->trace.push_back({t0, trace_now(), what});
}

// Bracket one launch with CUDA events on the launching stream when its kernel is profiled.
inline void prof_begin(xlb_ctx* c, const char* name, uint64_t bytes) {
    if (c->trace_on) trace_note(c, name, trace_now());
    if (c->prof_filter.empty()) return;
    if (c->prof_filter != "*") {  // a kernel name, or several separated by commas
        const std::string& f = c->prof_filter;
        const size_t len = strlen(name);
        bool hit = false;
        for (size_t at = f.find(name); at != std::string::npos && !hit; at = f.find(name, at + 1))
            hit = (at == 0 || f[at - 1] == ',') && (at + len == f.size() || f[at + len] == ',');
        if (!hit) return;
    }
    auto& e = c->prof[name];
    e.launches++;
    e.bytes += bytes;
    cudaEventCreate(&c->prof_e0);
    cudaEventRecord(c->prof_e0, c->stream);
    c->prof_open = &e;
}

// Bytes of a launch that the host learns only later (a count read back after the launch).
inline void prof_add_bytes(xlb_ctx* c, const char* name, uint64_t bytes) {
    if (c->prof_filter.empty()) return;
    auto it = c->prof.find(name);
    if (it != c->prof.end()) it->second.bytes += bytes;
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
        auto t0 = std::chrono::steady_clock::now();
        p = c->arena.alloc(n, c->stream);
        c->ms_alloc += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        if (!p)
            xlb_fail(XLB_ERR_RESOURCE_EXHAUSTED, "device memory exhausted: %llu bytes requested with %llu allocated and %llu reserved",
                     (unsigned long long)n, (unsigned long long)c->allocated, (unsigned long long)c->arena.reserved);
        c->allocated += n;
        if (c->allocated > c->peak) c->peak = c->allocated;
    }
    ~DevBuf() {
        if (p) {
            ctx->arena.release(p, bytes);
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
    const double tr0 = c->trace_on ? trace_now() : 0;
    if (c->wait_hook) {  // several ranks: never block for good on a stream a late peer may be holding up
        c->wait_hook(c);
        trace_note(c, "wait (communicator watched)", tr0);
        return;
    }
    auto t0 = std::chrono::steady_clock::now();
    static const bool spin = getenv("XLB_BLOCKING_WAIT") == nullptr;
    if (spin) {  // poll first: a fixpoint waits for a row count many times, and a blocked thread's wake-up
                 // costs milliseconds on a busy host; after 5 ms fall back to a blocking wait
        for (;;) {
            cudaError_t q = cudaStreamQuery(c->stream);
            if (q == cudaSuccess) break;
            if (q != cudaErrorNotReady) CUDA_OK(q);
            if (std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() > 5.0) break;
        }
    }
    CUDA_OK(cudaStreamSynchronize(c->stream));
    c->ms_sync_wait += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    c->syncs++;
    trace_note(c, "wait", tr0);
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
inline bool type_built(uint8_t t) { return t <= XLB_SYMBOL; }
inline bool type_unsigned(uint8_t t) { return t == XLB_U32 || t == XLB_SYMBOL || t == XLB_U64; }
inline bool rel_packable(const xlb_schema& s) {
    if (s.arity < 1 || s.arity > 2) return false;
    for (uint32_t i = 0; i < s.arity; ++i)
        if (s.types[i] != XLB_U32 && s.types[i] != XLB_SYMBOL) return false;
    return true;
}
