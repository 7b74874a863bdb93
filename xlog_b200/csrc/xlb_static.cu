// xlb_dedup_sorted_u64_static: duplicate removal over sorted keys with all scratch memory in a
// fixed device array that is part of the library image.
//
// Who this is for: code that must not allocate device memory at the point of the call — a
// host runtime that has handed the whole GPU to its own arena and forbids cudaMalloc from
// plug-ins, a latency-critical section where an allocation could synchronise the device, or a
// caller that simply has no allocator handle to pass down.  The ordinary entry points
// (xlb_dedup and friends) take their scratch from the context's stream-ordered pool; this one
// takes none: the caller passes device pointers for the input, the output and the count, and
// the tile counters, tile offsets and scan partials live in `g_static_scratch` below.
#include <atomic>

#include "xlb_kernels.cuh"

using namespace xk;

// Largest input the fixed scratch serves: 2^26 keys (512 MiB of keys).
static constexpr uint64_t STATIC_MAX_KEYS = 1ull << 26;
static constexpr uint64_t STATIC_MAX_TILES = STATIC_MAX_KEYS / SCAN_TILE;                    // 32768 tiles of 2048 keys
static constexpr uint64_t STATIC_MAX_SPINE = (STATIC_MAX_TILES + SCAN_TILE - 1) / SCAN_TILE;  // tiles of the scan over tile counts

// Layout (bytes): [0,8) total | tile counts u32 | tile offsets u64 | scan partials u64.
static constexpr uint64_t OFF_COUNTS = 256;
static constexpr uint64_t OFF_OFFS = OFF_COUNTS + STATIC_MAX_TILES * 4;
static constexpr uint64_t OFF_SPINE = OFF_OFFS + STATIC_MAX_TILES * 8;
static constexpr uint64_t STATIC_BYTES = OFF_SPINE + STATIC_MAX_SPINE * 8 + 256;

// About 385 KiB, resident on every GPU that loads the library until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_BYTES];

// In host code the array's name is only a handle for the runtime, not a device address; the
// address kernels can use comes from cudaGetSymbolAddress, per device.
// (looked up once per device; several host threads may race to store the same value)
static std::atomic<unsigned char*> g_scratch_ptr[64];

static thread_local char g_static_error[256] = "";

extern "C" const char* xlb_static_last_error(void) { return g_static_error; }

extern "C" uint64_t xlb_dedup_sorted_u64_static_max(void) { return STATIC_MAX_KEYS; }

extern "C" xlb_status xlb_dedup_sorted_u64_static(const uint64_t* d_sorted, uint64_t n, uint64_t* d_unique, uint64_t* d_count, void* cuda_stream) {
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    auto fail = [&](xlb_status st, const char* what, cudaError_t e) {
        snprintf(g_static_error, sizeof g_static_error, "%s%s%s", what, e != cudaSuccess ? ": " : "", e != cudaSuccess ? cudaGetErrorString(e) : "");
        return st;
    };
    if (!d_count || (n && (!d_sorted || !d_unique))) return fail(XLB_ERR_INVALID, "null pointer argument", cudaSuccess);
    if (n > STATIC_MAX_KEYS) {
        snprintf(g_static_error, sizeof g_static_error, "%llu keys exceed the %llu keys the fixed scratch serves; use xlb_dedup", (unsigned long long)n,
                 (unsigned long long)STATIC_MAX_KEYS);
        return XLB_ERR_CAPACITY;
    }
    if (n) {
        // blocks write output positions while other blocks still read input: the two ranges must not overlap
        const uintptr_t in0 = (uintptr_t)d_sorted, in1 = in0 + n * 8, out0 = (uintptr_t)d_unique, out1 = out0 + n * 8;
        if (in0 < out1 && out0 < in1) return fail(XLB_ERR_INVALID, "the input and output key ranges overlap; pass separate buffers", cudaSuccess);
    }
    // An error some earlier work of the caller left pending would be taken for (and cleared as) a
    // launch failure of this call: refuse to start, and leave it for the caller to read.
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return fail(XLB_ERR_CUDA, "a CUDA error was already pending when the call began", e);
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(XLB_ERR_CUDA, "cudaGetDevice", e);
    if (dev < 0 || dev >= 64) return fail(XLB_ERR_UNSUPPORTED, "device ordinal above 63", cudaSuccess);
    unsigned char* base = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!base) {
        // set-up, once per device, with that device current
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) return fail(XLB_ERR_CUDA, "cudaGetSymbolAddress(g_static_scratch)", e);
        base = (unsigned char*)p;
        g_scratch_ptr[dev].store(base, std::memory_order_release);
    }
    uint64_t* total = (uint64_t*)base;
    uint32_t* counts = (uint32_t*)(base + OFF_COUNTS);
    uint64_t* offs = (uint64_t*)(base + OFF_OFFS);
    uint64_t* spine = (uint64_t*)(base + OFF_SPINE);

    if (n == 0) {
        e = cudaMemsetAsync(d_count, 0, 8, stream);
        if (e != cudaSuccess) return fail(XLB_ERR_CUDA, "cudaMemsetAsync", e);
    } else {
        PredHead pred{d_sorted};
        EmitKey emit{d_sorted, d_unique};
        uint64_t ntiles = (n + SCAN_TILE - 1) / SCAN_TILE;
        if (ntiles == 1) {
            select_write_k<PredHead, EmitKey><<<1, BLOCK, 0, stream>>>(pred, emit, n, nullptr, d_count);
        } else {
            // every scratch word that is read below is written first by these launches, so nothing
            // left behind by an earlier call is ever observed
            select_count_k<PredHead><<<(unsigned)ntiles, BLOCK, 0, stream>>>(pred, n, counts);
            LoadU32 load{counts};
            uint64_t stiles = (ntiles + SCAN_TILE - 1) / SCAN_TILE;
            if (stiles == 1) {
                scan_apply_k<LoadU32, uint64_t><<<1, BLOCK, 0, stream>>>(load, ntiles, nullptr, offs, total);
            } else {
                scan_reduce_k<LoadU32, uint64_t><<<(unsigned)stiles, BLOCK, 0, stream>>>(load, ntiles, spine);
                scan_spine_k<uint64_t><<<1, 1024, 0, stream>>>(spine, stiles, total);
                scan_apply_k<LoadU32, uint64_t><<<(unsigned)stiles, BLOCK, 0, stream>>>(load, ntiles, spine, offs, nullptr);
            }
            select_write_k<PredHead, EmitKey><<<(unsigned)ntiles, BLOCK, 0, stream>>>(pred, emit, n, offs, nullptr);
            e = cudaMemcpyAsync(d_count, total, 8, cudaMemcpyDeviceToDevice, stream);
            if (e != cudaSuccess) return fail(XLB_ERR_CUDA, "cudaMemcpyAsync(count)", e);
        }
        e = cudaGetLastError();
        if (e != cudaSuccess) return fail(XLB_ERR_CUDA, "kernel launch", e);
    }
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(XLB_ERR_CUDA, "cudaStreamSynchronize", e);
    g_static_error[0] = 0;
    return XLB_OK;
}
