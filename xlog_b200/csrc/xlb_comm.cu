// NCCL exchange layer.  The library does not link NCCL: it binds the handful of entry points it
// needs at run time, from the NCCL already loaded into the process (the host program's, e.g.
// the one torch.distributed brought in) or else from libnccl.so.2 on the loader path, so a
// single-GPU user needs no NCCL at all.
#include <dlfcn.h>
#include <nccl.h>
#include <sched.h>

#include <chrono>
#include <cstdlib>

#include "xlb_comm.h"

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi& api() {
    static NcclApi a;
    if (a.handle) return a;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) xlb_fail(XLB_ERR_NCCL, "NCCL is not available: %s", dlerror());
#define BIND(name)                                                                  \
    a.name = (decltype(a.name))dlsym(h, "nccl" #name);                              \
    if (!a.name) xlb_fail(XLB_ERR_NCCL, "NCCL symbol nccl%s is missing", #name);
    BIND(GetUniqueId) BIND(CommInitRank) BIND(CommDestroy) BIND(CommAbort) BIND(CommGetAsyncError)
    BIND(GroupStart) BIND(GroupEnd) BIND(Send) BIND(Recv) BIND(AllReduce) BIND(AllGather) BIND(GetErrorString)
#undef BIND
    a.handle = h;
    return a;
}

#define NCCL_OK(expr)                                                                                   \
    do {                                                                                                \
        ncclResult_t r__ = (expr);                                                                      \
        if (r__ != ncclSuccess && r__ != ncclInProgress)                                                \
            xlb_fail(XLB_ERR_NCCL, "%s failed: %s", #expr, api().GetErrorString(r__));                  \
    } while (0)

// bit-wise OR of `parts` bitmaps of `words` words each, laid out back to back, into `out`
__global__ void bitmap_or_k(const unsigned int* __restrict__ gathered, uint32_t parts, uint64_t words, unsigned int* __restrict__ out) {
    for (uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (uint64_t)gridDim.x * blockDim.x) {
        unsigned int v = 0;
        for (uint32_t p = 0; p < parts; ++p) v |= gathered[(uint64_t)p * words + w];
        out[w] = v;
    }
}

}  // namespace

// Words per rank of the small host-visible staging area: a row of the count matrix (world counts,
// an OR bound, a spare) or an agreement vector of up to COMM_WORDS_MAX words.
static constexpr uint32_t STAGE_ROW = 64 + 2 + COMM_WORDS_MAX;

struct Comm {
    ncclComm_t comm = nullptr;
    bool aborted = false;     // set once the communicator was aborted: every later exchange fails at once
    double timeout_s = 120.0;
    Buf counts_dev;           // world rows of STAGE_ROW u64 (device side of the staging area)
    unsigned long long* h_stage = nullptr;  // pinned host copy of the gathered rows, plus one row to send from
};

static Comm* live_comm(xlb_ctx* c) {
    Comm* cm = c->comm;
    if (!cm) xlb_fail(XLB_ERR_INVALID, "internal: exchange without a communicator");
    if (cm->aborted || !cm->comm)
        xlb_fail(XLB_ERR_NCCL, "the communicator of this context was aborted after an earlier failure; create a new context");
    return cm;
}

static void abort_comm(Comm* cm) {
    if (cm->comm) api().CommAbort(cm->comm);
    cm->comm = nullptr;
    cm->aborted = true;
}

// Wait for the stream without ever blocking for good: poll the stream and the communicator's
// asynchronous error state (yielding the core between polls once the wait is not a short one);
// after the time limit abort the communicator and report a timeout.  Every host-visible result of
// an exchange is staged in pinned memory, so no copy blocks before this wait is reached.
static void comm_wait(xlb_ctx* c) {
    Comm* cm = c->comm;
    auto t0 = std::chrono::steady_clock::now();
    uint64_t polls = 0;
    for (;;) {
        cudaError_t q = cudaStreamQuery(c->stream);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady) xlb_fail(XLB_ERR_CUDA, "stream failed during an exchange: %s", cudaGetErrorString(q));
        if ((++polls & 15) == 0 && cm && cm->comm) {
            ncclResult_t ar = ncclSuccess;
            api().CommGetAsyncError(cm->comm, &ar);
            if (ar != ncclSuccess && ar != ncclInProgress) {
                abort_comm(cm);
                xlb_fail(XLB_ERR_NCCL, "NCCL reported an asynchronous error: %s", api().GetErrorString(ar));
            }
        }
        double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (cm && el > cm->timeout_s) {
            abort_comm(cm);
            xlb_fail(XLB_ERR_TIMEOUT, "exchange did not complete within %.0f s; communicator aborted", cm->timeout_s);
        }
        if (el > 100e-6) sched_yield();  // a peer is late: give the core to whoever may be feeding it
    }
    c->ms_sync_wait += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    c->syncs++;
}

void comm_destroy(xlb_ctx* c) {
    if (!c->comm) return;
    if (c->comm->comm) api().CommDestroy(c->comm->comm);
    if (c->comm->h_stage) cudaFreeHost(c->comm->h_stage);
    delete c->comm;
    c->comm = nullptr;
    c->wait_hook = nullptr;
    c->world = c->comm_world = 1;
    c->rank = c->comm_rank = 0;
}

bool comm_aborted(const xlb_ctx* c) { return c->comm && (c->comm->aborted || !c->comm->comm); }

extern "C" xlb_status xlb_comm_unique_id(uint8_t id[XLB_UNIQUE_ID_BYTES]) {
    try {
        static_assert(sizeof(ncclUniqueId) <= XLB_UNIQUE_ID_BYTES, "unique id size");
        ncclUniqueId u;
        NCCL_OK(api().GetUniqueId(&u));
        memset(id, 0, XLB_UNIQUE_ID_BYTES);
        memcpy(id, &u, sizeof u);
    } catch (const XlbError&) {
        return XLB_ERR_NCCL;
    }
    return XLB_OK;
}

extern "C" xlb_status xlb_comm_init(xlb_ctx* c, const uint8_t id[XLB_UNIQUE_ID_BYTES], uint32_t rank, uint32_t world) {
    if (!c || !id || world == 0 || rank >= world) return XLB_ERR_INVALID;
    try {
        if (world > 64) xlb_fail(XLB_ERR_UNSUPPORTED, "at most 64 ranks");
        comm_destroy(c);
        if (world == 1) return XLB_OK;
        CUDA_OK(cudaSetDevice(c->device));
        auto* cm = new Comm;
        c->comm = cm;
        if (const char* t = getenv("XLB_COMM_TIMEOUT_S")) cm->timeout_s = atof(t) > 0 ? atof(t) : cm->timeout_s;
        ncclUniqueId u;
        memcpy(&u, id, sizeof u);
        NCCL_OK(api().CommInitRank(&cm->comm, (int)world, u, (int)rank));
        c->rank = c->comm_rank = rank;
        c->world = c->comm_world = world;
        cm->counts_dev = make_buf(c, (uint64_t)world * STAGE_ROW * 8);
        CUDA_OK(cudaHostAlloc((void**)&cm->h_stage, (size_t)(world + 1) * STAGE_ROW * 8, cudaHostAllocDefault));
        c->wait_hook = comm_wait;  // every host wait of this context now watches the communicator too
    } catch (const XlbError& e) {
        c->last_error = e.msg;
        return e.st;
    }
    return XLB_OK;
}

// Test hook (no device work): puts the context into the state an aborted exchange leaves behind.
extern "C" xlb_status xlb_comm_mark_aborted_for_test(xlb_ctx* c) {
    if (!c) return XLB_ERR_INVALID;
    if (!c->comm) {
        c->comm = new Comm;
        c->world = c->comm_world = 2;
        c->rank = c->comm_rank = 0;
    }
    abort_comm(c->comm);
    return XLB_OK;
}

void comm_allgather_words(xlb_ctx* c, const uint64_t* mine, uint32_t k, uint64_t* all) {
    if (k > COMM_WORDS_MAX) xlb_fail(XLB_ERR_INVALID, "internal: agreement vector of %u words", k);
    Comm* cm = live_comm(c);
    const uint32_t W = c->comm_world;
    unsigned long long* dev = cm->counts_dev->as<unsigned long long>();
    unsigned long long* send = cm->h_stage + (size_t)W * STAGE_ROW;
    for (uint32_t i = 0; i < k; ++i) send[i] = mine[i];
    CUDA_OK(cudaMemcpyAsync(dev + (size_t)c->comm_rank * k, send, (size_t)k * 8, cudaMemcpyHostToDevice, c->stream));
    const double tr0 = c->trace_on ? trace_now() : 0;
    NCCL_OK(api().AllGather(dev + (size_t)c->comm_rank * k, dev, k, ncclUint64, cm->comm, c->stream));
    trace_note(c, "ncclAllGather (enqueue)", tr0);
    CUDA_OK(cudaMemcpyAsync(cm->h_stage, dev, (size_t)W * k * 8, cudaMemcpyDeviceToHost, c->stream));
    comm_wait(c);
    for (size_t i = 0; i < (size_t)W * k; ++i) all[i] = cm->h_stage[i];
}

uint64_t comm_allreduce_sum(xlb_ctx* c, uint64_t v) {
    if (c->comm_world <= 1) return v;
    std::vector<uint64_t> all(c->comm_world);
    comm_allgather_words(c, &v, 1, all.data());
    uint64_t s = 0;
    for (uint64_t x : all) s += x;
    return s;
}

Buf comm_gather_bitmaps(xlb_ctx* c, const unsigned int* bitmap, uint64_t words) {
    Comm* cm = live_comm(c);
    Buf gathered = make_buf(c, (uint64_t)c->comm_world * words * 4);
    const double tr0 = c->trace_on ? trace_now() : 0;
    NCCL_OK(api().AllGather(bitmap, gathered->p, words, ncclUint32, cm->comm, c->stream));
    trace_note(c, "ncclAllGather (enqueue)", tr0);
    return gathered;
}

void comm_or_bitmaps(xlb_ctx* c, unsigned int* bitmap, uint64_t words) {
    const uint32_t W = c->comm_world;
    Buf gathered = comm_gather_bitmaps(c, bitmap, words);
    uint64_t blocks = (words + 255) / 256;
    if (blocks > (uint64_t)c->sm_count * 8) blocks = (uint64_t)c->sm_count * 8;
    prof_begin(c, "bitmap_or", (uint64_t)W * words * 4 + words * 4);
    bitmap_or_k<<<(unsigned)blocks, 256, 0, c->stream>>>(gathered->as<unsigned int>(), W, words, bitmap);
    check_launch(c, "bitmap_or");
}

Keys comm_allgather_keys(xlb_ctx* c, const Keys& in) {
    Comm* cm = live_comm(c);
    const uint32_t W = c->comm_world;
    uint64_t mine[2] = {in.n, in.n ? in.bound : 0};
    std::vector<uint64_t> all((size_t)W * 2);
    comm_allgather_words(c, mine, 2, all.data());
    Keys out;
    out.bound = 0;
    for (uint32_t r = 0; r < W; ++r) {
        out.n += all[2 * r];
        out.bound |= all[2 * r + 1];
    }
    out.buf = make_buf(c, out.n * 8);
    NCCL_OK(api().GroupStart());
    uint64_t at = 0;
    for (uint32_t r = 0; r < W; ++r) {
        const uint64_t n = all[2 * r];
        if (r == c->comm_rank) {
            if (n) CUDA_OK(cudaMemcpyAsync(out.buf->as<uint64_t>() + at, in.ptr(), n * 8, cudaMemcpyDeviceToDevice, c->stream));
        } else {
            if (in.n) NCCL_OK(api().Send(in.ptr(), in.n, ncclUint64, (int)r, cm->comm, c->stream));
            if (n) NCCL_OK(api().Recv(out.buf->as<uint64_t>() + at, n, ncclUint64, (int)r, cm->comm, c->stream));
        }
        at += n;
    }
    NCCL_OK(api().GroupEnd());
    return out;
}

Keys comm_repartition(xlb_ctx* c, const Keys& in, int keysel, bool sorted_unique_result, xlb_run_stats& st) {
    if (c->comm_world <= 1) return in;
    Comm* cm = live_comm(c);
    uint32_t W = c->comm_world;
    // partition into one run per destination; the run lengths go straight from device memory into
    // the all-gather, so every rank learns the whole count matrix with a single host wait.  Each
    // row of the matrix carries one more word: the sender's OR bound of its rows, so the receiver
    // knows the bits of what it gets without looking at it.
    // and the number of rows the sender holds: a row of counts that does not add up to it is seen by
    // every rank in the gathered matrix, so all of them fail the same way before any receive is
    // posted with a size nobody will send.
    const uint32_t RW = W + 2;
    unsigned long long* dev = cm->counts_dev->as<unsigned long long>();
    unsigned long long* mine = dev + (uint64_t)c->comm_rank * RW;
    Keys part = ops_partition_by_owner_dev(c, in, keysel, W, mine);
    unsigned long long* send_tail = cm->h_stage + (size_t)W * STAGE_ROW;
    send_tail[0] = in.n ? in.bound : 0;
    send_tail[1] = in.n;
    CUDA_OK(cudaMemcpyAsync(mine + W, send_tail, 16, cudaMemcpyHostToDevice, c->stream));
    const double tr0 = c->trace_on ? trace_now() : 0;
    NCCL_OK(api().AllGather(mine, dev, RW, ncclUint64, cm->comm, c->stream));
    trace_note(c, "ncclAllGather (enqueue)", tr0);
    CUDA_OK(cudaMemcpyAsync(cm->h_stage, dev, (size_t)W * RW * 8, cudaMemcpyDeviceToHost, c->stream));
    comm_wait(c);
    const unsigned long long* all = cm->h_stage;
    std::vector<uint64_t> send(W), recv(W);
    uint64_t bound = 0, total = 0;
    for (uint32_t r = 0; r < W; ++r) {
        uint64_t row_sum = 0;
        for (uint32_t d = 0; d < W; ++d) row_sum += all[(size_t)r * RW + d];
        if (row_sum != all[(size_t)r * RW + W + 1])
            xlb_fail(XLB_ERR_NCCL, "exchange: the send counts of rank %u add up to %llu, it holds %llu rows", r, (unsigned long long)row_sum,
                     (unsigned long long)all[(size_t)r * RW + W + 1]);
        send[r] = all[(size_t)c->comm_rank * RW + r];
        recv[r] = all[(size_t)r * RW + c->comm_rank];
        bound |= all[(size_t)r * RW + W];
        total += recv[r];
    }
    Keys out;
    out.n = total;
    out.bound = bound;
    out.buf = make_buf(c, total * 8);
    // The rows this rank keeps are copied on the device; the others travel in one grouped
    // send / receive.  No host wait follows: what comes next is ordered behind it on the stream.
    NCCL_OK(api().GroupStart());
    uint64_t so = 0, ro = 0;
    for (uint32_t r = 0; r < W; ++r) {
        if (r == c->comm_rank) {
            if (send[r]) CUDA_OK(cudaMemcpyAsync(out.buf->as<uint64_t>() + ro, part.ptr() + so, send[r] * 8, cudaMemcpyDeviceToDevice, c->stream));
        } else {
            if (send[r]) NCCL_OK(api().Send(part.ptr() + so, send[r], ncclUint64, (int)r, cm->comm, c->stream));
            if (recv[r]) NCCL_OK(api().Recv(out.buf->as<uint64_t>() + ro, recv[r], ncclUint64, (int)r, cm->comm, c->stream));
            st.exchange_bytes += send[r] * 8;
        }
        so += send[r];
        ro += recv[r];
    }
    NCCL_OK(api().GroupEnd());
    if (sorted_unique_result) {
        ops_sort(c, out);
        ops_dedup_sorted(c, out);
    }
    return out;
}
