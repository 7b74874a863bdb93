// NCCL exchange layer.  The library does not link NCCL: it binds the handful of entry points it
// needs at run time, from the NCCL already loaded into the process (the host program's, e.g.
// the one torch.distributed brought in) or else from libnccl.so.2 on the loader path, so a
// single-GPU user needs no NCCL at all.
#include <dlfcn.h>
#include <nccl.h>

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

}  // namespace

struct Comm {
    ncclComm_t comm = nullptr;
    double timeout_s = 120.0;
    Buf counts_dev;  // world rows of world + 1 u64: row r = send counts of rank r, then its OR bound
};

// Wait for the stream without ever blocking for good: poll the stream and the communicator's
// asynchronous error state; after the time limit abort the communicator and report a timeout.
static void comm_wait(xlb_ctx* c) {
    Comm* cm = c->comm;
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t q = cudaStreamQuery(c->stream);
        if (q == cudaSuccess) return;
        if (q != cudaErrorNotReady) xlb_fail(XLB_ERR_CUDA, "stream failed during an exchange: %s", cudaGetErrorString(q));
        ncclResult_t ar = ncclSuccess;
        api().CommGetAsyncError(cm->comm, &ar);
        if (ar != ncclSuccess && ar != ncclInProgress) {
            api().CommAbort(cm->comm);
            cm->comm = nullptr;
            xlb_fail(XLB_ERR_NCCL, "NCCL reported an asynchronous error: %s", api().GetErrorString(ar));
        }
        double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (el > cm->timeout_s) {
            api().CommAbort(cm->comm);
            cm->comm = nullptr;
            xlb_fail(XLB_ERR_TIMEOUT, "exchange did not complete within %.0f s; communicator aborted", cm->timeout_s);
        }
    }
}

void comm_destroy(xlb_ctx* c) {
    if (!c->comm) return;
    if (c->comm->comm) api().CommDestroy(c->comm->comm);
    delete c->comm;
    c->comm = nullptr;
    c->world = 1;
    c->rank = 0;
}

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
        c->rank = rank;
        c->world = world;
        cm->counts_dev = make_buf(c, (uint64_t)world * (world + 1) * 8);
    } catch (const XlbError& e) {
        c->last_error = e.msg;
        return e.st;
    }
    return XLB_OK;
}

uint64_t comm_allreduce_sum(xlb_ctx* c, uint64_t v) {
    if (c->world <= 1) return v;
    Comm* cm = c->comm;
    Buf d = make_buf(c, 8);
    c->h_scalar[32] = v;
    CUDA_OK(cudaMemcpyAsync(d->p, &c->h_scalar[32], 8, cudaMemcpyHostToDevice, c->stream));
    NCCL_OK(api().AllReduce(d->p, d->p, 1, ncclUint64, ncclSum, cm->comm, c->stream));
    CUDA_OK(cudaMemcpyAsync(&c->h_scalar[33], d->p, 8, cudaMemcpyDeviceToHost, c->stream));
    comm_wait(c);
    return c->h_scalar[33];
}

Keys comm_repartition(xlb_ctx* c, const Keys& in, int keysel, bool sorted_unique_result, xlb_run_stats& st) {
    if (c->world <= 1) {
        Keys k = in;
        if (sorted_unique_result) { /* single rank: callers pass sorted data already */ }
        return k;
    }
    Comm* cm = c->comm;
    uint32_t W = c->world;
    // partition into one run per destination; the run lengths go straight from device memory into
    // the all-gather, so every rank learns the whole count matrix with a single host wait.  Each
    // row of the matrix carries one more word: the sender's OR bound of its rows, so the receiver
    // knows the bits of what it gets without looking at it.
    const uint32_t RW = W + 1;
    unsigned long long* mine = cm->counts_dev->as<unsigned long long>() + (uint64_t)c->rank * RW;
    Keys part = ops_partition_by_owner_dev(c, in, keysel, W, mine);
    c->h_scalar[60] = in.n ? in.bound : 0;
    CUDA_OK(cudaMemcpyAsync(mine + W, &c->h_scalar[60], 8, cudaMemcpyHostToDevice, c->stream));
    NCCL_OK(api().AllGather(mine, cm->counts_dev->p, RW, ncclUint64, cm->comm, c->stream));
    std::vector<unsigned long long> all((size_t)W * RW);
    CUDA_OK(cudaMemcpyAsync(all.data(), cm->counts_dev->p, (size_t)W * RW * 8, cudaMemcpyDeviceToHost, c->stream));
    comm_wait(c);
    std::vector<uint64_t> send(W);
    uint64_t bound = 0;
    for (uint32_t r = 0; r < W; ++r) {
        send[r] = all[(size_t)c->rank * RW + r];
        bound |= all[(size_t)r * RW + W];
    }
    std::vector<uint64_t> recv(W);
    uint64_t total = 0;
    for (uint32_t r = 0; r < W; ++r) {
        recv[r] = all[(size_t)r * RW + c->rank];
        total += recv[r];
    }
    Keys out;
    out.n = total;
    out.bound = bound;
    out.buf = make_buf(c, total * 8);
    NCCL_OK(api().GroupStart());
    uint64_t so = 0, ro = 0;
    for (uint32_t r = 0; r < W; ++r) {
        if (send[r]) NCCL_OK(api().Send(part.ptr() + so, send[r], ncclUint64, (int)r, cm->comm, c->stream));
        if (recv[r]) NCCL_OK(api().Recv(out.buf->as<uint64_t>() + ro, recv[r], ncclUint64, (int)r, cm->comm, c->stream));
        if (r != c->rank) st.exchange_bytes += send[r] * 8;
        so += send[r];
        ro += recv[r];
    }
    NCCL_OK(api().GroupEnd());
    comm_wait(c);
    if (sorted_unique_result) {
        ops_sort(c, out);
        ops_dedup_sorted(c, out);
    }
    return out;
}
