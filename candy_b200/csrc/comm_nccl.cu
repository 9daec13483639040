// NCCL all-reduce behind the C ABI: the stated baseline exchange for tensor-parallel linears, and the
// exchange for batches the fused peer-store path (comm.cu) does not take.  One process per GPU.
//
// NCCL is not linked: libnccl.so.2 is opened at cq_tp_init (the copy already loaded into the process if there
// is one, e.g. a host framework's; else the loader's search path; $CANDYQ_NCCL_LIBRARY overrides), so the
// library loads and every other entry point works on machines without NCCL.
//
// Waiting is bounded on the host: cq_tp_wait polls the stream and the communicator's asynchronous error
// state until the work is done, an error shows, or the deadline passes; on a deadline or an error the
// communicator is aborted (ncclCommAbort, which also releases kernels stuck on a peer that never arrived)
// and CQ_ERR_TIMEOUT / CQ_ERR_CUDA is returned.  The reference has no multi-device code: no counterpart.
#include <dlfcn.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "common.cuh"

namespace {

// The few NCCL declarations used (nccl.h 2.x ABI): results, the unique id, float32, sum.
typedef struct ncclComm *ncclComm_t;
typedef struct {
    char internal[128];
} ncclUniqueId;
enum { kNcclSuccess = 0, kNcclInProgress = 7, kNcclFloat32 = 7, kNcclSum = 0 };

struct NcclApi {
    void *handle = nullptr;
    int (*GetUniqueId)(ncclUniqueId *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*CommAbort)(ncclComm_t) = nullptr;
    int (*CommGetAsyncError)(ncclComm_t, int *) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    std::string error;
};

NcclApi &nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api;
    tried = true;
    const char *override_path = std::getenv("CANDYQ_NCCL_LIBRARY");
    const char *names[] = {override_path, "libnccl.so.2", "libnccl.so"};
    for (const char *nm : names) {
        if (!nm || !*nm) continue;
        api.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) break;
    }
    if (!api.handle) {
        api.error = std::string("libnccl.so.2 not found (set CANDYQ_NCCL_LIBRARY): ") + (dlerror() ? dlerror() : "");
        return api;
    }
#define CQ_NCCL_SYM(field, name)                                                     \
    api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, name));      \
    if (!api.field) api.error = std::string("symbol missing in NCCL library: ") + name;
    CQ_NCCL_SYM(GetUniqueId, "ncclGetUniqueId")
    CQ_NCCL_SYM(CommInitRank, "ncclCommInitRank")
    CQ_NCCL_SYM(AllReduce, "ncclAllReduce")
    CQ_NCCL_SYM(CommDestroy, "ncclCommDestroy")
    CQ_NCCL_SYM(CommAbort, "ncclCommAbort")
    CQ_NCCL_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
    CQ_NCCL_SYM(GetErrorString, "ncclGetErrorString")
#undef CQ_NCCL_SYM
    return api;
}

cq_status nccl_fail(cq_ctx *ctx, int r, const char *what) {
    NcclApi &api = nccl_api();
    return cq_fail(ctx, CQ_ERR_CUDA, std::string(what) + ": NCCL error " + std::to_string(r) + " (" + (api.GetErrorString ? api.GetErrorString(r) : "?") + ")");
}

}  // namespace

struct cq_tp {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    bool aborted = false;
};

extern "C" {

cq_status cq_tp_unique_id(cq_ctx *ctx, void *id128) {
    CQ_ENTER(ctx);
    if (!id128) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_tp_unique_id: null pointer");
    NcclApi &api = nccl_api();
    if (!api.error.empty() || !api.handle) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "cq_tp_unique_id: " + api.error);
    ncclUniqueId id;
    const int r = api.GetUniqueId(&id);
    if (r != kNcclSuccess) return nccl_fail(ctx, r, "ncclGetUniqueId");
    memcpy(id128, id.internal, sizeof(id.internal));
    return CQ_OK;
}

cq_status cq_tp_init(cq_ctx *ctx, int rank, int world, const void *nccl_unique_id, size_t id_bytes, cq_tp **out) {
    CQ_ENTER(ctx);
    if (!out || !nccl_unique_id || id_bytes != 128 || world < 1 || rank < 0 || rank >= world)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_tp_init: bad arguments (the unique id is 128 bytes)");
    *out = nullptr;
    NcclApi &api = nccl_api();
    if (!api.error.empty() || !api.handle) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "cq_tp_init: " + api.error);
    ncclUniqueId id;
    memcpy(id.internal, nccl_unique_id, sizeof(id.internal));
    cq_tp *tp = new cq_tp();
    tp->rank = rank, tp->world = world;
    const int r = api.CommInitRank(&tp->comm, world, id, rank);
    if (r != kNcclSuccess) {
        delete tp;
        return nccl_fail(ctx, r, "ncclCommInitRank");
    }
    *out = tp;
    return CQ_OK;
}

cq_status cq_tp_destroy(cq_ctx *ctx, cq_tp *tp) {
    CQ_ENTER(ctx);
    if (!tp) return CQ_OK;
    NcclApi &api = nccl_api();
    if (tp->comm && !tp->aborted) {
        cudaStreamSynchronize(ctx->stream);
        api.CommDestroy(tp->comm);
    }
    delete tp;
    return CQ_OK;
}

cq_status cq_allreduce_sum_f32(cq_ctx *ctx, cq_tp *tp, float *buf_dev, int64_t count) {
    CQ_ENTER(ctx);
    if (!tp || !buf_dev || count < 1) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_allreduce_sum_f32: bad arguments");
    if (tp->aborted) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_allreduce_sum_f32: the communicator was aborted after a timeout or an error");
    NcclApi &api = nccl_api();
    const int r = api.AllReduce(buf_dev, buf_dev, (size_t)count, kNcclFloat32, kNcclSum, tp->comm, ctx->stream);
    if (r != kNcclSuccess) return nccl_fail(ctx, r, "ncclAllReduce");
    return CQ_OK;
}

cq_status cq_tp_wait(cq_ctx *ctx, cq_tp *tp, int timeout_ms) {
    CQ_ENTER(ctx);
    if (!tp || timeout_ms < 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_tp_wait: bad arguments");
    if (tp->aborted) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_tp_wait: the communicator was aborted earlier");
    NcclApi &api = nccl_api();
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    for (;;) {
        const cudaError_t q = cudaStreamQuery(ctx->stream);
        if (q == cudaSuccess) return cq_synchronize(ctx);  // done: report any device-side error word too
        if (q != cudaErrorNotReady) return cq_cuda_fail(ctx, q, "cudaStreamQuery");
        int async_err = kNcclSuccess;
        const int r = api.CommGetAsyncError(tp->comm, &async_err);
        const bool failed = r != kNcclSuccess || (async_err != kNcclSuccess && async_err != kNcclInProgress);
        const bool late = std::chrono::steady_clock::now() >= deadline;
        if (failed || late) {
            api.CommAbort(tp->comm);  // releases collective kernels that are still waiting for a peer
            tp->aborted = true;
            cudaStreamSynchronize(ctx->stream);
            if (late && !failed)
                return cq_fail(ctx, CQ_ERR_TIMEOUT, "cq_tp_wait: the stream did not finish within " + std::to_string(timeout_ms) + " ms (a rank is late or gone); the communicator was aborted");
            return nccl_fail(ctx, r != kNcclSuccess ? r : async_err, "asynchronous NCCL error; the communicator was aborted");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

}  // extern "C"
