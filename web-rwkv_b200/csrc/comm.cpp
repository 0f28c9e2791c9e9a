// Tensor-parallel plumbing: an NCCL communicator bound to a context's stream and the all-reduce /
// all-gather ops the sharded layers need.  The ops are deferred like every other op (they can sit in op
// lists and be captured into CUDA graphs) and run on the context's stream, so they are ordered with the
// kernels around them.  The reference is single-GPU: nothing here has a counterpart in it.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

#include <string>

#include "common.h"

// NCCL is bound at first use, not at link time: a process that never shards does not load it, and one that
// has already loaded an NCCL (e.g. through torch.distributed) keeps using that single copy.
namespace {
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

const NcclApi& nccl() {
    static NcclApi api = [] {
        NcclApi a;
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) return a;
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(dlsym(h, "ncclCommAbort"));
        a.CommGetAsyncError = reinterpret_cast<decltype(a.CommGetAsyncError)>(dlsym(h, "ncclCommGetAsyncError"));
        a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
        a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
        a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommAbort && a.CommGetAsyncError && a.AllReduce && a.AllGather && a.GetErrorString;
        return a;
    }();
    return api;
}
}  // namespace
#define WRK_NEED_NCCL() WRK_REQUIRE(nccl().ok, WRK_ERR_NCCL, "libnccl.so.2 could not be loaded")

struct wrk_comm {
    std::atomic<int> refs{1};
    wrk_context* ctx = nullptr;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
};

namespace {

int32_t nccl_fail(const char* what, ncclResult_t r) {
    return wrk::set_error(WRK_ERR_NCCL, "%s failed: %s", what, nccl().GetErrorString(r));
}

// Shared by every op built on a communicator: the communicator is torn down only after the last op (and
// with it the last op list or command buffer) that may still launch on it is gone.
struct CommHold {
    wrk_comm* comm;
    explicit CommHold(wrk_comm* c) : comm(c) { c->refs.fetch_add(1); }
    CommHold(const CommHold&) = delete;
    CommHold& operator=(const CommHold&) = delete;
    ~CommHold() { wrk_comm_release(comm); }
};

bool nccl_dtype(int dtype, ncclDataType_t* out) {
    switch (dtype) {
        case WRK_F32: *out = ncclFloat32; return true;
        case WRK_F16: *out = ncclFloat16; return true;
        case WRK_U8: *out = ncclUint8; return true;
        case WRK_U32: *out = ncclUint32; return true;
        default: return false;
    }
}

}  // namespace

extern "C" {

int32_t wrk_comm_unique_id(uint8_t id[128]) {
    WRK_REQUIRE(id, WRK_ERR_INVALID_ARGUMENT, "null argument");
    static_assert(sizeof(ncclUniqueId) == 128, "the C ABI passes the id as 128 bytes");
    WRK_NEED_NCCL();
    ncclUniqueId uid;
    const ncclResult_t r = nccl().GetUniqueId(&uid);
    if (r != ncclSuccess) return nccl_fail("ncclGetUniqueId", r);
    std::memcpy(id, &uid, sizeof uid);
    return WRK_OK;
}

int32_t wrk_comm_create(wrk_context* ctx, const uint8_t id[128], int32_t rank, int32_t world, wrk_comm** out) {
    WRK_REQUIRE(ctx && id && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(world >= 1 && rank >= 0 && rank < world, WRK_ERR_INVALID_ARGUMENT, "rank %d of %d", rank, world);
    WRK_NEED_NCCL();
    WRK_CUDA(cudaSetDevice(ctx->device));
    // In-switch reduction binds every rank's buffers to one NVLink multicast object; a rank that dies while
    // bound faults its peers' GPUs.  Ranks of this library may leave (teardown is a local abort), so the
    // multicast path stays off unless the embedder has set the variable itself.
    setenv("NCCL_NVLS_ENABLE", "0", 0);
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof uid);
    ncclComm_t comm = nullptr;
    const ncclResult_t r = nccl().CommInitRank(&comm, world, uid, rank);
    if (r != ncclSuccess) return nccl_fail("ncclCommInitRank", r);
    auto c = new wrk_comm();
    c->ctx = ctx;
    c->comm = comm;
    c->rank = rank;
    c->world = world;
    *out = c;
    return WRK_OK;
}

int32_t wrk_comm_release(wrk_comm* comm) {
    if (comm == nullptr) return WRK_OK;
    if (comm->refs.fetch_sub(1) == 1) {
        if (comm->comm) {
            cudaSetDevice(comm->ctx->device);
            cudaStreamSynchronize(comm->ctx->stream);
            // local teardown: it does not wait for the other ranks (which may already be gone) nor for
            // CUDA graphs that still hold this communicator's kernels
            nccl().CommAbort(comm->comm);
        }
        delete comm;
    }
    return WRK_OK;
}

int32_t wrk_comm_retain(wrk_comm* comm) {
    WRK_REQUIRE(comm, WRK_ERR_INVALID_ARGUMENT, "null argument");
    comm->refs.fetch_add(1);
    return WRK_OK;
}

// The wait every rank of a split job makes in place of a plain stream synchronize: a peer that never enters a
// collective leaves this rank's kernel spinning on the device, which no CUDA call reports.  `done` and `failure`
// are polled every `poll_us` microseconds; the wait ends with WRK_OK when done() is non-zero, with WRK_ERR_NCCL
// when failure() is (its value is put in the message), with WRK_ERR_TIMEOUT after `timeout_ms`.
int32_t wrk_watchdog_wait(int32_t (*done)(void*), int32_t (*failure)(void*), void* user, uint32_t timeout_ms, uint32_t poll_us) {
    WRK_REQUIRE(done, WRK_ERR_INVALID_ARGUMENT, "null argument");
    const auto start = std::chrono::steady_clock::now();
    const auto limit = std::chrono::milliseconds(timeout_ms);
    for (;;) {
        if (done(user) != 0) return WRK_OK;
        if (failure) {
            const int32_t f = failure(user);
            if (f != 0) return wrk::set_error(WRK_ERR_NCCL, "a collective failed asynchronously (code %d)", f);
        }
        if (std::chrono::steady_clock::now() - start >= limit)
            return wrk::set_error(WRK_ERR_TIMEOUT, "work on the stream did not finish within %u ms: a peer may have left", timeout_ms);
        if (poll_us) std::this_thread::sleep_for(std::chrono::microseconds(poll_us));
    }
}

namespace {
struct CommWait {
    wrk_comm* comm;
    cudaEvent_t event;
};
int32_t comm_done(void* user) {
    const cudaError_t e = cudaEventQuery(static_cast<CommWait*>(user)->event);
    return e == cudaErrorNotReady ? 0 : 1;  // an error ends the wait too; the synchronize that follows reports it
}
int32_t comm_failure(void* user) {
    ncclResult_t async = ncclSuccess;
    const ncclResult_t r = nccl().CommGetAsyncError(static_cast<CommWait*>(user)->comm->comm, &async);
    if (r != ncclSuccess) return (int32_t)r;
    return async == ncclSuccess || async == ncclInProgress ? 0 : (int32_t)async;
}
}  // namespace

// Waits for everything submitted to the communicator's context so far, polling ncclCommGetAsyncError; on a failure
// or after timeout_ms the communicator is aborted (its kernels leave the device) and the error is returned: the
// context stays usable, the communicator does not.
int32_t wrk_comm_wait(wrk_comm* comm, uint32_t timeout_ms) {
    WRK_REQUIRE(comm, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(comm->comm, WRK_ERR_NCCL, "the communicator was aborted by an earlier failure");
    WRK_CUDA(cudaSetDevice(comm->ctx->device));
    CommWait w{comm, nullptr};
    WRK_CUDA(cudaEventCreateWithFlags(&w.event, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(w.event, comm->ctx->stream);
    int32_t status = e == cudaSuccess ? wrk_watchdog_wait(comm_done, comm_failure, &w, timeout_ms, 50)
                                      : wrk::set_error(WRK_ERR_CUDA, "cudaEventRecord failed: %s", cudaGetErrorString(e));
    if (status == WRK_ERR_TIMEOUT || status == WRK_ERR_NCCL) {
        const std::string message = wrk_last_error_message();
        nccl().CommAbort(comm->comm);
        comm->comm = nullptr;
        cudaStreamSynchronize(comm->ctx->stream);
        wrk::set_error(status, "%s; the communicator was aborted", message.c_str());
    }
    cudaEventDestroy(w.event);
    if (status == WRK_OK) WRK_CUDA(cudaStreamSynchronize(comm->ctx->stream));
    return status;
}

int32_t wrk_comm_rank(const wrk_comm* comm, int32_t* rank, int32_t* world) {
    WRK_REQUIRE(comm && rank && world, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *rank = comm->rank;
    *world = comm->world;
    return WRK_OK;
}

// x <- sum over ranks of x (in place).
int32_t wrk_op_all_reduce(wrk_comm* comm, wrk_tensor* x, wrk_op** out) {
    WRK_REQUIRE(comm && x && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(x->ctx == comm->ctx, WRK_ERR_INVALID_ARGUMENT, "tensor and communicator belong to different contexts");
    ncclDataType_t dt;
    WRK_REQUIRE(x->dtype != WRK_U8 && x->dtype != WRK_U32 && nccl_dtype(x->dtype, &dt), WRK_ERR_TYPE,
                "data type mismatch: all_reduce sums f16 or f32");
    void* ptr = x->ptr();
    const size_t count = x->len();
    auto hold = std::make_shared<CommHold>(comm);
    *out = wrk::new_atom("all_reduce",
                         [=](cudaStream_t s) {
                             ncclComm_t c = hold->comm->comm;  // null once a failed wait has aborted it
                             if (c == nullptr) return cudaErrorUnknown;
                             return nccl().AllReduce(ptr, ptr, count, dt, ncclSum, c, s) == ncclSuccess ? cudaSuccess : cudaErrorUnknown;
                         },
                         {x});
    return WRK_OK;
}

// output[rank r's slot] <- input of rank r, for every r: output holds world * len(input) elements.
int32_t wrk_op_all_gather(wrk_comm* comm, wrk_tensor* input, wrk_tensor* output, wrk_op** out) {
    WRK_REQUIRE(comm && input && output && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(input->ctx == comm->ctx && output->ctx == comm->ctx, WRK_ERR_INVALID_ARGUMENT,
                "tensors and communicator belong to different contexts");
    ncclDataType_t dt;
    WRK_REQUIRE(nccl_dtype(input->dtype, &dt) && output->dtype == input->dtype, WRK_ERR_TYPE, "data type mismatch");
    WRK_REQUIRE(output->len() == input->len() * (size_t)comm->world, WRK_ERR_SIZE, "all_gather output holds %zu elements, expected %zu",
                output->len(), input->len() * (size_t)comm->world);
    const void* src = input->ptr();
    void* dst = output->ptr();
    const size_t count = input->len();
    auto hold = std::make_shared<CommHold>(comm);
    *out = wrk::new_atom("all_gather",
                         [=](cudaStream_t s) {
                             ncclComm_t c = hold->comm->comm;
                             if (c == nullptr) return cudaErrorUnknown;
                             return nccl().AllGather(src, dst, count, dt, c, s) == ncclSuccess ? cudaSuccess : cudaErrorUnknown;
                         },
                         {input, output});
    return WRK_OK;
}

}  // extern "C"
