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
#include "kernels/kernels.h"

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

// The exchange region of the one-shot all-reduce over peer memory: this rank's two slots and flag words (plain
// cudaMalloc memory, exported with CUDA IPC) and the mappings of every other rank's region.
struct Exchange {
    int device = 0, rank = 0, world = 1;
    size_t slot_bytes = 0;
    void* local = nullptr;
    void* regions[wrk::k::kMaxPeers] = {};
    uint32_t* counters = nullptr;  // [0] sequence number of the last finished call, [1] CTAs done in the running call
    ~Exchange() {
        cudaSetDevice(device);
        for (int r = 0; r < world; ++r)
            if (r != rank && regions[r]) cudaIpcCloseMemHandle(regions[r]);
        if (local) cudaFree(local);
        if (counters) cudaFree(counters);
    }
};

struct wrk_comm {
    std::atomic<int> refs{1};
    wrk_context* ctx = nullptr;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    std::shared_ptr<Exchange> exchange;
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

// Collective over the ranks (every rank calls it at the same point): allocates this rank's exchange region, passes its IPC
// handle around with an NCCL all-gather and maps the peers' regions.
int32_t wrk_comm_enable_peer_reduce(wrk_comm* comm, size_t slot_bytes) {
    WRK_REQUIRE(comm, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(comm->comm, WRK_ERR_NCCL, "the communicator was aborted by an earlier failure");
    WRK_REQUIRE(comm->world <= wrk::k::kMaxPeers, WRK_ERR_UNSUPPORTED, "peer reduce is built for up to %d ranks", wrk::k::kMaxPeers);
    WRK_REQUIRE(slot_bytes >= 16 && slot_bytes % 256 == 0, WRK_ERR_INVALID_ARGUMENT, "slot of %zu bytes: a multiple of 256", slot_bytes);
    if (comm->exchange && comm->exchange->slot_bytes >= slot_bytes) return WRK_OK;
    WRK_REQUIRE(!comm->exchange, WRK_ERR_UNSUPPORTED, "the exchange region holds slots of %zu bytes; it is sized once", comm->exchange->slot_bytes);
    wrk_context* ctx = comm->ctx;
    WRK_CUDA(cudaSetDevice(ctx->device));
    auto ex = std::make_shared<Exchange>();
    ex->device = ctx->device;
    ex->rank = comm->rank;
    ex->world = comm->world;
    ex->slot_bytes = slot_bytes;
    const size_t region = 2 * slot_bytes + 256;
    WRK_CUDA(cudaMalloc(&ex->local, region));
    WRK_CUDA(cudaMemset(ex->local, 0, region));  // flags at zero before any peer can reach them
    WRK_CUDA(cudaMalloc(reinterpret_cast<void**>(&ex->counters), 256));
    WRK_CUDA(cudaMemset(ex->counters, 0, 256));
    cudaIpcMemHandle_t mine;
    WRK_CUDA(cudaIpcGetMemHandle(&mine, ex->local));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handles travel as 64 bytes");
    uint8_t* dev = nullptr;  // [world + 1][64]: this rank's handle, then every rank's
    WRK_CUDA(cudaMalloc(reinterpret_cast<void**>(&dev), (size_t)(comm->world + 1) * 64));
    std::vector<cudaIpcMemHandle_t> all(comm->world);
    cudaError_t e = cudaMemcpyAsync(dev, &mine, 64, cudaMemcpyHostToDevice, ctx->stream);
    ncclResult_t r = ncclSuccess;
    if (e == cudaSuccess) r = nccl().AllGather(dev, dev + 64, 64, ncclUint8, comm->comm, ctx->stream);
    if (e == cudaSuccess && r == ncclSuccess) e = cudaMemcpyAsync(all.data(), dev + 64, (size_t)comm->world * 64, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess && r == ncclSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(dev);
    if (r != ncclSuccess) return nccl_fail("ncclAllGather (IPC handles)", r);
    if (e != cudaSuccess) return wrk::set_error(WRK_ERR_CUDA, "exchanging IPC handles failed: %s", cudaGetErrorString(e));
    for (int p = 0; p < comm->world; ++p) {
        if (p == comm->rank) {
            ex->regions[p] = ex->local;
            continue;
        }
        e = cudaIpcOpenMemHandle(&ex->regions[p], all[p], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            ex->regions[p] = nullptr;
            return wrk::set_error(WRK_ERR_CUDA, "mapping rank %d's exchange region failed: %s", p, cudaGetErrorString(e));
        }
    }
    // nobody proceeds (and starts writing flags) before every rank has mapped every region
    float* token = nullptr;
    WRK_CUDA(cudaMalloc(reinterpret_cast<void**>(&token), 256));
    WRK_CUDA(cudaMemsetAsync(token, 0, 256, ctx->stream));
    r = nccl().AllReduce(token, token, 1, ncclFloat32, ncclSum, comm->comm, ctx->stream);
    e = cudaStreamSynchronize(ctx->stream);
    cudaFree(token);
    if (r != ncclSuccess) return nccl_fail("ncclAllReduce (barrier)", r);
    if (e != cudaSuccess) return wrk::set_error(WRK_ERR_CUDA, "barrier after mapping failed: %s", cudaGetErrorString(e));
    comm->exchange = ex;
    return WRK_OK;
}

int32_t wrk_comm_peer_slot_bytes(const wrk_comm* comm, size_t* slot_bytes) {
    WRK_REQUIRE(comm && slot_bytes, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *slot_bytes = comm->exchange ? comm->exchange->slot_bytes : 0;
    return WRK_OK;
}

// A tensor over slot `slot` (0 or 1) of this rank's exchange region: what a matmul writes its partial sums into.
int32_t wrk_comm_peer_slot(wrk_comm* comm, uint32_t slot, int32_t dtype, const uint32_t shape[4], wrk_tensor** out) {
    WRK_REQUIRE(comm && shape && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(comm->exchange, WRK_ERR_INVALID_ARGUMENT, "wrk_comm_enable_peer_reduce has not run on this communicator");
    WRK_REQUIRE(slot < 2, WRK_ERR_INVALID_ARGUMENT, "slot %u: 0 or 1", slot);
    auto t = new wrk_tensor();
    t->ctx = comm->ctx;
    t->dtype = dtype;
    for (int i = 0; i < 4; ++i) t->shape.v[i] = shape[i];
    if (wrk::dtype_size(dtype) == 0 || t->bytes() > comm->exchange->slot_bytes) {
        const size_t need = t->bytes();
        delete t;
        return wrk::set_error(WRK_ERR_SIZE, "a slot holds %zu bytes, the tensor needs %zu", comm->exchange->slot_bytes, need);
    }
    auto buf = std::make_shared<wrk::Buffer>(comm->ctx);
    buf->ptr = static_cast<uint8_t*>(comm->exchange->local) + (size_t)slot * comm->exchange->slot_bytes;
    buf->bytes = t->bytes();
    buf->external = comm->exchange;  // the region outlives the tensor
    t->buf = buf;
    *out = t;
    return WRK_OK;
}

// dst <- sum over the ranks of the first `count` f32 of slot `slot`, added in rank order by every rank from peer memory.
int32_t wrk_op_peer_all_reduce(wrk_comm* comm, uint32_t slot, size_t count, wrk_tensor* dst, wrk_op** out) {
    WRK_REQUIRE(comm && dst && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(comm->exchange, WRK_ERR_INVALID_ARGUMENT, "wrk_comm_enable_peer_reduce has not run on this communicator");
    WRK_REQUIRE(dst->ctx == comm->ctx, WRK_ERR_INVALID_ARGUMENT, "tensor and communicator belong to different contexts");
    WRK_REQUIRE(slot < 2 && count % 4 == 0 && count * 4 <= comm->exchange->slot_bytes, WRK_ERR_SIZE,
                "slot %u, %zu elements: slots are 0 or 1, counts multiples of 4 within %zu bytes", slot, count, comm->exchange->slot_bytes);
    WRK_REQUIRE((dst->dtype == WRK_F16 || dst->dtype == WRK_F32) && dst->len() == count, WRK_ERR_SIZE,
                "the destination holds %zu elements, the sum %zu", dst->len(), count);
    wrk::k::PeerReduceArgs a{};
    auto ex = comm->exchange;
    for (int r = 0; r < comm->world; ++r) a.regions[r] = ex->regions[r];
    a.world = (uint32_t)comm->world;
    a.rank = (uint32_t)comm->rank;
    a.slot = slot;
    a.slot_bytes = ex->slot_bytes;
    a.count = count;
    a.dst = dst->ptr();
    a.dst_dtype = dst->dtype;
    a.epoch = ex->counters;
    a.done = ex->counters + 1;
    a.status = comm->ctx->device_status;
    const int sms = comm->ctx->num_sms;
    auto hold = std::make_shared<CommHold>(comm);
    *out = wrk::new_atom("peer_all_reduce",
                         [=](cudaStream_t s) {
                             (void)hold;
                             (void)ex;
                             return wrk::k::peer_all_reduce(a, sms, s);
                         },
                         {dst});
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
