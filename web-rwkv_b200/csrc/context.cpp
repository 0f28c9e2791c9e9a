// Host side of libwrk: CUDA context, tensors, deferred ops, encode/submit.
//
// Stands in for the wgpu `Context` (src/context.rs), `TensorGpu` (src/tensor/mod.rs) and
// `Context::encode` (src/tensor/ops.rs:78-144) of the reference: one CUDA stream per context,
// device buffers from cudaMallocAsync's pool, pinned staging buffers for uploads and read-backs,
// and command lists that can be replayed as CUDA graphs.
#include <cstring>

#include "common.h"

namespace wrk {

static thread_local std::string g_last_error;

int32_t set_error(int32_t code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

// Tears the context down when its last reference (owner or buffer) goes.
static void context_unref(wrk_context* ctx) {
    if (ctx->refs.fetch_sub(1) != 1) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->ev_start) cudaEventDestroy(ctx->ev_start);
    if (ctx->ev_stop) cudaEventDestroy(ctx->ev_stop);
    if (ctx->device_status) cudaFree(ctx->device_status);
    if (ctx->host_status) cudaFreeHost(ctx->host_status);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

Buffer::Buffer(wrk_context* owner) : ctx(owner) { ctx->refs.fetch_add(1); }

Buffer::~Buffer() {
    if (ptr && !external) {
        cudaSetDevice(ctx->device);
        cudaFreeAsync(ptr, ctx->stream);
    }
    context_unref(ctx);
}

DView make_dview(const wrk_tensor* t) {
    DView d;
    d.base = t->ptr();
    d.dtype = t->dtype;
    for (int i = 0; i < 4; ++i) {
        d.shape[i] = t->shape.v[i];
        d.stride[i] = t->shape.v[i];
        d.offset[i] = 0;
    }
    return d;
}

DView make_dview(const wrk_view& v) {
    DView d;
    d.base = v.tensor->ptr();
    d.dtype = v.tensor->dtype;
    for (int i = 0; i < 4; ++i) {
        d.shape[i] = v.shape[i];
        d.stride[i] = v.stride[i];
        d.offset[i] = v.offset[i];
    }
    return d;
}

bool view_is(const wrk_view& v, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    return v.shape[0] == x && v.shape[1] == y && v.shape[2] == z && v.shape[3] == w;
}

bool is_float(int dtype) { return dtype == WRK_F32 || dtype == WRK_F16; }

int32_t check_shape(const char* what, const Shape4& have, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    if (have.v[0] == x && have.v[1] == y && have.v[2] == z && have.v[3] == w) return WRK_OK;
    return set_error(WRK_ERR_SHAPE, "tensor shape not match (%s): [%u, %u, %u, %u] vs. [%u, %u, %u, %u]", what,
                     have.v[0], have.v[1], have.v[2], have.v[3], x, y, z, w);
}

int32_t check_view(const char* what, const wrk_view* v, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    Shape4 s{{v->shape[0], v->shape[1], v->shape[2], v->shape[3]}};
    return check_shape(what, s, x, y, z, w);
}

int32_t tensor_alloc(wrk_context* ctx, int dtype, const uint32_t shape[4], bool zero, wrk_tensor** out) {
    WRK_REQUIRE(ctx && out && shape, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(dtype_size(dtype) != 0, WRK_ERR_TYPE, "data type mismatch: unknown dtype %d", dtype);
    WRK_CUDA(cudaSetDevice(ctx->device));
    auto t = new wrk_tensor();
    t->ctx = ctx;
    t->dtype = dtype;
    for (int i = 0; i < 4; ++i) t->shape.v[i] = shape[i];
    auto buf = std::make_shared<Buffer>(ctx);
    buf->bytes = t->bytes();
    const size_t alloc = buf->bytes ? (buf->bytes + 255) / 256 * 256 : 256;
    cudaError_t e = cudaMallocAsync(&buf->ptr, alloc, ctx->stream);
    if (e != cudaSuccess) {
        buf->ptr = nullptr;
        delete t;
        return set_error(WRK_ERR_CUDA, "cudaMallocAsync(%zu) failed: %s", alloc, cudaGetErrorString(e));
    }
    if (zero) {
        e = cudaMemsetAsync(buf->ptr, 0, alloc, ctx->stream);
        if (e != cudaSuccess) {
            delete t;
            return set_error(WRK_ERR_CUDA, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
        }
    }
    t->buf = buf;
    *out = t;
    return WRK_OK;
}

wrk_op* new_atom(const char* name, Launch launch, std::initializer_list<const wrk_tensor*> tensors,
                 uint32_t num_kernels) {
    auto op = new wrk_op();
    op->kind = wrk_op::Atom;
    op->name = name;
    op->launch = std::move(launch);
    op->num_kernels = num_kernels;
    for (auto t : tensors)
        if (t) op->keep.push_back(t->buf);
    return op;
}

}  // namespace wrk

using namespace wrk;

wrk_op::~wrk_op() {
    for (auto c : children) wrk_op_release(c);
}
wrk_commands::~wrk_commands() {
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    for (auto a : atoms) wrk_op_release(a);
}
wrk_matrix::~wrk_matrix() {
    if (w) wrk_tensor_release(w);
    if (m) wrk_tensor_release(m);
    if (q) wrk_tensor_release(q);
}

extern "C" {

const char* wrk_last_error_message(void) { return g_last_error.c_str(); }
const char* wrk_build_arch(void) { return "sm_100a"; }

int32_t wrk_context_create(int32_t device, wrk_context** out) {
    WRK_REQUIRE(out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return set_error(WRK_ERR_NO_DEVICE, "no CUDA device available: %s", cudaGetErrorString(e));
    WRK_REQUIRE(device >= 0 && device < count, WRK_ERR_INVALID_ARGUMENT, "device %d out of range (%d devices)", device,
                count);
    WRK_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    WRK_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return set_error(WRK_ERR_NO_DEVICE, "device %d is sm_%d%d; this library carries sm_100a code only", device,
                         prop.major, prop.minor);
    auto ctx = new wrk_context();
    ctx->device = device;
    ctx->num_sms = prop.multiProcessorCount;
    const int32_t status = [&]() -> int32_t {
        WRK_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
        WRK_CUDA(cudaEventCreate(&ctx->ev_start));
        WRK_CUDA(cudaEventCreate(&ctx->ev_stop));
        WRK_CUDA(cudaMalloc(&ctx->device_status, sizeof(int32_t)));
        WRK_CUDA(cudaMemset(ctx->device_status, 0, sizeof(int32_t)));
        WRK_CUDA(cudaMallocHost(&ctx->host_status, sizeof(int32_t)));
        // keep freed device memory in the pool instead of returning it to the driver on every sync
        cudaMemPool_t pool;
        WRK_CUDA(cudaDeviceGetDefaultMemPool(&pool, device));
        uint64_t threshold = UINT64_MAX;
        WRK_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold));
        return WRK_OK;
    }();
    if (status != WRK_OK) {
        context_unref(ctx);  // frees whatever was created before the failure
        return status;
    }
    *out = ctx;
    return WRK_OK;
}

// Drops the owner's reference.  Tensors, ops and command buffers released later still find the stream: the
// context is torn down when the last device buffer that belongs to it has been freed.
int32_t wrk_context_destroy(wrk_context* ctx) {
    if (!ctx) return WRK_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    context_unref(ctx);
    return WRK_OK;
}

int32_t wrk_context_synchronize(wrk_context* ctx) {
    WRK_REQUIRE(ctx, WRK_ERR_INVALID_ARGUMENT, "null context");
    WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    return WRK_OK;
}

int32_t wrk_context_stream(wrk_context* ctx, void** cuda_stream) {
    WRK_REQUIRE(ctx && cuda_stream, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *cuda_stream = ctx->stream;
    return WRK_OK;
}

int32_t wrk_context_device(wrk_context* ctx, int32_t* device) {
    WRK_REQUIRE(ctx && device, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *device = ctx->device;
    return WRK_OK;
}

int32_t wrk_context_device_status(wrk_context* ctx, int32_t* status) {
    WRK_REQUIRE(ctx && status, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_CUDA(cudaMemcpyAsync(ctx->host_status, ctx->device_status, sizeof(int32_t), cudaMemcpyDeviceToHost,
                             ctx->stream));
    WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    *status = *ctx->host_status;
    return WRK_OK;
}

int32_t wrk_pinned_alloc(wrk_context* ctx, size_t bytes, void** out) {
    WRK_REQUIRE(ctx && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_CUDA(cudaSetDevice(ctx->device));
    WRK_CUDA(cudaMallocHost(out, bytes ? bytes : 1));
    return WRK_OK;
}

int32_t wrk_pinned_free(wrk_context* ctx, void* ptr) {
    WRK_REQUIRE(ctx, WRK_ERR_INVALID_ARGUMENT, "null context");
    if (ptr) WRK_CUDA(cudaFreeHost(ptr));
    return WRK_OK;
}

int32_t wrk_timer_start(wrk_context* ctx) {
    WRK_REQUIRE(ctx, WRK_ERR_INVALID_ARGUMENT, "null context");
    WRK_CUDA(cudaEventRecord(ctx->ev_start, ctx->stream));
    return WRK_OK;
}

int32_t wrk_timer_stop(wrk_context* ctx, float* milliseconds) {
    WRK_REQUIRE(ctx && milliseconds, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_CUDA(cudaEventRecord(ctx->ev_stop, ctx->stream));
    WRK_CUDA(cudaEventSynchronize(ctx->ev_stop));
    WRK_CUDA(cudaEventElapsedTime(milliseconds, ctx->ev_start, ctx->ev_stop));
    return WRK_OK;
}

int32_t wrk_context_launch_count(wrk_context* ctx, uint64_t* count) {
    WRK_REQUIRE(ctx && count, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *count = ctx->launches.load();
    return WRK_OK;
}

// ---- tensors -------------------------------------------------------------------------

int32_t wrk_tensor_create(wrk_context* ctx, wrk_dtype dtype, const uint32_t shape[4], wrk_tensor** out) {
    return tensor_alloc(ctx, dtype, shape, false, out);
}

int32_t wrk_tensor_zeros(wrk_context* ctx, wrk_dtype dtype, const uint32_t shape[4], wrk_tensor** out) {
    return tensor_alloc(ctx, dtype, shape, true, out);
}

int32_t wrk_tensor_load(wrk_tensor* t, const void* host, size_t bytes) {
    WRK_REQUIRE(t && (host || bytes == 0), WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(bytes == t->bytes(), WRK_ERR_SIZE, "data size not match: %zu vs. %zu", bytes, t->bytes());
    if (bytes == 0) return WRK_OK;
    WRK_CUDA(cudaSetDevice(t->ctx->device));
    WRK_CUDA(cudaMemcpyAsync(t->ptr(), host, bytes, cudaMemcpyHostToDevice, t->ctx->stream));
    // pageable sources are staged by the runtime before the call returns; pinned sources must stay
    // valid until the stream reaches the copy, so wait here to keep the simple call safe for both
    WRK_CUDA(cudaStreamSynchronize(t->ctx->stream));
    return WRK_OK;
}

int32_t wrk_tensor_from_data(wrk_context* ctx, wrk_dtype dtype, const uint32_t shape[4], const void* host, size_t bytes,
                             wrk_tensor** out) {
    wrk_tensor* t = nullptr;
    WRK_TRY(tensor_alloc(ctx, dtype, shape, false, &t));
    int32_t s = wrk_tensor_load(t, host, bytes);
    if (s != WRK_OK) {
        wrk_tensor_release(t);
        return s;
    }
    *out = t;
    return WRK_OK;
}

int32_t wrk_tensor_back(wrk_tensor* t, void* host, size_t bytes) {
    WRK_REQUIRE(t && (host || bytes == 0), WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(bytes == t->bytes(), WRK_ERR_SIZE, "data size not match: %zu vs. %zu", bytes, t->bytes());
    if (bytes == 0) return WRK_OK;
    WRK_CUDA(cudaSetDevice(t->ctx->device));
    WRK_CUDA(cudaMemcpyAsync(host, t->ptr(), bytes, cudaMemcpyDeviceToHost, t->ctx->stream));
    WRK_CUDA(cudaStreamSynchronize(t->ctx->stream));
    return WRK_OK;
}

int32_t wrk_tensor_retain(wrk_tensor* t) {
    WRK_REQUIRE(t, WRK_ERR_INVALID_ARGUMENT, "null tensor");
    t->refs.fetch_add(1);
    return WRK_OK;
}

int32_t wrk_tensor_release(wrk_tensor* t) {
    if (!t) return WRK_OK;
    if (t->refs.fetch_sub(1) == 1) delete t;
    return WRK_OK;
}

int32_t wrk_tensor_deep_clone(wrk_tensor* t, wrk_tensor** out) {
    WRK_REQUIRE(t && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    wrk_tensor* c = nullptr;
    WRK_TRY(tensor_alloc(t->ctx, t->dtype, t->shape.v, false, &c));
    if (t->bytes()) {
        cudaError_t e = cudaMemcpyAsync(c->ptr(), t->ptr(), t->bytes(), cudaMemcpyDeviceToDevice, t->ctx->stream);
        if (e != cudaSuccess) {
            wrk_tensor_release(c);
            return set_error(WRK_ERR_CUDA, "cudaMemcpyAsync failed: %s", cudaGetErrorString(e));
        }
    }
    *out = c;
    return WRK_OK;
}

int32_t wrk_tensor_shape(const wrk_tensor* t, uint32_t shape[4]) {
    WRK_REQUIRE(t && shape, WRK_ERR_INVALID_ARGUMENT, "null argument");
    for (int i = 0; i < 4; ++i) shape[i] = t->shape.v[i];
    return WRK_OK;
}

int32_t wrk_tensor_dtype(const wrk_tensor* t, int32_t* dtype) {
    WRK_REQUIRE(t && dtype, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *dtype = t->dtype;
    return WRK_OK;
}

int32_t wrk_tensor_device_ptr(const wrk_tensor* t, void** ptr) {
    WRK_REQUIRE(t && ptr, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *ptr = t->ptr();
    return WRK_OK;
}

int32_t wrk_tensor_reshape(wrk_tensor* t, const uint32_t shape[4], wrk_tensor** out) {
    WRK_REQUIRE(t && shape && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    uint32_t s[4];
    int autos = 0, auto_at = -1;
    size_t known = 1;
    for (int i = 0; i < 4; ++i) {
        s[i] = shape[i];
        if (s[i] == WRK_DIM_AUTO) {
            ++autos;
            auto_at = i;
        } else {
            known *= s[i];
        }
    }
    WRK_REQUIRE(autos <= 1, WRK_ERR_DEDUCE, "cannot deduce dimension");
    if (autos == 1) {
        WRK_REQUIRE(known != 0 && t->len() % known == 0, WRK_ERR_DEDUCE, "cannot deduce dimension");
        s[auto_at] = (uint32_t)(t->len() / known);
    }
    const size_t n = (size_t)s[0] * s[1] * s[2] * s[3];
    WRK_REQUIRE(n == t->len(), WRK_ERR_SIZE, "data size not match: %zu vs. %zu", t->len(), n);
    auto r = new wrk_tensor();
    r->ctx = t->ctx;
    r->buf = t->buf;
    r->dtype = t->dtype;
    for (int i = 0; i < 4; ++i) r->shape.v[i] = s[i];
    *out = r;
    return WRK_OK;
}

int32_t wrk_tensor_view(wrk_tensor* t, const uint32_t start[4], const uint32_t end[4], wrk_view* out) {
    WRK_REQUIRE(t && start && end && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    for (int i = 0; i < 4; ++i) {
        if (start[i] > end[i] || end[i] > t->shape.v[i])
            return set_error(WRK_ERR_SLICE_OUT_OF_RANGE, "slice %u..%u out of range for dimension size %u", start[i],
                             end[i], t->shape.v[i]);
    }
    out->tensor = t;
    for (int i = 0; i < 4; ++i) {
        out->shape[i] = end[i] - start[i];
        out->stride[i] = t->shape.v[i];
        out->offset[i] = start[i];
    }
    return WRK_OK;
}

int32_t wrk_tensor_as_view(wrk_tensor* t, wrk_view* out) {
    WRK_REQUIRE(t && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    out->tensor = t;
    for (int i = 0; i < 4; ++i) {
        out->shape[i] = t->shape.v[i];
        out->stride[i] = t->shape.v[i];
        out->offset[i] = 0;
    }
    return WRK_OK;
}

// ---- ops -----------------------------------------------------------------------------

int32_t wrk_op_list(wrk_op* const* ops, size_t count, wrk_op** out) {
    WRK_REQUIRE(out && (ops || count == 0), WRK_ERR_INVALID_ARGUMENT, "null argument");
    auto op = new wrk_op();
    op->kind = wrk_op::List;
    op->name = "list";
    op->num_kernels = 0;
    for (size_t i = 0; i < count; ++i) {
        if (!ops[i]) {
            delete op;
            return set_error(WRK_ERR_INVALID_ARGUMENT, "null op at index %zu", i);
        }
        ops[i]->refs.fetch_add(1);
        op->children.push_back(ops[i]);
    }
    *out = op;
    return WRK_OK;
}

int32_t wrk_op_sep(wrk_op** out) {
    WRK_REQUIRE(out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    auto op = new wrk_op();
    op->kind = wrk_op::Sep;
    op->name = "sep";
    op->num_kernels = 0;
    *out = op;
    return WRK_OK;
}

int32_t wrk_op_release(wrk_op* op) {
    if (!op) return WRK_OK;
    if (op->refs.fetch_sub(1) == 1) delete op;
    return WRK_OK;
}

static void flatten(wrk_op* op, std::vector<wrk_op*>& atoms) {
    switch (op->kind) {
        case wrk_op::Atom: atoms.push_back(op); break;
        case wrk_op::List:
            for (auto c : op->children) flatten(c, atoms);
            break;
        case wrk_op::Sep: break;  // a stream already orders everything; the separator carries no work
    }
}

int32_t wrk_op_num_atoms(const wrk_op* op, uint64_t* count) {
    WRK_REQUIRE(op && count, WRK_ERR_INVALID_ARGUMENT, "null argument");
    std::vector<wrk_op*> atoms;
    flatten(const_cast<wrk_op*>(op), atoms);
    *count = atoms.size();
    return WRK_OK;
}

static int32_t launch_all(wrk_context* ctx, const std::vector<wrk_op*>& atoms, cudaStream_t stream) {
    for (auto a : atoms) {
        cudaError_t e = a->launch(stream);
        if (e != cudaSuccess)
            return set_error(WRK_ERR_CUDA, "launch of %s failed: %s", a->name.c_str(), cudaGetErrorString(e));
    }
    return WRK_OK;
}

int32_t wrk_encode(wrk_context* ctx, wrk_op* op, int32_t use_graph, wrk_commands** out) {
    WRK_REQUIRE(ctx && op && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    auto cmd = new wrk_commands();
    flatten(op, cmd->atoms);
    for (auto a : cmd->atoms) {
        a->refs.fetch_add(1);
        cmd->num_kernels += a->num_kernels;
    }
    if (use_graph && !cmd->atoms.empty()) {
        std::lock_guard<std::mutex> lock(ctx->mutex);
        cudaSetDevice(ctx->device);
        cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
        if (e != cudaSuccess) {
            delete cmd;
            return set_error(WRK_ERR_CUDA, "cudaStreamBeginCapture failed: %s", cudaGetErrorString(e));
        }
        int32_t s = launch_all(ctx, cmd->atoms, ctx->stream);
        e = cudaStreamEndCapture(ctx->stream, &cmd->graph);
        if (s != WRK_OK || e != cudaSuccess) {
            delete cmd;
            if (s != WRK_OK) return s;
            return set_error(WRK_ERR_CUDA, "cudaStreamEndCapture failed: %s", cudaGetErrorString(e));
        }
        e = cudaGraphInstantiate(&cmd->exec, cmd->graph, 0);
        if (e != cudaSuccess) {
            delete cmd;
            return set_error(WRK_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
        }
    }
    *out = cmd;
    return WRK_OK;
}

int32_t wrk_submit(wrk_context* ctx, wrk_commands* commands) {
    WRK_REQUIRE(ctx && commands, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_CUDA(cudaSetDevice(ctx->device));
    if (commands->exec) {
        WRK_CUDA(cudaGraphLaunch(commands->exec, ctx->stream));
    } else {
        WRK_TRY(launch_all(ctx, commands->atoms, ctx->stream));
    }
    ctx->launches.fetch_add(commands->num_kernels);
    return WRK_OK;
}

int32_t wrk_commands_release(wrk_commands* commands) {
    delete commands;
    return WRK_OK;
}

int32_t wrk_run(wrk_context* ctx, wrk_op* op) {
    WRK_REQUIRE(ctx && op, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_CUDA(cudaSetDevice(ctx->device));
    std::vector<wrk_op*> atoms;
    flatten(op, atoms);
    WRK_TRY(launch_all(ctx, atoms, ctx->stream));
    uint64_t n = 0;
    for (auto a : atoms) n += a->num_kernels;
    ctx->launches.fetch_add(n);
    return WRK_OK;
}

}  // extern "C"
