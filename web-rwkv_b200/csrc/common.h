// Internal declarations shared by the host side and the kernels of libwrk.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/wrk.h"

namespace wrk {

// ---- errors -------------------------------------------------------------------------
int32_t set_error(int32_t code, const char* fmt, ...);
#define WRK_CUDA(expr)                                                                         \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess)                                                                 \
            return wrk::set_error(WRK_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                \
                                  cudaGetErrorString(_e), __FILE__, __LINE__);                 \
    } while (0)
#define WRK_TRY(expr)                 \
    do {                              \
        int32_t _s = (expr);          \
        if (_s != WRK_OK) return _s;  \
    } while (0)
#define WRK_REQUIRE(cond, code, ...) \
    do {                             \
        if (!(cond)) return wrk::set_error(code, __VA_ARGS__); \
    } while (0)

inline size_t dtype_size(int dtype) {
    switch (dtype) {
        case WRK_F32: return 4;
        case WRK_F16: return 2;
        case WRK_U8: return 1;
        case WRK_U16: return 2;
        case WRK_U32: return 4;
        default: return 0;
    }
}

// ---- device-visible view ----------------------------------------------------------------
// Element (c, t, b) of a view lives at ((b + off.z) * stride.y + (t + off.y)) * stride.x + c + off.x
// elements from `base` (the reference's compute_index, e.g. matmul_vec_int8.wgsl:31-35).
struct DView {
    void* base;
    int32_t dtype;
    uint32_t shape[4];
    uint32_t stride[4];
    uint32_t offset[4];

    __host__ __device__ size_t index(uint32_t c, uint32_t t, uint32_t b) const {
        return ((size_t)(b + offset[2]) * stride[1] + (t + offset[1])) * stride[0] + c + offset[0];
    }
    __host__ __device__ size_t row(uint32_t t, uint32_t b) const { return index(0, t, b); }
};

// ---- host objects ---------------------------------------------------------------------
struct Buffer {
    wrk_context* ctx = nullptr;
    void* ptr = nullptr;
    size_t bytes = 0;
    std::shared_ptr<void> external;  // set: `ptr` lies in memory this object keeps alive and is not freed with the buffer
    explicit Buffer(wrk_context* owner);
    Buffer(const Buffer&) = delete;
    Buffer& operator=(const Buffer&) = delete;
    ~Buffer();
};

struct Shape4 {
    uint32_t v[4];
    uint32_t operator[](int i) const { return v[i]; }
    size_t len() const { return (size_t)v[0] * v[1] * v[2] * v[3]; }
    bool operator==(const Shape4& o) const { return v[0] == o.v[0] && v[1] == o.v[1] && v[2] == o.v[2] && v[3] == o.v[3]; }
};

using Launch = std::function<cudaError_t(cudaStream_t)>;

}  // namespace wrk

struct wrk_context {
    // One reference for the owner (dropped by wrk_context_destroy) and one per live device buffer: the stream
    // and the device outlive every tensor, op and command buffer that still holds memory of this context.
    std::atomic<int> refs{1};
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev_start = nullptr, ev_stop = nullptr;
    int num_sms = 0;
    int32_t* device_status = nullptr;  // device word: 0 = ok, else a wrk_status written by a kernel
    int32_t* host_status = nullptr;    // pinned mirror for reads
    std::atomic<uint64_t> launches{0};
    std::mutex mutex;
};

struct wrk_tensor {
    std::atomic<int> refs{1};
    wrk_context* ctx = nullptr;
    std::shared_ptr<wrk::Buffer> buf;
    int dtype = WRK_F32;
    wrk::Shape4 shape{{1, 1, 1, 1}};

    size_t len() const { return shape.len(); }
    size_t bytes() const { return len() * wrk::dtype_size(dtype); }
    void* ptr() const { return buf ? buf->ptr : nullptr; }
};

struct wrk_op {
    enum Kind { Atom, List, Sep };
    std::atomic<int> refs{1};
    Kind kind = Atom;
    std::string name;
    wrk::Launch launch;                              // Atom
    uint32_t num_kernels = 1;                        // kernels one launch() issues
    std::vector<std::shared_ptr<wrk::Buffer>> keep;  // buffers the atom touches
    std::vector<wrk_op*> children;                   // List (retained)
    ~wrk_op();
};

struct wrk_commands {
    std::vector<wrk_op*> atoms;  // retained, in order
    uint64_t num_kernels = 0;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    ~wrk_commands();
};

struct wrk_matrix {
    std::atomic<int> refs{1};
    int kind = 0;  // 0 Fp16, 1 Int8, 2 Fp4
    wrk_tensor* w = nullptr;
    wrk_tensor* m = nullptr;
    wrk_tensor* q = nullptr;
    ~wrk_matrix();
};

namespace wrk {

DView make_dview(const wrk_view& v);
DView make_dview(const wrk_tensor* t);
bool view_is(const wrk_view& v, uint32_t x, uint32_t y, uint32_t z, uint32_t w);
int32_t check_shape(const char* what, const Shape4& have, uint32_t x, uint32_t y, uint32_t z, uint32_t w);
int32_t check_view(const char* what, const wrk_view* v, uint32_t x, uint32_t y, uint32_t z, uint32_t w);
bool is_float(int dtype);
wrk_op* new_atom(const char* name, Launch launch, std::initializer_list<const wrk_tensor*> tensors,
                 uint32_t num_kernels = 1);
int32_t tensor_alloc(wrk_context* ctx, int dtype, const uint32_t shape[4], bool zero, wrk_tensor** out);

}  // namespace wrk
