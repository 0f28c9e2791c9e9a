// Vector forms of the elementwise kernels of support.cu for the shapes a prefill job produces: dense tensors
// [C, T (, Z)] with C a multiple of 8 and 16-byte-aligned rows.  A thread takes eight consecutive channels of one row
// with 16-byte loads and 32-bit index arithmetic (the general kernels divide 64-bit indices per element and move two
// bytes per access).  The arithmetic per element is the general kernels', expression for expression, so a tensor
// comes out with the same bits whichever kernel handled it.  Each entry point returns false when the operands do not
// fit; the caller then launches the general kernel.
//
// Same reference shaders as support.cu: token_shift.wgsl, binary.wgsl (add / mul with activations), activation.wgsl,
// blit.wgsl, channel_mix.wgsl / channel_mix_v7.wgsl, layer_norm.wgsl (src/tensor/ops.rs:1393-1462, 1656-1795, 1566-1650,
// 2015-2060, 407-470).
#include "device.cuh"

namespace wrk {
namespace k {

namespace {

constexpr int kVecThreads = 256;

inline int vec_grid(size_t n) {
    size_t g = (n + kVecThreads - 1) / kVecThreads;
    return (int)(g < 1 ? 1 : g > 148 * 16 ? 148 * 16 : g);
}

// eight consecutive elements of an f16 or f32 array, as floats
template <typename T>
__device__ __forceinline__ void load8(const T* p, float v[8]);
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float v[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float v[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float v[8]);
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float v[8]) {
    uint4 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __halves2half2(__float2half_rn(v[2 * i]), __float2half_rn(v[2 * i + 1]));
    *reinterpret_cast<uint4*>(p) = raw;
}
template <>
__device__ __forceinline__ void store8<float>(float* p, const float v[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}

// A view whose elements (c, t, b) lie at first + (b T + t) C + c: returns the element offset of (0, 0, 0).
bool dense(const DView& v, size_t* first) {
    if (v.offset[0] != 0 || v.stride[0] != v.shape[0]) return false;
    if (v.shape[2] != 1 && (v.offset[1] != 0 || v.stride[1] != v.shape[1])) return false;
    *first = v.index(0, 0, 0);
    return true;
}
template <typename T>
bool dense_as(const DView& v, T** p) {
    size_t first;
    if (v.dtype != (sizeof(T) == 2 ? WRK_F16 : WRK_F32) || v.shape[0] % 8 != 0 || !dense(v, &first)) return false;
    *p = static_cast<T*>(v.base) + first;
    return reinterpret_cast<uintptr_t>(*p) % 16 == 0;
}
bool fits32(size_t elements) { return elements / 8 < 0x7fffffffull; }

// ---- binary.wgsl: out <- act_out(act_x(in) (+|*) act_y(out)); `in` has out's shape, or one row [C] for the whole of
// out (plane8 = 0), or one row per plane [C, 1, Z] (plane8 = vectors per plane of out) ------------------------------
template <typename In, typename Out>
__global__ void binary_vec_kernel(int is_mul, const In* in, Out* out, uint32_t c8, uint32_t total8, int in_row, uint32_t plane8,
                                  int act_x, int act_y, int act_out) {
    for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < total8; o += gridDim.x * blockDim.x) {
        float x[8], y[8];
        load8(in + (size_t)(in_row ? (plane8 ? o / plane8 * c8 : 0u) + o % c8 : o) * 8, x);
        load8(out + (size_t)o * 8, y);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float ax = activate_f(act_x, x[i]), ay = activate_f(act_y, y[i]);
            y[i] = activate_f(act_out, is_mul ? ax * ay : ax + ay);
        }
        store8(out + (size_t)o * 8, y);
    }
}

template <typename In, typename Out>
bool binary_typed(int is_mul, const DView& input, const DView& output, int act_x, int act_y, int act_out, cudaStream_t stream) {
    In* in;
    Out* out;
    if (!dense_as<In>(input, &in) || !dense_as<Out>(output, &out)) return false;
    const bool same = input.shape[1] == output.shape[1] && input.shape[2] == output.shape[2];
    const bool row = input.shape[1] == 1 && input.shape[2] == 1;
    const bool plane_rows = input.shape[1] == 1 && input.shape[2] == output.shape[2];
    if (input.shape[0] != output.shape[0] || !(same || row || plane_rows)) return false;
    const size_t total = (size_t)output.shape[0] * output.shape[1] * output.shape[2];
    if (!fits32(total)) return false;
    const uint32_t c8 = output.shape[0] / 8;
    binary_vec_kernel<In, Out><<<vec_grid(total / 8), kVecThreads, 0, stream>>>(
        is_mul, in, out, c8, (uint32_t)(total / 8), same ? 0 : 1, same || row ? 0u : c8 * output.shape[1], act_x, act_y, act_out);
    return true;
}

// ---- activation.wgsl ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void activate_vec_kernel(T* x, uint32_t total8, int act) {
    for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < total8; o += gridDim.x * blockDim.x) {
        float v[8];
        load8(x + (size_t)o * 8, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = activate_f(act, v[i]);
        store8(x + (size_t)o * 8, v);
    }
}

// ---- blit.wgsl without a transpose (the data types may differ) --------------------------------------------------
template <typename In, typename Out>
__global__ void blit_vec_kernel(const In* in, Out* out, uint32_t total8) {
    for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < total8; o += gridDim.x * blockDim.x) {
        float v[8];
        load8(in + (size_t)o * 8, v);
        store8(out + (size_t)o * 8, v);
    }
}

template <typename In, typename Out>
bool blit_typed(const DView& input, const DView& output, cudaStream_t stream) {
    In* in;
    Out* out;
    if (!dense_as<In>(input, &in) || !dense_as<Out>(output, &out)) return false;
    const size_t total = (size_t)input.shape[0] * input.shape[1] * input.shape[2];
    if (!fits32(total)) return false;
    blit_vec_kernel<In, Out><<<vec_grid(total / 8), kVecThreads, 0, stream>>>(in, out, (uint32_t)(total / 8));
    return true;
}

// ---- token_shift.wgsl: out[c, t, z] <- mix(x_t, x_(t-1) or the carry row, f[c, (t,) z]) --------------------------
struct ShiftVecArgs {
    const uint32_t* cursors;
    int wide;
    DView state;  // f32, row 0 = the carry row
    const __half* in;  // [C, T]
    uint32_t c8, T, count;
    const __half* mix[kShiftMultiMax];  // factors of output i: one row [C] (mix_rows == 1) or one row per token
    const __half* bias[kShiftMultiMax]; // null, or one row [C] added to the factors first (the sum rounded to f16)
    __half* out[kShiftMultiMax];        // [C, T] each
    uint32_t mix_rows;
    int reversed;
};

__global__ void token_shift_vec_kernel(const ShiftVecArgs a) {
    const uint32_t total8 = a.c8 * a.T;
    for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < total8; o += gridDim.x * blockDim.x) {
        const uint32_t c = (o % a.c8) * 8, t = o / a.c8;
        const CursorD cu = cursor_at(a.cursors, a.wide, t);
        float cur[8], prev[8];
        load8(a.in + (size_t)o * 8, cur);
        if (t == cu.token) {
#pragma unroll
            for (int i = 0; i < 8; ++i) prev[i] = static_cast<const float*>(a.state.base)[a.state.index(c + i, 0, cu.batch)];
        } else {
            load8(a.in + (size_t)(o - a.c8) * 8, prev);
        }
#pragma unroll
        for (uint32_t k = 0; k < kShiftMultiMax; ++k) {
            if (k >= a.count) break;
            float f[8], y[8];
            load8(a.mix[k] + (size_t)(a.mix_rows == 1 ? o % a.c8 : o) * 8, f);
            if (a.bias[k] != nullptr) {
                float b[8];
                load8(a.bias[k] + (size_t)(o % a.c8) * 8, b);
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __half2float(__float2half_rn(b[i] + f[i]));
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = a.reversed ? mix_f(cur[i], prev[i], f[i]) : mix_f(prev[i], cur[i], f[i]);
            store8(a.out[k] + (size_t)o * 8, y);
        }
    }
}

// ---- channel_mix.wgsl / channel_mix_v7.wgsl ----------------------------------------------------------------------
// With `xres`, the residual stream takes the result as well: xres <- xres + x (x as stored, i.e. rounded to its type).
template <typename T>
__global__ void channel_mix_vec_kernel(const uint32_t* cursors, int wide, DView state, const T* r, const T* v, T* x, T* xres,
                                       uint32_t c8, uint32_t total8, int v7) {
    for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < total8; o += gridDim.x * blockDim.x) {
        const uint32_t c = (o % c8) * 8, t = o / c8;
        const CursorD cu = cursor_at(cursors, wide, t);
        float xv[8], vv[8];
        load8(x + (size_t)o * 8, xv);
        load8(v + (size_t)o * 8, vv);
        if (t - cu.token + 1u == cu.len) {
#pragma unroll
            for (int i = 0; i < 8; ++i) static_cast<float*>(state.base)[state.index(c + i, 0, cu.batch)] = xv[i];
        }
        if (!v7) {
            float rv[8];
            load8(r + (size_t)o * 8, rv);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float rr = 1.0f / (1.0f + expf(-rv[i]));
                vv[i] = rr * vv[i];
            }
        }
        store8(x + (size_t)o * 8, vv);
        if (xres != nullptr) {
            float res[8];
            load8(xres + (size_t)o * 8, res);
#pragma unroll
            for (int i = 0; i < 8; ++i) res[i] = (sizeof(T) == 2 ? __half2float(__float2half_rn(vv[i])) : vv[i]) + res[i];
            store8(xres + (size_t)o * 8, res);
        }
    }
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// ---- layer_norm.wgsl (and group norm: rows of one head) ----------------------------------------------------------
// (x - mean) * rsqrt(var + eps) * w + b with var = E[(x - mean)^2], the row read once.  With `delta`, src <- src + delta
// first (rounded to the data type, as the separate add stores it).
template <typename T>
__device__ __forceinline__ void norm_load(const T* delta, T* src, size_t at, float v[8]) {
    load8(src + at, v);
    if (delta != nullptr) {
        float d[8];
        load8(delta + at, d);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = sizeof(T) == 2 ? __half2float(__float2half_rn(d[i] + v[i])) : d[i] + v[i];
        store8(src + at, v);
    }
}
__device__ __forceinline__ void norm_store(const __half* w, const __half* b, size_t wat, float mean, float dev, float v[8]) {
    float wv[8], bv[8];
    load8(w + wat, wv);
    load8(b + wat, bv);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = fmaf((v[i] - mean) * dev, wv[i], bv[i]);
}

// Rows of up to 256 values: C / 8 lanes per row (a power of two), several rows per warp, sums by shuffles.
// With `gated`, the normalised row is not stored in x but rounded to f16 (the copy into an f16 tensor), multiplied by
// act(gate) and stored, rounded again, in `gated` (token-major [rows C] like x): group norm + blit + mul in one pass.
template <typename T>
__global__ void layer_norm_rows_kernel(const __half* w, const __half* b, const T* delta, T* src, T* x, uint32_t C, uint32_t rows,
                                       uint32_t wrows, float eps, const __half* gate, __half* gated, int gate_act) {
    const uint32_t lanes = C / 8;
    const uint32_t per_block = blockDim.x / lanes;
    for (uint32_t row0 = blockIdx.x * per_block; row0 < rows; row0 += gridDim.x * per_block) {  // uniform trip count per warp
        const uint32_t row = row0 + threadIdx.x / lanes, l = threadIdx.x % lanes;
        const bool live = row < rows;
        const size_t at = (size_t)row * C + l * 8;
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (live) norm_load(delta, src, at, v);
        float s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
        for (uint32_t off = lanes / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        const float mean = s / (float)C;
        float m2 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) m2 = fmaf(v[i] - mean, v[i] - mean, m2);
        for (uint32_t off = lanes / 2; off > 0; off >>= 1) m2 += __shfl_xor_sync(0xffffffffu, m2, off);
        const float dev = rsqrtf(m2 / (float)C + eps);
        if (live) {
            norm_store(w, b, (size_t)(row % wrows) * C + l * 8, mean, dev, v);
            if (gated == nullptr) {
                store8(x + at, v);
            } else {
                float g[8];
                load8(gate + at, g);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = activate_f(gate_act, g[i]) * __half2float(__float2half_rn(v[i]));
                store8(gated + at, v);
            }
        }
    }
}

// Rows of up to 8192 values: one CTA of 256 threads per row, up to four vectors of eight per thread.
constexpr int kNormIters = 4;
template <typename T>
__global__ void __launch_bounds__(256) layer_norm_wide_kernel(const __half* w, const __half* b, const T* delta, T* src, T* x,
                                                              uint32_t C, uint32_t rows, uint32_t wrows, float eps) {
    __shared__ float scratch[2][8];
    const uint32_t c8 = C / 8, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto block_total = [&](float s, int which) {
        s = warp_sum(s);
        if (lane == 0) scratch[which][warp] = s;
        __syncthreads();
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += scratch[which][i];
        return t;
    };
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * C, wb = (size_t)(row % wrows) * C;
        float v[kNormIters][8];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kNormIters; ++i) {
            const uint32_t k = threadIdx.x + i * 256;
#pragma unroll
            for (int e = 0; e < 8; ++e) v[i][e] = 0.f;
            if (k < c8) norm_load(delta, src, base + (size_t)k * 8, v[i]);
            s += ((v[i][0] + v[i][1]) + (v[i][2] + v[i][3])) + ((v[i][4] + v[i][5]) + (v[i][6] + v[i][7]));
        }
        const float mean = block_total(s, 0) / (float)C;
        float m2 = 0.f;
#pragma unroll
        for (int i = 0; i < kNormIters; ++i) {
            if (threadIdx.x + i * 256 < c8) {
#pragma unroll
                for (int e = 0; e < 8; ++e) m2 = fmaf(v[i][e] - mean, v[i][e] - mean, m2);
            }
        }
        const float dev = rsqrtf(block_total(m2, 1) / (float)C + eps);
#pragma unroll
        for (int i = 0; i < kNormIters; ++i) {
            const uint32_t k = threadIdx.x + i * 256;
            if (k < c8) {
                norm_store(w, b, wb + (size_t)k * 8, mean, dev, v[i]);
                store8(x + base + (size_t)k * 8, v[i]);
            }
        }
        __syncthreads();  // the scratch rows are rewritten by the next row
    }
}

template <typename T>
bool layer_norm_typed(const __half* w, const __half* b, const void* delta, void* src, void* x, uint32_t C, uint32_t rows,
                      uint32_t wrows, float eps, cudaStream_t stream) {
    const T* dp = static_cast<const T*>(delta);
    T *sp = static_cast<T*>(src), *xp = static_cast<T*>(x);
    const uint32_t lanes = C / 8;
    if (C <= 256 && (lanes & (lanes - 1)) == 0) {
        const uint32_t per_block = 256 / lanes, blocks = (rows + per_block - 1) / per_block;
        layer_norm_rows_kernel<T><<<blocks < 148u * 16u ? blocks : 148u * 16u, 256, 0, stream>>>(w, b, dp, sp, xp, C, rows, wrows, eps,
                                                                                                   nullptr, nullptr, 0);
        return true;
    }
    if (lanes <= (uint32_t)kNormIters * 256) {
        layer_norm_wide_kernel<T><<<rows < 148u * 8u ? rows : 148u * 8u, 256, 0, stream>>>(w, b, dp, sp, xp, C, rows, wrows, eps);
        return true;
    }
    return false;
}

}  // namespace

bool group_norm_gate_supported(const __half* w, const __half* b, const void* x, const __half* gate, const __half* out, uint32_t C) {
    const uint32_t lanes = C / 8;
    return C % 8 == 0 && C <= 256 && (lanes & (lanes - 1)) == 0 && aligned16(w) && aligned16(b) && aligned16(x) && aligned16(gate) &&
           aligned16(out);
}

cudaError_t group_norm_gate(const __half* w, const __half* b, int dtype, void* x, uint32_t C, uint32_t rows, uint32_t wrows, float eps,
                            const __half* gate, __half* out, int gate_act, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    if (!group_norm_gate_supported(w, b, x, gate, out, C)) return cudaErrorInvalidValue;
    const uint32_t per_block = 256 / (C / 8), blocks = (rows + per_block - 1) / per_block;
    const uint32_t grid = blocks < 148u * 16u ? blocks : 148u * 16u;
    if (dtype == WRK_F16)
        layer_norm_rows_kernel<__half><<<grid, 256, 0, stream>>>(w, b, nullptr, static_cast<__half*>(x), static_cast<__half*>(x), C, rows,
                                                                 wrows, eps, gate, out, gate_act);
    else
        layer_norm_rows_kernel<float><<<grid, 256, 0, stream>>>(w, b, nullptr, static_cast<float*>(x), static_cast<float*>(x), C, rows,
                                                                wrows, eps, gate, out, gate_act);
    return cudaGetLastError();
}

bool layer_norm_vec(const __half* w, const __half* b, int dtype, const void* delta, void* src, void* x, uint32_t C, uint32_t rows,
                    uint32_t wrows, float eps, cudaStream_t stream) {
    if (C % 8 != 0 || !aligned16(w) || !aligned16(b) || !aligned16(src) || !aligned16(x) || (delta && !aligned16(delta))) return false;
    return dtype == WRK_F16 ? layer_norm_typed<__half>(w, b, delta, src, x, C, rows, wrows, eps, stream)
                            : layer_norm_typed<float>(w, b, delta, src, x, C, rows, wrows, eps, stream);
}

bool binary_vec(int is_mul, const DView& input, const DView& output, int act_x, int act_y, int act_out, cudaStream_t stream) {
    if (input.dtype == WRK_F16 && output.dtype == WRK_F16)
        return binary_typed<__half, __half>(is_mul, input, output, act_x, act_y, act_out, stream);
    if (input.dtype == WRK_F16 && output.dtype == WRK_F32)
        return binary_typed<__half, float>(is_mul, input, output, act_x, act_y, act_out, stream);
    if (input.dtype == WRK_F32 && output.dtype == WRK_F32)
        return binary_typed<float, float>(is_mul, input, output, act_x, act_y, act_out, stream);
    return false;
}

bool activate_vec(const DView& x, int act, cudaStream_t stream) {
    const size_t total = (size_t)x.shape[0] * x.shape[1] * x.shape[2];
    if (!fits32(total)) return false;
    __half* h;
    float* f;
    if (dense_as<__half>(x, &h)) {
        activate_vec_kernel<__half><<<vec_grid(total / 8), kVecThreads, 0, stream>>>(h, (uint32_t)(total / 8), act);
        return true;
    }
    if (dense_as<float>(x, &f)) {
        activate_vec_kernel<float><<<vec_grid(total / 8), kVecThreads, 0, stream>>>(f, (uint32_t)(total / 8), act);
        return true;
    }
    return false;
}

bool blit_vec(const DView& input, const DView& output, cudaStream_t stream) {
    if (input.shape[0] != output.shape[0] || input.shape[1] != output.shape[1] || input.shape[2] != output.shape[2]) return false;
    if (input.dtype == WRK_F16 && output.dtype == WRK_F16) return blit_typed<__half, __half>(input, output, stream);
    if (input.dtype == WRK_F32 && output.dtype == WRK_F32) return blit_typed<float, float>(input, output, stream);
    if (input.dtype == WRK_F32 && output.dtype == WRK_F16) return blit_typed<float, __half>(input, output, stream);
    if (input.dtype == WRK_F16 && output.dtype == WRK_F32) return blit_typed<__half, float>(input, output, stream);
    return false;
}

namespace {
bool shift_vec_args(const uint32_t* cursors, int wide, const DView& time_mix, const DView* bias, const DView& state,
                    const DView& input, const DView& output, int reversed, ShiftVecArgs* out_args) {
    const uint32_t C = output.shape[0], T = output.shape[1], Z = output.shape[2];
    __half *in, *out, *mix, *bp = nullptr;
    if (bias != nullptr && (!dense_as<__half>(*bias, &bp) || bias->shape[0] != C || bias->shape[1] != 1 || bias->shape[2] != Z))
        return false;
    if (Z == 0 || Z > kShiftMultiMax || !dense_as<__half>(input, &in) || !dense_as<__half>(output, &out) ||
        !dense_as<__half>(time_mix, &mix))
        return false;
    if (input.shape[0] != C || input.shape[1] != T || input.shape[2] != 1) return false;  // one input for every plane
    const bool per_token = time_mix.shape[1] == T && time_mix.shape[2] == Z && T != 1;
    const bool one_row = time_mix.shape[1] == 1 && time_mix.shape[2] == Z;
    if (time_mix.shape[0] != C || !(per_token || one_row) || !fits32((size_t)C * T)) return false;
    ShiftVecArgs a{};
    a.cursors = cursors;
    a.wide = wide;
    a.state = state;
    a.in = in;
    a.c8 = C / 8;
    a.T = T;
    a.count = Z;
    a.mix_rows = one_row ? 1 : T;
    a.reversed = reversed;
    for (uint32_t z = 0; z < Z; ++z) {
        a.mix[z] = mix + (size_t)z * C * (one_row ? 1 : T);
        a.bias[z] = bp ? bp + (size_t)z * C : nullptr;
        a.out[z] = out + (size_t)z * C * T;
    }
    *out_args = a;
    return true;
}
}  // namespace

bool token_shift_vec_fits(const DView& time_mix, const DView* bias, const DView& state, const DView& input, const DView& output) {
    ShiftVecArgs a;
    return shift_vec_args(nullptr, 0, time_mix, bias, state, input, output, 0, &a);
}

bool token_shift_vec(const uint32_t* cursors, int wide, const DView& time_mix, const DView* bias, const DView& state,
                     const DView& input, const DView& output, int reversed, cudaStream_t stream) {
    ShiftVecArgs a;
    if (!shift_vec_args(cursors, wide, time_mix, bias, state, input, output, reversed, &a)) return false;
    token_shift_vec_kernel<<<vec_grid((size_t)a.c8 * a.T), kVecThreads, 0, stream>>>(a);
    return true;
}

bool token_shift_multi_vec(const ShiftMultiArgs& m, cudaStream_t stream) {
    if (m.C % 8 != 0 || !fits32((size_t)m.C * m.T) || !aligned16(m.in)) return false;
    ShiftVecArgs a{};
    a.cursors = m.cursors;
    a.wide = m.wide;
    a.state = m.state;
    a.in = m.in;
    a.c8 = m.C / 8;
    a.T = m.T;
    a.count = m.count;
    a.mix_rows = 1;
    a.reversed = m.reversed;
    for (uint32_t i = 0; i < m.count; ++i) {
        if (!aligned16(m.mix[i]) || !aligned16(m.out[i])) return false;
        a.mix[i] = m.mix[i];
        a.out[i] = m.out[i];
    }
    token_shift_vec_kernel<<<vec_grid((size_t)a.c8 * m.T), kVecThreads, 0, stream>>>(a);
    return true;
}

bool channel_mix_vec(const uint32_t* cursors, int wide, const DView& state, int dtype, const void* r, const void* v, void* x,
                     void* xres, uint32_t C, uint32_t T, int v7, cudaStream_t stream) {
    if (C % 8 != 0 || !fits32((size_t)C * T) || !aligned16(v) || !aligned16(x) || (!v7 && !aligned16(r)) || !aligned16(xres))
        return false;
    const uint32_t total8 = C / 8 * T;
    if (dtype == WRK_F16)
        channel_mix_vec_kernel<__half><<<vec_grid(total8), kVecThreads, 0, stream>>>(
            cursors, wide, state, static_cast<const __half*>(r), static_cast<const __half*>(v), static_cast<__half*>(x),
            static_cast<__half*>(xres), C / 8, total8, v7);
    else
        channel_mix_vec_kernel<float><<<vec_grid(total8), kVecThreads, 0, stream>>>(
            cursors, wide, state, static_cast<const float*>(r), static_cast<const float*>(v), static_cast<float*>(x),
            static_cast<float*>(xres), C / 8, total8, v7);
    return true;
}

}  // namespace k
}  // namespace wrk
