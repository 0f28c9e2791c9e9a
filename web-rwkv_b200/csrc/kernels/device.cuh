// Device-side helpers shared by the kernels.
#pragma once

#include "kernels.h"

namespace wrk {
namespace k {

__device__ __forceinline__ float dload(const void* base, int dtype, size_t i) {
    return dtype == WRK_F16 ? __half2float(static_cast<const __half*>(base)[i])
                            : static_cast<const float*>(base)[i];
}
__device__ __forceinline__ void dstore(void* base, int dtype, size_t i, float x) {
    if (dtype == WRK_F16) static_cast<__half*>(base)[i] = __float2half_rn(x);
    else static_cast<float*>(base)[i] = x;
}

// Activation functions of the reference (src/tensor/ops.rs:205-235), evaluated in f32.
__device__ __forceinline__ float activate_f(int act, float x) {
    switch (act) {
        case WRK_ACT_SQUARED_RELU: { const float p = fmaxf(x, 0.0f); return p * p; }
        case WRK_ACT_TANH: return x > 42.0f ? 1.0f : tanhf(x);
        case WRK_ACT_STABLE_EXP: return expf(-expf(x));
        case WRK_ACT_OPPOSITE_EXP: return -expf(x);
        case WRK_ACT_SOFTPLUS: return logf(1.0f + expf(x));
        case WRK_ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
        case WRK_ACT_SILU: return x / (1.0f + expf(-x));
        default: return x;
    }
}

// Roundings fixed by hand (no contraction left to the compiler), so that every kernel that evaluates one of these
// gives the same bits: the merged elementwise kernels are compared bit for bit with the single-op kernels.
// a (1 - f) + b f: the token shift and lerp of the reference (token_shift.wgsl, lerp.wgsl: mix(a, b, f))
__device__ __forceinline__ float mix_f(float a, float b, float f) { return __fmaf_rn(b, f, __fmul_rn(a, __fsub_rn(1.0f, f))); }
// k (1 + (a - 1) p): control_k_v7.wgsl
__device__ __forceinline__ float control_k_f(float k, float a, float p) {
    return __fmul_rn(k, __fmaf_rn(__fsub_rn(a, 1.0f), p, 1.0f));
}

struct CursorD { uint32_t batch, token, len; };
// Packed cursor: batch | token << 8 | len << 24 (src/tensor/mod.rs:53-60); wide: three u32 per token.
__device__ __forceinline__ CursorD cursor_at(const uint32_t* cursors, int wide, uint32_t t) {
    CursorD c;
    if (wide) {
        c.batch = cursors[3 * t];
        c.token = cursors[3 * t + 1];
        c.len = cursors[3 * t + 2];
    } else {
        const uint32_t x = cursors[t];
        c.batch = x & 0xffu;
        c.token = (x >> 8) & 0xffffu;
        c.len = (x >> 24) & 0xffu;
    }
    return c;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

}  // namespace k
}  // namespace wrk
