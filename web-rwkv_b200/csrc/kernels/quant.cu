// Int8 and NF4 weight quantizers (packing kernels) for sm_100a.
//
// Replaces quant_mat_int8.wgsl / quant_mat_nf4.wgsl of the reference.  Both are single fused
// passes (the reference reads the fp16 input twice and NF4 goes through an f32 scratch): a
// group of 16 (Int8) or 8 (NF4) lanes owns one quantization block, reads it with one 16-byte
// load per lane, reduces min/max or absmax with shuffles, and writes the packed bytes with one
// 8-byte or 4-byte store per lane.  HBM-bound: algorithmic bytes per element are
// 2 + 1 + 4/128 (Int8) and 2 + 1/2 + 2/64 (NF4).
//
// The packed bytes and scales must be bit-identical to the reference arithmetic, so every f32
// operation below uses an explicitly rounded intrinsic (no FMA contraction).
#include "kernels.h"

namespace wrk {
namespace k {

namespace {

__device__ __forceinline__ void unpack8(const uint4& raw, float v[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

// One lane handles 8 consecutive elements; 16 lanes share an Int8 block of 128.
__global__ void __launch_bounds__(256) quantize_int8_kernel(const __half* __restrict__ input, size_t len,
                                                            __half* __restrict__ minmax,
                                                            uint8_t* __restrict__ output) {
    const size_t nvec = (len + 7) / 8;
    const size_t nvec_pad = (nvec + 15) / 16 * 16;  // whole 16-lane groups stay converged for the shuffles
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec_pad;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t e0 = i * 8;
        float v[8];
        int valid = 0;
        if (e0 + 8 <= len) {
            unpack8(*reinterpret_cast<const uint4*>(input + e0), v);
            valid = 8;
        } else if (e0 < len) {
            valid = (int)(len - e0);
            for (int j = 0; j < 8; ++j) v[j] = j < valid ? __half2float(input[e0 + j]) : 0.0f;
        }
        float mn = 65504.0f, mx = -65504.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (j < valid) {
                mn = fminf(v[j], mn);
                mx = fmaxf(v[j], mx);
            }
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off, 16));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off, 16));
        }
        if (valid == 0) continue;
        if ((i & 15) == 0) {
            const size_t blk = e0 / 128;
            reinterpret_cast<__half2*>(minmax)[blk] = __floats2half2_rn(mn, mx);
        }
        const float range = __fsub_rn(mx, mn);
        uint32_t packed[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float x = __fdiv_rn(__fsub_rn(v[j], mn), range);
            x = (x > 0.0f) ? x : 0.0f;  // false for NaN: a degenerate block maps to 0
            x = (x > 1.0f) ? 1.0f : x;
            const float q = floorf(__fadd_rn(0.5f, __fmul_rn(255.0f, x)));
            packed[j >> 2] |= ((uint32_t)q & 0xffu) << ((j & 3) * 8);
        }
        if (valid == 8) {
            *reinterpret_cast<uint2*>(output + e0) = make_uint2(packed[0], packed[1]);
        } else {
            for (int j = 0; j < valid; ++j) output[e0 + j] = (uint8_t)(packed[j >> 2] >> ((j & 3) * 8));
        }
    }
}

// Nearest-entry search.  `literal` runs the reference loop: the last index j whose error
// |table[j] - x| is <= the running minimum, starting from (1.0, 0).  For an ascending table the
// same answer comes from locating the bracketing pair (4 comparisons) and applying the `<=` rule
// to the two rounded errors: errors are monotone on each side of x, so only the bracketing pair
// can tie for the minimum.
template <bool LITERAL>
__device__ __forceinline__ uint32_t nf4_index(const float* __restrict__ q, float x) {
    if (LITERAL) {
        float min_err = 1.0f;
        uint32_t min_index = 0;
#pragma unroll
        for (uint32_t j = 0; j < 16; ++j) {
            const float err = fabsf(__fsub_rn(q[j], x));
            if (err <= min_err) {
                min_err = err;
                min_index = j;
            }
        }
        return min_index;
    } else {
        // lo = largest index with q[lo] <= x (0 if none)
        uint32_t lo = (x >= q[8]) ? 8u : 0u;
        lo += (x >= q[lo + 4]) ? 4u : 0u;
        lo += (x >= q[lo + 2]) ? 2u : 0u;
        lo += (x >= q[lo + 1]) ? 1u : 0u;
        const uint32_t hi = lo < 15u ? lo + 1u : 15u;
        const float e_lo = fabsf(__fsub_rn(q[lo], x));
        const float e_hi = fabsf(__fsub_rn(q[hi], x));
        // literal rule restricted to {lo, hi}; both errors must also pass the initial 1.0 bound
        uint32_t idx = 0;
        float min_err = 1.0f;
        if (e_lo <= min_err) { min_err = e_lo; idx = lo; }
        if (e_hi <= min_err) { idx = hi; }
        return idx;
    }
}

// One lane handles 8 consecutive elements (one packed u32); 8 lanes share an NF4 block of 64.
template <bool LITERAL>
__global__ void __launch_bounds__(256) quantize_nf4_kernel(const __half* __restrict__ input, size_t len,
                                                           const float* __restrict__ table,
                                                           __half* __restrict__ absmax,
                                                           uint8_t* __restrict__ output) {
    __shared__ float q[16];
    if (threadIdx.x < 16) q[threadIdx.x] = table[threadIdx.x];
    __syncthreads();
    const size_t nvec = (len + 7) / 8;
    const size_t nvec_pad = (nvec + 7) / 8 * 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec_pad;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t e0 = i * 8;
        float v[8];
        int valid = 0;
        if (e0 + 8 <= len) {
            unpack8(*reinterpret_cast<const uint4*>(input + e0), v);
            valid = 8;
        } else if (e0 < len) {
            valid = (int)(len - e0);
            for (int j = 0; j < 8; ++j) v[j] = j < valid ? __half2float(input[e0 + j]) : 0.0f;
        }
        float mx = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (j < valid) mx = fmaxf(fabsf(v[j]), mx);
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off, 8));
        if (valid == 0) continue;
        if ((i & 7) == 0) absmax[e0 / 64] = __float2half_rn(mx);
        const float a = __fdiv_rn(1.0f, mx);
        uint32_t y = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (j < valid) y |= nf4_index<LITERAL>(q, __fmul_rn(v[j], a)) << (j * 4);
        }
        if (valid == 8) {
            *reinterpret_cast<uint32_t*>(output + e0 / 2) = y;
        } else {
            for (int j = 0; j < (valid + 1) / 2; ++j) output[e0 / 2 + j] = (uint8_t)(y >> (8 * j));
        }
    }
}

inline int grid_for(size_t work_items, int block, int num_sms) {
    const size_t need = (work_items + block - 1) / block;
    const size_t cap = (size_t)num_sms * 8;  // persistent grid-stride: 8 CTAs of 256 per SM
    return (int)(need < cap ? (need ? need : 1) : cap);
}

}  // namespace

cudaError_t quantize_int8(const __half* input, size_t len, __half* minmax, uint8_t* output, int num_sms,
                          cudaStream_t stream) {
    if (len == 0) return cudaSuccess;
    const int grid = grid_for((len + 7) / 8, 256, num_sms);
    quantize_int8_kernel<<<grid, 256, 0, stream>>>(input, len, minmax, output);
    return cudaGetLastError();
}

cudaError_t quantize_nf4(const __half* input, size_t len, const float* table, bool table_sorted, __half* absmax,
                         uint8_t* output, int num_sms, cudaStream_t stream) {
    if (len == 0) return cudaSuccess;
    const int grid = grid_for((len + 7) / 8, 256, num_sms);
    if (table_sorted)
        quantize_nf4_kernel<false><<<grid, 256, 0, stream>>>(input, len, table, absmax, output);
    else
        quantize_nf4_kernel<true><<<grid, 256, 0, stream>>>(input, len, table, absmax, output);
    return cudaGetLastError();
}

}  // namespace k
}  // namespace wrk
