// fp16 matmul with a short K: the second matrices of the low-rank adapters of v6 / v7 (32..256 -> C) at any number
// of tokens above the weight-streaming kernel's eight.  The matrices are 0.25-1 MB; the tensor-memory GEMM spends
// about 10 us of fixed work (TMEM allocation, tensor maps, pipeline fill) on each, as much as on a 4096 x 4096 Int8
// matrix; this kernel takes 6-7 us at 64 tokens.  A CTA of four warps owns a tile of 32 rows x 64 tokens, copies
// both operands into shared memory with 16-byte loads (all in flight before the first store) and multiplies with
// mma.sync.m16n8k16 (fp32 accumulate).  (A variant that also split a long K over CTAs, for the adapters' first
// matrices, measured 14 us against the tensor-memory kernel's 10 us and was dropped.)
//
// Replaces, for these shapes, the same reference shaders as the other matmul kernels: matmul_mat_fp16.wgsl
// (TensorOp::matmul_mat_fp16, src/tensor/ops.rs:999-1070) and matmul_vec_fp16.wgsl (TensorOp::matmul_vec_fp16,
// src/tensor/ops.rs:697-789).
#include <cuda_fp16.h>

#include <algorithm>

#include "device.cuh"
#include "kernels.h"

namespace wrk {
namespace k {

namespace {

constexpr int kTileM = 32, kTileN = 64, kChunk = 128, kPad = 8, kSmallThreads = 128;  // rows of 272 bytes: conflict-free fragments

struct SmallParams {
    const __half* w;  // [B][M][K]
    DView in, out;
    uint32_t K, M, N;
    int act;
};

__device__ __forceinline__ void mma16816(float c[4], const uint32_t a[4], const uint32_t b[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__global__ void __launch_bounds__(kSmallThreads) matmul_small_kernel(const SmallParams p) {
    __shared__ __align__(16) __half sw[kTileM][kChunk + kPad];
    __shared__ __align__(16) __half sx[kTileN][kChunk + kPad];
    const uint32_t m0 = blockIdx.x * kTileM, n0 = blockIdx.y * kTileN;
    const uint32_t batch = blockIdx.z;
    const uint32_t k_begin = 0, k_end = p.K;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const uint32_t wm = (warp & 1) * 16, wn = (warp >> 1) * 32;  // the warp's 16 rows x 32 tokens of the tile
    const __half* w = p.w + (size_t)batch * p.M * p.K;
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

    for (uint32_t kc = k_begin; kc < k_end; kc += kChunk) {
        const uint32_t len = min((uint32_t)kChunk, k_end - kc);  // a multiple of 16
        const uint32_t vecs = len / 8;
        __syncthreads();  // the previous chunk's readers are done
        // all of the thread's 16-byte loads of the chunk go out before the first store to shared memory
        constexpr uint32_t kWLoads = kTileM * (kChunk / 8) / kSmallThreads, kXLoads = kTileN * (kChunk / 8) / kSmallThreads;
        uint4 wv[kWLoads], xv[kXLoads];
#pragma unroll
        for (uint32_t q = 0; q < kWLoads; ++q) {
            const uint32_t i = threadIdx.x + q * kSmallThreads, r = i / vecs, v = i % vecs;
            wv[q] = make_uint4(0, 0, 0, 0);
            if (i < (uint32_t)kTileM * vecs && m0 + r < p.M) wv[q] = *reinterpret_cast<const uint4*>(w + (size_t)(m0 + r) * p.K + kc + v * 8);
        }
#pragma unroll
        for (uint32_t q = 0; q < kXLoads; ++q) {
            const uint32_t i = threadIdx.x + q * kSmallThreads, r = i / vecs, v = i % vecs;
            xv[q] = make_uint4(0, 0, 0, 0);
            if (i < (uint32_t)kTileN * vecs && n0 + r < p.N)
                xv[q] = *reinterpret_cast<const uint4*>(static_cast<const __half*>(p.in.base) + p.in.index(kc + v * 8, n0 + r, batch));
        }
#pragma unroll
        for (uint32_t q = 0; q < kWLoads; ++q) {
            const uint32_t i = threadIdx.x + q * kSmallThreads;
            if (i < (uint32_t)kTileM * vecs) *reinterpret_cast<uint4*>(&sw[i / vecs][(i % vecs) * 8]) = wv[q];
        }
#pragma unroll
        for (uint32_t q = 0; q < kXLoads; ++q) {
            const uint32_t i = threadIdx.x + q * kSmallThreads;
            if (i < (uint32_t)kTileN * vecs) *reinterpret_cast<uint4*>(&sx[i / vecs][(i % vecs) * 8]) = xv[q];
        }
        __syncthreads();
        for (uint32_t k = 0; k < len; k += 16) {
            uint32_t a[4];
            a[0] = *reinterpret_cast<const uint32_t*>(&sw[wm + g][k + 2 * t4]);
            a[1] = *reinterpret_cast<const uint32_t*>(&sw[wm + g + 8][k + 2 * t4]);
            a[2] = *reinterpret_cast<const uint32_t*>(&sw[wm + g][k + 2 * t4 + 8]);
            a[3] = *reinterpret_cast<const uint32_t*>(&sw[wm + g + 8][k + 2 * t4 + 8]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t b[2];
                b[0] = *reinterpret_cast<const uint32_t*>(&sx[wn + j * 8 + g][k + 2 * t4]);
                b[1] = *reinterpret_cast<const uint32_t*>(&sx[wn + j * 8 + g][k + 2 * t4 + 8]);
                mma16816(acc[j], a, b);
            }
        }
    }

    // accumulator element e of n-tile j: row wm + g + 8 (e / 2), token wn + 8 j + 2 t4 + (e & 1)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t m = m0 + wm + g + 8 * (e >> 1), n = n0 + wn + j * 8 + 2 * t4 + (e & 1);
            if (m < p.M && n < p.N) dstore(p.out.base, p.out.dtype, p.out.index(m, n, batch), activate_f(p.act, acc[j][e]));
        }
}

}  // namespace

bool matmul_small_supported(const MatmulArgs& a) {
    if (a.kind != MAT_FP16 || a.in.dtype != WRK_F16) return false;
    if (a.K > 256 || a.K % 16 != 0) return false;
    if (reinterpret_cast<uintptr_t>(a.matrix) % 16 != 0 || reinterpret_cast<uintptr_t>(a.in.base) % 16 != 0) return false;
    // 16-byte loads of the activations: every row and batch of the view starts on a multiple of 8 halves
    const DView& v = a.in;
    return v.stride[0] % 8 == 0 && v.offset[0] % 8 == 0 && ((size_t)v.stride[0] * v.stride[1]) % 8 == 0;
}

cudaError_t matmul_small(const MatmulArgs& a, int num_sms, cudaStream_t stream) {
    SmallParams p{};
    p.w = static_cast<const __half*>(a.matrix);
    p.in = a.in;
    p.out = a.out;
    p.K = a.K;
    p.M = a.M;
    p.N = a.N;
    p.act = a.act;
    (void)num_sms;
    dim3 grid((a.M + kTileM - 1) / kTileM, (a.N + kTileN - 1) / kTileN, a.B);
    matmul_small_kernel<<<grid, kSmallThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace k
}  // namespace wrk
