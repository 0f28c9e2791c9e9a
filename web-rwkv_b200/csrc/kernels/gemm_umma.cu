// Tensor-memory GEMM for the prefill / batched path (matmul_mat_fp16 / int8 / nf4 with more than a few
// tokens): out[n][m] = act(sum_k W[m][k] * x[n][k]).
//
// One CTA owns a 128-row slice of W and up to 256 tokens.  Eight producer warps walk K in steps of 64:
// they read the packed weights (u8 + per-128 (min, max), 4-bit + per-64 absmax, or fp16), dequantize them
// to fp16 in registers and store them, together with the fp16 activations of the step, into shared
// memory in the K-major 128-byte-swizzled layout tcgen05 reads.  A ninth warp issues the MMAs
// (tcgen05.mma.cta_group::1.kind::f16, M = 128, N = token tile, K = 16 per instruction) into a TMEM
// accumulator of 128 lanes x N fp32 columns and releases each stage through tcgen05.commit.  After the
// last step the producer warps read the accumulator back with tcgen05.ld (warp w reads lanes
// 32 (w % 4) ..), apply the activation and store token-major rows.
//
// Weights enter the MMA as fp16(fma(q, (max - min) / 255, min)) resp. fp16(table[nib] * absmax), computed in
// f32 and rounded once; the accumulation is fp32.  Every wait on an mbarrier is bounded: on a timeout the kernel records
// WRK_ERR_TIMEOUT in the context's status word, stops waiting and still frees its TMEM columns.
#include "device.cuh"
#include "kernels.h"

namespace wrk {
namespace k {

namespace {

constexpr int BM = 128;             // weight rows per CTA (UMMA M)
constexpr int BK = 64;              // K per stage: one 128-byte swizzle atom of fp16
constexpr int kProducerWarps = 8;
constexpr int kUmmaThreads = (kProducerWarps + 1) * 32;
constexpr int kMaxStages = 6;
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr uint32_t A_STAGE_BYTES = BM * BK * 2;  // 16 KB

struct UmmaParams {
    const uint8_t* w;
    const __half* scale;
    const float* table;
    int kind;
    uint32_t K, M, N;
    DView in, out;
    int act;
    uint32_t n_tile;    // tokens per CTA: multiple of 16, <= 256
    uint32_t tmem_cols; // power of two >= max(32, n_tile)
    uint32_t stages;
    int vec_in;         // activations readable as 16-byte (fp16) / 32-byte (fp32) groups
    int32_t* status;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
// Waits for the phase with the given parity; gives up after kSpinLimit polls (or at once when another
// wait of this CTA has already given up) and reports it.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* status) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(ok)
            : "r"(smem_addr(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    if (status != nullptr) atomicExch(status, (int32_t)WRK_ERR_TIMEOUT);
    return false;
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// K-major, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart, 16-byte chunk index XOR row % 8.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4);
}
// Shared-memory matrix descriptor of such a tile (start address, LBO = 1, SBO = 1024 bytes, version 1, SWIZZLE_128B).
__device__ __forceinline__ uint64_t sw128_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor: fp16 x fp16 -> fp32, both operands K-major, M x N.
__device__ __forceinline__ uint32_t f16_idesc(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t v[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_half2(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// 32 consecutive weights of one row (k0 .. k0 + 31) as four 16-byte groups of fp16.
__device__ __forceinline__ void dequant32(const UmmaParams& p, uint32_t m, uint32_t k0, const float2* lut2, uint4 out[4]) {
    if (m >= p.M) {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = make_uint4(0, 0, 0, 0);
        return;
    }
    if (p.kind == MAT_FP16) {
        const uint4* src = reinterpret_cast<const uint4*>(p.w + ((size_t)m * p.K + k0) * 2);
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = __ldg(src + j);
    } else if (p.kind == MAT_INT8) {
        // f32 dequantization (q / 255 scaled as in the reference up to the order of the two roundings), one
        // rounding to fp16 per weight: the errors of a row are independent, none is shared by a whole block
        const size_t e = (size_t)m * p.K + k0;
        const uint4* src = reinterpret_cast<const uint4*>(p.w + e);
        const uint4 q0 = __ldg(src), q1 = __ldg(src + 1);
        const float2 mm = __half22float2(__ldg(reinterpret_cast<const __half2*>(p.scale) + e / 128));
        const float sc = (mm.y - mm.x) * (1.0f / 255.0f), mn = mm.x;
        const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint32_t h[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // byte b -> float 8388608 + b (0x4B000000 | b), minus 8388608: b exactly
            const float f0 = __uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7650)) - 8388608.0f;
            const float f1 = __uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7651)) - 8388608.0f;
            const float f2 = __uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7652)) - 8388608.0f;
            const float f3 = __uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7653)) - 8388608.0f;
            h[2 * i] = pack_half2(__floats2half2_rn(fmaf(f0, sc, mn), fmaf(f1, sc, mn)));
            h[2 * i + 1] = pack_half2(__floats2half2_rn(fmaf(f2, sc, mn), fmaf(f3, sc, mn)));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
    } else {
        // NF4: 16 bytes, low nibble first; one absmax per 64 weights; f32 product rounded once
        const size_t e = (size_t)m * p.K + k0;
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(p.w + e / 2));
        const float am = __half2float(__ldg(p.scale + e / 64));
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
        uint32_t h[16];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float2 pair = lut2[(words[i] >> (8 * b)) & 0xffu];  // (table[lo nibble], table[hi nibble])
                h[4 * i + b] = pack_half2(__floats2half2_rn(pair.x * am, pair.y * am));
            }
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
    }
}

// Eight activations x[n][k0 .. k0 + 7] as fp16 (zeros beyond the last token).
__device__ __forceinline__ uint4 load_x8(const UmmaParams& p, uint32_t n, uint32_t k0) {
    if (n >= p.N) return make_uint4(0, 0, 0, 0);
    const size_t i = p.in.index(k0, n, 0);
    if (p.in.dtype == WRK_F16) {
        const __half* src = static_cast<const __half*>(p.in.base) + i;
        if (p.vec_in) return *reinterpret_cast<const uint4*>(src);
        __half v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = src[e];
        return *reinterpret_cast<uint4*>(v);
    }
    const float* src = static_cast<const float*>(p.in.base) + i;
    float f[8];
    if (p.vec_in) {
        const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
        f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = src[e];
    }
    uint4 r;
    r.x = pack_half2(__floats2half2_rn(f[0], f[1]));
    r.y = pack_half2(__floats2half2_rn(f[2], f[3]));
    r.z = pack_half2(__floats2half2_rn(f[4], f[5]));
    r.w = pack_half2(__floats2half2_rn(f[6], f[7]));
    return r;
}

__global__ void __launch_bounds__(kUmmaThreads, 1) matmul_umma_kernel(const UmmaParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ float2 lut2[256];
    __shared__ int abort_flag;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t b_bytes = p.n_tile * BK * 2;
    const uint32_t stage_bytes = A_STAGE_BYTES + b_bytes;
    const uint32_t m0 = blockIdx.x * BM, n0 = blockIdx.y * p.n_tile;
    const uint32_t nk = p.K / BK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(&full_bar[s], kProducerWarps);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&done_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (p.kind == MAT_NF4 && threadIdx.x < 256) {
        lut2[threadIdx.x] = make_float2(p.table[threadIdx.x & 15], p.table[threadIdx.x >> 4]);
    }
    if (warp == kProducerWarps) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&tmem_base_slot)), "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = tmem_base_slot;

    if (warp < kProducerWarps) {
        // ---- producers: dequantized weights and activations of one K step per stage ----
        const uint32_t row = threadIdx.x >> 1, half = threadIdx.x & 1;  // 256 threads: 128 rows x two 32-weight halves
        for (uint32_t kt = 0; kt < nk; ++kt) {
            const uint32_t s = kt % p.stages, use = kt / p.stages;
            if (use > 0) mbar_wait(&empty_bar[s], (use - 1) & 1, &abort_flag, p.status);
            uint8_t* sa = smem + (size_t)s * stage_bytes;
            uint8_t* sb = sa + A_STAGE_BYTES;
            uint4 wv[4];
            dequant32(p, m0 + row, kt * BK + half * 32, lut2, wv);
#pragma unroll
            for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(sa + sw128_offset(row, half * 4 + j)) = wv[j];
            for (uint32_t q = threadIdx.x; q < p.n_tile * 8; q += kProducerWarps * 32) {
                const uint32_t tok = q >> 3, ch = q & 7;
                *reinterpret_cast<uint4*>(sb + sw128_offset(tok, ch)) = load_x8(p, n0 + tok, kt * BK + ch * 8);
            }
            fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[s]);
        }
        // ---- epilogue: TMEM -> registers -> activation -> token-major rows ----
        mbar_wait(&done_bar, 0, &abort_flag, p.status);
        tc_fence_after();
        const uint32_t quad = warp & 3, side = warp >> 2;  // lanes 32 quad .., half of the columns each
        const uint32_t m = m0 + quad * 32 + lane;
        const uint32_t c_begin = side * (p.n_tile / 2), c_end = c_begin + p.n_tile / 2;
        for (uint32_t c = c_begin; c < c_end; c += 8) {
            uint32_t v[8];
            tmem_ld8(tmem_d + ((quad * 32) << 16) + c, v);
            tmem_ld_wait();
            if (m < p.M) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t n = n0 + c + j;
                    if (n < p.N) dstore(p.out.base, p.out.dtype, p.out.index(m, n, 0), activate_f(p.act, __uint_as_float(v[j])));
                }
            }
        }
    } else {
        // ---- MMA issuer ----
        const uint32_t idesc = f16_idesc(BM, p.n_tile);
        for (uint32_t kt = 0; kt < nk; ++kt) {
            const uint32_t s = kt % p.stages, use = kt / p.stages;
            mbar_wait(&full_bar[s], use & 1, &abort_flag, p.status);
            tc_fence_after();
            if (lane == 0) {
                const uint32_t sa = smem_addr(smem + (size_t)s * stage_bytes);
                const uint64_t da = sw128_desc(sa), db = sw128_desc(sa + A_STAGE_BYTES);
#pragma unroll
                for (uint32_t kk = 0; kk < BK / 16; ++kk)  // 32 bytes of K per instruction: + 2 in the address field
                    umma_f16(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (kt | kk) != 0 ? 1u : 0u);
                umma_commit(&empty_bar[s]);  // arrives when the MMAs above have read the stage
            }
            __syncwarp();
        }
        if (lane == 0) umma_commit(&done_bar);
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kProducerWarps) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_d), "r"(p.tmem_cols) : "memory");
    }
}

}  // namespace

bool matmul_umma_supported(const MatmulArgs& a) {
    if (a.B != 1 || a.N < 16 || a.M == 0) return false;
    if (a.K % BK != 0 || (a.kind == MAT_INT8 && a.K % 128 != 0)) return false;
    if (reinterpret_cast<uintptr_t>(a.matrix) % 16 != 0) return false;
    if (a.scale != nullptr && reinterpret_cast<uintptr_t>(a.scale) % 4 != 0) return false;
    return true;
}

cudaError_t matmul_umma(const MatmulArgs& a, int32_t* status, cudaStream_t stream) {
    UmmaParams p{};
    p.w = static_cast<const uint8_t*>(a.matrix);
    p.scale = a.scale;
    p.table = a.table;
    p.kind = a.kind;
    p.K = a.K;
    p.M = a.M;
    p.N = a.N;
    p.in = a.in;
    p.out = a.out;
    p.act = a.act;
    p.status = status;
    p.n_tile = std::min<uint32_t>(256, (a.N + 15) / 16 * 16);
    p.tmem_cols = 32;
    while (p.tmem_cols < p.n_tile) p.tmem_cols *= 2;
    const uint32_t stage_bytes = A_STAGE_BYTES + p.n_tile * BK * 2;
    p.stages = std::min<uint32_t>(kMaxStages, std::max<uint32_t>(2, (200u * 1024) / stage_bytes));
    p.stages = std::min<uint32_t>(p.stages, std::max<uint32_t>(2, a.K / BK));
    const size_t esz = a.in.dtype == WRK_F16 ? 2 : 4;
    p.vec_in = (a.in.stride[0] % 8 == 0) && (a.in.offset[0] % 8 == 0) && (reinterpret_cast<uintptr_t>(a.in.base) % (8 * esz) == 0);
    const size_t smem = (size_t)p.stages * stage_bytes + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(matmul_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const dim3 grid((a.M + BM - 1) / BM, (a.N + p.n_tile - 1) / p.n_tile);
    matmul_umma_kernel<<<grid, kUmmaThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace k
}  // namespace wrk
