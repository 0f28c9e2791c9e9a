// Weight-streaming matmul for fp16 / Int8 / NF4 weights on sm_100a (decode GEMV and small-N GEMM).
//
// Replaces matmul_vec_{fp16,int8,nf4}.wgsl (and, until the tensor-memory GEMM takes over for large
// token counts, matmul_mat_*.wgsl).  The kernel is HBM-bound: every weight byte is read exactly once
// per group of 8*NT tokens with 16-byte loads, expanded to fp16 in registers and fed to
// mma.sync.m16n8k16 (fp32 accumulate), so the ALU only pays for the byte->half expansion.
//
// Work split: one CTA (8 warps) owns 16 weight rows and up to 8*NT tokens; its warps split K in
// interleaved chunks (consecutive warps read consecutive 64..128-byte pieces of the same rows) and
// reduce through shared memory.  The activations of the CTA's tokens are staged in shared memory as
// fp16 once per K-stage, together with their per-chunk sums, which turns the Int8 affine dequant
//   sum_k (q_k/255 * (max-min) + min) * x_k  =  (max-min)/255 * sum_k q_k x_k + min * sum_k x_k
// into one MMA chain on the raw bytes plus two FMAs per 128-element block.
//
// Fragment mapping (lane = 4*g + t): the MMA's k index is a permutation of the physical k, the same
// for A and B: in k-step s lane t supplies physical elements 4s..4s+3 of its own 16-byte piece.
#include "device.cuh"

namespace wrk {
namespace k {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kRows = 16;

struct MmParams {
    const uint8_t* matrix;
    const __half* scale;
    const float* table;
    uint32_t K, M, N;
    DView in, out;
    int act;
    uint32_t KS;       // K elements staged per pass (multiple of 128)
    uint32_t xstride;  // halfs per staged token row (KS + 8: rows shift by one 16-byte bank group)
    uint32_t ntok;     // token rows allocated in shared memory (min(8*NT, N))
    int vec_in;        // input rows can be read with 4-element vector loads
};

__device__ __forceinline__ void mma16816(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two bytes of `w` (selected by `sel`) -> half2 of their integer values: 0x6400 | q is 1024 + q.
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t w, uint32_t sel) {
    const uint32_t h = __byte_perm(w, 0x64646464u, sel);
    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&h), __float2half2_rn(1024.0f));
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ uint2 ldg_stream8(const void* p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}

// Stage activations [ntok][k0, k0 + kse) as fp16 and (Int8) their sums per 128-element unit.
template <int KIND>
__device__ __forceinline__ void stage_input(const MmParams& p, uint32_t n0, uint32_t b, uint32_t k0, uint32_t kse,
                                            __half* xs, float* sx) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t units = (kse + 127) / 128;
    for (uint32_t u = warp; u < p.ntok * units; u += kWarps) {
        const uint32_t tok = u / units, unit = u % units;
        const uint32_t n = n0 + tok;
        const uint32_t kk = unit * 128 + lane * 4;  // within the stage
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (n < p.N && kk < kse) {
            const size_t base = p.in.index(k0 + kk, n, b);
            if (p.vec_in && kk + 4 <= kse) {
                if (p.in.dtype == WRK_F16) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __half*>(p.in.base) + base);
                    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
                } else {
                    const float4 raw = *reinterpret_cast<const float4*>(static_cast<const float*>(p.in.base) + base);
                    v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
                }
            } else {
                for (int j = 0; j < 4; ++j)
                    if (kk + j < kse) v[j] = dload(p.in.base, p.in.dtype, base + j);
            }
        }
        const __half2 h0 = __floats2half2_rn(v[0], v[1]);
        const __half2 h1 = __floats2half2_rn(v[2], v[3]);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&h0);
        packed.y = *reinterpret_cast<const uint32_t*>(&h1);
        *reinterpret_cast<uint2*>(xs + (size_t)tok * p.xstride + kk) = packed;
        if (KIND == MAT_INT8) {
            // sum of the values the MMA will actually see (after rounding to fp16)
            const float2 r0 = __half22float2(h0), r1 = __half22float2(h1);
            const float s = warp_sum((r0.x + r0.y) + (r1.x + r1.y));
            if (lane == 0) sx[tok * units + unit] = s;
        }
    }
}

template <int KIND, int NT>
__global__ void __launch_bounds__(kThreads) matmul_mma_kernel(const MmParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ __half lut[16];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t row0 = blockIdx.x * kRows;
    const uint32_t n0 = blockIdx.y * (8 * NT);
    const uint32_t b = blockIdx.z;

    const uint32_t units_max = p.KS / 128;
    __half* xs = reinterpret_cast<__half*>(smem);
    float* sx = reinterpret_cast<float*>(smem + (size_t)p.ntok * p.xstride * sizeof(__half));
    float* red = sx + (size_t)p.ntok * units_max;  // [kWarps][kRows][8 * NT]

    if (KIND == MAT_NF4 && threadIdx.x < 16) lut[threadIdx.x] = __float2half_rn(p.table[threadIdx.x]);

    const uint32_t rA = row0 + g, rB = row0 + g + 8;
    const bool vA = rA < p.M, vB = rB < p.M;
    // bytes per weight row
    const size_t row_bytes = KIND == MAT_FP16 ? (size_t)p.K * 2 : KIND == MAT_INT8 ? (size_t)p.K : (size_t)p.K / 2;
    const uint8_t* pA = p.matrix + ((size_t)b * p.M + (vA ? rA : 0)) * row_bytes;
    const uint8_t* pB = p.matrix + ((size_t)b * p.M + (vB ? rB : 0)) * row_bytes;

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.0f;

    const __half* xrow[NT];
    bool xvalid[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const uint32_t tok = 8 * j + g;
        xvalid[j] = tok < p.ntok && n0 + tok < p.N;
        xrow[j] = xs + (size_t)(xvalid[j] ? tok : 0) * p.xstride;
    }

    for (uint32_t k0 = 0; k0 < p.K; k0 += p.KS) {
        const uint32_t kse = min(p.KS, p.K - k0);
        __syncthreads();  // previous stage fully consumed
        stage_input<KIND>(p, n0, b, k0, kse, xs, sx);
        __syncthreads();
        const uint32_t units = (kse + 127) / 128;

        if (KIND == MAT_INT8) {
            // chunk = one 128-element quantization block per row: two 16-byte pieces per lane and row
            const uint32_t nch = kse / 128;
            const size_t blkA = ((size_t)b * p.M + (vA ? rA : 0)) * (p.K / 128) + k0 / 128;
            const size_t blkB = ((size_t)b * p.M + (vB ? rB : 0)) * (p.K / 128) + k0 / 128;
            const __half2* sc = reinterpret_cast<const __half2*>(p.scale);
            for (uint32_t c = warp; c < nch; c += kWarps) {
                const size_t off = (size_t)k0 + (size_t)c * 128 + 16 * t;
                uint4 wa0 = make_uint4(0, 0, 0, 0), wa1 = wa0, wb0 = wa0, wb1 = wa0;
                float2 mmA = make_float2(0.f, 0.f), mmB = mmA;
                if (vA) {
                    wa0 = ldg_stream(pA + off);
                    wa1 = ldg_stream(pA + off + 64);
                    mmA = __half22float2(sc[blkA + c]);
                }
                if (vB) {
                    wb0 = ldg_stream(pB + off);
                    wb1 = ldg_stream(pB + off + 64);
                    mmB = __half22float2(sc[blkB + c]);
                }
                float d[NT][4];
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) d[j][e] = 0.0f;
                const uint32_t wa[8] = {wa0.x, wa0.y, wa0.z, wa0.w, wa1.x, wa1.y, wa1.z, wa1.w};
                const uint32_t wb[8] = {wb0.x, wb0.y, wb0.z, wb0.w, wb1.x, wb1.y, wb1.z, wb1.w};
#pragma unroll
                for (int s2 = 0; s2 < 4; ++s2) {  // two k-steps per 16-byte activation read
                    const uint32_t kk = c * 128 + (s2 < 2 ? 16 * t + 8 * s2 : 64 + 16 * t + 8 * (s2 - 2));
                    uint32_t a[2][4];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int s = 2 * s2 + h;
                        a[h][0] = bytes_to_half2(wa[s], 0x4140);
                        a[h][1] = bytes_to_half2(wb[s], 0x4140);
                        a[h][2] = bytes_to_half2(wa[s], 0x4342);
                        a[h][3] = bytes_to_half2(wb[s], 0x4342);
                    }
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        uint4 xv = make_uint4(0, 0, 0, 0);
                        if (xvalid[j]) xv = *reinterpret_cast<const uint4*>(xrow[j] + kk);
                        mma16816(d[j], a[0][0], a[0][1], a[0][2], a[0][3], xv.x, xv.y);
                        mma16816(d[j], a[1][0], a[1][1], a[1][2], a[1][3], xv.z, xv.w);
                    }
                }
                const float sA = (mmA.y - mmA.x) * (1.0f / 255.0f), sB = (mmB.y - mmB.x) * (1.0f / 255.0f);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const uint32_t tk0 = 8 * j + 2 * t, tk1 = tk0 + 1;
                    const float s0 = tk0 < p.ntok ? sx[tk0 * units + c] : 0.0f;
                    const float s1 = tk1 < p.ntok ? sx[tk1 * units + c] : 0.0f;
                    acc[j][0] += sA * d[j][0] + mmA.x * s0;
                    acc[j][1] += sA * d[j][1] + mmA.x * s1;
                    acc[j][2] += sB * d[j][2] + mmB.x * s0;
                    acc[j][3] += sB * d[j][3] + mmB.x * s1;
                }
            }
        } else if (KIND == MAT_NF4) {
            // chunk = one 64-element absmax block per row: one 8-byte piece (16 nibbles) per lane and row
            const uint32_t nch = kse / 64;
            const size_t blkA = ((size_t)b * p.M + (vA ? rA : 0)) * (p.K / 64) + k0 / 64;
            const size_t blkB = ((size_t)b * p.M + (vB ? rB : 0)) * (p.K / 64) + k0 / 64;
            for (uint32_t c = warp; c < nch; c += kWarps) {
                const size_t off = ((size_t)k0 + (size_t)c * 64) / 2 + 8 * t;
                uint2 wa = make_uint2(0x77777777u, 0x77777777u), wb = wa;
                float aA = 0.f, aB = 0.f;
                if (vA) { wa = ldg_stream8(pA + off); aA = __half2float(p.scale[blkA + c]); }
                if (vB) { wb = ldg_stream8(pB + off); aB = __half2float(p.scale[blkB + c]); }
                float d[NT][4];
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) d[j][e] = 0.0f;
                const uint32_t wau[2] = {wa.x, wa.y}, wbu[2] = {wb.x, wb.y};
#pragma unroll
                for (int s2 = 0; s2 < 2; ++s2) {  // one u32 = 8 nibbles = two k-steps
                    const uint32_t kk = c * 64 + 16 * t + 8 * s2;
                    uint32_t a[2][4];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t qa = wau[s2] >> (16 * h), qb = wbu[s2] >> (16 * h);
                        const __half2 a0 = __halves2half2(lut[qa & 15u], lut[(qa >> 4) & 15u]);
                        const __half2 a2 = __halves2half2(lut[(qa >> 8) & 15u], lut[(qa >> 12) & 15u]);
                        const __half2 a1 = __halves2half2(lut[qb & 15u], lut[(qb >> 4) & 15u]);
                        const __half2 a3 = __halves2half2(lut[(qb >> 8) & 15u], lut[(qb >> 12) & 15u]);
                        a[h][0] = *reinterpret_cast<const uint32_t*>(&a0);
                        a[h][1] = *reinterpret_cast<const uint32_t*>(&a1);
                        a[h][2] = *reinterpret_cast<const uint32_t*>(&a2);
                        a[h][3] = *reinterpret_cast<const uint32_t*>(&a3);
                    }
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        uint4 xv = make_uint4(0, 0, 0, 0);
                        if (xvalid[j]) xv = *reinterpret_cast<const uint4*>(xrow[j] + kk);
                        mma16816(d[j], a[0][0], a[0][1], a[0][2], a[0][3], xv.x, xv.y);
                        mma16816(d[j], a[1][0], a[1][1], a[1][2], a[1][3], xv.z, xv.w);
                    }
                }
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    acc[j][0] = fmaf(d[j][0], aA, acc[j][0]);
                    acc[j][1] = fmaf(d[j][1], aA, acc[j][1]);
                    acc[j][2] = fmaf(d[j][2], aB, acc[j][2]);
                    acc[j][3] = fmaf(d[j][3], aB, acc[j][3]);
                }
            }
        } else {
            // fp16 weights: chunk = 32 elements per row, one 16-byte piece (8 halfs) per lane and row
            const uint32_t nch = kse / 32;
            for (uint32_t c = warp; c < nch; c += kWarps) {
                const size_t off = ((size_t)k0 + (size_t)c * 32 + 8 * t) * 2;
                uint4 wa = make_uint4(0, 0, 0, 0), wb = wa;
                if (vA) wa = ldg_stream(pA + off);
                if (vB) wb = ldg_stream(pB + off);
                const uint32_t kk = c * 32 + 8 * t;
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    uint4 xv = make_uint4(0, 0, 0, 0);
                    if (xvalid[j]) xv = *reinterpret_cast<const uint4*>(xrow[j] + kk);
                    mma16816(acc[j], wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
                    mma16816(acc[j], wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
                }
            }
        }
    }

    // cross-warp reduction, activation, store
    constexpr int NTOK = 8 * NT;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        float* r = red + ((size_t)warp * kRows) * NTOK;
        r[(size_t)g * NTOK + 8 * j + 2 * t] = acc[j][0];
        r[(size_t)g * NTOK + 8 * j + 2 * t + 1] = acc[j][1];
        r[(size_t)(g + 8) * NTOK + 8 * j + 2 * t] = acc[j][2];
        r[(size_t)(g + 8) * NTOK + 8 * j + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    for (int o = threadIdx.x; o < kRows * NTOK; o += kThreads) {
        const int row = o % kRows, tok = o / kRows;
        const uint32_t m = row0 + row, n = n0 + tok;
        if (m >= p.M || n >= p.N || (uint32_t)tok >= p.ntok) continue;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) s += red[((size_t)w * kRows + row) * NTOK + tok];
        dstore(p.out.base, p.out.dtype, p.out.index(m, n, b), activate_f(p.act, s));
    }
}

// Shape-agnostic fallback (K not a multiple of the quantization block, unaligned rows): one thread
// per output element, the reference's arithmetic verbatim.  Correctness path only.
__global__ void matmul_generic_kernel(int kind, const uint8_t* matrix, const __half* scale, const float* table,
                                      uint32_t K, uint32_t M, uint32_t N, uint32_t B, DView in, DView out, int act) {
    const size_t total = (size_t)M * N * B;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t m = o % M, n = (o / M) % N, b = o / ((size_t)M * N);
        const size_t row = ((size_t)b * M + m) * K;
        float acc = 0.0f;
        for (uint32_t k = 0; k < K; ++k) {
            float w;
            if (kind == MAT_FP16) {
                w = __half2float(reinterpret_cast<const __half*>(matrix)[row + k]);
            } else if (kind == MAT_INT8) {
                const size_t blk = (row + k) / 128;
                const float mn = __half2float(scale[2 * blk]), mx = __half2float(scale[2 * blk + 1]);
                w = fmaf((float)matrix[row + k] / 255.0f, mx - mn, mn);
            } else {
                const uint32_t nib = (matrix[(row + k) >> 1] >> (((row + k) & 1) * 4)) & 15u;
                w = table[nib] * __half2float(scale[(row + k) / 64]);
            }
            acc = fmaf(w, dload(in.base, in.dtype, in.index(k, n, b)), acc);
        }
        dstore(out.base, out.dtype, out.index(m, n, b), activate_f(act, acc));
    }
}

template <int KIND, int NT>
cudaError_t launch_mma(const MmParams& p, uint32_t B, cudaStream_t stream) {
    const size_t smem = (size_t)p.ntok * p.xstride * sizeof(__half) + (size_t)p.ntok * (p.KS / 128) * sizeof(float) +
                        (size_t)kWarps * kRows * 8 * NT * sizeof(float);
    static SmemOptIn opt_in;  // one per instantiation
    if (cudaError_t e = opt_in.ensure(matmul_mma_kernel<KIND, NT>, 160 * 1024); e != cudaSuccess) return e;
    dim3 grid((p.M + kRows - 1) / kRows, (p.N + 8 * NT - 1) / (8 * NT), B);
    matmul_mma_kernel<KIND, NT><<<grid, kThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

template <int KIND>
cudaError_t dispatch_nt(MmParams& p, uint32_t B, cudaStream_t stream) {
    const uint32_t ntile = p.N <= 8 ? 1 : p.N <= 16 ? 2 : 4;
    p.ntok = p.N < 8 * ntile ? p.N : 8 * ntile;
    // stage as much of K as fits in ~96 KB of fp16 activations
    const size_t budget = 96 * 1024;
    uint32_t ks = (p.K + 127) / 128 * 128;
    while ((size_t)p.ntok * (ks + 8) * 2 > budget && ks > 1024) ks = (ks / 2 + 1023) / 1024 * 1024;
    p.KS = ks;
    p.xstride = ks + 8;
    switch (ntile) {
        case 1: return launch_mma<KIND, 1>(p, B, stream);
        case 2: return launch_mma<KIND, 2>(p, B, stream);
        default: return launch_mma<KIND, 4>(p, B, stream);
    }
}

}  // namespace

cudaError_t matmul(const MatmulArgs& a, int num_sms, cudaStream_t stream) {
    if (a.M == 0 || a.N == 0 || a.B == 0) return cudaSuccess;
    // more tokens than the weight-streaming kernel takes (8) and a short K: the adapters' second matrices
    if (a.N > 8 && matmul_small_supported(a)) return matmul_small(a, num_sms, stream);
    if (matmul_umma_supported(a)) return matmul_umma(a, a.status, stream);
    const uint32_t ck = a.kind == MAT_INT8 ? 128 : a.kind == MAT_NF4 ? 64 : 32;
    const bool aligned = (reinterpret_cast<uintptr_t>(a.matrix) % 16 == 0) && a.K % ck == 0 &&
                         (a.scale == nullptr || reinterpret_cast<uintptr_t>(a.scale) % 4 == 0);
    if (!aligned) {
        const size_t total = (size_t)a.M * a.N * a.B;
        const int grid = (int)std::min<size_t>((total + 127) / 128, (size_t)num_sms * 16);
        matmul_generic_kernel<<<grid, 128, 0, stream>>>(a.kind, static_cast<const uint8_t*>(a.matrix), a.scale, a.table,
                                                        a.K, a.M, a.N, a.B, a.in, a.out, a.act);
        return cudaGetLastError();
    }
    MmParams p;
    p.matrix = static_cast<const uint8_t*>(a.matrix);
    p.scale = a.scale;
    p.table = a.table;
    p.K = a.K;
    p.M = a.M;
    p.N = a.N;
    p.in = a.in;
    p.out = a.out;
    p.act = a.act;
    const size_t esz = a.in.dtype == WRK_F16 ? 2 : 4;
    p.vec_in = (a.in.stride[0] % 4 == 0) && (a.in.offset[0] % 4 == 0) &&
               (reinterpret_cast<uintptr_t>(a.in.base) % (4 * esz) == 0);
    switch (a.kind) {
        case MAT_INT8: return dispatch_nt<MAT_INT8>(p, a.B, stream);
        case MAT_NF4: return dispatch_nt<MAT_NF4>(p, a.B, stream);
        default: return dispatch_nt<MAT_FP16>(p, a.B, stream);
    }
}

}  // namespace k
}  // namespace wrk
