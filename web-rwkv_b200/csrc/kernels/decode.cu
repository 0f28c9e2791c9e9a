// Fused decode path for jobs of a few tokens (T <= 8): the whole v5/v6 layer in seven launches.
//
// The quantized matmuls of a decode step are pure weight streaming, and at model widths of 2048-4096
// a single matrix is only a few microseconds of HBM time, so the structure of this file is built
// around never letting the stream of weights stop:
//   * fused_gemv_kernel is a grouped weight-streaming kernel.  A launch covers several matrices (e.g.
//     key / value / receptance / gate + the decay adapter); the concatenated row space is cut into one
//     contiguous row range per CTA (balanced by bytes, one CTA per SM slot), and each CTA pulls exactly its
//     rows into shared memory with asynchronous 16-byte copies (cp.async, one commit group per tile part of
//     16 rows x 1 KB + its block scales), four to six tile parts in flight.  Per-row bulk-TMA copies were
//     measured first: the TMA unit serialises them (~50 ns each, 32 per tile part), which cost more than
//     the copy itself; a 2-D tensor-map box would fetch whole 16-row boxes and over-read the 13.8-row
//     shares a 2048-row matrix leaves per SM.
//   * every kernel here is launched with programmatic dependent launch: it signals its dependents at
//     once, issues the copies of its first weight tiles, and only then executes griddepcontrol.wait.
//     Weights are never written during a job, so the next kernel's weights are already landing in shared
//     memory while the previous kernel is still finishing.
//   * layer norm + token shift run as a per-CTA prologue (every CTA recomputes the few-KB vector instead
//     of a separate launch and a grid-wide dependency); residual add, squared ReLU, channel mix and the
//     carry-row updates run as epilogues.
// The math on the tiles is the mma.sync scheme of matmul.cu (bytes expanded to fp16 in registers, fp32
// accumulate, Int8 affine term through per-block activation sums).  Every tensor the reference stores as
// fp16 is rounded to fp16 here at the same point.
#include "decode.cuh"
#include "device.cuh"

namespace wrk {
namespace k {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int PB = 1024;          // bytes of one weight row per tile part
constexpr int PITCH = PB + 16;    // shared-memory row pitch: consecutive rows shift by one 16-byte bank group
constexpr int SCP = 80;           // pitch of a row's scales inside a slot (<= 64 bytes of data)
constexpr int SLOT = 16 * PITCH + 16 * SCP;  // one tile part: 16 rows of weights, then their scales
constexpr int MAX_SLOTS = 6;
constexpr int GROUP_ROWS = 64;    // rows accumulated in registers at a time (4 MMA row tiles)

// floats reserved for the per-block activation sums (keeps what follows 16-byte aligned)
__host__ __device__ inline uint32_t sums_floats(uint32_t T, uint32_t kmax) {
    return (T * ((kmax + 127) / 128) + 3) / 4 * 4 + 4;
}

// Optional stage timestamps (builds with -DWRK_TRACE only): CTA 0 records (stage, globaltimer ns) in
// shared memory and appends them to a global log when the kernel ends.
#ifdef WRK_TRACE
__device__ unsigned long long g_trace[1 << 16];
__device__ unsigned int g_trace_n;
__shared__ unsigned long long s_trace[128];
__shared__ unsigned int s_trace_n;
__device__ __forceinline__ void trace(int stage) {
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        if (stage == 100) s_trace_n = 0;
        if (s_trace_n < 64) {
            s_trace[2 * s_trace_n] = (unsigned long long)stage;
            s_trace[2 * s_trace_n + 1] = t;
            ++s_trace_n;
        }
        if (stage == 107) {
            const unsigned int base = atomicAdd(&g_trace_n, s_trace_n);
            for (unsigned int i = 0; i < s_trace_n && base + i < (1u << 15); ++i) {
                g_trace[2 * (base + i)] = s_trace[2 * i];
                g_trace[2 * (base + i) + 1] = s_trace[2 * i + 1];
            }
        }
    }
}
#else
__device__ __forceinline__ void trace(int) {}
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

__device__ __forceinline__ void mma16816(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t w, uint32_t sel) {
    const uint32_t h = __byte_perm(w, 0x64646464u, sel);  // 0x6400 | q = 1024 + q
    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&h), __float2half2_rn(1024.0f));
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t row_bytes(const GemvProblem& p) {
    return p.kind == MAT_FP16 ? p.K * 2 : p.kind == MAT_INT8 ? p.K : p.K / 2;
}
__device__ __forceinline__ uint32_t part_elems(int kind) { return kind == MAT_FP16 ? PB / 2 : kind == MAT_INT8 ? PB : PB * 2; }

// Position in a CTA's sequence of tile parts: segment -> group of <= 64 rows -> K part -> row tile.
struct TileIter {
    int seg, group0, part, tile;
    int ntile, nparts, gend;  // of the current group
    bool valid;

    __device__ void enter(const FusedGemvArgs& a, const GemvSegment* segs) {
        while (seg < kSegmentsPerCta && segs[seg].row0 >= segs[seg].row1) ++seg;
        valid = seg < kSegmentsPerCta;
        if (!valid) return;
        const GemvSegment& s = segs[seg];
        gend = min(group0 + GROUP_ROWS, s.row1);
        ntile = (gend - group0 + 15) / 16;
        nparts = (row_bytes(a.p[s.problem]) + PB - 1) / PB;
    }
    __device__ void start(const FusedGemvArgs& a, const GemvSegment* segs) {
        seg = 0;
        part = tile = 0;
        while (seg < kSegmentsPerCta && segs[seg].row0 >= segs[seg].row1) ++seg;
        group0 = seg < kSegmentsPerCta ? segs[seg].row0 : 0;
        enter(a, segs);
    }
    __device__ void next(const FusedGemvArgs& a, const GemvSegment* segs) {
        if (++tile < ntile) return;
        tile = 0;
        if (++part < nparts) return;
        part = 0;
        group0 += GROUP_ROWS;
        if (group0 >= segs[seg].row1) {
            ++seg;
            while (seg < kSegmentsPerCta && segs[seg].row0 >= segs[seg].row1) ++seg;
            if (seg < kSegmentsPerCta) group0 = segs[seg].row0;
        }
        enter(a, segs);
    }
    __device__ bool last_part_of_group() const { return part == nparts - 1 && tile == ntile - 1; }
};

// Asynchronous global -> shared copies (LDGSTS): 16 bytes for weights, 4 bytes for block scales.
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait(int pending) {
    switch (pending) {
        case 0: asm volatile("cp.async.wait_group 0;\n" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;\n" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;\n" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;\n" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;\n" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 5;\n" ::: "memory"); break;
    }
}

// Block scales ride along with the tile when pairs of them are 4-byte aligned in every row.
__device__ __forceinline__ bool scales_async(const GemvProblem& p) {
    return p.kind == MAT_INT8 || (p.kind == MAT_NF4 && p.K % 128 == 0);
}

// All threads issue the copies of one tile part: exactly the CTA's rows, nothing more.
__device__ __forceinline__ void issue_tile(const FusedGemvArgs& a, const GemvSegment* segs, const TileIter& it,
                                           uint8_t* slot) {
    const GemvProblem& p = a.p[segs[it.seg].problem];
    const uint32_t rb = row_bytes(p);
    const uint32_t bytes = min((uint32_t)PB, rb - it.part * PB);
    const int row0 = it.group0 + 16 * it.tile;
    const int nr = min(16, it.gend - row0);
    const uint32_t cpr = bytes / 16;
    const uint8_t* src = p.w + (size_t)row0 * rb + (size_t)it.part * PB;
    for (uint32_t i = threadIdx.x; i < (uint32_t)nr * cpr; i += kThreads) {
        const uint32_t r = i / cpr, c = i % cpr;
        cp_async16(slot + r * PITCH + c * 16, src + (size_t)r * rb + c * 16);
    }
    if (scales_async(p)) {
        // Int8: one (min, max) pair = 4 bytes per 128 weights; NF4: two absmax = 4 bytes per 128 weights
        const uint32_t per_row = p.kind == MAT_INT8 ? bytes / 128 : bytes / 64;  // 4-byte units in this part
        const uint32_t row_units = p.K / 128;
        const uint32_t part_units = p.kind == MAT_INT8 ? PB / 128 : PB / 64;
        const uint8_t* sc = reinterpret_cast<const uint8_t*>(p.scale);
        uint8_t* sslot = slot + 16 * PITCH;
        for (uint32_t i = threadIdx.x; i < (uint32_t)nr * per_row; i += kThreads) {
            const uint32_t r = i / per_row, u = i % per_row;
            cp_async4(sslot + r * SCP + u * 4, sc + ((size_t)(row0 + r) * row_units + it.part * part_units + u) * 4);
        }
    }
}

__device__ __forceinline__ float block_sum_256(float v, float* scratch) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) s += scratch[w];
    return s;
}

// Layer norm of a.ln_x rows (+ token shift) into xgen[v][t][c] (fp16, pitch xp).
// Each thread keeps its channels of a row in registers (C <= 8 * kThreads * kLnVec).
constexpr int kLnVec = 4;  // groups of 8 channels per thread: C <= 8192
__device__ void run_prologue(const FusedGemvArgs& a, __half* xgen, uint32_t xp, __half* lnrow, float* scratch) {
    const uint32_t C = a.C, T = a.T;
    const uint32_t ngrp = C / 8;  // 16-byte groups per row
    for (uint32_t t = 0; t < T; ++t) {
        float v[kLnVec][8];
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < kLnVec; ++q) {
            const uint32_t gi = threadIdx.x + q * kThreads;
            if (gi < ngrp) {
                const uint4 raw = *reinterpret_cast<const uint4*>(a.ln_x + (size_t)t * C + gi * 8);
                const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h[e]);
                    v[q][2 * e] = f.x;
                    v[q][2 * e + 1] = f.y;
                    s += f.x + f.y;
                }
            }
        }
        const float mean = block_sum_256(s, scratch) / (float)C;
        float m2 = 0.f;
#pragma unroll
        for (int q = 0; q < kLnVec; ++q)
            if (threadIdx.x + q * kThreads < ngrp)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float d = v[q][e] - mean;
                    m2 += d * d;
                }
        const float dev = rsqrtf(block_sum_256(m2, scratch) / (float)C + a.ln_eps);
#pragma unroll
        for (int q = 0; q < kLnVec; ++q) {
            const uint32_t gi = threadIdx.x + q * kThreads;
            if (gi < ngrp) {
                const uint4 wraw = *reinterpret_cast<const uint4*>(a.ln_w + gi * 8);
                const uint4 braw = *reinterpret_cast<const uint4*>(a.ln_b + gi * 8);
                const __half* wh = reinterpret_cast<const __half*>(&wraw);
                const __half* bh = reinterpret_cast<const __half*>(&braw);
                uint4 outv;
                __half* oh = reinterpret_cast<__half*>(&outv);
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    oh[e] = __float2half_rn(fmaf((v[q][e] - mean) * dev, __half2float(wh[e]), __half2float(bh[e])));
                *reinterpret_cast<uint4*>(lnrow + (size_t)t * xp + gi * 8) = outv;
                if (a.ln_out != nullptr && blockIdx.x == 0) *reinterpret_cast<uint4*>(a.ln_out + (size_t)t * C + gi * 8) = outv;
            }
        }
    }
    __syncthreads();
    if (a.prologue == PRO_LN) return;  // the vectors are the normalised rows themselves
    const int nv = a.prologue == PRO_LN_SHIFT2 ? 2 : 1;
    for (uint32_t t = 0; t < T; ++t) {
        const CursorD cu = cursor_at(a.cursors, a.wide, t);
        for (uint32_t c = threadIdx.x; c < C; c += kThreads) {
            const float cur = __half2float(lnrow[(size_t)t * xp + c]);
            const float prev = (t == cu.token) ? static_cast<const float*>(a.state.base)[a.state.index(c, 0, cu.batch)]
                                               : __half2float(lnrow[(size_t)(t - 1) * xp + c]);
            const float lhs = a.reversed ? cur : prev, rhs = a.reversed ? prev : cur;
            for (int vi = 0; vi < nv; ++vi) {
                const float f = __half2float((vi == 0 ? a.mix0 : a.mix1)[c]);
                xgen[((size_t)vi * T + t) * xp + c] = __float2half_rn(lhs * (1.0f - f) + rhs * f);
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kThreads, 2) fused_gemv_kernel(const FusedGemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float scratch[kWarps];
    __shared__ __half lut[16];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const uint32_t T = a.T;
    const GemvSegment* segs = a.segments + (size_t)blockIdx.x * kSegmentsPerCta;

    // shared memory carve-up (all offsets multiples of 16 bytes)
    uint32_t kmax = 0;
    for (int i = 0; i < a.num_problems; ++i) kmax = max(kmax, a.p[i].K);
    const uint32_t xp = (a.prologue != PRO_NONE ? a.C : kmax) + 8;  // halfs per activation row
    uint8_t* slots = smem;
    const int NSLOT = a.num_slots;
    float* red = reinterpret_cast<float*>(slots + (size_t)NSLOT * SLOT);   // [kWarps][GROUP_ROWS][T]
    float* sums = red + (size_t)kWarps * GROUP_ROWS * T;                    // [T][kmax / 128]
    __half* xs = reinterpret_cast<__half*>(sums + sums_floats(T, kmax));    // staged x or prologue rows
    __half* lnrow = xs;                                                     // PRO_LN: vectors = normalised rows
    __half* xgen = a.prologue == PRO_LN ? xs : xs + (size_t)T * xp;         // shifted vectors follow the rows

    if (threadIdx.x < 16 && a.table != nullptr) lut[threadIdx.x] = __float2half_rn(a.table[threadIdx.x]);
    __syncthreads();
    trace(100);
    pdl_launch_dependents();
    trace(109);

    // weights do not depend on earlier kernels: start streaming before waiting for them
    TileIter prod, cons;
    prod.start(a, segs);
    cons = prod;
    uint32_t issued = 0;
    trace(110);
    for (int s = 0; s < NSLOT; ++s) {
        if (prod.valid) {
            issue_tile(a, segs, prod, slots + s * SLOT);
            prod.next(a, segs);
            ++issued;
        }
        cp_async_commit();  // one group per slot, empty or not: the group count stays uniform
    }
    trace(111);
    trace(101);
    pdl_wait();
    trace(102);

    if (a.prologue != PRO_NONE && (cons.valid || blockIdx.x == 0)) run_prologue(a, xgen, xp, lnrow, scratch);

    trace(103);
    float acc[GROUP_ROWS / 16][4];
    int staged_problem = -1;
    uint32_t consumed = 0;
    while (cons.valid) {
        const GemvSegment& sg = segs[cons.seg];
        const GemvProblem& p = a.p[sg.problem];
        const __half* xv;  // this problem's activations in shared memory, pitch xp
        if (p.x == nullptr) {
            xv = xgen + (size_t)p.x_sel * T * xp;
        } else {
            xv = xs;
        }
        if (staged_problem != sg.problem) {
            // stage x (explicit inputs) and the per-128-block sums of the values the MMA will see:
            // 16 consecutive lanes cover one block of 128, so the sums come from the registers in flight
            __syncthreads();
            if (p.x != nullptr) {
                const uint32_t groups = p.K / 8, total = T * groups;
                for (uint32_t i0 = 0; i0 < total; i0 += kThreads) {
                    const uint32_t i = i0 + threadIdx.x;
                    float sum = 0.f;
                    uint32_t tok = 0, k8 = 0;
                    if (i < total) {
                        tok = i / groups;
                        k8 = i % groups;
                        const uint4 raw = *reinterpret_cast<const uint4*>(p.x + (size_t)tok * p.x_stride + k8 * 8);
                        *reinterpret_cast<uint4*>(xs + (size_t)tok * xp + k8 * 8) = raw;
                        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __half22float2(h[e]);
                            sum += f.x + f.y;
                        }
                    }
                    if (p.kind == MAT_INT8) {
#pragma unroll
                        for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off, 16);
                        if (i < total && (k8 & 15) == 0) sums[tok * (p.K / 128) + (k8 >> 4)] = sum;
                    }
                }
            } else if (p.kind == MAT_INT8) {
                const uint32_t nblk = p.K / 128;
                for (uint32_t u = warp; u < T * nblk; u += kWarps) {
                    const uint32_t tok = u / nblk, blk = u % nblk;
                    const uint2 raw = *reinterpret_cast<const uint2*>(xv + (size_t)tok * xp + blk * 128 + lane * 4);
                    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    const float s = warp_sum((lo.x + lo.y) + (hi.x + hi.y));
                    if (lane == 0) sums[tok * nblk + blk] = s;
                }
            }
            __syncthreads();
            staged_problem = sg.problem;
        }
        if (cons.part == 0 && cons.tile == 0) {
#pragma unroll
            for (int i = 0; i < GROUP_ROWS / 16; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
        }

        const int slot_i = consumed % NSLOT;
        trace(104);
        cp_async_wait(NSLOT - 1);  // this thread's copies of tile part `consumed` have landed ...
        __syncthreads();           // ... and everyone else's
        trace(105);
        const uint8_t* slot = slots + slot_i * SLOT;
        const uint32_t rb = row_bytes(p);
        const uint32_t bytes = min((uint32_t)PB, rb - cons.part * PB);
        const int rowA = cons.group0 + 16 * cons.tile + g, rowB = rowA + 8;
        const bool xval = (uint32_t)g < T;
        const bool stma = scales_async(p);
        const __half* xrow = xv + (size_t)(xval ? g : 0) * xp + (size_t)cons.part * part_elems(p.kind);
        float ac[4];
#pragma unroll
        for (int i = 0; i < GROUP_ROWS / 16; ++i)
            if (i == cons.tile) {
                ac[0] = acc[i][0]; ac[1] = acc[i][1]; ac[2] = acc[i][2]; ac[3] = acc[i][3];
            }
        const uint8_t* sslot = slot + 16 * PITCH;  // this tile part's scales, SCP bytes per row

        if (p.kind == MAT_INT8) {
            const uint32_t nblk = p.K / 128;
            const __half2* sc = reinterpret_cast<const __half2*>(p.scale);
            const bool vA = rowA < cons.gend, vB = rowB < cons.gend;
            for (uint32_t c = warp; c < bytes / 128; c += kWarps) {
                const uint32_t blk = cons.part * (PB / 128) + c;
                const uint8_t* pa = slot + g * PITCH + c * 128 + 16 * t4;
                const uint4 wa0 = *reinterpret_cast<const uint4*>(pa), wa1 = *reinterpret_cast<const uint4*>(pa + 64);
                const uint4 wb0 = *reinterpret_cast<const uint4*>(pa + 8 * PITCH),
                            wb1 = *reinterpret_cast<const uint4*>(pa + 8 * PITCH + 64);
                float2 mmA = make_float2(0.f, 0.f), mmB = mmA;
                if (stma) {
                    mmA = __half22float2(*reinterpret_cast<const __half2*>(sslot + g * SCP + c * 4));
                    mmB = __half22float2(*reinterpret_cast<const __half2*>(sslot + (g + 8) * SCP + c * 4));
                } else {
                    if (vA) mmA = __half22float2(__ldg(sc + (size_t)rowA * nblk + blk));
                    if (vB) mmB = __half22float2(__ldg(sc + (size_t)rowB * nblk + blk));
                }
                const uint32_t wa[8] = {wa0.x, wa0.y, wa0.z, wa0.w, wa1.x, wa1.y, wa1.z, wa1.w};
                const uint32_t wb[8] = {wb0.x, wb0.y, wb0.z, wb0.w, wb1.x, wb1.y, wb1.z, wb1.w};
                float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s2 = 0; s2 < 4; ++s2) {
                    const uint32_t kk = c * 128 + (s2 < 2 ? 16 * t4 + 8 * s2 : 64 + 16 * t4 + 8 * (s2 - 2));
                    uint4 xq = make_uint4(0, 0, 0, 0);
                    if (xval) xq = *reinterpret_cast<const uint4*>(xrow + kk);
                    mma16816(d, bytes_to_half2(wa[2 * s2], 0x4140), bytes_to_half2(wb[2 * s2], 0x4140),
                             bytes_to_half2(wa[2 * s2], 0x4342), bytes_to_half2(wb[2 * s2], 0x4342), xq.x, xq.y);
                    mma16816(d, bytes_to_half2(wa[2 * s2 + 1], 0x4140), bytes_to_half2(wb[2 * s2 + 1], 0x4140),
                             bytes_to_half2(wa[2 * s2 + 1], 0x4342), bytes_to_half2(wb[2 * s2 + 1], 0x4342), xq.z, xq.w);
                }
                const uint32_t tk0 = 2 * t4, tk1 = tk0 + 1;
                const float s0 = tk0 < T ? sums[tk0 * nblk + blk] : 0.f, s1 = tk1 < T ? sums[tk1 * nblk + blk] : 0.f;
                const float sA = (mmA.y - mmA.x) * (1.0f / 255.0f), sB = (mmB.y - mmB.x) * (1.0f / 255.0f);
                ac[0] += sA * d[0] + mmA.x * s0;
                ac[1] += sA * d[1] + mmA.x * s1;
                ac[2] += sB * d[2] + mmB.x * s0;
                ac[3] += sB * d[3] + mmB.x * s1;
            }
        } else if (p.kind == MAT_NF4) {
            const uint32_t nblk = p.K / 64;
            const bool vA = rowA < cons.gend, vB = rowB < cons.gend;
            for (uint32_t c = warp; c < bytes / 32; c += kWarps) {
                const uint32_t blk = cons.part * (PB / 32) + c;
                const uint8_t* pa = slot + g * PITCH + c * 32 + 8 * t4;
                const uint2 wa = *reinterpret_cast<const uint2*>(pa), wb = *reinterpret_cast<const uint2*>(pa + 8 * PITCH);
                float aA, aB;
                if (stma) {
                    aA = __half2float(*reinterpret_cast<const __half*>(sslot + g * SCP + c * 2));
                    aB = __half2float(*reinterpret_cast<const __half*>(sslot + (g + 8) * SCP + c * 2));
                } else {
                    aA = vA ? __half2float(__ldg(p.scale + (size_t)rowA * nblk + blk)) : 0.f;
                    aB = vB ? __half2float(__ldg(p.scale + (size_t)rowB * nblk + blk)) : 0.f;
                }
                const uint32_t wau[2] = {wa.x, wa.y}, wbu[2] = {wb.x, wb.y};
                float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s2 = 0; s2 < 2; ++s2) {
                    uint4 xq = make_uint4(0, 0, 0, 0);
                    if (xval) xq = *reinterpret_cast<const uint4*>(xrow + c * 64 + 16 * t4 + 8 * s2);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t qa = wau[s2] >> (16 * h), qb = wbu[s2] >> (16 * h);
                        const __half2 a0 = __halves2half2(lut[qa & 15u], lut[(qa >> 4) & 15u]);
                        const __half2 a2 = __halves2half2(lut[(qa >> 8) & 15u], lut[(qa >> 12) & 15u]);
                        const __half2 a1 = __halves2half2(lut[qb & 15u], lut[(qb >> 4) & 15u]);
                        const __half2 a3 = __halves2half2(lut[(qb >> 8) & 15u], lut[(qb >> 12) & 15u]);
                        mma16816(d, *reinterpret_cast<const uint32_t*>(&a0), *reinterpret_cast<const uint32_t*>(&a1),
                                 *reinterpret_cast<const uint32_t*>(&a2), *reinterpret_cast<const uint32_t*>(&a3),
                                 h == 0 ? xq.x : xq.z, h == 0 ? xq.y : xq.w);
                    }
                }
                ac[0] = fmaf(d[0], aA, ac[0]);
                ac[1] = fmaf(d[1], aA, ac[1]);
                ac[2] = fmaf(d[2], aB, ac[2]);
                ac[3] = fmaf(d[3], aB, ac[3]);
            }
        } else {
            for (uint32_t c = warp; c < bytes / 64; c += kWarps) {
                const uint8_t* pa = slot + g * PITCH + c * 64 + 16 * t4;
                const uint4 wa = *reinterpret_cast<const uint4*>(pa), wb = *reinterpret_cast<const uint4*>(pa + 8 * PITCH);
                uint4 xq = make_uint4(0, 0, 0, 0);
                if (xval) xq = *reinterpret_cast<const uint4*>(xrow + c * 32 + 8 * t4);
                mma16816(ac, wa.x, wb.x, wa.y, wb.y, xq.x, xq.y);
                mma16816(ac, wa.z, wb.z, wa.w, wb.w, xq.z, xq.w);
            }
        }

#pragma unroll
        for (int i = 0; i < GROUP_ROWS / 16; ++i)
            if (i == cons.tile) {
                acc[i][0] = ac[0]; acc[i][1] = ac[1]; acc[i][2] = ac[2]; acc[i][3] = ac[3];
            }
        const bool finish = cons.last_part_of_group();
        const int fin_group0 = cons.group0, fin_gend = cons.gend, fin_problem = sg.problem;
        __syncthreads();  // everyone is done with this slot (and with `red` of the previous group)
        ++consumed;
        cons.next(a, segs);
        if (prod.valid) {
            // refill the slot just released with the tile part NSLOT steps ahead
            issue_tile(a, segs, prod, slots + slot_i * SLOT);
            prod.next(a, segs);
            ++issued;
        }
        cp_async_commit();
        if (!finish) continue;

        // ---- group finished: cross-warp reduction and epilogue ----
        const GemvProblem& fp = a.p[fin_problem];
#pragma unroll
        for (int i = 0; i < GROUP_ROWS / 16; ++i) {
            const int r0 = 16 * i + g;
            const uint32_t tk0 = 2 * t4, tk1 = tk0 + 1;
            float* r = red + (size_t)warp * GROUP_ROWS * T;
            if (tk0 < T) {
                r[(size_t)r0 * T + tk0] = acc[i][0];
                r[(size_t)(r0 + 8) * T + tk0] = acc[i][2];
            }
            if (tk1 < T) {
                r[(size_t)r0 * T + tk1] = acc[i][1];
                r[(size_t)(r0 + 8) * T + tk1] = acc[i][3];
            }
        }
        __syncthreads();
        const int nrows = fin_gend - fin_group0;
        for (int o = threadIdx.x; o < nrows * (int)T; o += kThreads) {
            const int row = o % nrows, tok = o / nrows;
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += red[((size_t)w * GROUP_ROWS + row) * T + tok];
            s = activate_f(fp.act, s);
            const uint32_t m = fin_group0 + row;
            const size_t oi = (size_t)tok * fp.M + m;
            if (a.epilogue == EPI_STORE) {
                dstore(fp.out, fp.out_dtype, (size_t)tok * fp.out_stride + m, s);
            } else if (a.epilogue == EPI_RESIDUAL) {
                // att_o is an fp16 tensor in the reference; x += att_o is rounded to fp16 again
                const float o16 = __half2float(__float2half_rn(s));
                a.xres[oi] = __float2half_rn(a.rescale * __half2float(__float2half_rn(__half2float(a.xres[oi]) + o16)));
            } else {
                // channel mix: carry row <- normalised ffn input at a sequence's last token;
                // x += sigmoid(r) * v with the reference's fp16 rounding points
                const CursorD cu = cursor_at(a.cursors, a.wide, tok);
                if ((uint32_t)tok - cu.token + 1u == cu.len)
                    static_cast<float*>(a.cm_state.base)[a.cm_state.index(m, 0, cu.batch)] = __half2float(a.cm_x[oi]);
                const float v16 = __half2float(__float2half_rn(s));
                float mixed = v16;
                if (a.cm_r != nullptr) {
                    const float rr = 1.0f / (1.0f + expf(-__half2float(a.cm_r[oi])));
                    mixed = rr * v16;
                }
                const float o16 = __half2float(__float2half_rn(mixed));
                const __half sum16 = __float2half_rn(__half2float(a.xres[oi]) + o16);
                a.xres[oi] = a.rescale == 1.0f ? sum16 : __float2half_rn(a.rescale * __half2float(sum16));
            }
        }
        // `red` is reused by the next group only after the __syncthreads that follows its first tile part
        trace(106);
    }
    trace(107);
}

#ifdef WRK_TRACE
}  // namespace
cudaError_t debug_trace_read(unsigned long long* host, unsigned int* n) {
    cudaError_t e = cudaMemcpyFromSymbol(n, g_trace_n, sizeof(unsigned int));
    if (e != cudaSuccess) return e;
    e = cudaMemcpyFromSymbol(host, g_trace, sizeof(unsigned long long) * (1 << 16));
    unsigned int zero = 0;
    cudaMemcpyToSymbol(g_trace_n, &zero, sizeof zero);
    return e;
}
namespace {
#endif


// ---- v6 data-dependent token shift ---------------------------------------------------------------
// sx[i][t][c] = mix(att_x[t][c], prev[t][c], f16(f16(W2[i][c][:] . tmx[t][i*D:(i+1)*D]) + mix[i][c]))
__global__ void __launch_bounds__(256) tmix_shift_kernel(const TmixArgs a) {
    extern __shared__ __half s_tmx[];  // [T][5 * D]
    pdl_launch_dependents();
    const uint32_t C = a.C, D = a.D, T = a.T;
    // the adapter weights of this thread do not depend on earlier kernels
    const uint32_t o = blockIdx.x * blockDim.x + threadIdx.x;  // (i, c)
    const bool active = o < 5 * C;
    const uint32_t i = active ? o / C : 0, c = active ? o % C : 0;
    uint4 wreg[8];  // D <= 64 halfs
    if (active) {
        const uint4* wp = reinterpret_cast<const uint4*>(a.w2 + ((size_t)i * C + c) * D);
        for (uint32_t j = 0; j < D / 8; ++j) wreg[j] = wp[j];
    }
    pdl_wait();
    for (uint32_t j = threadIdx.x; j < T * 5 * D; j += blockDim.x) s_tmx[j] = a.tmx[j];
    __syncthreads();
    if (!active) return;
    const float mu = __half2float(a.mix[(size_t)i * C + c]);
    for (uint32_t t = 0; t < T; ++t) {
        float acc = 0.f;
        const __half* xv = s_tmx + (size_t)t * 5 * D + i * D;
        for (uint32_t j = 0; j < D / 8; ++j) {
            const __half2* w2 = reinterpret_cast<const __half2*>(&wreg[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 wf = __half22float2(w2[e]);
                acc = fmaf(wf.x, __half2float(xv[j * 8 + 2 * e]), acc);
                acc = fmaf(wf.y, __half2float(xv[j * 8 + 2 * e + 1]), acc);
            }
        }
        // time_mix buffer is fp16: matmul result rounded, then the static mix added and rounded again
        const float f = __half2float(__float2half_rn(__half2float(__float2half_rn(acc)) + mu));
        const CursorD cu = cursor_at(a.cursors, a.wide, t);
        const float cur = __half2float(a.att_x[(size_t)t * C + c]);
        const float prev = (t == cu.token) ? static_cast<const float*>(a.state.base)[a.state.index(c, 0, cu.batch)]
                                           : __half2float(a.att_x[(size_t)(t - 1) * C + c]);
        a.sx[((size_t)i * T + t) * C + c] = __float2half_rn(cur * (1.0f - f) + prev * f);
    }
}

// ---- v5 / v6 time-mix block: decay adapter, WKV, group norm, gate --------------------------------
template <int S>
__global__ void __launch_bounds__(S) wkv56_fused_kernel(const Wkv6Args a) {
    __shared__ float sk[S], sr[S], sw[S], su[S], red[4];
    __shared__ __half s_tdw[64 * kDecodeMaxTokens];
    __shared__ uint32_t s_start, s_count;
    pdl_launch_dependents();
    const uint32_t h = blockIdx.x, slot = blockIdx.y, j = threadIdx.x;
    const uint32_t C = S * a.H, c = h * S + j;

    // state column, decay-adapter row and per-channel constants do not depend on this job's kernels...
    uint4 w2reg[8];
    if (a.per_token_decay) {
        const uint4* wp = reinterpret_cast<const uint4*>(a.td_w2 + (size_t)c * a.D);
        for (uint32_t q = 0; q < a.D / 8; ++q) w2reg[q] = wp[q];
    }
    su[j] = a.time_first[c];
    const float td_static = a.per_token_decay ? __half2float(a.td0[c]) : 0.f;
    const float gw = __half2float(a.gn_w[c]), gb = __half2float(a.gn_b[c]);
    pdl_wait();  // ...the state does (the previous token's job wrote it), and so do the cursors

    // run of tokens of this batch slot
    if (j == 0) {
        s_start = 0xffffffffu;
        s_count = 0;
    }
    __syncthreads();
    {
        uint32_t mn = 0xffffffffu, cnt = 0;
        for (uint32_t t = j; t < a.T; t += S) {
            const CursorD cu = cursor_at(a.cursors, a.wide, t);
            if (cu.batch == slot) {
                mn = min(mn, t);
                ++cnt;
            }
        }
        if (cnt) {
            atomicMin(&s_start, mn);
            atomicAdd(&s_count, cnt);
        }
    }
    __syncthreads();
    const uint32_t start = s_start, count = s_count;
    if (count == 0) return;

    float st[S];
#pragma unroll
    for (int i = 0; i < S; ++i) st[i] = static_cast<const float*>(a.state.base)[a.state.index(c, 1 + i, slot)];

    for (uint32_t n = 0; n < count; ++n) {
        const uint32_t t = start + n;
        const size_t ti = (size_t)t * C + c;
        __syncthreads();
        if (a.per_token_decay)
            for (uint32_t q = j; q < a.D; q += S) s_tdw[q] = a.tdw[(size_t)t * a.D + q];
        sk[j] = a.k[ti];
        sr[j] = a.r[ti];
        __syncthreads();
        float wj;
        if (a.per_token_decay) {
            float acc = 0.f;
            for (uint32_t q = 0; q < a.D / 8; ++q) {
                const __half2* w2 = reinterpret_cast<const __half2*>(&w2reg[q]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 wf = __half22float2(w2[e]);
                    acc = fmaf(wf.x, __half2float(s_tdw[q * 8 + 2 * e]), acc);
                    acc = fmaf(wf.y, __half2float(s_tdw[q * 8 + 2 * e + 1]), acc);
                }
            }
            wj = expf(-expf(acc + td_static));  // time_decay buffer is f32: no rounding before the activation
        } else {
            wj = a.td5[c];
        }
        sw[j] = wj;
        __syncthreads();
        const float vj = a.v[ti];
        float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
        for (int i = 0; i < S; i += 4) {
            float kv;
            kv = sk[i] * vj;     y0 += sr[i] * fmaf(su[i], kv, st[i]);             st[i] = fmaf(sw[i], st[i], kv);
            kv = sk[i + 1] * vj; y1 += sr[i + 1] * fmaf(su[i + 1], kv, st[i + 1]); st[i + 1] = fmaf(sw[i + 1], st[i + 1], kv);
            kv = sk[i + 2] * vj; y2 += sr[i + 2] * fmaf(su[i + 2], kv, st[i + 2]); st[i + 2] = fmaf(sw[i + 2], st[i + 2], kv);
            kv = sk[i + 3] * vj; y3 += sr[i + 3] * fmaf(su[i + 3], kv, st[i + 3]); st[i + 3] = fmaf(sw[i + 3], st[i + 3], kv);
        }
        const float y = (y0 + y1) + (y2 + y3);
        const CursorD cu = cursor_at(a.cursors, a.wide, t);
        if (t - cu.token + 1u == cu.len)
            static_cast<float*>(a.state.base)[a.state.index(c, 0, slot)] = __half2float(a.att_x[ti]);
        // group norm over the head's S outputs (f32 buffer in the reference), then fp16, then the gate
        float s = warp_sum(y);
        if ((j & 31) == 0) red[j >> 5] = s;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < S / 32; ++w) tot += red[w];
        const float mean = tot / (float)S;
        const float dlt = y - mean;
        __syncthreads();
        s = warp_sum(dlt * dlt);
        if ((j & 31) == 0) red[j >> 5] = s;
        __syncthreads();
        tot = 0.f;
        for (int w = 0; w < S / 32; ++w) tot += red[w];
        const float dev = rsqrtf(tot / (float)S + a.gn_eps);
        const float gn16 = __half2float(__float2half_rn(fmaf(dlt * dev, gw, gb)));
        const float gg = __half2float(a.g[ti]);
        const float silu = gg / (1.0f + expf(-gg));
        a.out[ti] = __float2half_rn(silu * gn16);
    }
#pragma unroll
    for (int i = 0; i < S; ++i) static_cast<float*>(a.state.base)[a.state.index(c, 1 + i, slot)] = st[i];
}

template <typename Kernel, typename Args>
cudaError_t launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const Args& args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args);
}

}  // namespace

// Cuts the concatenated rows of the launch's matrices into one contiguous range per CTA, balanced by
// weight bytes.  Returns false when a CTA would need more than kSegmentsPerCta ranges.
bool fused_gemv_partition(const FusedGemvArgs& a, int grid, std::vector<GemvSegment>& table) {
    table.assign((size_t)grid * kSegmentsPerCta, GemvSegment{0, 0, 0, 0});
    double total = 0;
    std::vector<double> cost(a.num_problems);
    for (int i = 0; i < a.num_problems; ++i) {
        const GemvProblem& p = a.p[i];
        cost[i] = p.kind == MAT_FP16 ? p.K * 2.0 : p.kind == MAT_INT8 ? p.K * 1.03125 : p.K * 0.53125;
        total += cost[i] * p.M;
    }
    int prob = 0;
    uint32_t row = 0;
    double done = 0;
    for (int c = 0; c < grid; ++c) {
        const bool last = c == grid - 1;
        const double target = total * (c + 1) / grid;
        int nseg = 0;
        while (prob < a.num_problems && nseg < kSegmentsPerCta) {
            const GemvProblem& p = a.p[prob];
            uint32_t take = p.M - row;
            if (!last) {
                const double want = std::ceil((target - done) / cost[prob] - 1e-9);
                take = (uint32_t)std::min<double>(take, std::max(0.0, want));
            }
            if (take > 0) {
                table[(size_t)c * kSegmentsPerCta + nseg++] = GemvSegment{prob, (int32_t)row, (int32_t)(row + take), 0};
                row += take;
                done += take * cost[prob];
            }
            if (row == p.M) {
                ++prob;
                row = 0;
            }
            if (!last && done >= target - 1e-6) break;
        }
    }
    return prob == a.num_problems;
}

size_t fused_gemv_smem(uint32_t T, uint32_t Kmax, uint32_t C, int prologue, int num_slots) {
    const uint32_t xp = (prologue != PRO_NONE ? C : Kmax) + 8;
    size_t bytes = (size_t)num_slots * SLOT;
    bytes += (size_t)kWarps * GROUP_ROWS * T * sizeof(float);
    bytes += (size_t)sums_floats(T, Kmax) * sizeof(float);
    const size_t rows = prologue == PRO_NONE || prologue == PRO_LN ? T : prologue == PRO_LN_SHIFT1 ? 2 * T : 3 * T;
    bytes += rows * xp * sizeof(__half);
    return bytes + 64;
}

int fused_gemv_slots(uint32_t T, uint32_t Kmax, uint32_t C, int prologue) {
    // as many slots as keep two CTAs (this kernel's and the next one's) resident per SM
    int n = MAX_SLOTS;
    while (n > 2 && fused_gemv_smem(T, Kmax, C, prologue, n) > 100 * 1024) --n;
    return n;
}

cudaError_t fused_gemv(const FusedGemvArgs& a_in, int grid, cudaStream_t stream) {
    FusedGemvArgs a = a_in;
    uint32_t kmax = 0;
    for (int i = 0; i < a.num_problems; ++i) kmax = std::max(kmax, a.p[i].K);
    a.num_slots = fused_gemv_slots(a.T, kmax, a.C, a.prologue);
    const size_t smem = fused_gemv_smem(a.T, kmax, a.C, a.prologue, a.num_slots);
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(fused_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured = 200 * 1024;
    }
    return launch_pdl(fused_gemv_kernel, dim3(grid), dim3(kThreads), smem, stream, a);
}

cudaError_t tmix_shift_v6(const TmixArgs& a, cudaStream_t stream) {
    const uint32_t threads = 5 * a.C;
    const size_t smem = (size_t)a.T * 5 * a.D * sizeof(__half);
    return launch_pdl(tmix_shift_kernel, dim3((threads + 255) / 256), dim3(256), smem, stream, a);
}

cudaError_t wkv56_fused(const Wkv6Args& a, cudaStream_t stream) {
    return launch_pdl(wkv56_fused_kernel<64>, dim3(a.H, a.B), dim3(64), 0, stream, a);
}

}  // namespace k
}  // namespace wrk
