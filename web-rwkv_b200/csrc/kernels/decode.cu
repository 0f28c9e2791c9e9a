// Fused decode path for jobs of a few tokens (T <= 8): the whole v6 layer in seven launches.
//
// The quantized matmuls of a decode step are pure weight streaming, and at model widths of 2048-4096
// a single matrix is only a few microseconds of HBM time, so the structure of this file is built
// around never letting the stream of weights stop:
//   * fused_gemv_kernel is a grouped weight-streaming kernel.  A launch covers several matrices (e.g.
//     key / value / receptance / gate + the decay adapter); the concatenated row space is cut into one
//     contiguous row range per CTA (balanced by bytes, one CTA per SM).  A CTA walks its rows in MMA row tiles of 16; its 16 warps split a tile's 128-byte
//     chunks and each streams its own items through a private ring in shared memory with cp.async.
//     (A variant that re-laid the weights per CTA at load time and fetched 34 KB stages with one
//     cp.async.bulk each was measured: faster alone, slower inside the model, twice the weight memory;
//     it is not kept.)
//   * every kernel here is launched with programmatic dependent launch: it signals its dependents at
//     once, issues the copies of its first weight items, and only then executes griddepcontrol.wait.
//     Weights are never written during a job, so a CTA that becomes resident while the previous kernel is
//     still draining already has its first weights landing in shared memory.
//   * layer norm + token shift run as a per-CTA prologue (every CTA recomputes the few-KB vector instead
//     of a separate launch and a grid-wide dependency); residual add, squared ReLU, channel mix and the
//     carry-row updates run as epilogues.
// The math on the tiles is the mma.sync scheme of matmul.cu (bytes expanded to fp16 in registers, fp32
// accumulate, Int8 affine term through per-block activation sums).  Every tensor the reference stores as
// fp16 is rounded to fp16 here at the same point.
#include "decode.cuh"
#include "device.cuh"

#include <mutex>

namespace wrk {
namespace k {

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = 16;
constexpr int GROUP_ROWS = 64;  // rows (4 MMA row tiles) whose partial results meet in shared memory at once

// floats reserved for the per-block activation sums (keeps what follows 16-byte aligned)
__host__ __device__ inline uint32_t sums_floats(uint32_t T, uint32_t kmax) {
    return (T * ((kmax + 127) / 128) + 3) / 4 * 4 + 4;
}

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
__device__ __forceinline__ uint32_t row_bytes(const GemvProblem& p) {
    return p.kind == MAT_FP16 ? p.K * 2 : p.kind == MAT_INT8 ? p.K : p.K / 2;
}

// One warp-level work item covers CHUNK_BYTES of 16 weight rows (an MMA row tile): Int8 one 128-weight
// block per row, fp16 64 weights, NF4 four 64-weight blocks.  Lane (g, t4) reads 16-byte (NF4: 8-byte)
// pieces of rows g and g + 8.
constexpr int CHUNK_BYTES = 128;

// One work item in registers: this lane's pieces of rows g and g + 8 and their block scales.
struct Item {
    uint4 q[4];     // Int8 / fp16: rowA lo, rowA hi, rowB lo, rowB hi; NF4: blocks (0,1) A, (2,3) A, (0,1) B, (2,3) B
    uint32_t s[4];  // Int8: s[0] = (min, max) of rowA as half2, s[2] = rowB; NF4: absmax pairs A01, A23, B01, B23
};

// The CTA's row ranges, kept in registers.
struct Segs {
    int prob[kSegmentsPerCta], r0[kSegmentsPerCta], r1[kSegmentsPerCta];
    __device__ __forceinline__ int P(int s) const { return s == 0 ? prob[0] : s == 1 ? prob[1] : prob[2]; }
    __device__ __forceinline__ int R0(int s) const { return s == 0 ? r0[0] : s == 1 ? r0[1] : r0[2]; }
    __device__ __forceinline__ int R1(int s) const { return s == 0 ? r1[0] : s == 1 ? r1[1] : r1[2]; }
};

// ---- per-warp staging ring --------------------------------------------------------------------
// Each warp streams its own work items through a private ring of cells in shared memory with cp.async.  A
// lane copies exactly the 16-byte pieces it will later feed to the MMA into its own slots, so reading them
// back is conflict free; the block scales of the item's 16 rows are copied once per row (by the lanes
// t4 = 0 / 2 for Int8, all four for NF4) and read after a warp barrier.
constexpr int kMinRing = 2, kMaxRing = 5;          // items in flight per warp (chosen per launch)
constexpr int CELL_DATA = 32 * 4 * 16;             // per lane: four 16-byte pieces
constexpr int CELL_BYTES = CELL_DATA + 16 * 8;     // + 8 bytes of block scales per row

__device__ __forceinline__ void cp_async16z(void* dst, const void* src, bool valid) {
    const uint32_t n = valid ? 16u : 0u;  // src-size 0: the cell is zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async8z(void* dst, const void* src, bool valid) {
    const uint32_t n = valid ? 8u : 0u;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async4z(void* dst, const void* src, bool valid) {
    const uint32_t n = valid ? 4u : 0u;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
// all but the newest n groups of this thread have landed (n = 1 .. kMaxRing)
__device__ __forceinline__ void cp_async_wait_dyn(int n) {
    if (n <= 1) cp_async_wait<1>();
    else if (n == 2) cp_async_wait<2>();
    else if (n == 3) cp_async_wait<3>();
    else if (n == 4) cp_async_wait<4>();
    else if (n == 5) cp_async_wait<5>();
    else cp_async_wait<6>();
}

// Work mapping inside a CTA: its row ranges are walked in MMA row tiles of 16 rows; the 16 warps split a
// tile's chunks (warp w takes chunks w, w + 16, ...), keep their partial results in registers, and meet in
// shared memory once per tile.  The copy side of a warp walks the same (range, tile, chunk) sequence as its
// compute side, `depth` items ahead.  Tiles are taken in groups of four: one barrier and one pass of sums
// and epilogues per 64 rows.
struct Loader {
    int seg, row0, r1, c, nchunk;  // seg == kSegmentsPerCta: the CTA's work is exhausted
    int kind;
    uint32_t rb, srow;             // bytes per weight row / per row of the scale table
    const uint8_t* wbase;          // matrix + this lane's byte offset inside a chunk
    const uint8_t* sbase;          // scale table

    __device__ __forceinline__ bool valid() const { return seg < kSegmentsPerCta; }

    // first range at or after `seg` in which this warp has chunks
    __device__ __forceinline__ void enter(const FusedGemvArgs& a, const Segs& sg, int warp, int lane) {
        for (; seg < kSegmentsPerCta; ++seg) {
            if (sg.R0(seg) >= sg.R1(seg)) continue;
            const GemvProblem& p = a.p[sg.P(seg)];
            rb = row_bytes(p);
            nchunk = (int)((rb + CHUNK_BYTES - 1) / CHUNK_BYTES);
            if (warp >= nchunk) continue;
            kind = p.kind;
            srow = kind == MAT_INT8 ? (p.K / 128) * 4 : kind == MAT_NF4 ? (p.K / 64) * 2 : 0;
            wbase = p.w + (kind == MAT_NF4 ? 8 : 16) * (lane & 3);
            sbase = reinterpret_cast<const uint8_t*>(p.scale);
            row0 = sg.R0(seg);
            r1 = sg.R1(seg);
            c = warp;
            return;
        }
    }
    // Issues the copies of the current item into `cell` (nothing when exhausted) and steps to the next one.
    __device__ __forceinline__ void issue(const FusedGemvArgs& a, const Segs& sg, uint8_t* cell, int warp, int lane) {
        if (!valid()) return;
        const int g = lane >> 2, t4 = lane & 3;
        const bool vA = row0 + g < r1, vB = row0 + g + 8 < r1;
        const uint32_t off = (uint32_t)c * CHUNK_BYTES;
        const uint8_t* A = wbase + (size_t)(vA ? row0 + g : row0) * rb + off;
        const uint8_t* B = vB ? A + 8 * (size_t)rb : A;
        uint8_t* wq = cell + lane * 16;  // piece i at wq + i * 512
        const int sr = g + 8 * (t4 >> 1), sh = t4 & 1;  // scale row / half copied by this lane
        const bool vS = row0 + sr < r1;
        const uint8_t* S = sbase + (size_t)(vS ? row0 + sr : row0) * srow;
        uint8_t* ws = cell + CELL_DATA + sr * 8 + sh * 4;
        if (kind == MAT_NF4) {
            // four 64-weight blocks of 32 bytes, 8 bytes of each per lane: slots hold (blk0, blk1), (blk2, blk3)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool in = off + 32 * j < rb;
                cp_async8z(wq + (j >> 1) * 512 + (j & 1) * 8, A + 32 * j, in && vA);
                cp_async8z(wq + (2 + (j >> 1)) * 512 + (j & 1) * 8, B + 32 * j, in && vB);
            }
            // absmax of blocks (0, 1) or (2, 3): K is a multiple of 128, so the pairs are 4-byte aligned
            cp_async4z(ws, S + (off >> 4) + sh * 4, vS && off + 64 * sh < rb);
        } else {
            const bool hi = off + 64 < rb;  // fp16 rows may end after the first 64 bytes of the chunk
            cp_async16z(wq, A, vA);
            cp_async16z(wq + 512, A + 64, vA && hi);
            cp_async16z(wq + 1024, B, vB);
            cp_async16z(wq + 1536, B + 64, vB && hi);
            if (kind == MAT_INT8 && sh == 0) cp_async4z(ws, S + (off >> 5), vS);
        }
        c += kWarps;
        if (c >= nchunk) {
            c = warp;
            row0 += 16;
            if (row0 >= r1) {
                ++seg;
                enter(a, sg, warp, lane);
            }
        }
    }
};

// This lane's registers of the item in `cell` (after its copies have landed and the warp has synchronised).
__device__ __forceinline__ Item read_item(const uint8_t* cell, int lane) {
    Item it;
    const int g = lane >> 2;
#pragma unroll
    for (int i = 0; i < 4; ++i) it.q[i] = *reinterpret_cast<const uint4*>(cell + i * 512 + lane * 16);
    const uint2 sa = *reinterpret_cast<const uint2*>(cell + CELL_DATA + g * 8);
    const uint2 sb = *reinterpret_cast<const uint2*>(cell + CELL_DATA + (g + 8) * 8);
    it.s[0] = sa.x;  // Int8: (min, max) of row g; NF4: absmax of blocks 0, 1
    it.s[1] = sa.y;  //                            NF4: absmax of blocks 2, 3
    it.s[2] = sb.x;  // same for row g + 8
    it.s[3] = sb.y;
    return it;
}

// Sum over the CTA.  One barrier: the caller alternates between two scratch arrays, so the readers of one
// use are past a barrier before the array is written again.
__device__ __forceinline__ float block_sum_256(float v, float* scratch) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) s += scratch[w];
    return s;
}

// Layer norm of a.ln_x rows (+ token shift) into xgen[v][t][c] (fp16, pitch xp).
// Each thread owns kLnVec groups of 8 channels (C <= 8 * kThreads * kLnVec) through both passes.  The
// per-channel parameters were copied into shared memory before the grid dependency was awaited
// (stage_prologue_params): the norm weight sits in row 0 of lnrow, the bias in pbias, the shift factors in
// row 0 of each xgen region.  Rows are produced last token first, so every parameter row is consumed by its
// owner thread before that thread overwrites it with row 0's result.
constexpr int kLnVec = 2;  // groups of 8 channels per thread: C <= 8192
template <int PRO>
__device__ __forceinline__ void stage_prologue_params(const FusedGemvArgs& a, __half* xgen, uint32_t xp, __half* lnrow,
                                                      __half* pbias) {
    const uint32_t ngrp = a.C / 8;
    constexpr int nv = PRO == PRO_LN ? 0 : PRO == PRO_LN_SHIFT2 ? 2 : 1;
#pragma unroll
    for (int q = 0; q < kLnVec; ++q) {
        const uint32_t gi = threadIdx.x + q * kThreads;
        if (gi < ngrp) {
            cp_async16z(lnrow + gi * 8, a.ln_w + gi * 8, true);
            cp_async16z(pbias + gi * 8, a.ln_b + gi * 8, true);
            for (int vi = 0; vi < nv; ++vi)
                cp_async16z(xgen + (size_t)vi * a.T * xp + gi * 8, (vi == 0 ? a.mix0 : a.mix1) + gi * 8, true);
        }
    }
}

template <int PRO>
__device__ void run_prologue(const FusedGemvArgs& a, __half* xgen, uint32_t xp, __half* lnrow, const __half* pbias,
                             float* scratch) {
    const uint32_t C = a.C, T = a.T;
    const uint32_t ngrp = C / 8;  // 16-byte groups per row
    constexpr bool shift = PRO != PRO_LN;
    // decode (T == 1): the carry row of the token shift goes in flight together with the input row
    const bool early = shift && T == 1;
    float prev1[kLnVec][8];
    CursorD cu0 = CursorD{0, 0, 1};
    if (early) cu0 = cursor_at(a.cursors, a.wide, 0);
    for (int t = (int)T - 1; t >= 0; --t) {
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
        if (early) {
#pragma unroll
            for (int q = 0; q < kLnVec; ++q) {
                const uint32_t gi = threadIdx.x + q * kThreads;
                if (gi < ngrp)
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        prev1[q][e] = static_cast<const float*>(a.state.base)[a.state.index(gi * 8 + e, 0, cu0.batch)];
            }
        }
        const float mean = block_sum_256(s, scratch) / (float)C;  // scratch: [2][kWarps]
        float m2 = 0.f;
#pragma unroll
        for (int q = 0; q < kLnVec; ++q)
            if (threadIdx.x + q * kThreads < ngrp)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float d = v[q][e] - mean;
                    m2 += d * d;
                }
        const float dev = rsqrtf(block_sum_256(m2, scratch + kWarps) / (float)C + a.ln_eps);
#pragma unroll
        for (int q = 0; q < kLnVec; ++q) {
            const uint32_t gi = threadIdx.x + q * kThreads;
            if (gi < ngrp) {
                const uint4 wraw = *reinterpret_cast<const uint4*>(lnrow + gi * 8);
                const uint4 braw = *reinterpret_cast<const uint4*>(pbias + gi * 8);
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
    if (shift) {
        constexpr int nv = PRO == PRO_LN_SHIFT2 ? 2 : 1;
        for (int t = (int)T - 1; t >= 0; --t) {
            const CursorD cu = early ? cu0 : cursor_at(a.cursors, a.wide, (uint32_t)t);
#pragma unroll
            for (int q = 0; q < kLnVec; ++q) {
                const uint32_t gi = threadIdx.x + q * kThreads;
                if (gi >= ngrp) continue;
                const uint4 craw = *reinterpret_cast<const uint4*>(lnrow + (size_t)t * xp + gi * 8);
                const __half* ch = reinterpret_cast<const __half*>(&craw);
                float prev[8];
                if (early) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) prev[e] = prev1[q][e];
                } else if ((uint32_t)t == cu.token) {
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        prev[e] = static_cast<const float*>(a.state.base)[a.state.index(gi * 8 + e, 0, cu.batch)];
                } else {
                    const uint4 praw = *reinterpret_cast<const uint4*>(lnrow + (size_t)(t - 1) * xp + gi * 8);
                    const __half* ph = reinterpret_cast<const __half*>(&praw);
#pragma unroll
                    for (int e = 0; e < 8; ++e) prev[e] = __half2float(ph[e]);
                }
                for (int vi = 0; vi < nv; ++vi) {
                    __half* region = xgen + (size_t)vi * T * xp;
                    const uint4 fraw = *reinterpret_cast<const uint4*>(region + gi * 8);  // shift factors (row 0)
                    const __half* fh = reinterpret_cast<const __half*>(&fraw);
                    uint4 outv;
                    __half* oh = reinterpret_cast<__half*>(&outv);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float cur = __half2float(ch[e]), f = __half2float(fh[e]);
                        const float lhs = a.reversed ? cur : prev[e], rhs = a.reversed ? prev[e] : cur;
                        oh[e] = __float2half_rn(lhs * (1.0f - f) + rhs * f);
                    }
                    *reinterpret_cast<uint4*>(region + (size_t)t * xp + gi * 8) = outv;
                }
            }
        }
    }
    __syncthreads();
}

// Operands of the launch's epilogue for one output, fetched before the weights are multiplied so that
// their memory round trip overlaps the main loop.
struct EpiOperands {
    float xres, r, cmx;
    CursorD cu;
};
template <int EPI>
__device__ __forceinline__ EpiOperands epilogue_fetch(const FusedGemvArgs& a, const GemvProblem& p, uint32_t m, int tok) {
    EpiOperands e;
    e.xres = e.r = e.cmx = 0.f;
    e.cu = CursorD{0, 0, 1};
    if (EPI == EPI_STORE) return e;
    const size_t oi = (size_t)tok * p.M + m;
    e.xres = __half2float(a.xres[oi]);
    if (EPI == EPI_CHANNEL_MIX) {
        e.cu = cursor_at(a.cursors, a.wide, tok);
        e.cmx = __half2float(a.cm_x[oi]);
        if (a.cm_r != nullptr) e.r = __half2float(a.cm_r[oi]);
    }
    return e;
}

// Activation + the launch's epilogue for output (token tok, row m) of problem p.
template <int EPI>
__device__ __forceinline__ void epilogue_one(const FusedGemvArgs& a, const GemvProblem& p, uint32_t m, int tok, float s,
                                             const EpiOperands& e) {
    s = activate_f(p.act, s);
    const size_t oi = (size_t)tok * p.M + m;
    if (EPI == EPI_STORE) {
        dstore(p.out, p.out_dtype, (size_t)tok * p.out_stride + m, s);
    } else if (EPI == EPI_RESIDUAL) {
        // att_o is an fp16 tensor in the reference; x += att_o is rounded to fp16 again
        const float o16 = __half2float(__float2half_rn(s));
        a.xres[oi] = __float2half_rn(a.rescale * __half2float(__float2half_rn(e.xres + o16)));
    } else {
        // channel mix: carry row <- normalised ffn input at a sequence's last token;
        // x += sigmoid(r) * v with the reference's fp16 rounding points
        if ((uint32_t)tok - e.cu.token + 1u == e.cu.len)
            static_cast<float*>(a.cm_state.base)[a.cm_state.index(m, 0, e.cu.batch)] = e.cmx;
        const float v16 = __half2float(__float2half_rn(s));
        float mixed = v16;
        if (a.cm_r != nullptr) {
            const float rr = 1.0f / (1.0f + expf(-e.r));
            mixed = rr * v16;
        }
        const float o16 = __half2float(__float2half_rn(mixed));
        const __half sum16 = __float2half_rn(e.xres + o16);
        a.xres[oi] = a.rescale == 1.0f ? sum16 : __float2half_rn(a.rescale * __half2float(sum16));
    }
}

// Multiplies one work item with the staged activations: out[0..3] = rows g / g + 8 x tokens 2 t4 / 2 t4 + 1.
// The four k-steps of an Int8 item go to four independent accumulators (chains of two MMAs).
__device__ __forceinline__ void consume_item(const GemvProblem& p, const Item& it, int c, const __half* xrow, bool xval,
                                             const float* sums, uint32_t T, int t4, const uint32_t* lut2, float out[4]) {
    if (p.kind == MAT_INT8) {
        const uint32_t wa[8] = {it.q[0].x, it.q[0].y, it.q[0].z, it.q[0].w, it.q[1].x, it.q[1].y, it.q[1].z, it.q[1].w};
        const uint32_t wb[8] = {it.q[2].x, it.q[2].y, it.q[2].z, it.q[2].w, it.q[3].x, it.q[3].y, it.q[3].z, it.q[3].w};
        float d[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) d[i][0] = d[i][1] = d[i][2] = d[i][3] = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < 4; ++s2) {
            const uint32_t kk = c * 128 + (s2 < 2 ? 16 * t4 + 8 * s2 : 64 + 16 * t4 + 8 * (s2 - 2));
            uint4 xq = make_uint4(0, 0, 0, 0);
            if (xval) xq = *reinterpret_cast<const uint4*>(xrow + kk);
            // bytes enter as 1024 + q (0x6400 | q): exact in fp16; the offset leaves through the block's sum of x
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t ua = wa[2 * s2 + h], ub = wb[2 * s2 + h];
                mma16816(d[s2], __byte_perm(ua, 0x64646464u, 0x4140), __byte_perm(ub, 0x64646464u, 0x4140),
                         __byte_perm(ua, 0x64646464u, 0x4342), __byte_perm(ub, 0x64646464u, 0x4342), h == 0 ? xq.x : xq.z,
                         h == 0 ? xq.y : xq.w);
            }
        }
        const float2 mmA = __half22float2(*reinterpret_cast<const __half2*>(&it.s[0]));
        const float2 mmB = __half22float2(*reinterpret_cast<const __half2*>(&it.s[2]));
        const uint32_t nblk = p.K / 128;
        const uint32_t tk0 = 2 * t4, tk1 = tk0 + 1;
        const float s0 = tk0 < T ? sums[tk0 * nblk + c] : 0.f, s1 = tk1 < T ? sums[tk1 * nblk + c] : 0.f;
        const float sA = (mmA.y - mmA.x) * (1.0f / 255.0f), sB = (mmB.y - mmB.x) * (1.0f / 255.0f);
        const float oA = mmA.x - 1024.0f * sA, oB = mmB.x - 1024.0f * sB;
        out[0] = sA * ((d[0][0] + d[1][0]) + (d[2][0] + d[3][0])) + oA * s0;
        out[1] = sA * ((d[0][1] + d[1][1]) + (d[2][1] + d[3][1])) + oA * s1;
        out[2] = sB * ((d[0][2] + d[1][2]) + (d[2][2] + d[3][2])) + oB * s0;
        out[3] = sB * ((d[0][3] + d[1][3]) + (d[2][3] + d[3][3])) + oB * s1;
    } else if (p.kind == MAT_NF4) {
        const uint32_t qa[8] = {it.q[0].x, it.q[0].y, it.q[0].z, it.q[0].w, it.q[1].x, it.q[1].y, it.q[1].z, it.q[1].w};
        const uint32_t qb[8] = {it.q[2].x, it.q[2].y, it.q[2].z, it.q[2].w, it.q[3].x, it.q[3].y, it.q[3].z, it.q[3].w};
        out[0] = out[1] = out[2] = out[3] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // four absmax blocks of 64 weights
            const __half2 sa2 = *reinterpret_cast<const __half2*>(&it.s[j >> 1]);
            const __half2 sb2 = *reinterpret_cast<const __half2*>(&it.s[2 + (j >> 1)]);
            const float aA = __half2float((j & 1) ? __high2half(sa2) : __low2half(sa2));
            const float aB = __half2float((j & 1) ? __high2half(sb2) : __low2half(sb2));
            float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2) {
                uint4 xq = make_uint4(0, 0, 0, 0);
                if (xval && (uint32_t)(c * 256 + j * 64) < p.K)
                    xq = *reinterpret_cast<const uint4*>(xrow + c * 256 + j * 64 + 16 * t4 + 8 * s2);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    // a byte holds two consecutive weights: one lookup gives both as a half2
                    const uint32_t ua = qa[2 * j + s2] >> (16 * h), ub = qb[2 * j + s2] >> (16 * h);
                    mma16816(d, lut2[ua & 0xffu], lut2[ub & 0xffu], lut2[(ua >> 8) & 0xffu], lut2[(ub >> 8) & 0xffu],
                             h == 0 ? xq.x : xq.z, h == 0 ? xq.y : xq.w);
                }
            }
            out[0] = fmaf(d[0], aA, out[0]);
            out[1] = fmaf(d[1], aA, out[1]);
            out[2] = fmaf(d[2], aB, out[2]);
            out[3] = fmaf(d[3], aB, out[3]);
        }
    } else {
        // 64 fp16 weights per row: two 16-byte pieces per lane and row, independent accumulators
        float d[2][4];
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
            d[hlf][0] = d[hlf][1] = d[hlf][2] = d[hlf][3] = 0.f;
            const uint4 wa = it.q[hlf], wb = it.q[2 + hlf];
            uint4 xq = make_uint4(0, 0, 0, 0);
            if (xval && (uint32_t)(c * 64 + hlf * 32) < p.K)
                xq = *reinterpret_cast<const uint4*>(xrow + c * 64 + hlf * 32 + 8 * t4);
            mma16816(d[hlf], wa.x, wb.x, wa.y, wb.y, xq.x, xq.y);
            mma16816(d[hlf], wa.z, wb.z, wa.w, wb.w, xq.z, xq.w);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) out[e] = d[0][e] + d[1][e];
    }
}

// One CTA per SM: the kernel then has 128 registers per thread (under a 64-register cap it spills inside the
// item loop) and room for a deep ring; measured, that is worth far more than letting the next launch's CTAs
// become resident early to prefetch (727 -> 932 tokens/s on the 1.6B-shaped bench model).
#ifndef WRK_GEMV_MIN_CTAS
#define WRK_GEMV_MIN_CTAS 1
#endif
template <int PRO, int EPI>
__global__ void __launch_bounds__(kThreads, WRK_GEMV_MIN_CTAS) fused_gemv_kernel(const FusedGemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float scratch[2 * kWarps];
    __shared__ uint32_t lut2[256];  // NF4: byte -> half2(table[low nibble], table[high nibble])

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const uint32_t T = a.T;
    const int depth = a.ring_depth;

    // shared memory carve-up (all offsets multiples of 16 bytes)
    const uint32_t xp = (PRO != PRO_NONE ? a.C : a.kmax) + 8;            // halfs per activation row
    uint8_t* ring = smem + (size_t)warp * depth * CELL_BYTES;            // this warp's staging cells
    float* part = reinterpret_cast<float*>(smem + (size_t)kWarps * depth * CELL_BYTES);  // [kWarps][GROUP_ROWS * T] partial results
    float* sums = part + kWarps * GROUP_ROWS * T;                        // [T][kmax / 128]
    __half* xs = reinterpret_cast<__half*>(sums + sums_floats(T, a.kmax));  // staged x or prologue rows
    __half* lnrow = xs;                                                  // PRO_LN: vectors = normalised rows
    __half* xgen = PRO == PRO_LN ? xs : xs + (size_t)T * xp;             // shifted vectors follow the rows
    const uint32_t pro_rows = PRO == PRO_LN ? T : PRO == PRO_LN_SHIFT1 ? 2 * T : 3 * T;
    __half* pbias = xs + (size_t)pro_rows * xp;                          // layer-norm bias (prologues only)

    if (threadIdx.x < 256 && a.table != nullptr) {
        const __half2 v = __floats2half2_rn(a.table[threadIdx.x & 15], a.table[threadIdx.x >> 4]);
        lut2[threadIdx.x] = *reinterpret_cast<const uint32_t*>(&v);
    }
    pdl_launch_dependents();

    // ---- everything up to the wait touches only weights: each warp fetches its first items ----
    Segs sg;
    if (a.inline_partition) {
        // this CTA's slice of the concatenated row space, cut at the matrices' boundaries
        const uint32_t g0 = a.cta_row_start[blockIdx.x], g1 = a.cta_row_start[blockIdx.x + 1];
#pragma unroll
        for (int i = 0; i < kSegmentsPerCta; ++i) sg.prob[i] = 0, sg.r0[i] = 0, sg.r1[i] = 0;
        uint32_t base = 0;
        int n = 0;
#pragma unroll
        for (int pi = 0; pi < kMaxProblems; ++pi) {
            if (pi < a.num_problems) {
                const uint32_t lo = max(g0, base), hi = min(g1, base + a.p[pi].M);
                if (lo < hi) {
                    if (n == 0) sg.prob[0] = pi, sg.r0[0] = (int)(lo - base), sg.r1[0] = (int)(hi - base);
                    else if (n == 1) sg.prob[1] = pi, sg.r0[1] = (int)(lo - base), sg.r1[1] = (int)(hi - base);
                    else if (n == 2) sg.prob[2] = pi, sg.r0[2] = (int)(lo - base), sg.r1[2] = (int)(hi - base);
                    ++n;
                }
                base += a.p[pi].M;
            }
        }
    } else {
        const int4* tab = reinterpret_cast<const int4*>(a.segments + (size_t)blockIdx.x * kSegmentsPerCta);
#pragma unroll
        for (int i = 0; i < kSegmentsPerCta; ++i) {
            const int4 e = __ldg(tab + i);
            sg.prob[i] = e.x;
            sg.r0[i] = e.y;
            sg.r1[i] = e.z;
        }
    }
    const bool any_work = sg.r0[0] < sg.r1[0] || sg.r0[1] < sg.r1[1] || sg.r0[2] < sg.r1[2];
    const bool pro = PRO != PRO_NONE && (any_work || blockIdx.x == 0);
    if (PRO != PRO_NONE) {
        if (pro) stage_prologue_params<PRO>(a, xgen, xp, lnrow, pbias);
        cp_async_commit();
    }
    Loader ld;
    ld.seg = 0;
    ld.enter(a, sg, warp, lane);
    int cs_slot = 0;
#pragma unroll 1
    for (int d = 0; d < depth; ++d) {
        ld.issue(a, sg, ring + d * CELL_BYTES, warp, lane);
        cp_async_commit();  // one group per cell, empty or not
    }
    pdl_wait();

    if (PRO != PRO_NONE && pro) {
        cp_async_wait_dyn(depth);  // this thread's parameter copies (it is their only reader)
        run_prologue<PRO>(a, xgen, xp, lnrow, pbias, scratch);
    }

    int staged_problem = -1;
    const int last_seg = sg.r0[2] < sg.r1[2] ? 2 : sg.r0[1] < sg.r1[1] ? 1 : 0;
#pragma unroll 1
    for (int seg = 0; seg < kSegmentsPerCta; ++seg) {
        const int r0 = sg.R0(seg), r1 = sg.R1(seg);
        if (r0 >= r1) continue;
        const int problem = sg.P(seg);
        const GemvProblem& p = a.p[problem];
        const __half* xv = p.x == nullptr ? xgen + (size_t)p.x_sel * T * xp : xs;
        if (staged_problem != problem) {
            // stage x (explicit inputs) and the per-128-block sums of the values the MMA will see:
            // 16 consecutive lanes cover one block of 128, so the sums come from the registers in flight
            __syncthreads();
            if (p.x != nullptr) {
                const uint32_t groups = p.K / 8, total = T * groups;
                // four 16-byte loads per thread go in flight before any of them is used
                for (uint32_t i0 = 0; i0 < total; i0 += 4 * kThreads) {
                    uint4 raw[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t i = i0 + u * kThreads + threadIdx.x;
                        raw[u] = make_uint4(0, 0, 0, 0);
                        if (i < total) {
                            const uint32_t tok = i / groups, k8 = i - tok * groups;
                            raw[u] = *reinterpret_cast<const uint4*>(p.x + (size_t)tok * p.x_stride + k8 * 8);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t i = i0 + u * kThreads + threadIdx.x;
                        if (i0 + u * kThreads >= total) break;  // uniform across the CTA
                        float sum = 0.f;
                        uint32_t tok = 0, k8 = 0;
                        if (i < total) {
                            tok = i / groups;
                            k8 = i - tok * groups;
                            *reinterpret_cast<uint4*>(xs + (size_t)tok * xp + k8 * 8) = raw[u];
                            const __half2* h = reinterpret_cast<const __half2*>(&raw[u]);
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
                }
            } else if (p.kind == MAT_INT8) {
                const uint32_t nblk = p.K / 128;
                for (uint32_t u = warp; u < T * nblk; u += kWarps) {
                    const uint32_t tok = u / nblk, blk = u - tok * nblk;
                    const uint2 raw = *reinterpret_cast<const uint2*>(xv + (size_t)tok * xp + blk * 128 + lane * 4);
                    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    const float s = warp_sum((lo.x + lo.y) + (hi.x + hi.y));
                    if (lane == 0) sums[tok * nblk + blk] = s;
                }
            }
            __syncthreads();
            staged_problem = problem;
        }
        const bool xval = (uint32_t)g < T;
        const __half* xrow = xv + (size_t)(xval ? g : 0) * xp;
        const int nchunk = (int)((row_bytes(p) + CHUNK_BYTES - 1) / CHUNK_BYTES);

#pragma unroll 1
        for (int group0 = r0; group0 < r1; group0 += GROUP_ROWS) {
            const int gn = min(GROUP_ROWS, r1 - group0);
            // the group's outputs belong to the first gn * T threads; their epilogue operands go in flight now
            const int orow = (int)threadIdx.x / (int)T, otok = (int)threadIdx.x - orow * (int)T;
            const bool has_out = (int)threadIdx.x < gn * (int)T;
            EpiOperands eo;
            if (has_out) eo = epilogue_fetch<EPI>(a, p, (uint32_t)(group0 + orow), otok);

            float* mine = part + (size_t)warp * GROUP_ROWS * T;
#pragma unroll 1
            for (int row0 = group0; row0 < group0 + gn; row0 += 16) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
                for (int c = warp; c < nchunk; c += kWarps) {
                    cp_async_wait_dyn(depth - 1);  // this lane's copies of the oldest item in flight have landed
                    __syncwarp();                  // ... and so have the other lanes' (the rows' block scales)
                    uint8_t* cell = ring + cs_slot * CELL_BYTES;
                    const Item it = read_item(cell, lane);
                    __syncwarp();  // every lane has read the cell: refill it with the item `depth` steps ahead
                    ld.issue(a, sg, cell, warp, lane);
                    cp_async_commit();
                    if (++cs_slot == depth) cs_slot = 0;
                    float out[4];
                    consume_item(p, it, c, xrow, xval, sums, T, t4, lut2, out);
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[e] += out[e];
                }
                // this warp's partial results of the tile's 16 rows
                const uint32_t tk0 = 2 * t4, tk1 = tk0 + 1;
                float* dst = mine + (size_t)(row0 - group0) * T;
                if (tk0 < T) {
                    dst[g * T + tk0] = acc[0];
                    dst[(g + 8) * T + tk0] = acc[2];
                }
                if (tk1 < T) {
                    dst[g * T + tk1] = acc[1];
                    dst[(g + 8) * T + tk1] = acc[3];
                }
            }
            __syncthreads();
            // the 16 warps' partial results are summed in warp order (deterministic)
            if (has_out) {
                const float* src = part + threadIdx.x;
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) s += src[(size_t)w * GROUP_ROWS * T];
                epilogue_one<EPI>(a, p, (uint32_t)(group0 + orow), otok, s, eo);
            }
            if (group0 + GROUP_ROWS < r1 || seg < last_seg) __syncthreads();  // the slabs are written again
        }
    }
}


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
    float mu = 0.f;
    if (active) {
        const uint4* wp = reinterpret_cast<const uint4*>(a.w2 + ((size_t)i * C + c) * D);
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j)
            if (j < D / 8) wreg[j] = wp[j];
        mu = __half2float(a.mix[(size_t)i * C + c]);
    }
    pdl_wait();
    // every input of token 0 goes in flight before the first barrier: one memory round trip, not four
    for (uint32_t j = threadIdx.x; j < T * 5 * D; j += blockDim.x) s_tmx[j] = a.tmx[j];
    const CursorD cu0 = cursor_at(a.cursors, a.wide, 0);
    const float cur0 = active ? __half2float(a.att_x[c]) : 0.f;
    const float prev0 = (active && cu0.token == 0) ? static_cast<const float*>(a.state.base)[a.state.index(c, 0, cu0.batch)] : 0.f;
    __syncthreads();
    if (!active) return;
    for (uint32_t t = 0; t < T; ++t) {
        float acc = 0.f;
        const __half* xv = s_tmx + (size_t)t * 5 * D + i * D;
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            if (j >= D / 8) break;
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
        float cur, prev;
        if (t == 0) {
            cur = cur0;
            prev = prev0;
        } else {
            const CursorD cu = cursor_at(a.cursors, a.wide, t);
            cur = __half2float(a.att_x[(size_t)t * C + c]);
            prev = (t == cu.token) ? static_cast<const float*>(a.state.base)[a.state.index(c, 0, cu.batch)]
                                   : __half2float(a.att_x[(size_t)(t - 1) * C + c]);
        }
        a.sx[((size_t)i * T + t) * C + c] = __float2half_rn(cur * (1.0f - f) + prev * f);
    }
}

// ---- v5 / v6 time-mix block: decay adapter, WKV, group norm, gate --------------------------------
// One CTA per (head, batch slot), 4 * S threads: thread (q, j) owns rows [q S/4, (q+1) S/4) of state column j,
// a quarter of the decay-adapter dot product of channel j and a quarter of output j's sum.
template <int S>
__global__ void __launch_bounds__(4 * S) wkv56_fused_kernel(const Wkv6Args a) {
    constexpr int Q = 4, SI = S / Q;
    __shared__ float sk[S], sr[S], sw[S], su[S], part[Q][S], red[Q * S / 32];
    __shared__ __half s_tdw[128];
    __shared__ uint32_t s_start, s_count;
    pdl_launch_dependents();
    const uint32_t h = blockIdx.x, slot = blockIdx.y, j = threadIdx.x % S, q = threadIdx.x / S;
    const uint32_t C = S * a.H, c = h * S + j;
    const uint32_t dq = a.D / Q;  // adapter inputs per quarter (a multiple of 8, at most 32)

    // the decay-adapter row and the per-channel constants do not depend on this job's kernels...
    uint4 w2reg[4];
    float td_static = 0.f, td5 = 0.f;
    if (a.per_token_decay) {
        const uint4* wp = reinterpret_cast<const uint4*>(a.td_w2 + (size_t)c * a.D + q * dq);
#pragma unroll
        for (uint32_t e = 0; e < 4; ++e)
            if (e < dq / 8) w2reg[e] = wp[e];
        td_static = __half2float(a.td0[c]);
    } else {
        td5 = a.td5[c];
    }
    if (q == 0) su[j] = a.time_first[c];
    const float gw = __half2float(a.gn_w[c]), gb = __half2float(a.gn_b[c]);
    // ...nor do the WKV state rows: within a job only this kernel writes them, and every job begins with
    // launches that are not programmatic dependents, i.e. after the previous job has completed
    float st[SI];
#pragma unroll
    for (int i = 0; i < SI; ++i) st[i] = static_cast<const float*>(a.state.base)[a.state.index(c, 1 + q * SI + i, slot)];
    pdl_wait();  // the token's k, v, r, g and adapter activations come from the kernels before this one

    // run of tokens of this batch slot
    uint32_t start, count;
    if (a.T == 1) {
        start = 0;
        count = cursor_at(a.cursors, a.wide, 0).batch == slot ? 1u : 0u;
    } else {
        if (threadIdx.x == 0) {
            s_start = 0xffffffffu;
            s_count = 0;
        }
        __syncthreads();
        uint32_t mn = 0xffffffffu, cnt = 0;
        for (uint32_t t = threadIdx.x; t < a.T; t += Q * S) {
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
        __syncthreads();
        start = s_start;
        count = s_count;
    }
    if (count == 0) return;

    for (uint32_t n = 0; n < count; ++n) {
        const uint32_t t = start + n;
        const size_t ti = (size_t)t * C + c;
        // all of the token's inputs go in flight together
        const float kj = a.k[ti], rj = a.r[ti], vj = a.v[ti];
        const float gg = __half2float(a.g[ti]), ax = __half2float(a.att_x[ti]);
        __half tdh = __float2half_rn(0.f);
        if (a.per_token_decay && threadIdx.x < a.D) tdh = a.tdw[(size_t)t * a.D + threadIdx.x];
        const CursorD cu = cursor_at(a.cursors, a.wide, t);
        __syncthreads();  // the previous token's readers are done
        if (q == 0) {
            sk[j] = kj;
            sr[j] = rj;
        }
        if (a.per_token_decay && threadIdx.x < a.D) s_tdw[threadIdx.x] = tdh;
        __syncthreads();
        if (a.per_token_decay) {
            float acc = 0.f;
            const __half* xv = s_tdw + q * dq;
#pragma unroll
            for (uint32_t e = 0; e < 4; ++e) {
                if (e >= dq / 8) break;
                const __half2* w2 = reinterpret_cast<const __half2*>(&w2reg[e]);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 wf = __half22float2(w2[u]);
                    acc = fmaf(wf.x, __half2float(xv[e * 8 + 2 * u]), acc);
                    acc = fmaf(wf.y, __half2float(xv[e * 8 + 2 * u + 1]), acc);
                }
            }
            part[q][j] = acc;
            __syncthreads();
            // time_decay buffer is f32: no rounding before the activation
            if (q == 0) sw[j] = expf(-expf(((part[0][j] + part[1][j]) + (part[2][j] + part[3][j])) + td_static));
        } else if (q == 0) {
            sw[j] = td5;
        }
        __syncthreads();
        float y0 = 0.f, y1 = 0.f;
#pragma unroll
        for (int ii = 0; ii < SI; ii += 2) {
            const int i = q * SI + ii;
            float kv;
            kv = sk[i] * vj;     y0 += sr[i] * fmaf(su[i], kv, st[ii]);             st[ii] = fmaf(sw[i], st[ii], kv);
            kv = sk[i + 1] * vj; y1 += sr[i + 1] * fmaf(su[i + 1], kv, st[ii + 1]); st[ii + 1] = fmaf(sw[i + 1], st[ii + 1], kv);
        }
        part[q][j] = y0 + y1;
        if (q == 0 && t - cu.token + 1u == cu.len) static_cast<float*>(a.state.base)[a.state.index(c, 0, slot)] = ax;
        __syncthreads();
        const float y = (part[0][j] + part[1][j]) + (part[2][j] + part[3][j]);
        // group norm over the head's S outputs (f32 buffer in the reference), then fp16, then the gate;
        // every quarter repeats it on the same values, quarter 0 stores
        const uint32_t wbase = q * (S / 32);
        float s = warp_sum(y);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < S / 32; ++w) tot += red[wbase + w];
        const float mean = tot / (float)S;
        const float dlt = y - mean;
        __syncthreads();
        s = warp_sum(dlt * dlt);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
        __syncthreads();
        tot = 0.f;
        for (int w = 0; w < S / 32; ++w) tot += red[wbase + w];
        const float dev = rsqrtf(tot / (float)S + a.gn_eps);
        const float gn16 = __half2float(__float2half_rn(fmaf(dlt * dev, gw, gb)));
        const float silu = gg / (1.0f + expf(-gg));
        if (q == 0) a.out[ti] = __float2half_rn(silu * gn16);
    }
#pragma unroll
    for (int i = 0; i < SI; ++i) static_cast<float*>(a.state.base)[a.state.index(c, 1 + q * SI + i, slot)] = st[i];
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
// weight bytes (a single matrix: a running byte count; several: whole CTAs per matrix).  Returns false when a
// CTA would need more than kSegmentsPerCta ranges.
bool fused_gemv_partition(const FusedGemvArgs& a, int grid, std::vector<GemvSegment>& table) {
    table.assign((size_t)grid * kSegmentsPerCta, GemvSegment{0, 0, 0, 0});
    double total = 0;
    std::vector<double> cost(a.num_problems);
    for (int i = 0; i < a.num_problems; ++i) {
        const GemvProblem& p = a.p[i];
        cost[i] = p.kind == MAT_FP16 ? p.K * 2.0 : p.kind == MAT_INT8 ? p.K * 1.03125 : p.K * 0.53125;
        total += cost[i] * p.M;
    }
    if (a.num_problems > 1 && a.num_problems <= grid) {
        // Several matrices: every matrix gets a whole number of CTAs in proportion to its bytes (largest
        // remainders first, at least one each) and splits its rows evenly among them.  No CTA then crosses a
        // matrix boundary: a crossing CTA re-stages its activations mid-way and ends up with an extra partial
        // tile, which made it finish microseconds after the others.
        std::vector<int> n(a.num_problems, 1);
        std::vector<double> share(a.num_problems);
        int used = a.num_problems;
        for (int i = 0; i < a.num_problems; ++i) {
            share[i] = cost[i] * a.p[i].M / total * grid;
            const int extra = std::max(0, (int)std::floor(share[i]) - 1);
            n[i] += extra;
            used += extra;
        }
        while (used < grid) {  // hand out the remaining CTAs by largest load per CTA
            int best = 0;
            double worst = -1;
            for (int i = 0; i < a.num_problems; ++i) {
                const double load = cost[i] * a.p[i].M / n[i];
                if (load > worst && (uint32_t)n[i] < a.p[i].M) worst = load, best = i;
            }
            ++n[best];
            ++used;
        }
        while (used > grid) {  // more minimum CTAs than the proportional split: take from the lightest loads
            int best = -1;
            double lightest = 1e300;
            for (int i = 0; i < a.num_problems; ++i) {
                const double load = cost[i] * a.p[i].M / n[i];
                if (n[i] > 1 && load < lightest) lightest = load, best = i;
            }
            if (best < 0) break;
            --n[best];
            --used;
        }
        if (used == grid) {
            int c = 0;
            for (int i = 0; i < a.num_problems; ++i)
                for (int j = 0; j < n[i]; ++j, ++c) {
                    const int32_t r0 = (int32_t)((uint64_t)a.p[i].M * j / n[i]), r1 = (int32_t)((uint64_t)a.p[i].M * (j + 1) / n[i]);
                    table[(size_t)c * kSegmentsPerCta] = GemvSegment{i, r0, r1, 0};
                }
            return true;
        }
        table.assign((size_t)grid * kSegmentsPerCta, GemvSegment{0, 0, 0, 0});
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

void fused_gemv_inline_partition(FusedGemvArgs& a, int grid, const std::vector<GemvSegment>& table) {
    a.inline_partition = 0;
    if (grid > kInlineCtas) return;
    uint32_t cur = 0;
    for (int c = 0; c < grid; ++c) {
        a.cta_row_start[c] = cur;
        for (int i = 0; i < kSegmentsPerCta; ++i) {
            const GemvSegment& sg = table[(size_t)c * kSegmentsPerCta + i];
            if (sg.row1 > sg.row0) cur += (uint32_t)(sg.row1 - sg.row0);
        }
    }
    a.cta_row_start[grid] = cur;
    a.inline_partition = 1;
}

size_t fused_gemv_smem(uint32_t T, uint32_t Kmax, uint32_t C, int prologue, int depth) {
    depth = std::min(std::max(depth, kMinRing), kMaxRing);
    const uint32_t xp = (prologue != PRO_NONE ? C : Kmax) + 8;
    size_t bytes = (size_t)kWarps * depth * CELL_BYTES + (size_t)kWarps * GROUP_ROWS * T * sizeof(float);
    bytes += (size_t)sums_floats(T, Kmax) * sizeof(float);
    // activation rows (+ one row of layer-norm bias for the prologues)
    const size_t rows = prologue == PRO_NONE ? T : (prologue == PRO_LN ? T : prologue == PRO_LN_SHIFT1 ? 2 * T : 3 * T) + 1;
    bytes += rows * xp * sizeof(__half);
    return bytes + 64;
}

namespace {

// Dynamic shared memory a launch may ask for (the ring takes what the activations leave).
constexpr size_t kMaxGemvSmem = 200 * 1024;

// Fills the launch-derived fields (largest K, ring depth) and returns the dynamic shared memory size.
size_t fused_gemv_prepare(FusedGemvArgs& a) {
    uint32_t kmax = 0;
    for (int i = 0; i < a.num_problems; ++i) kmax = std::max(kmax, a.p[i].K);
    a.kmax = kmax;
    int depth = kMaxRing;
    while (depth > kMinRing && fused_gemv_smem(a.T, kmax, a.C, a.prologue, depth) > kMaxGemvSmem) --depth;
    a.ring_depth = depth;
    return fused_gemv_smem(a.T, kmax, a.C, a.prologue, depth);
}

template <int PRO, int EPI>
cudaError_t launch_fused_gemv(const FusedGemvArgs& a, int grid, size_t smem, cudaStream_t stream, bool pdl) {
    static SmemOptIn opt_in;  // one per instantiation
    if (cudaError_t e = opt_in.ensure(fused_gemv_kernel<PRO, EPI>, 200 * 1024); e != cudaSuccess) return e;
    if (pdl) return launch_pdl(fused_gemv_kernel<PRO, EPI>, dim3(grid), dim3(kThreads), smem, stream, a);
    fused_gemv_kernel<PRO, EPI><<<grid, kThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t dispatch_fused_gemv(const FusedGemvArgs& a, int grid, size_t smem, cudaStream_t stream, bool pdl) {
    if (a.prologue == PRO_NONE) {
        if (a.epilogue == EPI_STORE) return launch_fused_gemv<PRO_NONE, EPI_STORE>(a, grid, smem, stream, pdl);
        if (a.epilogue == EPI_RESIDUAL) return launch_fused_gemv<PRO_NONE, EPI_RESIDUAL>(a, grid, smem, stream, pdl);
        if (a.epilogue == EPI_CHANNEL_MIX) return launch_fused_gemv<PRO_NONE, EPI_CHANNEL_MIX>(a, grid, smem, stream, pdl);
    } else if (a.epilogue == EPI_STORE) {
        if (a.prologue == PRO_LN) return launch_fused_gemv<PRO_LN, EPI_STORE>(a, grid, smem, stream, pdl);
        if (a.prologue == PRO_LN_SHIFT1) return launch_fused_gemv<PRO_LN_SHIFT1, EPI_STORE>(a, grid, smem, stream, pdl);
        if (a.prologue == PRO_LN_SHIFT2) return launch_fused_gemv<PRO_LN_SHIFT2, EPI_STORE>(a, grid, smem, stream, pdl);
    }
    return cudaErrorInvalidValue;  // a prologue with a residual epilogue is not instantiated
}

}  // namespace

cudaError_t fused_gemv(const FusedGemvArgs& a_in, int grid, cudaStream_t stream) {
    FusedGemvArgs a = a_in;
    const size_t smem = fused_gemv_prepare(a);
    return dispatch_fused_gemv(a, grid, smem, stream, true);
}

cudaError_t tmix_shift_v6(const TmixArgs& a, cudaStream_t stream) {
    const uint32_t threads = 5 * a.C;
    const size_t smem = (size_t)a.T * 5 * a.D * sizeof(__half);
    return launch_pdl(tmix_shift_kernel, dim3((threads + 255) / 256), dim3(256), smem, stream, a);
}

cudaError_t wkv56_fused(const Wkv6Args& a, cudaStream_t stream) {
    return launch_pdl(wkv56_fused_kernel<64>, dim3(a.H, a.B), dim3(256), 0, stream, a);
}

// ---- Int8 GEMV with its row-range table in static device memory -------------------------------------
// Same kernel as fused_gemv; the table it reads sits in the array below instead of in a tensor, and a
// one-thread kernel fills it on the caller's stream right before the multiply, so no call allocates.
// Every call on a device uses the same array: calls that overlap in time (two streams, two threads) race.
namespace {

static __device__ __align__(256) GemvSegment g_static_segments[kStaticGemvMaxCtas * kSegmentsPerCta];

// The partition fused_gemv_partition computes for a single matrix, with the same double arithmetic
// (explicitly rounded operations, so no fused multiply-add changes a row split).  Every entry of the
// CTAs' ranges is written, so the array needs no particular contents beforehand.
__global__ void static_partition_kernel(GemvSegment* table, uint32_t K, uint32_t M, int grid) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    const double cost = __dmul_rn((double)K, 1.03125);
    const double total = __dmul_rn(cost, (double)M);
    uint32_t row = 0;
    double done = 0.0;
    for (int c = 0; c < grid; ++c) {
        GemvSegment* e = table + (size_t)c * kSegmentsPerCta;
        for (int i = 0; i < kSegmentsPerCta; ++i) e[i] = GemvSegment{0, 0, 0, 0};
        if (row >= M) continue;
        uint32_t take = M - row;
        if (c != grid - 1) {
            const double target = __ddiv_rn(__dmul_rn(total, (double)(c + 1)), (double)grid);
            const double want = ceil(__dsub_rn(__ddiv_rn(__dsub_rn(target, done), cost), 1e-9));
            take = (uint32_t)fmin((double)take, fmax(0.0, want));
        }
        if (take > 0) {
            e[0] = GemvSegment{0, (int32_t)row, (int32_t)(row + take), 0};
            row += take;
            done = __dadd_rn(done, __dmul_rn((double)take, cost));
        }
    }
}

struct StaticSetup {
    GemvSegment* table = nullptr;
    int sms = 0;
    std::atomic<bool> ready{false};
};
StaticSetup g_static_setup[kStaticGemvMaxDevices];
std::mutex g_static_mutex;

}  // namespace

int gemv_int8_static(int device, cudaStream_t stream, const uint8_t* w, const __half* minmax, const __half* x, float* y,
                     uint32_t K, uint32_t M, uint32_t T, int act, uint32_t num_ctas, cudaError_t* cuda_error) {
    *cuda_error = cudaSuccess;
    if (device < 0 || device >= kStaticGemvMaxDevices) return SG_BAD_DEVICE;
    int current = -1;
    if ((*cuda_error = cudaGetDevice(&current)) != cudaSuccess) return SG_CUDA;
    if (current != device) return SG_BAD_DEVICE;
    StaticSetup& su = g_static_setup[device];
    if (!su.ready.load(std::memory_order_acquire)) {
        // first call on this device: the array's address and the SM count (later calls take no lock)
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!su.ready.load(std::memory_order_relaxed)) {
            void* ptr = nullptr;
            if ((*cuda_error = cudaGetSymbolAddress(&ptr, g_static_segments)) != cudaSuccess) return SG_CUDA;
            if ((*cuda_error = cudaDeviceGetAttribute(&su.sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess)
                return SG_CUDA;
            su.table = static_cast<GemvSegment*>(ptr);
            su.ready.store(true, std::memory_order_release);
        }
    }
    if (K == 0 || M == 0 || K % 128 != 0 || T == 0 || T > (uint32_t)kDecodeMaxTokens || M > 0x7fffffffu) return SG_BAD_SHAPE;
    if (fused_gemv_smem(T, K, K, PRO_NONE, kMinRing) > 200 * 1024) return SG_BAD_SHAPE;
    const int grid = num_ctas == 0 ? su.sms : (int)num_ctas;
    if (num_ctas > (uint32_t)kStaticGemvMaxCtas || grid > kStaticGemvMaxCtas) return SG_TOO_MANY_CTAS;

    FusedGemvArgs a{};
    a.T = T;
    a.C = K;
    a.prologue = PRO_NONE;
    a.epilogue = EPI_STORE;
    a.rescale = 1.0f;
    a.num_problems = 1;
    a.segments = su.table;
    GemvProblem& p = a.p[0];
    p.w = w;
    p.scale = minmax;
    p.kind = MAT_INT8;
    p.K = K;
    p.M = M;
    p.x = x;
    p.x_stride = K;
    p.out = y;
    p.out_stride = M;
    p.out_dtype = WRK_F32;
    p.act = act;
    const size_t smem = fused_gemv_prepare(a);
    static_partition_kernel<<<1, 32, 0, stream>>>(su.table, K, M, grid);
    if ((*cuda_error = cudaGetLastError()) != cudaSuccess) return SG_CUDA;
    // a plain launch: the multiply reads the table at once, so it must not start before the fill kernel ends
    if ((*cuda_error = dispatch_fused_gemv(a, grid, smem, stream, false)) != cudaSuccess) return SG_CUDA;
    return SG_OK;
}

}  // namespace k
}  // namespace wrk
