// Device code shared by the weight-streaming kernels: the per-warp staging ring, the MMA item math, the
// layer-norm / token-shift prologue and the residual / channel-mix epilogues.  Included by decode.cu (one launch
// per group of matrices) and decode_step.cu (the whole decode step in one persistent kernel).
#pragma once

#include "decode.cuh"
#include "device.cuh"

// Barrier over the kThreads compute threads of a CTA.  A kernel that carries extra warps outside the compute
// group (a producer warp that never joins) defines it as a named barrier of kThreads threads before including this.
#ifndef WRK_CTA_SYNC
#define WRK_CTA_SYNC() __syncthreads()
#endif

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
struct LoaderCore {
    int row0, r1, c, nchunk;
    int kind;
    uint32_t rb, srow;             // bytes per weight row / per row of the scale table
    const uint8_t* wbase;          // matrix + this lane's byte offset inside a chunk
    const uint8_t* sbase;          // scale table

    // Points the loader at rows [first, last) of a matrix; false when this warp has no chunk of its rows.
    __device__ __forceinline__ bool open(int mat_kind, uint32_t K, const uint8_t* w, const __half* scale, int first, int last,
                                         int warp, int lane) {
        rb = mat_kind == MAT_FP16 ? K * 2 : mat_kind == MAT_INT8 ? K : K / 2;
        nchunk = (int)((rb + CHUNK_BYTES - 1) / CHUNK_BYTES);
        if (warp >= nchunk) return false;
        kind = mat_kind;
        srow = kind == MAT_INT8 ? (K / 128) * 4 : kind == MAT_NF4 ? (K / 64) * 2 : 0;
        wbase = w + (kind == MAT_NF4 ? 8 : 16) * (lane & 3);
        sbase = reinterpret_cast<const uint8_t*>(scale);
        row0 = first;
        r1 = last;
        c = warp;
        return true;
    }
    // Issues the copies of the current item into `cell` and steps to the next one; true when the range is done.
    __device__ __forceinline__ bool copy_and_step(uint8_t* cell, int warp, int lane) {
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
            if (row0 >= r1) return true;
        }
        return false;
    }
};

// The loader of a single launch: walks the CTA's (at most kSegmentsPerCta) row ranges.
struct Loader : LoaderCore {
    int seg;  // seg == kSegmentsPerCta: the CTA's work is exhausted

    __device__ __forceinline__ bool valid() const { return seg < kSegmentsPerCta; }

    // first range at or after `seg` in which this warp has chunks
    __device__ __forceinline__ void enter(const GemvCore& a, const Segs& sg, int warp, int lane) {
        for (; seg < kSegmentsPerCta; ++seg) {
            if (sg.R0(seg) >= sg.R1(seg)) continue;
            const GemvProblem& p = a.p[sg.P(seg)];
            if (open(p.kind, p.K, p.w, p.scale, sg.R0(seg), sg.R1(seg), warp, lane)) return;
        }
    }
    // Issues the copies of the current item into `cell` (nothing when exhausted) and steps to the next one.
    __device__ __forceinline__ void issue(const GemvCore& a, const Segs& sg, uint8_t* cell, int warp, int lane) {
        if (!valid()) return;
        if (copy_and_step(cell, warp, lane)) {
            ++seg;
            enter(a, sg, warp, lane);
        }
    }
};

// The loader of the step kernel: walks the CTA's work list (one row range per weight-streaming phase, in
// shared memory) from the first phase to the last, regardless of which phase the math is in.
struct StepLoader : LoaderCore {
    int entry, count;
    const StepWork* work;

    __device__ __forceinline__ bool valid() const { return entry < count; }
    __device__ __forceinline__ void enter(int warp, int lane) {
        for (; entry < count; ++entry) {
            const StepWork wk = work[entry];
            if (wk.r0 >= wk.r1) continue;
            if (open(wk.kind, wk.K, wk.w, wk.scale, wk.r0, wk.r1, warp, lane)) return;
        }
    }
    __device__ __forceinline__ void issue(uint8_t* cell, int warp, int lane) {
        if (!valid()) return;
        if (copy_and_step(cell, warp, lane)) {
            ++entry;
            enter(warp, lane);
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
    WRK_CTA_SYNC();
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
__device__ __forceinline__ void stage_prologue_params(const GemvCore& a, __half* xgen, uint32_t xp, __half* lnrow,
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
__device__ void run_prologue(const GemvCore& a, __half* xgen, uint32_t xp, __half* lnrow, const __half* pbias,
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
                const uint4 raw = *reinterpret_cast<const uint4*>(a.ln_x + (size_t)(t + a.ln_row_off[t]) * C + gi * 8);
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
    WRK_CTA_SYNC();
}

// Operands of the launch's epilogue for one output, fetched before the weights are multiplied so that
// their memory round trip overlaps the main loop.
struct EpiOperands {
    float xres, r, cmx;
    CursorD cu;
};
template <int EPI>
__device__ __forceinline__ EpiOperands epilogue_fetch(const GemvCore& a, const GemvProblem& p, uint32_t m, int tok) {
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
__device__ __forceinline__ void epilogue_one(const GemvCore& a, const GemvProblem& p, uint32_t m, int tok, float s,
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
__device__ __forceinline__ void consume_item(int kind, uint32_t K, const Item& it, int c, const __half* xrow, bool xval,
                                             const float* sums, uint32_t T, int t4, const uint32_t* lut2, float out[4]) {
    if (kind == MAT_INT8) {
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
        const uint32_t nblk = K / 128;
        const uint32_t tk0 = 2 * t4, tk1 = tk0 + 1;
        const float s0 = tk0 < T ? sums[tk0 * nblk + c] : 0.f, s1 = tk1 < T ? sums[tk1 * nblk + c] : 0.f;
        const float sA = (mmA.y - mmA.x) * (1.0f / 255.0f), sB = (mmB.y - mmB.x) * (1.0f / 255.0f);
        const float oA = mmA.x - 1024.0f * sA, oB = mmB.x - 1024.0f * sB;
        out[0] = sA * ((d[0][0] + d[1][0]) + (d[2][0] + d[3][0])) + oA * s0;
        out[1] = sA * ((d[0][1] + d[1][1]) + (d[2][1] + d[3][1])) + oA * s1;
        out[2] = sB * ((d[0][2] + d[1][2]) + (d[2][2] + d[3][2])) + oB * s0;
        out[3] = sB * ((d[0][3] + d[1][3]) + (d[2][3] + d[3][3])) + oB * s1;
    } else if (kind == MAT_NF4) {
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
                if (xval && (uint32_t)(c * 256 + j * 64) < K)
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
            if (xval && (uint32_t)(c * 64 + hlf * 32) < K)
                xq = *reinterpret_cast<const uint4*>(xrow + c * 64 + hlf * 32 + 8 * t4);
            mma16816(d[hlf], wa.x, wb.x, wa.y, wb.y, xq.x, xq.y);
            mma16816(d[hlf], wa.z, wb.z, wa.w, wb.w, xq.z, xq.w);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) out[e] = d[0][e] + d[1][e];
    }
}

}  // namespace
}  // namespace k
}  // namespace wrk
