// The whole decode step of a v5 / v6 job (a few tokens) in one persistent kernel.
//
// One CTA per SM, launched cooperatively, walks a list of phases: weight-streaming phases (the grouped GEMV of
// decode.cu with its layer-norm / token-shift prologues and residual / channel-mix epilogues), the v6
// data-dependent token shift and the WKV block.  Between phases the CTAs meet at a grid-wide barrier (one
// atomic arrival per CTA, a bounded poll: a wait that gives up writes WRK_ERR_TIMEOUT to the context's status
// word and the CTA leaves the kernel).
//
// Why one kernel: at model widths of 2048-4096 a phase is a few microseconds of HBM time, and a kernel boundary
// costs about as much again (the next kernel's CTAs cannot become resident while this one fills the SM's shared
// memory, so every launch starts with an empty pipeline).  Here a CTA's copy side never stops at a boundary: the
// work list of the CTA (its row range of every weight-streaming phase of the job, kept in shared memory) is
// walked by each warp's loader `depth` items ahead of its math, across phases, because weights do not depend on
// anything the job computes.  While the CTAs wait at a barrier, normalise a vector or run the WKV recurrence,
// the rings fill with the next matrices' rows (about 25 MB over the chip), and the math after the barrier starts
// on data that is already in shared memory.
//
// Phase descriptors are fetched two phases ahead into shared memory with one bulk copy each (completion on an
// mbarrier); what a phase needs from memory that no earlier phase of the job writes (layer-norm parameters,
// adapter rows, the WKV state) is requested before the barrier wait, so that it is in flight while the CTA waits.
#include "decode_step_common.cuh"

#include <cstdlib>

namespace wrk {
namespace k {

namespace {

// The CTA's shared memory as the weight-streaming phases use it.
struct GemvShared {
    uint8_t* ring;   // this warp's cells
    float* part;
    float* sums;
    __half* xs;
    float* scratch;  // [2 * kWarps]
    const uint32_t* lut2;
    int depth;
};

// ---- weight-streaming phase ------------------------------------------------------------------------
// The body of fused_gemv_kernel for one row range, with the loader running over the whole job.  Prologue and
// epilogue are chosen at run time and the row loop exists once per weight format: every phase of every layer
// runs the same few KB of loop code, which therefore stays in the instruction caches from phase to phase (six
// template copies of the loop, one per prologue / epilogue pair, starved the warps of instructions: each phase
// began with a cold loop fetched through a memory system that is busy streaming weights).
// Rows [r0, r1) of one matrix of format KIND against the staged activations: the item loop and, per group of 64
// rows, the sum over the warps and the epilogue.
template <int KIND>
__device__ __noinline__ void stream_rows(const GemvShared sm, const GemvCore& a, const GemvProblem& p, int epi, uint32_t K, int r0,
                                         int r1, const __half* xv, uint32_t xp, StepLoader& ld_io, int& cs_slot_io, int warp, int lane) {
    const int g = lane >> 2, t4 = lane & 3;
    const uint32_t T = a.T;
    const int depth = sm.depth;
    float* part = sm.part;
    const float* sums = sm.sums;
    const bool xval = (uint32_t)g < T;
    const __half* xrow = xv + (size_t)(xval ? g : 0) * xp;
    const uint32_t rb = KIND == MAT_FP16 ? K * 2 : KIND == MAT_INT8 ? K : K / 2;
    const int nchunk = (int)((rb + CHUNK_BYTES - 1) / CHUNK_BYTES);
    uint8_t* ring = sm.ring;
    const uint32_t* lut2 = sm.lut2;
    int cs_slot = cs_slot_io;
    StepLoader ld = ld_io;  // the loader and the ring cursor live in registers through the loop

#pragma unroll 1
    for (int group0 = r0; group0 < r1; group0 += GROUP_ROWS) {
        const int gn = min(GROUP_ROWS, r1 - group0);
        // the group's outputs belong to the first gn * T threads; their epilogue operands go in flight now
        const int orow = (int)threadIdx.x / (int)T, otok = (int)threadIdx.x - orow * (int)T;
        const bool has_out = (int)threadIdx.x < gn * (int)T;
        EpiOperands eo;
        if (has_out) eo = epilogue_fetch_rt(epi, a, p, (uint32_t)(group0 + orow), otok);

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
                ld.issue(cell, warp, lane);
                cp_async_commit();
                if (++cs_slot == depth) cs_slot = 0;
                float out[4];
                consume_item(KIND, K, it, c, xrow, xval, sums, T, t4, lut2, out);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] += out[e];
            }
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
            float total = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) total += src[(size_t)w * GROUP_ROWS * T];
            epilogue_one_rt(epi, a, p, (uint32_t)(group0 + orow), otok, total, eo);
        }
        if (group0 + GROUP_ROWS < r1) __syncthreads();  // the slabs are written again
    }
    cs_slot_io = cs_slot;
    ld_io = ld;
}

// Stages the phase's activations: the layer-norm / token-shift prologue or the explicit input rows, and the
// per-128-block sums of the values an Int8 matrix will be multiplied with.  Returns the rows the matrix reads.
__device__ __noinline__ const __half* stage_activations(const GridSync gs, const GemvShared sm, const GemvCore& a, const StepWork wk,
                                                       bool* alive) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pro_kind = a.prologue;
    const uint32_t T = a.T;
    const uint32_t xp = (pro_kind != PRO_NONE ? a.C : a.kmax) + 8;  // halfs per activation row
    __half* xs = sm.xs;
    __half* lnrow = xs;
    __half* xgen = pro_kind == PRO_LN || pro_kind == PRO_NONE ? xs : xs + (size_t)T * xp;
    const uint32_t pro_rows = pro_kind == PRO_LN ? T : pro_kind == PRO_LN_SHIFT1 ? 2 * T : 3 * T;
    __half* pbias = xs + (size_t)pro_rows * xp;
    float* sums = sm.sums;

    const bool any_work = wk.r0 < wk.r1;
    const bool pro = pro_kind != PRO_NONE && (any_work || blockIdx.x == 0);
    if (pro_kind != PRO_NONE) {
        // parameters of the prologue: in flight while the CTA waits for the previous phase
        if (pro) {
            if (pro_kind == PRO_LN) stage_prologue_params<PRO_LN>(a, xgen, xp, lnrow, pbias);
            else if (pro_kind == PRO_LN_SHIFT1) stage_prologue_params<PRO_LN_SHIFT1>(a, xgen, xp, lnrow, pbias);
            else stage_prologue_params<PRO_LN_SHIFT2>(a, xgen, xp, lnrow, pbias);
        }
        cp_async_commit();
    }
    *alive = gs.wait();
    if (!*alive) return nullptr;
    if (pro) {
        // the parameter group is the newest of this thread: waiting for it waits for the ring's groups too,
        // which were issued before the barrier and have had its whole wait to land
        cp_async_wait<0>();
        if (pro_kind == PRO_LN) run_prologue<PRO_LN>(a, xgen, xp, lnrow, pbias, sm.scratch);
        else if (pro_kind == PRO_LN_SHIFT1) run_prologue<PRO_LN_SHIFT1>(a, xgen, xp, lnrow, pbias, sm.scratch);
        else run_prologue<PRO_LN_SHIFT2>(a, xgen, xp, lnrow, pbias, sm.scratch);
    }
    if (!any_work) return nullptr;

    const GemvProblem& p = a.p[wk.problem];
    const int kind = wk.kind;
    const uint32_t K = wk.K;
    const __half* xv = p.x == nullptr ? xgen + (size_t)p.x_sel * T * xp : xs;
    // stage x (explicit inputs) and the per-128-block sums of the values the MMA will see
    if (p.x != nullptr) {
        const uint32_t groups = K / 8, total = T * groups;
        const __half* px = p.x;
        const uint32_t x_stride = p.x_stride;
        for (uint32_t i0 = 0; i0 < total; i0 += 4 * kThreads) {
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = i0 + u * kThreads + threadIdx.x;
                raw[u] = make_uint4(0, 0, 0, 0);
                if (i < total) {
                    const uint32_t tok = i / groups, k8 = i - tok * groups;
                    raw[u] = *reinterpret_cast<const uint4*>(px + (size_t)tok * x_stride + k8 * 8);
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
                if (kind == MAT_INT8) {
#pragma unroll
                    for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off, 16);
                    if (i < total && (k8 & 15) == 0) sums[tok * (K / 128) + (k8 >> 4)] = sum;
                }
            }
        }
    } else if (kind == MAT_INT8) {
        const uint32_t nblk = K / 128;
        for (uint32_t u = warp; u < T * nblk; u += kWarps) {
            const uint32_t tok = u / nblk, blk = u - tok * nblk;
            const uint2 raw = *reinterpret_cast<const uint2*>(xv + (size_t)tok * xp + blk * 128 + lane * 4);
            const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            const float total = warp_sum((lo.x + lo.y) + (hi.x + hi.y));
            if (lane == 0) sums[tok * nblk + blk] = total;
        }
    }
    __syncthreads();
    return xv;
}

__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const StepArgs s) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float scratch[2 * kWarps];
    __shared__ uint32_t lut2[256];  // NF4: byte -> half2(table[low nibble], table[high nibble])
    __shared__ __align__(16) StepPhase desc[2];
    __shared__ __align__(8) uint64_t desc_bar[2];
    __shared__ __align__(8) uint64_t work_bar;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t T = s.T;
    const int depth = s.ring_depth;
    const uint32_t work_bytes = ((uint32_t)s.num_gemv * (uint32_t)sizeof(StepWork) + 127u) / 128u * 128u;
    StepWork* work = reinterpret_cast<StepWork*>(smem);
    uint8_t* ring0 = smem + work_bytes;
    GemvShared sm;
    sm.ring = ring0 + (size_t)warp * depth * CELL_BYTES;
    sm.part = reinterpret_cast<float*>(ring0 + (size_t)kWarps * depth * CELL_BYTES);
    sm.sums = sm.part + kWarps * GROUP_ROWS * T;
    sm.xs = reinterpret_cast<__half*>(sm.sums + sums_floats(T, s.kmax));
    sm.scratch = scratch;
    sm.lut2 = lut2;
    sm.depth = depth;
    GridSync gs{s.barrier, s.status, s.timeline, &abort_flag, 0};

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&desc_bar[0], 1);
        mbar_init(&desc_bar[1], 1);
        mbar_init(&work_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        if (s.num_gemv > 0) {
            mbar_expect_tx(&work_bar, (uint32_t)s.num_gemv * (uint32_t)sizeof(StepWork));
            bulk_load(work, s.work + (size_t)blockIdx.x * s.num_gemv, (uint32_t)s.num_gemv * (uint32_t)sizeof(StepWork), &work_bar);
        }
        for (int i = 0; i < 2 && i < s.num_phases; ++i) {
            mbar_expect_tx(&desc_bar[i], (uint32_t)sizeof(StepPhase));
            bulk_load(&desc[i], s.phases + i, (uint32_t)sizeof(StepPhase), &desc_bar[i]);
        }
    }
    if (threadIdx.x < 256 && s.table != nullptr) {
        const __half2 v = __floats2half2_rn(s.table[threadIdx.x & 15], s.table[threadIdx.x >> 4]);
        lut2[threadIdx.x] = *reinterpret_cast<const uint32_t*>(&v);
    }
    __syncthreads();

    // the work list, then each warp's first items
    bool alive = true;
    if (s.num_gemv > 0 && threadIdx.x == 0) {
        uint32_t polls = 0;
        while (!mbar_try_wait(&work_bar, 0)) {
            if (++polls >= kStepSpinLimit) {
                abort_flag = 1;
                atomicExch(s.status, (int32_t)WRK_ERR_TIMEOUT);
                break;
            }
        }
    }
    __syncthreads();
    alive = abort_flag == 0;
    if (alive && s.num_gemv > 0)
        for (uint32_t polls = 0; polls < 1024 && !mbar_try_wait(&work_bar, 0); ++polls) {}
    StepLoader ld;
    ld.entry = 0;
    ld.count = alive ? s.num_gemv : 0;
    ld.work = work;
    ld.enter(warp, lane);
    int cs_slot = 0;
#pragma unroll 1
    for (int d = 0; d < depth; ++d) {
        ld.issue(sm.ring + d * CELL_BYTES, warp, lane);
        cp_async_commit();  // one group per cell, empty or not
    }

#pragma unroll 1
    for (int ph = 0; alive && ph < s.num_phases; ++ph) {
        gs.phase = ph;
        // the phase's descriptor has landed: one thread waits (bounded), the others follow it through a barrier
        // and then observe the completed phase of the mbarrier themselves
        if (threadIdx.x == 0) {
            uint32_t polls = 0;
            while (!mbar_try_wait(&desc_bar[ph & 1], (uint32_t)(ph >> 1) & 1u)) {
                if (++polls >= kStepSpinLimit) {
                    abort_flag = 1;
                    atomicExch(s.status, (int32_t)WRK_ERR_TIMEOUT);
                    break;
                }
            }
        }
        __syncthreads();
        if (abort_flag != 0) break;
        for (uint32_t polls = 0; polls < 1024 && !mbar_try_wait(&desc_bar[ph & 1], (uint32_t)(ph >> 1) & 1u); ++polls) {}
        const StepPhase& d = desc[ph & 1];
        if (d.type == PH_GEMV) {
            const GemvCore& a = d.gemv;
            StepWork wk{};
            if (d.gemv_index >= 0) wk = work[d.gemv_index];
            const __half* xv = stage_activations(gs, sm, a, wk, &alive);
            if (alive && xv != nullptr) {
                const GemvProblem& p = a.p[wk.problem];
                const uint32_t xp = (a.prologue != PRO_NONE ? a.C : a.kmax) + 8;
                if (wk.kind == MAT_INT8) stream_rows<MAT_INT8>(sm, a, p, a.epilogue, wk.K, wk.r0, wk.r1, xv, xp, ld, cs_slot, warp, lane);
                else if (wk.kind == MAT_NF4) stream_rows<MAT_NF4>(sm, a, p, a.epilogue, wk.K, wk.r0, wk.r1, xv, xp, ld, cs_slot, warp, lane);
                else stream_rows<MAT_FP16>(sm, a, p, a.epilogue, wk.K, wk.r0, wk.r1, xv, xp, ld, cs_slot, warp, lane);
            }
        } else if (d.type == PH_TMIX) {
            alive = tmix_phase(gs, d.tmix, sm.xs);
        } else {
            alive = wkv_phase(gs, d.wkv, sm.xs);
        }
        if (!alive) break;
        if (ph + 1 < s.num_phases) {
            gs.arrive();
            // desc[ph & 1] is free (every thread is past the phase): fetch the descriptor two phases ahead
            if (threadIdx.x == 0 && ph + 2 < s.num_phases) {
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                mbar_expect_tx(&desc_bar[ph & 1], (uint32_t)sizeof(StepPhase));
                bulk_load(&desc[ph & 1], s.phases + ph + 2, (uint32_t)sizeof(StepPhase), &desc_bar[ph & 1]);
            }
        } else {
            gs.stamp(1);
        }
    }
    cp_async_wait<0>();  // nothing of this CTA is in flight when it leaves
}

// Shared memory outside the ring for a job shape.
size_t step_fixed_smem(const StepArgs& s) {
    const size_t work_bytes = ((size_t)s.num_gemv * sizeof(StepWork) + 127) / 128 * 128;
    return work_bytes + (size_t)kWarps * GROUP_ROWS * s.T * sizeof(float) + (size_t)sums_floats(s.T, s.kmax) * sizeof(float) +
           (size_t)s.x_halfs * sizeof(__half) + 64;
}

constexpr size_t kMaxStepSmem = 224 * 1024;  // dynamic; the kernel's static arrays take about 2.5 KB of the 227 KB a CTA may have

}  // namespace

size_t decode_step_prepare(StepArgs& s, bool any_prologue) {
    // activation rows: a prologue keeps T normalised rows, up to 2 T shifted rows and a row of bias (pitch C + 8);
    // a phase with explicit inputs stages T rows of its K; the token-shift and WKV phases need a few KB
    size_t halfs = (size_t)s.T * (s.kmax + 8);
    if (any_prologue) halfs = std::max(halfs, (size_t)(3 * s.T + 1) * (s.C + 8));
    halfs = std::max<size_t>(halfs, 4096);
    s.x_halfs = (uint32_t)((halfs + 63) / 64 * 64);
    const size_t fixed = step_fixed_smem(s);
    int depth = kMaxRing;
    while (depth >= kMinRing && fixed + (size_t)kWarps * depth * CELL_BYTES > kMaxStepSmem) --depth;
    if (depth < kMinRing) return 0;
    s.ring_depth = depth;
    return fixed + (size_t)kWarps * depth * CELL_BYTES;
}

cudaError_t decode_step(const StepArgs& s, int grid, cudaStream_t stream) {
    static SmemOptIn opt_in;
    if (cudaError_t e = opt_in.ensure(decode_step_kernel, (int)kMaxStepSmem); e != cudaSuccess) return e;
    const size_t smem = step_fixed_smem(s) + (size_t)kWarps * s.ring_depth * CELL_BYTES;
    if (s.ring_depth < kMinRing || s.ring_depth > kMaxRing || smem > kMaxStepSmem) return cudaErrorInvalidValue;
    // the barrier counts arrivals from zero in every launch
    if (cudaError_t e = cudaMemsetAsync(s.barrier, 0, sizeof(uint32_t), stream); e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    // cooperative: the launch fails instead of starting when the CTAs cannot all be resident at once
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_step_kernel, s);
}

}  // namespace k
}  // namespace wrk
