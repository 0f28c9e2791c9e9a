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
#include "gemv_device.cuh"

namespace wrk {
namespace k {

namespace {

constexpr uint32_t kStepSpinLimit = 1u << 21;  // polls before a wait gives up (about a second)

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bar_sync_256() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }

// What a CTA carries from phase to phase.
struct Step {
    const StepArgs& s;
    int phase;
    volatile int* abort_flag;
    // shared memory
    StepWork* work;
    uint8_t* ring;   // this warp's cells
    float* part;
    float* sums;
    __half* xs;
    float* scratch;  // [2 * kWarps]
    const uint32_t* lut2;
    StepLoader ld;
    int cs_slot;
    int warp, lane;

    __device__ __forceinline__ Step(const StepArgs& args) : s(args) {}

    __device__ __forceinline__ void stamp(int which) {
        if (s.timeline != nullptr && threadIdx.x == 0)
            s.timeline[(size_t)(2 * phase + which) * gridDim.x + blockIdx.x] = global_timer();
    }
    // Every CTA has finished the previous phase and its results are visible.  False: the wait gave up.
    __device__ __forceinline__ bool wait_grid() {
        if (phase > 0) {
            if (threadIdx.x == 0) {
                const uint32_t target = (uint32_t)phase * gridDim.x;
                uint32_t polls = 0;
                while (ld_acquire_gpu(s.barrier) < target) {
                    if (++polls >= kStepSpinLimit) {
                        *abort_flag = 1;
                        atomicExch(s.status, (int32_t)WRK_ERR_TIMEOUT);
                        break;
                    }
                }
                __threadfence();
            }
            __syncthreads();
        }
        stamp(0);
        return *abort_flag == 0;
    }
    // This CTA's results of the phase are written: arrive at the barrier.
    __device__ __forceinline__ void arrive_grid() {
        __syncthreads();
        stamp(1);
        if (threadIdx.x == 0) {
            __threadfence();
            atomicAdd(s.barrier, 1u);
        }
    }
};

// ---- weight-streaming phase ------------------------------------------------------------------------
// The body of fused_gemv_kernel for one row range, with the loader running over the whole job.
template <int PRO, int EPI>
__device__ __noinline__ bool gemv_phase(Step& st, const GemvCore& a, const StepWork wk) {
    const int warp = st.warp, lane = st.lane, g = lane >> 2, t4 = lane & 3;
    const uint32_t T = a.T;
    const int depth = st.s.ring_depth;
    const uint32_t xp = (PRO != PRO_NONE ? a.C : a.kmax) + 8;  // halfs per activation row
    __half* xs = st.xs;
    __half* lnrow = xs;
    __half* xgen = PRO == PRO_LN ? xs : xs + (size_t)T * xp;
    const uint32_t pro_rows = PRO == PRO_LN ? T : PRO == PRO_LN_SHIFT1 ? 2 * T : 3 * T;
    __half* pbias = xs + (size_t)pro_rows * xp;
    float* part = st.part;
    float* sums = st.sums;

    const bool any_work = wk.r0 < wk.r1;
    const bool pro = PRO != PRO_NONE && (any_work || blockIdx.x == 0);
    if (PRO != PRO_NONE) {
        // parameters of the prologue: in flight while the CTA waits for the previous phase
        if (pro) stage_prologue_params<PRO>(a, xgen, xp, lnrow, pbias);
        cp_async_commit();
    }
    if (!st.wait_grid()) return false;
    if (PRO != PRO_NONE && pro) {
        // the parameter group is the newest of this thread: waiting for it waits for the ring's groups too,
        // which were issued before the barrier and have had its whole wait to land
        cp_async_wait<0>();
        run_prologue<PRO>(a, xgen, xp, lnrow, pbias, st.scratch);
    }
    if (!any_work) return true;

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
            const float sm = warp_sum((lo.x + lo.y) + (hi.x + hi.y));
            if (lane == 0) sums[tok * nblk + blk] = sm;
        }
    }
    __syncthreads();

    const bool xval = (uint32_t)g < T;
    const __half* xrow = xv + (size_t)(xval ? g : 0) * xp;
    const uint32_t rb = kind == MAT_FP16 ? K * 2 : kind == MAT_INT8 ? K : K / 2;
    const int nchunk = (int)((rb + CHUNK_BYTES - 1) / CHUNK_BYTES);
    const int r0 = wk.r0, r1 = wk.r1;
    uint8_t* ring = st.ring;
    const uint32_t* lut2 = st.lut2;
    int cs_slot = st.cs_slot;
    StepLoader ld = st.ld;  // the loader and the ring cursor live in registers through the loop

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
                ld.issue(cell, warp, lane);
                cp_async_commit();
                if (++cs_slot == depth) cs_slot = 0;
                float out[4];
                consume_item(kind, K, it, c, xrow, xval, sums, T, t4, lut2, out);
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
            float sm = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) sm += src[(size_t)w * GROUP_ROWS * T];
            epilogue_one<EPI>(a, p, (uint32_t)(group0 + orow), otok, sm, eo);
        }
        if (group0 + GROUP_ROWS < r1) __syncthreads();  // the slabs are written again
    }
    st.cs_slot = cs_slot;
    st.ld = ld;
    return true;
}

// ---- v6 data-dependent token shift -------------------------------------------------------------------
// sx[i][t][c] = mix(att_x[t][c], prev[t][c], f16(f16(W2[i][c][:] . tmx[t][i*D:(i+1)*D]) + mix[i][c])); the 5 C
// outputs are spread evenly over the CTAs, one per thread.
__device__ __noinline__ bool tmix_phase(Step& st, const TmixArgs& a) {
    __half* s_tmx = st.xs;  // [T][5 * D]
    const uint32_t C = a.C, D = a.D, T = a.T;
    const uint32_t per = (5 * C + gridDim.x - 1) / gridDim.x;  // at most kThreads (checked by the host)
    const uint32_t o = blockIdx.x * per + threadIdx.x;
    const bool active = threadIdx.x < per && o < 5 * C;
    const uint32_t i = active ? o / C : 0, c = active ? o % C : 0;
    // the adapter weights of this thread do not depend on earlier phases
    uint4 wreg[8];  // D <= 64 halfs
    float mu = 0.f;
    if (active) {
        const uint4* wp = reinterpret_cast<const uint4*>(a.w2 + ((size_t)i * C + c) * D);
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j)
            if (j < D / 8) wreg[j] = wp[j];
        mu = __half2float(a.mix[(size_t)i * C + c]);
    }
    if (!st.wait_grid()) return false;
    for (uint32_t j = threadIdx.x; j < T * 5 * D; j += kThreads) s_tmx[j] = a.tmx[j];
    const CursorD cu0 = cursor_at(a.cursors, a.wide, 0);
    const float cur0 = active ? __half2float(a.att_x[c]) : 0.f;
    const float prev0 = (active && cu0.token == 0) ? static_cast<const float*>(a.state.base)[a.state.index(c, 0, cu0.batch)] : 0.f;
    __syncthreads();
    if (!active) return true;
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
    return true;
}

// ---- v5 / v6 time-mix block: decay adapter, WKV, group norm, gate ------------------------------------------
// A (head, sequence) pair is worked by 4 * S = 256 threads of a CTA: thread (q, j) owns rows [q S/4, (q+1) S/4) of
// state column j, a quarter of the decay-adapter dot product of channel j and a quarter of output j's sum.  Pairs
// are spread over the CTAs (every fourth SM or so at 64 heads), so each state column is fetched by its own SM.
struct WkvStatic {
    uint4 w2reg[4];
    float td_static, td5, u, gw, gb;
    float st[16];
};
__device__ __forceinline__ void wkv_load(const Wkv6Args& a, uint32_t h, uint32_t slot, uint32_t j, uint32_t q, WkvStatic& r) {
    constexpr int S = 64, SI = 16;
    const uint32_t c = h * S + j;
    const uint32_t dq = a.D / 4;
    r.td_static = r.td5 = 0.f;
    if (a.per_token_decay) {
        const uint4* wp = reinterpret_cast<const uint4*>(a.td_w2 + (size_t)c * a.D + q * dq);
#pragma unroll
        for (uint32_t e = 0; e < 4; ++e)
            if (e < dq / 8) r.w2reg[e] = wp[e];
        r.td_static = __half2float(a.td0[c]);
    } else {
        r.td5 = a.td5[c];
    }
    r.u = a.time_first[c];
    r.gw = __half2float(a.gn_w[c]);
    r.gb = __half2float(a.gn_b[c]);
    // within a job only this phase writes the WKV rows of its layer
#pragma unroll
    for (int i = 0; i < SI; ++i) r.st[i] = static_cast<const float*>(a.state.base)[a.state.index(c, 1 + q * SI + i, slot)];
}

__device__ __forceinline__ void wkv_pair(const Wkv6Args& a, uint32_t h, uint32_t slot, uint32_t start, uint32_t count, WkvStatic& r, float* fs,
                         __half* s_tdw) {
    constexpr int S = 64, Q = 4, SI = S / Q;
    float* sk = fs;
    float* sr = fs + S;
    float* sw = fs + 2 * S;
    float* su = fs + 3 * S;
    float* part = fs + 4 * S;     // [Q][S]
    float* red = fs + 8 * S;      // [Q * S / 32]
    const uint32_t j = threadIdx.x % S, q = threadIdx.x / S;
    const uint32_t C = S * a.H, c = h * S + j;
    const uint32_t dq = a.D / Q;
    if (q == 0) su[j] = r.u;
    for (uint32_t n = 0; n < count; ++n) {
        const uint32_t t = start + n;
        const size_t ti = (size_t)t * C + c;
        // all of the token's inputs go in flight together
        const float kj = a.k[ti], rj = a.r[ti], vj = a.v[ti];
        const float gg = __half2float(a.g[ti]), ax = __half2float(a.att_x[ti]);
        __half tdh = __float2half_rn(0.f);
        if (a.per_token_decay && threadIdx.x < a.D) tdh = a.tdw[(size_t)t * a.D + threadIdx.x];
        const CursorD cu = cursor_at(a.cursors, a.wide, t);
        bar_sync_256();  // the previous token's readers are done
        if (q == 0) {
            sk[j] = kj;
            sr[j] = rj;
        }
        if (a.per_token_decay && threadIdx.x < a.D) s_tdw[threadIdx.x] = tdh;
        bar_sync_256();
        if (a.per_token_decay) {
            float acc = 0.f;
            const __half* xv = s_tdw + q * dq;
#pragma unroll
            for (uint32_t e = 0; e < 4; ++e) {
                if (e >= dq / 8) break;
                const __half2* w2 = reinterpret_cast<const __half2*>(&r.w2reg[e]);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 wf = __half22float2(w2[u]);
                    acc = fmaf(wf.x, __half2float(xv[e * 8 + 2 * u]), acc);
                    acc = fmaf(wf.y, __half2float(xv[e * 8 + 2 * u + 1]), acc);
                }
            }
            part[q * S + j] = acc;
            bar_sync_256();
            // time_decay buffer is f32: no rounding before the activation
            if (q == 0)
                sw[j] = expf(-expf(((part[j] + part[S + j]) + (part[2 * S + j] + part[3 * S + j])) + r.td_static));
        } else if (q == 0) {
            sw[j] = r.td5;
        }
        bar_sync_256();
        float y0 = 0.f, y1 = 0.f;
#pragma unroll
        for (int ii = 0; ii < SI; ii += 2) {
            const int i = q * SI + ii;
            float kv;
            kv = sk[i] * vj;     y0 += sr[i] * fmaf(su[i], kv, r.st[ii]);             r.st[ii] = fmaf(sw[i], r.st[ii], kv);
            kv = sk[i + 1] * vj; y1 += sr[i + 1] * fmaf(su[i + 1], kv, r.st[ii + 1]); r.st[ii + 1] = fmaf(sw[i + 1], r.st[ii + 1], kv);
        }
        bar_sync_256();  // the adapter sums in part[] have been read
        part[q * S + j] = y0 + y1;
        if (q == 0 && t - cu.token + 1u == cu.len) static_cast<float*>(a.state.base)[a.state.index(c, 0, slot)] = ax;
        bar_sync_256();
        const float y = (part[j] + part[S + j]) + (part[2 * S + j] + part[3 * S + j]);
        // group norm over the head's S outputs (f32 buffer in the reference), then fp16, then the gate;
        // every quarter repeats it on the same values, quarter 0 stores
        const uint32_t wbase = q * (S / 32);
        float sm = warp_sum(y);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sm;
        bar_sync_256();
        float tot = 0.f;
        for (int w = 0; w < S / 32; ++w) tot += red[wbase + w];
        const float mean = tot / (float)S;
        const float dlt = y - mean;
        bar_sync_256();
        sm = warp_sum(dlt * dlt);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sm;
        bar_sync_256();
        tot = 0.f;
        for (int w = 0; w < S / 32; ++w) tot += red[wbase + w];
        const float dev = rsqrtf(tot / (float)S + a.gn_eps);
        const float gn16 = __half2float(__float2half_rn(fmaf(dlt * dev, r.gw, r.gb)));
        const float silu = gg / (1.0f + expf(-gg));
        if (q == 0) a.out[ti] = __float2half_rn(silu * gn16);
    }
#pragma unroll
    for (int i = 0; i < SI; ++i) static_cast<float*>(a.state.base)[a.state.index(c, 1 + q * SI + i, slot)] = r.st[i];
    bar_sync_256();  // the arrays are reused by the CTA's next pair
}

__device__ __noinline__ bool wkv_phase(Step& st, const Wkv6Args& a) {
    constexpr int S = 64;
    // the sequences of the job's tokens: (slot, first token, count), in token order (cursors are uploaded before
    // the launch; no phase writes them)
    uint32_t* runs = reinterpret_cast<uint32_t*>(st.xs);           // [3 * kDecodeMaxTokens + 1]
    float* fs = reinterpret_cast<float*>(st.xs) + 32;               // 8 * S + 8 floats
    __half* s_tdw = reinterpret_cast<__half*>(fs + 8 * S + 8);      // 128 halfs
    if (threadIdx.x == 0) {
        uint32_t n = 0;
        for (uint32_t t = 0; t < a.T;) {
            const CursorD cu = cursor_at(a.cursors, a.wide, t);
            uint32_t e = t + 1;
            while (e < a.T && cursor_at(a.cursors, a.wide, e).batch == cu.batch) ++e;
            runs[3 * n] = cu.batch;
            runs[3 * n + 1] = t;
            runs[3 * n + 2] = e - t;
            ++n;
            t = e;
        }
        runs[3 * kDecodeMaxTokens] = n;
    }
    __syncthreads();
    const uint32_t npairs = runs[3 * kDecodeMaxTokens] * a.H;
    // pairs are spread over the grid: with fewer pairs than CTAs, pair p sits on CTA floor(p * grid / npairs)
    uint32_t first = 0xffffffffu, stride = gridDim.x;
    if (npairs <= gridDim.x) {
        const uint32_t p = (blockIdx.x * npairs + gridDim.x - 1) / gridDim.x;
        if (p < npairs && p * gridDim.x / npairs == blockIdx.x) first = p;
        stride = npairs;  // one pair at most
    } else {
        first = blockIdx.x;
    }
    const bool worker = threadIdx.x < 4 * S;
    const uint32_t j = threadIdx.x % S, q = (threadIdx.x / S) & 3;
    WkvStatic regs;
    if (worker && first < npairs) wkv_load(a, first % a.H, runs[3 * (first / a.H)], j, q, regs);
    if (!st.wait_grid()) return false;
    if (!worker) return true;
    for (uint32_t p = first; p < npairs; p += stride) {
        const uint32_t run = p / a.H, h = p % a.H;
        if (p != first) wkv_load(a, h, runs[3 * run], j, q, regs);
        wkv_pair(a, h, runs[3 * run], runs[3 * run + 1], runs[3 * run + 2], regs, fs, s_tdw);
    }
    return true;
}

__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const StepArgs s) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float scratch[2 * kWarps];
    __shared__ uint32_t lut2[256];  // NF4: byte -> half2(table[low nibble], table[high nibble])
    __shared__ __align__(16) StepPhase desc[2];
    __shared__ __align__(8) uint64_t desc_bar[2];
    __shared__ __align__(8) uint64_t work_bar;
    __shared__ int abort_flag;

    Step st(s);
    st.warp = threadIdx.x >> 5;
    st.lane = threadIdx.x & 31;
    st.abort_flag = &abort_flag;
    st.phase = 0;
    st.scratch = scratch;
    st.lut2 = lut2;
    const uint32_t T = s.T;
    const int depth = s.ring_depth;
    const uint32_t work_bytes = ((uint32_t)s.num_gemv * (uint32_t)sizeof(StepWork) + 127u) / 128u * 128u;
    st.work = reinterpret_cast<StepWork*>(smem);
    uint8_t* ring0 = smem + work_bytes;
    st.ring = ring0 + (size_t)st.warp * depth * CELL_BYTES;
    st.part = reinterpret_cast<float*>(ring0 + (size_t)kWarps * depth * CELL_BYTES);
    st.sums = st.part + kWarps * GROUP_ROWS * T;
    st.xs = reinterpret_cast<__half*>(st.sums + sums_floats(T, s.kmax));

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&desc_bar[0], 1);
        mbar_init(&desc_bar[1], 1);
        mbar_init(&work_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        if (s.num_gemv > 0) {
            mbar_expect_tx(&work_bar, (uint32_t)s.num_gemv * (uint32_t)sizeof(StepWork));
            bulk_load(st.work, s.work + (size_t)blockIdx.x * s.num_gemv, (uint32_t)s.num_gemv * (uint32_t)sizeof(StepWork), &work_bar);
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
    st.ld.entry = 0;
    st.ld.count = alive ? s.num_gemv : 0;
    st.ld.work = st.work;
    st.ld.enter(st.warp, st.lane);
    st.cs_slot = 0;
#pragma unroll 1
    for (int d = 0; d < depth; ++d) {
        st.ld.issue(st.ring + d * CELL_BYTES, st.warp, st.lane);
        cp_async_commit();  // one group per cell, empty or not
    }

#pragma unroll 1
    for (int ph = 0; alive && ph < s.num_phases; ++ph) {
        st.phase = ph;
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
            if (d.gemv_index >= 0) wk = st.work[d.gemv_index];
            const int pe = a.prologue * 4 + a.epilogue;
            if (pe == PRO_NONE * 4 + EPI_STORE) alive = gemv_phase<PRO_NONE, EPI_STORE>(st, a, wk);
            else if (pe == PRO_NONE * 4 + EPI_RESIDUAL) alive = gemv_phase<PRO_NONE, EPI_RESIDUAL>(st, a, wk);
            else if (pe == PRO_NONE * 4 + EPI_CHANNEL_MIX) alive = gemv_phase<PRO_NONE, EPI_CHANNEL_MIX>(st, a, wk);
            else if (pe == PRO_LN * 4 + EPI_STORE) alive = gemv_phase<PRO_LN, EPI_STORE>(st, a, wk);
            else if (pe == PRO_LN_SHIFT1 * 4 + EPI_STORE) alive = gemv_phase<PRO_LN_SHIFT1, EPI_STORE>(st, a, wk);
            else alive = gemv_phase<PRO_LN_SHIFT2, EPI_STORE>(st, a, wk);
        } else if (d.type == PH_TMIX) {
            alive = tmix_phase(st, d.tmix);
        } else {
            alive = wkv_phase(st, d.wkv);
        }
        if (!alive) break;
        if (ph + 1 < s.num_phases) {
            st.arrive_grid();
            // desc[ph & 1] is free (every thread is past the phase): fetch the descriptor two phases ahead
            if (threadIdx.x == 0 && ph + 2 < s.num_phases) {
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                mbar_expect_tx(&desc_bar[ph & 1], (uint32_t)sizeof(StepPhase));
                bulk_load(&desc[ph & 1], s.phases + ph + 2, (uint32_t)sizeof(StepPhase), &desc_bar[ph & 1]);
            }
        } else {
            st.stamp(1);
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
