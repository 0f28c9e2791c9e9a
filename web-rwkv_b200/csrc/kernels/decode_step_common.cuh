// Shared by the two persistent decode kernels (decode_step.cu: per-warp cp.async rings + mma.sync;
// decode_step_umma.cu: TMA stages + tcgen05): the grid barrier, the mbarrier / bulk-copy helpers and the phases
// that stream no weights (v6 data-dependent token shift, WKV block).
#pragma once

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

// The grid barrier as a CTA sees it (passed by value: a handful of registers).
struct GridSync {
    uint32_t* barrier;
    int32_t* status;
    unsigned long long* timeline;
    volatile int* abort_flag;  // shared memory
    int phase;

    __device__ __forceinline__ void stamp(int which) const {
        if (timeline != nullptr && threadIdx.x == 0)
            timeline[(size_t)(2 * phase + which) * gridDim.x + blockIdx.x] = global_timer();
    }
    // Every CTA has finished the previous phase and its results are visible.  False: the wait gave up.
    __device__ __forceinline__ bool wait() const {
        if (phase > 0) {
            if (threadIdx.x == 0) {
                const uint32_t target = (uint32_t)phase * gridDim.x;
                uint32_t polls = 0;
                while (ld_acquire_gpu(barrier) < target) {
                    if (++polls >= kStepSpinLimit) {
                        *abort_flag = 1;
                        atomicExch(status, (int32_t)WRK_ERR_TIMEOUT);
                        break;
                    }
                }
                __threadfence();
            }
            WRK_CTA_SYNC();
        }
        stamp(0);
        return *abort_flag == 0;
    }
    // This CTA's results of the phase are written: arrive at the barrier.
    __device__ __forceinline__ void arrive() const {
        WRK_CTA_SYNC();
        stamp(1);
        if (threadIdx.x == 0) {
            __threadfence();
            atomicAdd(barrier, 1u);
        }
    }
};

// Epilogue of a weight-streaming phase, chosen at run time.
__device__ __forceinline__ EpiOperands epilogue_fetch_rt(int epi, const GemvCore& a, const GemvProblem& p, uint32_t m, int tok) {
    if (epi == EPI_RESIDUAL) return epilogue_fetch<EPI_RESIDUAL>(a, p, m, tok);
    if (epi == EPI_CHANNEL_MIX) return epilogue_fetch<EPI_CHANNEL_MIX>(a, p, m, tok);
    return epilogue_fetch<EPI_STORE>(a, p, m, tok);
}
__device__ __forceinline__ void epilogue_one_rt(int epi, const GemvCore& a, const GemvProblem& p, uint32_t m, int tok, float sm,
                                                const EpiOperands& e) {
    if (epi == EPI_RESIDUAL) epilogue_one<EPI_RESIDUAL>(a, p, m, tok, sm, e);
    else if (epi == EPI_CHANNEL_MIX) epilogue_one<EPI_CHANNEL_MIX>(a, p, m, tok, sm, e);
    else epilogue_one<EPI_STORE>(a, p, m, tok, sm, e);
}

// ---- v6 data-dependent token shift -------------------------------------------------------------------
// sx[i][t][c] = mix(att_x[t][c], prev[t][c], f16(f16(W2[i][c][:] . tmx[t][i*D:(i+1)*D]) + mix[i][c])); the 5 C
// outputs are spread evenly over the CTAs, one per thread.
__device__ __noinline__ bool tmix_phase(const GridSync gs, const TmixArgs& a, __half* s_tmx /* [T][5 * D] */) {
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
    if (!gs.wait()) return false;
    for (uint32_t j = threadIdx.x; j < T * 5 * D; j += kThreads) s_tmx[j] = a.tmx[j];
    const CursorD cu0 = cursor_at(a.cursors, a.wide, 0);
    const float cur0 = active ? __half2float(a.att_x[c]) : 0.f;
    const float prev0 = (active && cu0.token == 0) ? static_cast<const float*>(a.state.base)[a.state.index(c, 0, cu0.batch)] : 0.f;
    WRK_CTA_SYNC();
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

__device__ __noinline__ bool wkv_phase(const GridSync gs, const Wkv6Args& a, __half* xs) {
    constexpr int S = 64;
    // the sequences of the job's tokens: (slot, first token, count), in token order (cursors are uploaded before
    // the launch; no phase writes them)
    uint32_t* runs = reinterpret_cast<uint32_t*>(xs);           // [3 * kDecodeMaxTokens + 1]
    float* fs = reinterpret_cast<float*>(xs) + 32;               // 8 * S + 8 floats
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
    WRK_CTA_SYNC();
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
    if (!gs.wait()) return false;
    if (!worker) return true;
    for (uint32_t p = first; p < npairs; p += stride) {
        const uint32_t run = p / a.H, h = p % a.H;
        if (p != first) wkv_load(a, h, runs[3 * run], j, q, regs);
        wkv_pair(a, h, runs[3 * run], runs[3 * run + 1], runs[3 * run + 2], regs, fs, s_tdw);
    }
    return true;
}

}  // namespace
}  // namespace k
}  // namespace wrk
