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
#include "gemv_device.cuh"

#include <mutex>

namespace wrk {
namespace k {

namespace {

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
                    consume_item(p.kind, p.K, it, c, xrow, xval, sums, T, t4, lut2, out);
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
