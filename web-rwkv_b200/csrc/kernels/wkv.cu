// WKV state recurrences of RWKV v5 / v6 / v7 for sm_100a.
//
// Replaces time_mix_v5.wgsl, time_mix_v6.wgsl and time_mix_v7.wgsl.  The reference runs one
// dispatch with C/4 threads that is serial over every token of the job and round-trips the whole
// S x S state through global memory on each token.  Here one CTA of S threads owns one
// (sequence, head) pair: thread j keeps column j of the head's state (S fp32 values) in registers
// for the sequence's whole run of tokens, the per-token vectors shared by the head (k, r, w, ...)
// are broadcast through double-buffered shared memory (one barrier per token, next token's loads
// issued before the current token's math), and the state touches HBM once on the way in and once
// on the way out.  Sequences are independent, so the grid is (heads, batch slots).
//
// State layout (reference: src/runtime/v6.rs:187-197): f32 view [C, S+1, B]; row 0 = token-shift
// carry, row 1+i = key index i for all heads side by side (column h*S + j = value index j).
#include "device.cuh"

namespace wrk {
namespace k {

namespace {

// Finds the contiguous run of tokens that belongs to batch slot `slot`.  Returns false when the
// slot has no token in this job.  `carry` (when given) receives 1 + the last token of the run whose cursor says it
// ends its sequence's part of the job (t - token + 1 == len), or 0 when there is none: the token whose layer input
// becomes the token-shift carry row.
struct RunScratch {
    uint32_t start, count, carry;
};
__device__ __forceinline__ bool find_run(const uint32_t* cursors, int wide, uint32_t T, uint32_t slot, RunScratch* sh,
                                         uint32_t& start, uint32_t& count, uint32_t* carry = nullptr) {
    if (threadIdx.x == 0) {
        sh->start = 0xffffffffu;
        sh->count = 0;
        sh->carry = 0;
    }
    __syncthreads();
    uint32_t my_min = 0xffffffffu, my_cnt = 0, my_carry = 0;
    for (uint32_t t = threadIdx.x; t < T; t += blockDim.x) {
        const CursorD c = cursor_at(cursors, wide, t);
        if (c.batch == slot) {
            my_min = min(my_min, t);
            ++my_cnt;
            if (t - c.token + 1u == c.len) my_carry = t + 1;
        }
    }
    if (my_cnt) {
        atomicMin(&sh->start, my_min);
        atomicAdd(&sh->count, my_cnt);
        if (my_carry) atomicMax(&sh->carry, my_carry);
    }
    __syncthreads();
    start = sh->start;
    count = sh->count;
    if (carry) *carry = sh->carry;
    return count != 0;
}

// One CTA of (S / 4) (S / CW) threads per (head, batch slot): a thread keeps a 4 x CW tile of the head's S x S state
// in registers for the sequence's whole run of tokens (rows = key index, columns = value index), so every k, r, w
// value it fetches from shared memory feeds CW columns and every v value four rows.  (Measured at S = 64, 64 heads:
// CW = 4, 8 warps: 0.34 us per token; CW = 2, 16 warps: 0.40 us.)  The S / 4 row groups of a column
// group are lanes of ONE warp: a token's output column is summed by shuffles alone, and nothing but the state's own
// recurrence (one fma deep per token) ties a token to the one before it - no barrier, no shared-memory partials.  The
// tokens' k, r, w and v rows reach shared memory a chunk of TC tokens at a time, loaded a chunk ahead into registers
// while the current chunk is computed (one barrier per chunk), so a token's step never waits for global memory.
template <int S, int CW>
__global__ void __launch_bounds__((S / 4) * (S / CW)) time_mix_v56_kernel(const WkvArgs a) {
    constexpr int RG = S / 4, NT = RG * (S / CW), CGW = 32 / RG, TC = S <= 64 ? 16 : 4, PI = (4 * S + NT - 1) / NT;
    static_assert(CW == 2 || CW == 4, "columns per thread");
    static_assert(RG == 8 || RG == 16 || RG == 32, "the row groups of a column group are lanes of one warp");
    enum { IN_K = 0, IN_R = 1, IN_W = 2, IN_V = 3 };
    __shared__ __align__(16) float sin[2][4][TC][S];
    __shared__ RunScratch run;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rg = lane % RG, cg = warp * CGW + lane / RG;  // rows 4 rg .. 4 rg + 3, columns CW cg .. CW cg + CW - 1
    const uint32_t h = blockIdx.x, slot = blockIdx.y, C = a.S * a.H, c0 = h * S;

    uint32_t start, count, carry;
    if (!find_run(a.cursors, a.wide, a.T, slot, &run, start, count, &carry)) return;
    // The token-shift carry row takes the layer input of the run's closing token.  Nothing in this kernel reads that
    // row, so it is written now, before the token's input is overwritten with its output; the token loop below then
    // has no cursor to look at and no branch.
    if (carry != 0) {
        for (uint32_t j = tid; j < S; j += NT)
            static_cast<float*>(a.state.base)[a.state.index(c0 + j, 0, slot)] = dload(a.x, a.dtype, (size_t)(carry - 1) * C + c0 + j);
    }

    float st[4][CW], u[4];  // st[row][column]
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        u[r] = a.time_first[c0 + 4 * rg + r];
#pragma unroll
        for (int cc = 0; cc < CW; ++cc)
            st[r][cc] = static_cast<const float*>(a.state.base)[a.state.index(c0 + CW * cg + cc, 1 + 4 * rg + r, slot)];
    }

    // staging: (tensor, channel) pairs tid, tid + NT, ... of the 4 S pairs; element (token, channel) of chunk `chunk`
    // (zero past the run's end)
    float stage[PI][TC];
    auto load_chunk = [&](uint32_t chunk) {
#pragma unroll
        for (int pi = 0; pi < PI; ++pi) {
            const uint32_t pair = tid + pi * NT, tensor = pair / S, c = c0 + pair % S;
#pragma unroll
            for (int n = 0; n < TC; ++n) {
                const uint32_t m = chunk * TC + n;
                const size_t ti = (size_t)(start + m) * C + c;
                float v = 0.f;
                if (pair < 4 * S && m < count) {
                    if (tensor == IN_K) v = dload(a.k, a.dtype, ti);
                    else if (tensor == IN_R) v = dload(a.r, a.dtype, ti);
                    else if (tensor == IN_W) v = a.per_token_decay ? a.time_decay[ti] : a.time_decay[c];
                    else v = dload(a.v, a.dtype, ti);
                }
                stage[pi][n] = v;
            }
        }
    };
    auto store_chunk = [&](int buf) {
#pragma unroll
        for (int pi = 0; pi < PI; ++pi) {
            const uint32_t pair = tid + pi * NT;
            if (pair < 4 * S) {
#pragma unroll
                for (int n = 0; n < TC; ++n) sin[buf][pair / S][n][pair % S] = stage[pi][n];
            }
        }
    };
    // one token: the tile's share of the four output columns, summed over the row groups; lane rg == 0 stores them
    auto token = [&](int buf, uint32_t n, uint32_t t) {
        const float4 kq = *reinterpret_cast<const float4*>(&sin[buf][IN_K][n][4 * rg]);
        const float4 rq = *reinterpret_cast<const float4*>(&sin[buf][IN_R][n][4 * rg]);
        const float4 wq = *reinterpret_cast<const float4*>(&sin[buf][IN_W][n][4 * rg]);
        const float kr[4] = {kq.x, kq.y, kq.z, kq.w}, rr[4] = {rq.x, rq.y, rq.z, rq.w}, wr[4] = {wq.x, wq.y, wq.z, wq.w};
        float vc[CW], y[CW];
#pragma unroll
        for (int cc = 0; cc < CW; cc += 2) {
            const float2 vq = *reinterpret_cast<const float2*>(&sin[buf][IN_V][n][CW * cg + cc]);
            vc[cc] = vq.x, vc[cc + 1] = vq.y;
            y[cc] = y[cc + 1] = 0.f;
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int cc = 0; cc < CW; ++cc) {
                const float kv = kr[r] * vc[cc];
                y[cc] = fmaf(rr[r], fmaf(u[r], kv, st[r][cc]), y[cc]);
                st[r][cc] = fmaf(wr[r], st[r][cc], kv);
            }
        }
#pragma unroll
        for (int off = 1; off < RG; off <<= 1) {
#pragma unroll
            for (int cc = 0; cc < CW; ++cc) y[cc] += __shfl_xor_sync(0xffffffffu, y[cc], off);
        }
        if (rg == 0) {
            const size_t ti = (size_t)t * C + c0 + CW * cg;
#pragma unroll
            for (int cc = 0; cc < CW; ++cc) dstore(a.x, a.dtype, ti + cc, y[cc]);
        }
    };
    const uint32_t chunks = (count + TC - 1) / TC;
    load_chunk(0);
    store_chunk(0);
    __syncthreads();

    for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
        const int buf = chunk & 1;
        const bool more = chunk + 1 < chunks;
        if (more) load_chunk(chunk + 1);  // in flight while this chunk's tokens are computed
        const uint32_t len = min((uint32_t)TC, count - chunk * TC), t0 = start + chunk * TC;
        if (len == TC) {
#pragma unroll 4
            for (uint32_t n = 0; n < TC; ++n) token(buf, n, t0 + n);
        } else {
            for (uint32_t n = 0; n < len; ++n) token(buf, n, t0 + n);
        }
        if (more) store_chunk(buf ^ 1);  // last read during the previous chunk, before its closing barrier
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int cc = 0; cc < CW; ++cc)
            static_cast<float*>(a.state.base)[a.state.index(c0 + CW * cg + cc, 1 + 4 * rg + r, slot)] = st[r][cc];
}

// ---- v5 / v6 in blocks of 16 tokens ("chunk-parallel") ------------------------------------------------------------
// The recurrence  y_t = r_t . (u k_t v_t^T + S_(t-1)),  S_t = diag(w_t) S_(t-1) + k_t v_t^T  unrolled over a block of
// L = 16 tokens that starts from state S0 (rows i = key index, columns j = value index, per head):
//   y_t   = (r_t Pe_t) S0  +  sum_(s<=t) A[t][s] v_s,      S_end = diag(Pe_L) S0 + sum_s (k_s E_s) v_s^T
//   Pe_t  = prod_(m<t) w_m   (Pe_0 = 1),   E_s = prod_(m>s) w_m,
//   A[t][s] = sum_i r_t[i] k_s[i] prod_(s<m<t) w_m[i]  (s < t),   A[t][t] = sum_i r_t[i] u[i] k_t[i].
// Every product of decays is taken forwards (no division, nothing can overflow; what underflows is a contribution that
// has decayed to nothing).  The work of a block is then three small matrix products - [16 x 64][64 x 64] for the state's
// share of y, [16 x 16][16 x 64] for the block's own tokens and [64 x 16][16 x 64] for the new state - in which no
// element waits for another: 4 x 4 register tiles in fp32 on the CUDA cores, operands from shared memory.  The serial
// kernel above spends about 650 cycles on a token's chain of dependent steps; this one about 130 per token.
// One CTA of 256 threads per (head of 64 channels, batch slot); the state tile of a thread stays in registers from
// block to block; the tokens' rows are staged a block ahead as in the serial kernel.
constexpr int kBlockTokens = 16;
constexpr int kQtStride = 20;  // row stride of Qt in floats: 16-byte rows whose vector stores do not collide
constexpr size_t kChunkedSmemFloats = 2 * 4 * kBlockTokens * 64 + 64 * kQtStride + kBlockTokens * 64 + kBlockTokens * kBlockTokens + 64 +
                                      64 * 64 + 4 * kBlockTokens * 64;
__global__ void __launch_bounds__(256) time_mix_v56_chunked_kernel(const WkvArgs a) {
    constexpr int S = 64, L = kBlockTokens;
    enum { IN_K = 0, IN_R = 1, IN_W = 2, IN_V = 3 };
    extern __shared__ __align__(16) float wkv_smem[];
    float(*sin)[4][L][S] = reinterpret_cast<float(*)[4][L][S]>(wkv_smem);              // [2]: staged k, r, w, v
    float(*Qt)[kQtStride] = reinterpret_cast<float(*)[kQtStride]>(wkv_smem + 2 * 4 * L * S);  // [S]: Qt[i][t] = r_t[i] Pe_t[i]
    float(*Kd)[S] = reinterpret_cast<float(*)[S]>(&Qt[S][0]);                            // [L]: Kd[s][i] = k_s[i] E_s[i]
    float(*At)[L] = reinterpret_cast<float(*)[L]>(&Kd[L][0]);                            // [L]: At[s][t] = A[t][s], 0 for s > t
    float* PL = &At[L][0];                                                               // [S]: the block's whole decay
    float(*S0)[S] = reinterpret_cast<float(*)[S]>(PL + S);                               // [S]: the state at the block's start
    float* red = &S0[S][0];  // [4][L][S] partial outputs of the four key ranges; before that [L s][L t][16] partials of A
    __shared__ RunScratch run;
    const uint32_t tid = threadIdx.x;
    const uint32_t h = blockIdx.x, slot = blockIdx.y, C = a.S * a.H, c0 = h * S;
    const uint32_t ri = tid / 16, cj = tid % 16;               // state tile: rows 4 ri .., columns 4 cj ..
    const uint32_t tg = tid / 64, tt = (tid % 64) / 16;        // output tile: key range 16 tg .., tokens 4 tt .., columns 4 cj ..

    uint32_t start, count, carry;
    if (!find_run(a.cursors, a.wide, a.T, slot, &run, start, count, &carry)) return;
    if (carry != 0 && tid < S)  // the carry row takes the layer input of the run's closing token (nothing here reads the row)
        static_cast<float*>(a.state.base)[a.state.index(c0 + tid, 0, slot)] = dload(a.x, a.dtype, (size_t)(carry - 1) * C + c0 + tid);

    float st[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
            st[r][cc] = static_cast<const float*>(a.state.base)[a.state.index(c0 + 4 * cj + cc, 1 + 4 * ri + r, slot)];
    float u4[4];  // time_first of the keys this thread takes in the A partials: 4 (tid % 16) ..
#pragma unroll
    for (int e = 0; e < 4; ++e) u4[e] = a.time_first[c0 + 4 * cj + e];

    // staging: thread (tensor = tid / 64, channel = tid % 64) takes the block's 16 tokens of its tensor and channel;
    // past the run's end k, r, v are 0 and w is 1 (such a token changes nothing)
    float stage[L];
    const uint32_t tensor = tid / S, ch = tid % S;
    auto load_chunk = [&](uint32_t chunk) {
#pragma unroll
        for (int n = 0; n < L; ++n) {
            const uint32_t m = chunk * L + n;
            const size_t ti = (size_t)(start + m) * C + c0 + ch;
            float v = tensor == IN_W ? 1.0f : 0.0f;
            if (m < count) {
                if (tensor == IN_K) v = dload(a.k, a.dtype, ti);
                else if (tensor == IN_R) v = dload(a.r, a.dtype, ti);
                else if (tensor == IN_W) v = a.per_token_decay ? a.time_decay[ti] : a.time_decay[c0 + ch];
                else v = dload(a.v, a.dtype, ti);
            }
            stage[n] = v;
        }
    };
    auto store_chunk = [&](int buf) {
#pragma unroll
        for (int n = 0; n < L; ++n) sin[buf][tensor][n][ch] = stage[n];
    };
    const uint32_t chunks = (count + L - 1) / L;
    load_chunk(0);
    store_chunk(0);
    __syncthreads();

    for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
        const int buf = chunk & 1;
        const bool more = chunk + 1 < chunks;
        if (more) load_chunk(chunk + 1);  // in flight while this block is computed
        const float(*sk)[S] = sin[buf][IN_K];
        const float(*sr)[S] = sin[buf][IN_R];
        const float(*sw)[S] = sin[buf][IN_W];
        const float(*sv)[S] = sin[buf][IN_V];

        // (1) the state tile to shared memory; the decay products; the partial sums of A
#pragma unroll
        for (int r = 0; r < 4; ++r) *reinterpret_cast<float4*>(&S0[4 * ri + r][4 * cj]) = make_float4(st[r][0], st[r][1], st[r][2], st[r][3]);
        {
            // thread (key i = tid % 64, quarter tq = tid / 64): Qt[i][4 tq ..], Kd[4 tq ..][i]; quarter 3 ends on the whole product
            const uint32_t i = tid % S, tq = tid / S;
            float pe = 1.0f;
            for (uint32_t t = 0; t < 4 * tq; ++t) pe *= sw[t][i];
            float q[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                q[e] = sr[4 * tq + e][i] * pe;
                pe *= sw[4 * tq + e][i];
            }
            *reinterpret_cast<float4*>(&Qt[i][4 * tq]) = make_float4(q[0], q[1], q[2], q[3]);
            if (tq == 3) PL[i] = pe;
            float en = 1.0f;
            for (uint32_t s2 = L - 1; s2 > 4 * tq + 3; --s2) en *= sw[s2][i];
#pragma unroll
            for (int e = 3; e >= 0; --e) {
                Kd[4 * tq + e][i] = sk[4 * tq + e][i] * en;
                en *= sw[4 * tq + e][i];
            }
        }
        {
            // thread (s = tid / 16, keys 4 cj ..): its share of A[t][s] for t = s .. L - 1, into red[s][t][cj]
            const uint32_t s2 = tid / 16;
            const float4 kq = *reinterpret_cast<const float4*>(&sk[s2][4 * cj]);
            const float kk[4] = {kq.x, kq.y, kq.z, kq.w};
            float d[4] = {1.0f, 1.0f, 1.0f, 1.0f};
            for (uint32_t t = 0; t < s2; ++t) red[(s2 * L + t) * 16 + cj] = 0.0f;
            {
                const float4 rq = *reinterpret_cast<const float4*>(&sr[s2][4 * cj]);
                red[(s2 * L + s2) * 16 + cj] = (rq.x * kk[0] * u4[0] + rq.y * kk[1] * u4[1]) + (rq.z * kk[2] * u4[2] + rq.w * kk[3] * u4[3]);
            }
            for (uint32_t t = s2 + 1; t < L; ++t) {
                const float4 rq = *reinterpret_cast<const float4*>(&sr[t][4 * cj]);
                const float4 wq = *reinterpret_cast<const float4*>(&sw[t][4 * cj]);
                red[(s2 * L + t) * 16 + cj] = (rq.x * kk[0] * d[0] + rq.y * kk[1] * d[1]) + (rq.z * kk[2] * d[2] + rq.w * kk[3] * d[3]);
                d[0] *= wq.x, d[1] *= wq.y, d[2] *= wq.z, d[3] *= wq.w;
            }
        }
        __syncthreads();
        // (2) A[t][s] summed over the 16 key groups: thread (s, t) = (tid / 16, tid % 16)
        {
            const float4* p4 = reinterpret_cast<const float4*>(red + (size_t)tid * 16);
            const float4 p0 = p4[0], p1 = p4[1], p2 = p4[2], p3 = p4[3];
            At[tid / 16][tid % 16] = ((p0.x + p0.y) + (p0.z + p0.w)) + ((p1.x + p1.y) + (p1.z + p1.w)) +
                                     (((p2.x + p2.y) + (p2.z + p2.w)) + ((p3.x + p3.y) + (p3.z + p3.w)));
        }
        __syncthreads();
        // (3) the outputs of tokens 4 tt .. and columns 4 cj .., summed over keys 16 tg .. (the state's share) and over the
        // block's tokens 4 tg .. (their own share); then the new state tile
        {
            float acc[4][4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) acc[e][cc] = 0.0f;
#pragma unroll 4
            for (uint32_t i = 16 * tg; i < 16 * tg + 16; ++i) {
                const float4 q4 = *reinterpret_cast<const float4*>(&Qt[i][4 * tt]);
                const float4 s4 = *reinterpret_cast<const float4*>(&S0[i][4 * cj]);
                const float qv[4] = {q4.x, q4.y, q4.z, q4.w}, sv4[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) acc[e][cc] = fmaf(qv[e], sv4[cc], acc[e][cc]);
            }
#pragma unroll
            for (uint32_t s2 = 4 * tg; s2 < 4 * tg + 4; ++s2) {
                const float4 a4 = *reinterpret_cast<const float4*>(&At[s2][4 * tt]);
                const float4 v4 = *reinterpret_cast<const float4*>(&sv[s2][4 * cj]);
                const float av[4] = {a4.x, a4.y, a4.z, a4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) acc[e][cc] = fmaf(av[e], vv[cc], acc[e][cc]);
            }
            // red is free again: every thread has passed the barrier that follows its last read in (2)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                *reinterpret_cast<float4*>(&red[((size_t)tg * L + 4 * tt + e) * S + 4 * cj]) = make_float4(acc[e][0], acc[e][1], acc[e][2], acc[e][3]);
        }
        {
            const float4 pl = *reinterpret_cast<const float4*>(&PL[4 * ri]);
            const float plv[4] = {pl.x, pl.y, pl.z, pl.w};
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) st[r][cc] *= plv[r];
#pragma unroll 4
            for (uint32_t s2 = 0; s2 < L; ++s2) {
                const float4 k4 = *reinterpret_cast<const float4*>(&Kd[s2][4 * ri]);
                const float4 v4 = *reinterpret_cast<const float4*>(&sv[s2][4 * cj]);
                const float kv[4] = {k4.x, k4.y, k4.z, k4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) st[r][cc] = fmaf(kv[r], vv[cc], st[r][cc]);
            }
        }
        __syncthreads();
        // (4) token t = tid / 16, columns 4 cj ..: the four key ranges' partial outputs
        {
            const uint32_t t = tid / 16, m = chunk * L + t;
            if (m < count) {
                float4 y = *reinterpret_cast<const float4*>(&red[((size_t)0 * L + t) * S + 4 * cj]);
#pragma unroll
                for (int g = 1; g < 4; ++g) {
                    const float4 p = *reinterpret_cast<const float4*>(&red[((size_t)g * L + t) * S + 4 * cj]);
                    y.x += p.x, y.y += p.y, y.z += p.z, y.w += p.w;
                }
                const size_t ti = (size_t)(start + m) * C + c0 + 4 * cj;
                dstore(a.x, a.dtype, ti, y.x);
                dstore(a.x, a.dtype, ti + 1, y.y);
                dstore(a.x, a.dtype, ti + 2, y.z);
                dstore(a.x, a.dtype, ti + 3, y.w);
            }
        }
        if (more) store_chunk(buf ^ 1);  // last read during the previous block, before its closing barrier
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
            static_cast<float*>(a.state.base)[a.state.index(c0 + 4 * cj + cc, 1 + 4 * ri + r, slot)] = st[r][cc];
}

// v7: one CTA of (1 + G) * S threads per (head, batch slot).  Thread j of the first S keeps the whole column j of the
// state in registers, so a token needs no exchange between threads; the other G groups of S threads fetch the tokens'
// rows a chunk of 768 / S tokens ahead (three pairs: r and the decay; k and v; a and kk, 3 / G pairs per group), apply
// the per-token transforms (w -> exp(-0.606531 sigmoid(w)), -kk, kk a) and hand them over through shared memory, one
// barrier per chunk.
template <int S, int G>
__global__ void __launch_bounds__((1 + G) * S) time_mix_v7_kernel(const WkvArgs a) {
    static_assert(G == 1 || G == 3, "three pairs of rows over the loader groups");
    constexpr int TC = 768 / S, P = 3 / G;
    enum { IN_R = 0, IN_W = 1, IN_K = 2, IN_V = 3, IN_A = 4, IN_B = 5 };
    __shared__ __align__(16) float sin[2][6][TC][S];
    __shared__ RunScratch run;
    const uint32_t h = blockIdx.x, slot = blockIdx.y, j = threadIdx.x % S, q = threadIdx.x / S;
    const uint32_t C = a.S * a.H, c = h * S + j;
    const size_t plane = (size_t)a.T * C;

    uint32_t start, count, carry;
    if (!find_run(a.cursors, a.wide, a.T, slot, &run, start, count, &carry)) return;
    // the carry row takes the layer input of the run's closing token: written now (nothing here reads the row), before
    // the token's input is overwritten with its output
    if (carry != 0 && q == 0)
        static_cast<float*>(a.state.base)[a.state.index(c, 0, slot)] = dload(a.x, a.dtype, (size_t)(carry - 1) * C + c);

    float st[S];
    if (q == 0) {
#pragma unroll
        for (int i = 0; i < S; ++i) st[i] = static_cast<const float*>(a.state.base)[a.state.index(c, 1 + i, slot)];
    }

    auto decay = [](float w) { return expf(-0.606531f * (1.0f / (1.0f + expf(-w)))); };
    // loader group q (1..G): the pairs of staged rows it owns, element (token, channel j) of chunk `chunk` (zero past
    // the run's end)
    float s0[P][TC], s1[P][TC];
    auto load_chunk = [&](uint32_t chunk) {
#pragma unroll
        for (int pi = 0; pi < P; ++pi) {
            const uint32_t pair = G == 1 ? (uint32_t)pi : q - 1;
#pragma unroll
            for (int n = 0; n < TC; ++n) {
                const uint32_t m = chunk * TC + n;
                const size_t ti = (size_t)(start + m) * C + c;
                float x0 = 0.f, x1 = 0.f;
                if (m < count) {
                    if (pair == 0) x0 = dload(a.r, a.dtype, ti), x1 = dload(a.w, a.dtype, ti);
                    else if (pair == 1) x0 = dload(a.n, a.dtype, ti), x1 = dload(a.n, a.dtype, ti + plane);
                    else x0 = dload(a.n, a.dtype, ti + 2 * plane), x1 = dload(a.n, a.dtype, ti + 3 * plane);
                }
                s0[pi][n] = x0;
                s1[pi][n] = x1;
            }
        }
    };
    auto store_chunk = [&](int buf) {
#pragma unroll
        for (int pi = 0; pi < P; ++pi) {
            const uint32_t pair = G == 1 ? (uint32_t)pi : q - 1;
#pragma unroll
            for (int n = 0; n < TC; ++n) {
                if (pair == 0) sin[buf][IN_R][n][j] = s0[pi][n], sin[buf][IN_W][n][j] = decay(s1[pi][n]);
                else if (pair == 1) sin[buf][IN_K][n][j] = s0[pi][n], sin[buf][IN_V][n][j] = s1[pi][n];
                else sin[buf][IN_A][n][j] = -s1[pi][n], sin[buf][IN_B][n][j] = s1[pi][n] * s0[pi][n];
            }
        }
    };
    const uint32_t chunks = (count + TC - 1) / TC;
    if (q != 0) {
        load_chunk(0);
        store_chunk(0);
    }
    __syncthreads();

    for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
        const int buf = chunk & 1;
        const bool more = chunk + 1 < chunks;
        if (q != 0) {
            if (more) {
                load_chunk(chunk + 1);
                store_chunk(buf ^ 1);  // last read two chunks ago, before that chunk's closing barrier
            }
        } else {
            const uint32_t len = min((uint32_t)TC, count - chunk * TC);
            for (uint32_t n = 0; n < len; ++n) {
                const uint32_t t = start + chunk * TC + n;
                const size_t ti = (size_t)t * C + c;
                const float vj = sin[buf][IN_V][n][j];
                const float4* r4 = reinterpret_cast<const float4*>(sin[buf][IN_R][n]);
                const float4* w4 = reinterpret_cast<const float4*>(sin[buf][IN_W][n]);
                const float4* k4 = reinterpret_cast<const float4*>(sin[buf][IN_K][n]);
                const float4* a4 = reinterpret_cast<const float4*>(sin[buf][IN_A][n]);
                const float4* b4 = reinterpret_cast<const float4*>(sin[buf][IN_B][n]);
                float z0 = 0.f, z1 = 0.f, z2 = 0.f, z3 = 0.f;
#pragma unroll
                for (int i = 0; i < S; i += 4) {
                    const float4 av = a4[i / 4];
                    z0 = fmaf(st[i], av.x, z0);
                    z1 = fmaf(st[i + 1], av.y, z1);
                    z2 = fmaf(st[i + 2], av.z, z2);
                    z3 = fmaf(st[i + 3], av.w, z3);
                }
                const float sav = (z0 + z1) + (z2 + z3);
                float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
                for (int i = 0; i < S; i += 4) {
                    const float4 wv = w4[i / 4], kv = k4[i / 4], bv = b4[i / 4], rv = r4[i / 4];
                    st[i] = st[i] * wv.x + kv.x * vj + sav * bv.x;
                    y0 = fmaf(rv.x, st[i], y0);
                    st[i + 1] = st[i + 1] * wv.y + kv.y * vj + sav * bv.y;
                    y1 = fmaf(rv.y, st[i + 1], y1);
                    st[i + 2] = st[i + 2] * wv.z + kv.z * vj + sav * bv.z;
                    y2 = fmaf(rv.z, st[i + 2], y2);
                    st[i + 3] = st[i + 3] * wv.w + kv.w * vj + sav * bv.w;
                    y3 = fmaf(rv.w, st[i + 3], y3);
                }
                dstore(a.x, a.dtype, ti, (y0 + y1) + (y2 + y3));
            }
        }
        __syncthreads();
    }
    if (q == 0) {
#pragma unroll
        for (int i = 0; i < S; ++i) static_cast<float*>(a.state.base)[a.state.index(c, 1 + i, slot)] = st[i];
    }
}

// v7, runs of a few tokens (batched decode: many sequences, a token or two each): S threads per (head, batch slot),
// thread j with column j of the state, a token's shared vectors through double-buffered shared memory.  Such a job
// streams the states (S x S floats per head and sequence, in and out) and little else; the small CTA keeps six of
// them on an SM where the staged kernel above fits one.
template <int S>
__global__ void __launch_bounds__(S) time_mix_v7_short_kernel(const WkvArgs a) {
    __shared__ float sr[2][S], sw[2][S], sk[2][S], sa[2][S], sb[2][S];
    __shared__ RunScratch run;
    const uint32_t h = blockIdx.x, slot = blockIdx.y, j = threadIdx.x;
    const uint32_t C = a.S * a.H, c = h * S + j;
    const size_t plane = (size_t)a.T * C;

    uint32_t start, count;
    if (!find_run(a.cursors, a.wide, a.T, slot, &run, start, count)) return;

    float st[S];
#pragma unroll
    for (int i = 0; i < S; ++i) st[i] = static_cast<const float*>(a.state.base)[a.state.index(c, 1 + i, slot)];

    auto decay = [](float w) { return expf(-0.606531f * (1.0f / (1.0f + expf(-w)))); };
    {
        const size_t ti = (size_t)start * C + c;
        sr[0][j] = dload(a.r, a.dtype, ti);
        sw[0][j] = decay(dload(a.w, a.dtype, ti));
        sk[0][j] = dload(a.n, a.dtype, ti);
        const float av = dload(a.n, a.dtype, ti + 2 * plane), kk = dload(a.n, a.dtype, ti + 3 * plane);
        sa[0][j] = -kk;
        sb[0][j] = kk * av;
    }
    __syncthreads();

    for (uint32_t n = 0; n < count; ++n) {
        const uint32_t t = start + n;
        const int cur = n & 1, nxt = cur ^ 1;
        const size_t ti = (size_t)t * C + c;
        const bool more = n + 1 < count;
        float nr = 0.f, nw = 0.f, nk = 0.f, na = 0.f, nkk = 0.f;
        if (more) {
            nr = dload(a.r, a.dtype, ti + C);
            nw = dload(a.w, a.dtype, ti + C);
            nk = dload(a.n, a.dtype, ti + C);
            na = dload(a.n, a.dtype, ti + C + 2 * plane);
            nkk = dload(a.n, a.dtype, ti + C + 3 * plane);
        }
        const float vj = dload(a.n, a.dtype, ti + plane);
        const float xin = dload(a.x, a.dtype, ti);
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
        for (int i = 0; i < S; i += 4) {
            s0 = fmaf(st[i], sa[cur][i], s0);
            s1 = fmaf(st[i + 1], sa[cur][i + 1], s1);
            s2 = fmaf(st[i + 2], sa[cur][i + 2], s2);
            s3 = fmaf(st[i + 3], sa[cur][i + 3], s3);
        }
        const float sav = (s0 + s1) + (s2 + s3);
        float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
        for (int i = 0; i < S; i += 4) {
            st[i] = st[i] * sw[cur][i] + sk[cur][i] * vj + sav * sb[cur][i];
            y0 = fmaf(sr[cur][i], st[i], y0);
            st[i + 1] = st[i + 1] * sw[cur][i + 1] + sk[cur][i + 1] * vj + sav * sb[cur][i + 1];
            y1 = fmaf(sr[cur][i + 1], st[i + 1], y1);
            st[i + 2] = st[i + 2] * sw[cur][i + 2] + sk[cur][i + 2] * vj + sav * sb[cur][i + 2];
            y2 = fmaf(sr[cur][i + 2], st[i + 2], y2);
            st[i + 3] = st[i + 3] * sw[cur][i + 3] + sk[cur][i + 3] * vj + sav * sb[cur][i + 3];
            y3 = fmaf(sr[cur][i + 3], st[i + 3], y3);
        }
        const CursorD cu = cursor_at(a.cursors, a.wide, t);
        if (t - cu.token + 1u == cu.len)
            static_cast<float*>(a.state.base)[a.state.index(c, 0, slot)] = xin;
        dstore(a.x, a.dtype, ti, (y0 + y1) + (y2 + y3));
        if (more) {
            sr[nxt][j] = nr;
            sw[nxt][j] = decay(nw);
            sk[nxt][j] = nk;
            sa[nxt][j] = -nkk;
            sb[nxt][j] = nkk * na;
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < S; ++i) static_cast<float*>(a.state.base)[a.state.index(c, 1 + i, slot)] = st[i];
}

// x_j += (sum_i u_i k_i r_i) * v_j per (token, head): one warp per (token, head).
__global__ void time_first_v7_kernel(const __half* u, int dtype, const void* r, const void* n, void* x, uint32_t S,
                                     uint32_t H, uint32_t T) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= T * H) return;
    const uint32_t t = warp / H, h = warp % H;
    const uint32_t C = S * H;
    const size_t base = (size_t)t * C + h * S, plane = (size_t)T * C;
    float s = 0.f;
    for (uint32_t i = lane; i < S; i += 32)
        s += __half2float(u[h * S + i]) * dload(n, dtype, base + i) * dload(r, dtype, base + i);
    s = warp_sum(s);
    for (uint32_t i = lane; i < S; i += 32)
        dstore(x, dtype, base + i, dload(x, dtype, base + i) + s * dload(n, dtype, base + i + plane));
}

}  // namespace

cudaError_t time_mix_v56(const WkvArgs& a, cudaStream_t stream) {
    if (a.T == 0 || a.B == 0) return cudaSuccess;
    dim3 grid(a.H, a.B);
    switch (a.S) {
        case 32: time_mix_v56_kernel<32, 4><<<grid, 64, 0, stream>>>(a); break;
        case 64: time_mix_v56_kernel<64, 4><<<grid, 256, 0, stream>>>(a); break;
        case 128: time_mix_v56_kernel<128, 4><<<grid, 1024, 0, stream>>>(a); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// The block form of time_mix_v56 (heads of 64 channels only).
bool time_mix_v56_chunked_supported(const WkvArgs& a) { return a.S == 64; }

cudaError_t time_mix_v56_chunked(const WkvArgs& a, cudaStream_t stream) {
    if (a.T == 0 || a.B == 0) return cudaSuccess;
    if (!time_mix_v56_chunked_supported(a)) return cudaErrorInvalidValue;
    static SmemOptIn opt_in;
    const size_t smem = kChunkedSmemFloats * sizeof(float);
    if (cudaError_t e = opt_in.ensure(time_mix_v56_chunked_kernel, (int)smem); e != cudaSuccess) return e;
    time_mix_v56_chunked_kernel<<<dim3(a.H, a.B), 256, smem, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t time_mix_v7(const WkvArgs& a, cudaStream_t stream) {
    if (a.T == 0 || a.B == 0) return cudaSuccess;
    dim3 grid(a.H, a.B);
    if (a.T <= 4 * a.B) {  // at most four tokens per sequence on average
        switch (a.S) {
            case 32: time_mix_v7_short_kernel<32><<<grid, 32, 0, stream>>>(a); break;
            case 64: time_mix_v7_short_kernel<64><<<grid, 64, 0, stream>>>(a); break;
            case 128: time_mix_v7_short_kernel<128><<<grid, 128, 0, stream>>>(a); break;
            default: return cudaErrorInvalidValue;
        }
        return cudaGetLastError();
    }
    switch (a.S) {
        case 32: time_mix_v7_kernel<32, 3><<<grid, 128, 0, stream>>>(a); break;
        case 64: time_mix_v7_kernel<64, 3><<<grid, 256, 0, stream>>>(a); break;
        case 128: time_mix_v7_kernel<128, 1><<<grid, 256, 0, stream>>>(a); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// time_mix_v4.wgsl: per channel c and token t (batch from the cursor), with (aa, bb, pp) = state rows 1..3:
//   x_t = sigmoid(r_t) * (e1 aa + e2 v_t) / (e1 bb + e2),   e1 = exp(pp - q), e2 = exp(u + k_t - q), q = max(pp, u + k_t)
//   (aa, bb, pp) <- (e1' aa + e2' v_t, e1' bb + e2', q'),      e1' = exp(w + pp - q'), e2' = exp(k_t - q'), q' = max(w + pp, k_t)
// and state row 0 <- the input x of the sequence's last token in the job.  One thread per channel walks the tokens in
// order and keeps (aa, bb, pp) in registers while consecutive tokens belong to one batch slot.
__global__ void time_mix_v4_kernel(const uint32_t* cursors, int wide, const float* time_decay, const float* time_first,
                                   DView state, int dtype, const void* k, const void* v, const void* r, void* x,
                                   uint32_t C, uint32_t T) {
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float u = time_first[c], w = time_decay[c];
    float* st = static_cast<float*>(state.base);
    uint32_t held = 0xffffffffu;  // batch slot whose recurrence is in registers
    float aa = 0.f, bb = 0.f, pp = 0.f;
    for (uint32_t t = 0; t < T; ++t) {
        const CursorD cu = cursor_at(cursors, wide, t);
        if (cu.batch != held) {
            if (held != 0xffffffffu) {
                st[state.index(c, 1, held)] = aa;
                st[state.index(c, 2, held)] = bb;
                st[state.index(c, 3, held)] = pp;
            }
            held = cu.batch;
            aa = st[state.index(c, 1, held)];
            bb = st[state.index(c, 2, held)];
            pp = st[state.index(c, 3, held)];
        }
        const size_t ti = (size_t)t * C + c;
        // the token-shift carry: read before this token's slot of x is overwritten (the last token's slot is >= t)
        const uint32_t last = cu.token + cu.len - 1u;
        if ((t == last || t == cu.token) && last >= t && last < T)
            st[state.index(c, 0, held)] = dload(x, dtype, (size_t)last * C + c);
        const float kk = dload(k, dtype, ti), vv = dload(v, dtype, ti);
        const float rr = 1.0f / (1.0f + expf(-dload(r, dtype, ti)));
        float ww = u + kk;
        float q = fmaxf(pp, ww);
        float e1 = expf(pp - q), e2 = expf(ww - q);
        dstore(x, dtype, ti, rr * (e1 * aa + e2 * vv) / (e1 * bb + e2));
        ww = w + pp;
        q = fmaxf(ww, kk);
        e1 = expf(ww - q);
        e2 = expf(kk - q);
        aa = e1 * aa + e2 * vv;
        bb = e1 * bb + e2;
        pp = q;
    }
    if (held != 0xffffffffu) {
        st[state.index(c, 1, held)] = aa;
        st[state.index(c, 2, held)] = bb;
        st[state.index(c, 3, held)] = pp;
    }
}

cudaError_t time_mix_v4(const uint32_t* cursors, int wide, const float* time_decay, const float* time_first, DView state,
                        int dtype, const void* k, const void* v, const void* r, void* x, uint32_t C, uint32_t T,
                        cudaStream_t stream) {
    if (T == 0 || C == 0) return cudaSuccess;
    time_mix_v4_kernel<<<(C + 127) / 128, 128, 0, stream>>>(cursors, wide, time_decay, time_first, state, dtype, k, v, r, x,
                                                            C, T);
    return cudaGetLastError();
}

cudaError_t time_first_v7(const __half* u, int dtype, const void* r, const void* n, void* x, uint32_t S, uint32_t H,
                          uint32_t T, cudaStream_t stream) {
    if (T == 0) return cudaSuccess;
    const uint32_t warps = T * H;
    const uint32_t blocks = (warps * 32 + 255) / 256;
    time_first_v7_kernel<<<blocks, 256, 0, stream>>>(u, dtype, r, n, x, S, H, T);
    return cudaGetLastError();
}

}  // namespace k
}  // namespace wrk
