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
// slot has no token in this job.
__device__ __forceinline__ bool find_run(const uint32_t* cursors, int wide, uint32_t T, uint32_t slot,
                                         uint32_t* s_start, uint32_t* s_count, uint32_t& start, uint32_t& count) {
    if (threadIdx.x == 0) {
        *s_start = 0xffffffffu;
        *s_count = 0;
    }
    __syncthreads();
    uint32_t my_min = 0xffffffffu, my_cnt = 0;
    for (uint32_t t = threadIdx.x; t < T; t += blockDim.x) {
        const CursorD c = cursor_at(cursors, wide, t);
        if (c.batch == slot) {
            my_min = min(my_min, t);
            ++my_cnt;
        }
    }
    if (my_cnt) {
        atomicMin(s_start, my_min);
        atomicAdd(s_count, my_cnt);
    }
    __syncthreads();
    start = *s_start;
    count = *s_count;
    return count != 0;
}

// One CTA of Q * S threads per (head, batch slot): thread (q, j) keeps rows [q S/Q, (q+1) S/Q) of state
// column j in registers for the sequence's whole run of tokens and adds its part of output j; the Q parts
// meet in shared memory (one barrier per token, buffers alternate).
template <int S, int Q>
__global__ void __launch_bounds__(S * Q) time_mix_v56_kernel(const WkvArgs a) {
    constexpr int SI = S / Q;
    __shared__ float sk[2][S], sr[2][S], sw[2][S], su[S], part[2][Q][S];
    __shared__ uint32_t s_start, s_count;
    const uint32_t h = blockIdx.x, slot = blockIdx.y, j = threadIdx.x % S, q = threadIdx.x / S;
    const uint32_t C = a.S * a.H, c = h * S + j;

    uint32_t start, count;
    if (!find_run(a.cursors, a.wide, a.T, slot, &s_start, &s_count, start, count)) return;

    float st[SI];
#pragma unroll
    for (int i = 0; i < SI; ++i) st[i] = static_cast<const float*>(a.state.base)[a.state.index(c, 1 + q * SI + i, slot)];
    if (q == 0) {
        su[j] = a.time_first[c];
        if (!a.per_token_decay) sw[0][j] = sw[1][j] = a.time_decay[c];
        const size_t ti = (size_t)start * C + c;
        sk[0][j] = dload(a.k, a.dtype, ti);
        sr[0][j] = dload(a.r, a.dtype, ti);
        if (a.per_token_decay) sw[0][j] = a.time_decay[ti];
    }
    __syncthreads();

    for (uint32_t n = 0; n < count; ++n) {
        const uint32_t t = start + n;
        const int cur = n & 1, nxt = cur ^ 1;
        const size_t ti = (size_t)t * C + c;
        // next token's shared vectors: issue the loads before this token's math
        float nk = 0.f, nr = 0.f, nw = 0.f, xin = 0.f;
        const bool more = n + 1 < count;
        if (q == 0) {
            if (more) {
                nk = dload(a.k, a.dtype, ti + C);
                nr = dload(a.r, a.dtype, ti + C);
                if (a.per_token_decay) nw = a.time_decay[ti + C];
            }
            xin = dload(a.x, a.dtype, ti);
        }
        const float vj = dload(a.v, a.dtype, ti);
        float y0 = 0.f, y1 = 0.f;
#pragma unroll
        for (int ii = 0; ii < SI; ii += 2) {
            const int i = q * SI + ii;
            float kv;
            kv = sk[cur][i] * vj;     y0 += sr[cur][i] * fmaf(su[i], kv, st[ii]);             st[ii] = fmaf(sw[cur][i], st[ii], kv);
            kv = sk[cur][i + 1] * vj; y1 += sr[cur][i + 1] * fmaf(su[i + 1], kv, st[ii + 1]); st[ii + 1] = fmaf(sw[cur][i + 1], st[ii + 1], kv);
        }
        part[cur][q][j] = y0 + y1;
        if (q == 0 && more) {
            sk[nxt][j] = nk;
            sr[nxt][j] = nr;
            if (a.per_token_decay) sw[nxt][j] = nw;
        }
        __syncthreads();
        if (q == 0) {
            float y = part[cur][0][j];
#pragma unroll
            for (int p2 = 1; p2 < Q; ++p2) y += part[cur][p2][j];
            const CursorD cu = cursor_at(a.cursors, a.wide, t);
            if (t - cu.token + 1u == cu.len)  // last token of the run: token-shift carry takes the layer input
                static_cast<float*>(a.state.base)[a.state.index(c, 0, slot)] = xin;
            dstore(a.x, a.dtype, ti, y);
        }
    }
#pragma unroll
    for (int i = 0; i < SI; ++i) static_cast<float*>(a.state.base)[a.state.index(c, 1 + q * SI + i, slot)] = st[i];
}

template <int S>
__global__ void __launch_bounds__(S) time_mix_v7_kernel(const WkvArgs a) {
    __shared__ float sr[2][S], sw[2][S], sk[2][S], sa[2][S], sb[2][S];
    __shared__ uint32_t s_start, s_count;
    const uint32_t h = blockIdx.x, slot = blockIdx.y, j = threadIdx.x;
    const uint32_t C = a.S * a.H, c = h * S + j;
    const size_t plane = (size_t)a.T * C;

    uint32_t start, count;
    if (!find_run(a.cursors, a.wide, a.T, slot, &s_start, &s_count, start, count)) return;

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
        case 32: time_mix_v56_kernel<32, 4><<<grid, 128, 0, stream>>>(a); break;
        case 64: time_mix_v56_kernel<64, 4><<<grid, 256, 0, stream>>>(a); break;
        case 128: time_mix_v56_kernel<128, 4><<<grid, 512, 0, stream>>>(a); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t time_mix_v7(const WkvArgs& a, cudaStream_t stream) {
    if (a.T == 0 || a.B == 0) return cudaSuccess;
    dim3 grid(a.H, a.B);
    switch (a.S) {
        case 32: time_mix_v7_kernel<32><<<grid, 32, 0, stream>>>(a); break;
        case 64: time_mix_v7_kernel<64><<<grid, 64, 0, stream>>>(a); break;
        case 128: time_mix_v7_kernel<128><<<grid, 128, 0, stream>>>(a); break;
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
