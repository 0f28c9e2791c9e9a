// Supporting ops of the v5/v6/v7 jobs: normalisation, token shift, channel mix and the
// elementwise/broadcast/copy ops.  These are the op-by-op ("strict") forms that mirror the
// reference's operator list one to one; every tensor the reference stores as fp16 is a rounding
// point here as well.  They are latency-bound on the activations of a single job and are not
// individually roofline-graded.
#include "device.cuh"

namespace wrk {
namespace k {

namespace {

constexpr int kEw = 256;

inline int ew_grid(size_t n) {
    size_t g = (n + kEw - 1) / kEw;
    if (g < 1) g = 1;
    if (g > 148 * 16) g = 148 * 16;
    return (int)g;
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (nw == 1) return v;
    __syncthreads();  // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int w = 0; w < nw; ++w) s += scratch[w];
    return s;
}

// layer_norm.wgsl: per row of C, (x - mean) * rsqrt(var + eps) * w + b; var = E[(x - mean)^2].
// Rows of up to kLnRegs * blockDim values are read once and kept in registers (one round of loads in flight instead
// of three dependent passes over global memory); longer rows take the three passes.
constexpr int kLnRegs = 32;
// With `delta`, src <- src + delta first (rounded to the data type, as the separate add stores it).
__global__ void layer_norm_kernel(const __half* w, const __half* b, int dtype, const void* delta, void* src, void* x, uint32_t C,
                                  uint32_t rows, uint32_t wrows, float eps) {
    __shared__ float scratch[32];
    const bool cached = C <= (uint32_t)kLnRegs * blockDim.x;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * C;
        const size_t wb = (size_t)(row % wrows) * C;
        if (cached) {
            float v[kLnRegs];
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < kLnRegs; ++i) {
                const uint32_t c = threadIdx.x + (uint32_t)i * blockDim.x;
                v[i] = c < C ? dload(src, dtype, base + c) : 0.f;
                if (delta && c < C) {
                    v[i] = dtype == WRK_F16 ? __half2float(__float2half_rn(dload(delta, dtype, base + c) + v[i]))
                                            : dload(delta, dtype, base + c) + v[i];
                    dstore(src, dtype, base + c, v[i]);
                }
                s += v[i];
            }
            const float mean = block_sum(s, scratch) / (float)C;
            float m2 = 0.f;
#pragma unroll
            for (int i = 0; i < kLnRegs; ++i) {
                const uint32_t c = threadIdx.x + (uint32_t)i * blockDim.x;
                const float d = v[i] - mean;
                if (c < C) m2 += d * d;
            }
            const float dev = rsqrtf(block_sum(m2, scratch) / (float)C + eps);
#pragma unroll
            for (int i = 0; i < kLnRegs; ++i) {
                const uint32_t c = threadIdx.x + (uint32_t)i * blockDim.x;
                if (c < C) dstore(x, dtype, base + c, fmaf((v[i] - mean) * dev, __half2float(w[wb + c]), __half2float(b[wb + c])));
            }
            continue;
        }
        if (delta)  // each thread reads back only what it wrote
            for (uint32_t c = threadIdx.x; c < C; c += blockDim.x)
                dstore(src, dtype, base + c, dload(delta, dtype, base + c) + dload(src, dtype, base + c));
        float s = 0.f;
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) s += dload(src, dtype, base + c);
        const float mean = block_sum(s, scratch) / (float)C;
        float m2 = 0.f;
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) {
            const float d = dload(src, dtype, base + c) - mean;
            m2 += d * d;
        }
        const float var = block_sum(m2, scratch) / (float)C + eps;
        const float dev = rsqrtf(var);
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) {
            const float v = (dload(src, dtype, base + c) - mean) * dev;
            dstore(x, dtype, base + c, fmaf(v, __half2float(w[wb + c]), __half2float(b[wb + c])));
        }
    }
}

// normalize.wgsl l2_norm: x * rsqrt(sum x^2 + eps) per row of C.
__global__ void l2_norm_kernel(int dtype, void* x, uint32_t C, uint32_t rows, float eps) {
    __shared__ float scratch[32];
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * C;
        float s = 0.f;
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) {
            const float v = dload(x, dtype, base + c);
            s = __fmaf_rn(v, v, s);
        }
        const float norm = rsqrtf(block_sum(s, scratch) + eps);
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x)
            dstore(x, dtype, base + c, dload(x, dtype, base + c) * norm);
    }
}

// normalize.wgsl recenter: x - mean(x) per row of C.
__global__ void recenter_kernel(int dtype, void* x, uint32_t C, uint32_t rows) {
    __shared__ float scratch[32];
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * C;
        float s = 0.f;
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) s += dload(x, dtype, base + c);
        const float mean = block_sum(s, scratch) / (float)C;
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) dstore(x, dtype, base + c, dload(x, dtype, base + c) - mean);
    }
}

// normalize.wgsl rms_norm: fma(x * rsqrt(mean x^2 + eps), w, b) per row of C.
__global__ void rms_norm_kernel(const __half* w, const __half* b, int dtype, void* x, uint32_t C, uint32_t rows,
                                float eps) {
    __shared__ float scratch[32];
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * C;
        float s = 0.f;
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) {
            const float v = dload(x, dtype, base + c);
            s += v * v;
        }
        const float norm = rsqrtf(block_sum(s, scratch) / (float)C + eps);
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x)
            dstore(x, dtype, base + c, fmaf(dload(x, dtype, base + c) * norm, __half2float(w[c]), __half2float(b[c])));
    }
}

// embed.wgsl: output[:, t, b] = input[:, tokens[t, b]] (fp16 rows of the embedding matrix, widened if the output is f32).
__global__ void embed_kernel(const uint32_t* tokens, const __half* input, int dtype, void* output, uint32_t C,
                             uint32_t rows, uint32_t vocab, int32_t* status) {
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint32_t tok = tokens[row];
        if (tok >= vocab) {  // the reference reads out of bounds here; report instead
            if (threadIdx.x == 0) atomicCAS(status, 0, WRK_ERR_BATCH_OUT_OF_RANGE);
            continue;
        }
        const __half* src = input + (size_t)tok * C;
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) dstore(output, dtype, (size_t)row * C + c, __half2float(src[c]));
    }
}

// reshape.wgsl broadcast: output[c, t, b] = input[c, t % in.T, b % in.B].
__global__ void broadcast_kernel(DView in, DView out) {
    const uint32_t C = out.shape[0], T = out.shape[1], B = out.shape[2];
    const size_t total = (size_t)C * T * B;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % C, t = (o / C) % T, b = o / ((size_t)C * T);
        dstore(out.base, out.dtype, out.index(c, t, b),
               dload(in.base, in.dtype, in.index(c, t % in.shape[1], b % in.shape[2])));
    }
}

// blend.wgsl: output = factor[0] * input + factor[1] * output.
__global__ void blend_kernel(const float* factor, DView in, DView out) {
    const uint32_t C = out.shape[0], T = out.shape[1], B = out.shape[2];
    const size_t total = (size_t)C * T * B;
    const float fx = factor[0], fy = factor[1];
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % C, t = (o / C) % T, b = o / ((size_t)C * T);
        const size_t oi = out.index(c, t, b);
        dstore(out.base, out.dtype, oi,
               fx * dload(in.base, in.dtype, in.index(c, t, b)) + fy * dload(out.base, out.dtype, oi));
    }
}

// blend_lora.wgsl: output[m, n, b] = factor[0] * sum_k xa[k, m, b] * xb[k, n, b] + factor[1] * output[m, n, b], all fp16
// tensors, f32 sum over the common rank K.  One warp per 32 consecutive m of one n: lanes read xa rows, xb's row of K
// is shared by the warp.
__global__ void blend_lora_kernel(const float* factor, DView xa, DView xb, DView out, uint32_t K) {
    const uint32_t M = out.shape[0], N = out.shape[1], B = out.shape[2];
    const size_t total = (size_t)M * N * B;
    const float fx = factor[0], fy = factor[1];
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t m = o % M, n = (o / M) % N, b = o / ((size_t)M * N);
        const __half* a = static_cast<const __half*>(xa.base) + xa.index(0, m, b);
        const __half* bb = static_cast<const __half*>(xb.base) + xb.index(0, n, b);
        float sum = 0.f;
        for (uint32_t k = 0; k < K; ++k) sum = fmaf(__half2float(a[k]), __half2float(bb[k]), sum);
        const size_t oi = out.index(m, n, b);
        dstore(out.base, out.dtype, oi, fx * sum + fy * dload(out.base, out.dtype, oi));
    }
}

// softmax.wgsl: x <- exp(x - max) / sum exp(x - max) per row of C (two reductions, then the write).
__global__ void softmax_kernel(int dtype, void* x, uint32_t C, uint32_t rows) {
    __shared__ float scratch[32];
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * C;
        float m = -1.0e30f;
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) m = fmaxf(m, dload(x, dtype, base + c));
        // block maximum through the sum helper's scratch: warp maxima, then the first warp's maximum of those
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        __syncthreads();
        if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
        __syncthreads();
        float mx = -1.0e30f;
        for (uint32_t w = 0; w < (blockDim.x + 31) / 32; ++w) mx = fmaxf(mx, scratch[w]);
        __syncthreads();
        float s = 0.f;
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x) s += expf(dload(x, dtype, base + c) - mx);
        const float sum = block_sum(s, scratch);
        for (uint32_t c = threadIdx.x; c < C; c += blockDim.x)
            dstore(x, dtype, base + c, expf(dload(x, dtype, base + c) - mx) / sum);
    }
}

// token_shift.wgsl: out[c, t, z] = mix(x_t, prev, f) (reversed) or mix(prev, x_t, f); prev is the
// previous token of the same sequence or, at the sequence's first token of the job, the carry row.
__global__ void token_shift_kernel(const uint32_t* cursors, int wide, DView tm, DView state, DView in, DView out,
                                   int reversed) {
    const uint32_t C = out.shape[0], T = out.shape[1], Z = out.shape[2];
    const size_t total = (size_t)C * T * Z;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % C, t = (o / C) % T, z = o / ((size_t)C * T);
        const CursorD cu = cursor_at(cursors, wide, t);
        const float f = dload(tm.base, tm.dtype, tm.index(c, tm.shape[1] == 1 ? 0 : t, z));
        const float cur = dload(in.base, in.dtype, in.index(c, t, 0));
        const float prev = (t == cu.token) ? static_cast<const float*>(state.base)[state.index(c, 0, cu.batch)]
                                           : dload(in.base, in.dtype, in.index(c, t - 1, 0));
        const float a = reversed ? cur : prev, b = reversed ? prev : cur;
        dstore(out.base, out.dtype, out.index(c, t, z), mix_f(a, b, f));
    }
}

// Several token shifts of one input in one launch: out_i[c, t] = mix(x_t, prev, f_i[c]) as token_shift_kernel computes it,
// with the input and the previous row read once.
__global__ void token_shift_multi_kernel(const ShiftMultiArgs a) {
    const size_t total = (size_t)a.C * a.T;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % a.C, t = o / a.C;
        const CursorD cu = cursor_at(a.cursors, a.wide, t);
        const float cur = __half2float(a.in[o]);
        const float prev = (t == cu.token) ? static_cast<const float*>(a.state.base)[a.state.index(c, 0, cu.batch)]
                                           : __half2float(a.in[o - a.C]);
        const float x = a.reversed ? cur : prev, y = a.reversed ? prev : cur;
#pragma unroll
        for (uint32_t i = 0; i < kShiftMultiMax; ++i) {
            if (i >= a.count) break;
            const float f = __half2float(a.mix[i][c]);
            a.out[i][o] = __float2half_rn(mix_f(x, y, f));
        }
    }
}

// The v7 time-mix operand in one launch, one warp per head and token (a row of S channels of [S, H, T]):
//   kk <- l2_norm(k * k_k)  (blit + mul + l2_norm, each rounding to f16 where the separate ops store f16),
//   k  <- k * (1 + (a - 1) * k_a)  (control_k_kernel),  n[.., 0..3] <- k, v, a, kk  (four blits).
// Sums run in l2_norm_kernel's order for a block of 32 threads, so the results are bit-identical to the separate ops.
__global__ void pack_v7_kernel(const PackV7Args p) {
    const uint32_t lane = threadIdx.x;
    const size_t plane = (size_t)p.rows * p.S;
    for (uint32_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const size_t base = (size_t)row * p.S;
        const uint32_t c0 = (row % p.H) * p.S;
        float s = 0.f;
        for (uint32_t c = lane; c < p.S; c += 32) {
            const float v = __half2float(__float2half_rn(__half2float(p.k_k[c0 + c]) * __half2float(p.k[base + c])));
            s = __fmaf_rn(v, v, s);
        }
        const float norm = rsqrtf(warp_sum(s) + p.eps);
        for (uint32_t c = lane; c < p.S; c += 32) {
            const size_t i = base + c;
            const float kv = __half2float(p.k[i]), av = __half2float(p.a[i]);
            const float v = __half2float(__float2half_rn(__half2float(p.k_k[c0 + c]) * kv));
            const __half kk = __float2half_rn(v * norm);
            const __half kn = __float2half_rn(control_k_f(kv, av, __half2float(p.k_a[c0 + c])));
            p.kk[i] = kk;
            p.k[i] = kn;
            p.n[i] = kn;
            p.n[plane + i] = p.v[i];
            p.n[2 * plane + i] = p.a[i];
            p.n[3 * plane + i] = kk;
        }
    }
}

// channel_mix.wgsl: carry row <- x_in at the sequence's last token; x = sigmoid(r) * v (v7: x = v).
__global__ void channel_mix_kernel(const uint32_t* cursors, int wide, DView state, int dtype, const void* r,
                                   const void* v, void* x, uint32_t C, uint32_t T, int v7) {
    const size_t total = (size_t)C * T;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % C, t = o / C;
        const CursorD cu = cursor_at(cursors, wide, t);
        if (t - cu.token + 1u == cu.len)
            static_cast<float*>(state.base)[state.index(c, 0, cu.batch)] = dload(x, dtype, o);
        if (v7) {
            dstore(x, dtype, o, dload(v, dtype, o));
        } else {
            const float rr = 1.0f / (1.0f + expf(-dload(r, dtype, o)));
            dstore(x, dtype, o, rr * dload(v, dtype, o));
        }
    }
}

// The shift row of every sequence that has tokens in the job <- x at the sequence's last token (what the time-mix
// and channel-mix ops do for their own channels, as an op of its own).
__global__ void shift_carry_kernel(const uint32_t* cursors, int wide, DView state, int dtype, const void* x, uint32_t C, uint32_t T) {
    const size_t total = (size_t)C * T;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % C, t = o / C;
        const CursorD cu = cursor_at(cursors, wide, t);
        if (t - cu.token + 1u == cu.len) static_cast<float*>(state.base)[state.index(c, 0, cu.batch)] = dload(x, dtype, o);
    }
}

__global__ void binary_kernel(int is_mul, DView in, DView out, int act_x, int act_y, int act_out) {
    const uint32_t C = out.shape[0], T = out.shape[1], B = out.shape[2];
    const size_t total = (size_t)C * T * B;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % C, t = (o / C) % T, b = o / ((size_t)C * T);
        const float xi = dload(in.base, in.dtype, in.index(c, in.shape[1] == 1 ? 0 : t, in.shape[2] == 1 ? 0 : b));
        const size_t oi = out.index(c, t, b);
        const float ax = activate_f(act_x, xi), ay = activate_f(act_y, dload(out.base, out.dtype, oi));
        dstore(out.base, out.dtype, oi, activate_f(act_out, is_mul ? ax * ay : ax + ay));
    }
}

__global__ void activate_kernel(DView x, int act) {
    const uint32_t C = x.shape[0], T = x.shape[1], B = x.shape[2];
    const size_t total = (size_t)C * T * B;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % C, t = (o / C) % T, b = o / ((size_t)C * T);
        const size_t i = x.index(c, t, b);
        dstore(x.base, x.dtype, i, activate_f(act, dload(x.base, x.dtype, i)));
    }
}

__global__ void blit_kernel(DView in, DView out, int transpose) {
    const uint32_t C = in.shape[0], T = in.shape[1], B = in.shape[2];
    const size_t total = (size_t)C * T * B;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % C, t = (o / C) % T, b = o / ((size_t)C * T);
        const float v = dload(in.base, in.dtype, in.index(c, t, b));
        dstore(out.base, out.dtype, transpose ? out.index(c, b, t) : out.index(c, t, b), v);
    }
}

__global__ void lerp_kernel(DView in, DView out, DView f, int reversed) {
    const uint32_t C = out.shape[0], T = out.shape[1], B = out.shape[2];
    const size_t total = (size_t)C * T * B;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % C, t = (o / C) % T, b = o / ((size_t)C * T);
        const float ff = dload(f.base, f.dtype, f.index(c, f.shape[1] == 1 ? 0 : t, f.shape[2] == 1 ? 0 : b));
        const float xi = dload(in.base, in.dtype, in.index(c, t, b));
        const size_t oi = out.index(c, t, b);
        const float yo = dload(out.base, out.dtype, oi);
        const float a = reversed ? yo : xi, bb = reversed ? xi : yo;
        dstore(out.base, out.dtype, oi, mix_f(a, bb, ff));
    }
}

__global__ void affine_kernel(int dtype, void* x, size_t len, float scale, float bias) {
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < len; o += (size_t)gridDim.x * blockDim.x)
        dstore(x, dtype, o, scale * dload(x, dtype, o) + bias);
}

__global__ void control_k_kernel(const __half* p, DView a, DView k) {
    const uint32_t C = k.shape[0], T = k.shape[1], B = k.shape[2];
    const size_t total = (size_t)C * T * B;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total; o += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = o % C, t = (o / C) % T, b = o / ((size_t)C * T);
        const float pp = __half2float(p[c]);
        const float av = dload(a.base, a.dtype, a.index(c, t, b));
        const size_t ki = k.index(c, t, b);
        dstore(k.base, k.dtype, ki, control_k_f(dload(k.base, k.dtype, ki), av, pp));
    }
}

}  // namespace

cudaError_t layer_norm(const __half* w, const __half* b, int dtype, void* x, uint32_t C, uint32_t rows, uint32_t wrows,
                       float eps, cudaStream_t stream) {
    return layer_norm_copy(w, b, dtype, nullptr, x, x, C, rows, wrows, eps, stream);
}

// src <- src + delta when `delta` is given; x <- layer norm of `src` (the same dtype and shape; src == x: in place)
cudaError_t layer_norm_copy(const __half* w, const __half* b, int dtype, const void* delta, void* src, void* x, uint32_t C,
                            uint32_t rows, uint32_t wrows, float eps, cudaStream_t stream) {
    if (rows == 0 || C == 0) return cudaSuccess;
    if (layer_norm_vec(w, b, dtype, delta, src, x, C, rows, wrows, eps, stream)) return cudaGetLastError();
    const int block = C <= 256 ? 32 : 256;
    const uint32_t grid = rows < 148u * 32u ? rows : 148u * 32u;
    layer_norm_kernel<<<grid, block, 0, stream>>>(w, b, dtype, delta, src, x, C, rows, wrows, eps);
    return cudaGetLastError();
}

cudaError_t l2_norm(int dtype, void* x, uint32_t C, uint32_t rows, float eps, cudaStream_t stream) {
    if (rows == 0 || C == 0) return cudaSuccess;
    const int block = C <= 256 ? 32 : 256;
    const uint32_t grid = rows < 148u * 32u ? rows : 148u * 32u;
    l2_norm_kernel<<<grid, block, 0, stream>>>(dtype, x, C, rows, eps);
    return cudaGetLastError();
}

cudaError_t softmax(int dtype, void* x, uint32_t C, uint32_t rows, cudaStream_t stream) {
    if (rows == 0 || C == 0) return cudaSuccess;
    const int block = C <= 256 ? 32 : C <= 4096 ? 256 : 1024;
    const uint32_t grid = rows < 148u * 32u ? rows : 148u * 32u;
    softmax_kernel<<<grid, block, 0, stream>>>(dtype, x, C, rows);
    return cudaGetLastError();
}

cudaError_t recenter(int dtype, void* x, uint32_t C, uint32_t rows, cudaStream_t stream) {
    if (rows == 0 || C == 0) return cudaSuccess;
    const int block = C <= 256 ? 32 : 256;
    const uint32_t grid = rows < 148u * 32u ? rows : 148u * 32u;
    recenter_kernel<<<grid, block, 0, stream>>>(dtype, x, C, rows);
    return cudaGetLastError();
}

cudaError_t rms_norm(const __half* w, const __half* b, int dtype, void* x, uint32_t C, uint32_t rows, float eps,
                     cudaStream_t stream) {
    if (rows == 0 || C == 0) return cudaSuccess;
    const int block = C <= 256 ? 32 : 256;
    const uint32_t grid = rows < 148u * 32u ? rows : 148u * 32u;
    rms_norm_kernel<<<grid, block, 0, stream>>>(w, b, dtype, x, C, rows, eps);
    return cudaGetLastError();
}

cudaError_t embed(const uint32_t* tokens, const __half* input, int dtype, void* output, uint32_t C, uint32_t rows,
                  uint32_t vocab, int32_t* status, cudaStream_t stream) {
    if (rows == 0 || C == 0) return cudaSuccess;
    const uint32_t grid = rows < 148u * 32u ? rows : 148u * 32u;
    embed_kernel<<<grid, 256, 0, stream>>>(tokens, input, dtype, output, C, rows, vocab, status);
    return cudaGetLastError();
}

cudaError_t broadcast(DView input, DView output, cudaStream_t stream) {
    const size_t total = (size_t)output.shape[0] * output.shape[1] * output.shape[2];
    if (total == 0) return cudaSuccess;
    broadcast_kernel<<<ew_grid(total), kEw, 0, stream>>>(input, output);
    return cudaGetLastError();
}

cudaError_t blend(const float* factor, DView input, DView output, cudaStream_t stream) {
    const size_t total = (size_t)output.shape[0] * output.shape[1] * output.shape[2];
    if (total == 0) return cudaSuccess;
    blend_kernel<<<ew_grid(total), kEw, 0, stream>>>(factor, input, output);
    return cudaGetLastError();
}

cudaError_t blend_lora(const float* factor, DView xa, DView xb, DView output, uint32_t K, cudaStream_t stream) {
    const size_t total = (size_t)output.shape[0] * output.shape[1] * output.shape[2];
    if (total == 0) return cudaSuccess;
    blend_lora_kernel<<<ew_grid(total), kEw, 0, stream>>>(factor, xa, xb, output, K);
    return cudaGetLastError();
}

cudaError_t token_shift(const uint32_t* cursors, int wide, DView time_mix, DView state, DView input, DView output,
                        int reversed, cudaStream_t stream) {
    const size_t total = (size_t)output.shape[0] * output.shape[1] * output.shape[2];
    if (total == 0) return cudaSuccess;
    if (token_shift_vec(cursors, wide, time_mix, nullptr, state, input, output, reversed, stream)) return cudaGetLastError();
    token_shift_kernel<<<ew_grid(total), kEw, 0, stream>>>(cursors, wide, time_mix, state, input, output, reversed);
    return cudaGetLastError();
}

cudaError_t token_shift_multi(const ShiftMultiArgs& a, cudaStream_t stream) {
    const size_t total = (size_t)a.C * a.T;
    if (total == 0 || a.count == 0) return cudaSuccess;
    if (token_shift_multi_vec(a, stream)) return cudaGetLastError();
    token_shift_multi_kernel<<<ew_grid(total), kEw, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t pack_v7(const PackV7Args& p, cudaStream_t stream) {
    if (p.rows == 0 || p.S == 0) return cudaSuccess;
    const uint32_t grid = p.rows < 148u * 32u ? p.rows : 148u * 32u;
    pack_v7_kernel<<<grid, 32, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t shift_carry(const uint32_t* cursors, int wide, DView state, int dtype, const void* x, uint32_t C, uint32_t T,
                        cudaStream_t stream) {
    const size_t total = (size_t)C * T;
    if (total == 0) return cudaSuccess;
    shift_carry_kernel<<<ew_grid(total), kEw, 0, stream>>>(cursors, wide, state, dtype, x, C, T);
    return cudaGetLastError();
}

cudaError_t channel_mix(const uint32_t* cursors, int wide, DView state, int dtype, const void* r, const void* v,
                        void* x, uint32_t C, uint32_t T, int v7, cudaStream_t stream) {
    const size_t total = (size_t)C * T;
    if (total == 0) return cudaSuccess;
    if (channel_mix_vec(cursors, wide, state, dtype, r, v, x, nullptr, C, T, v7, stream)) return cudaGetLastError();
    channel_mix_kernel<<<ew_grid(total), kEw, 0, stream>>>(cursors, wide, state, dtype, r, v, x, C, T, v7);
    return cudaGetLastError();
}

cudaError_t binary(int is_mul, DView input, DView output, int act_x, int act_y, int act_out, cudaStream_t stream) {
    const size_t total = (size_t)output.shape[0] * output.shape[1] * output.shape[2];
    if (total == 0) return cudaSuccess;
    if (binary_vec(is_mul, input, output, act_x, act_y, act_out, stream)) return cudaGetLastError();
    binary_kernel<<<ew_grid(total), kEw, 0, stream>>>(is_mul, input, output, act_x, act_y, act_out);
    return cudaGetLastError();
}

cudaError_t activate(DView x, int act, cudaStream_t stream) {
    const size_t total = (size_t)x.shape[0] * x.shape[1] * x.shape[2];
    if (total == 0) return cudaSuccess;
    if (activate_vec(x, act, stream)) return cudaGetLastError();
    activate_kernel<<<ew_grid(total), kEw, 0, stream>>>(x, act);
    return cudaGetLastError();
}

cudaError_t blit(DView input, DView output, int transpose, cudaStream_t stream) {
    const size_t total = (size_t)input.shape[0] * input.shape[1] * input.shape[2];
    if (total == 0) return cudaSuccess;
    if (!transpose && blit_vec(input, output, stream)) return cudaGetLastError();
    blit_kernel<<<ew_grid(total), kEw, 0, stream>>>(input, output, transpose);
    return cudaGetLastError();
}

cudaError_t lerp(DView input, DView output, DView factor, int reversed, cudaStream_t stream) {
    const size_t total = (size_t)output.shape[0] * output.shape[1] * output.shape[2];
    if (total == 0) return cudaSuccess;
    lerp_kernel<<<ew_grid(total), kEw, 0, stream>>>(input, output, factor, reversed);
    return cudaGetLastError();
}

cudaError_t affine(int dtype, void* x, size_t len, float scale, float bias, cudaStream_t stream) {
    if (len == 0) return cudaSuccess;
    affine_kernel<<<ew_grid(len), kEw, 0, stream>>>(dtype, x, len, scale, bias);
    return cudaGetLastError();
}

cudaError_t control_k_v7(const __half* p, DView a, DView k, cudaStream_t stream) {
    const size_t total = (size_t)k.shape[0] * k.shape[1] * k.shape[2];
    if (total == 0) return cudaSuccess;
    control_k_kernel<<<ew_grid(total), kEw, 0, stream>>>(p, a, k);
    return cudaGetLastError();
}

}  // namespace k
}  // namespace wrk
