// CPU oracle for the quantized-matmul + WKV inference path of web-rwkv.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain scalar C++, the arithmetic of
// the reference's compute shaders so that the CUDA kernels can be checked against it.
// It is never linked into, imported by, or called from the product library; only the
// test-suite, the smoke check and the CPU-baseline leg of the benchmark may load it.
//
// Parity status: the reference ships no stored golden vectors for this path (its own
// tests regenerate inputs from a third-party RNG and assert tolerances only), and the
// reference itself (Rust + WGSL through wgpu) cannot be built or run where this oracle
// is developed.  The quantizers and matmuls are pinned against the *properties* asserted
// by the reference's tests (src/tensor/ops.rs:2914-3257) and the scheduler against its
// three known-answer tests; the WKV recurrences, token shift, channel mix, group norm and
// end-to-end logits have no reference test at all: for those, PARITY IS UNPINNED and this
// restatement of the shader text is the only arbiter.
//
// Build: g++ -O2 -ffp-contract=off -mf16c -fopenmp -shared -fPIC (see oracle/Makefile).
// Every function cites the reference file:line it follows.
//
// Conventions (reference: src/tensor/shape.rs:96-99, src/tensor/mod.rs:28-32):
//   shape [x, y, z, w] with x fastest; a view keeps {shape, stride, offset}; element
//   (c, t, b) of a view lives at ((b + off.z) * stride.y + (t + off.y)) * stride.x + c + off.x.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

enum { ORC_F32 = 0, ORC_F16 = 1 };
enum { ORC_ACT_NONE = 0, ORC_ACT_SQUARED_RELU, ORC_ACT_TANH, ORC_ACT_STABLE_EXP, ORC_ACT_OPPOSITE_EXP,
       ORC_ACT_SOFTPLUS, ORC_ACT_SIGMOID, ORC_ACT_SILU };
enum { ORC_MAT_FP16 = 0, ORC_MAT_INT8 = 1, ORC_MAT_NF4 = 2 };

typedef struct {
    void* data;
    int32_t dtype;  // ORC_F32 / ORC_F16
    uint32_t shape[4];
    uint32_t stride[4];
    uint32_t offset[4];
} orc_view;

}  // extern "C"

namespace {

inline float h2f(uint16_t u) {
    _Float16 h;
    std::memcpy(&h, &u, 2);
    return (float)h;
}
inline uint16_t f2h(float f) {
    _Float16 h = (_Float16)f;  // round-to-nearest-even, as pack2x16float
    uint16_t u;
    std::memcpy(&u, &h, 2);
    return u;
}

inline size_t vindex(const orc_view& v, uint32_t c, uint32_t t, uint32_t b) {
    return ((size_t)(b + v.offset[2]) * v.stride[1] + (t + v.offset[1])) * v.stride[0] + c + v.offset[0];
}
inline float vload(const orc_view& v, size_t i) {
    return v.dtype == ORC_F16 ? h2f(((const uint16_t*)v.data)[i]) : ((const float*)v.data)[i];
}
inline void vstore(const orc_view& v, size_t i, float x) {
    if (v.dtype == ORC_F16) ((uint16_t*)v.data)[i] = f2h(x);
    else ((float*)v.data)[i] = x;
}

// Activation functions: src/tensor/ops.rs:205-235.
inline float activate(int act, float x) {
    switch (act) {
        case ORC_ACT_SQUARED_RELU: { float p = std::max(x, 0.0f); return p * p; }
        case ORC_ACT_TANH: return x > 42.0f ? 1.0f : std::tanh(x);
        case ORC_ACT_STABLE_EXP: return std::exp(-std::exp(x));
        case ORC_ACT_OPPOSITE_EXP: return -std::exp(x);
        case ORC_ACT_SOFTPLUS: return std::log(1.0f + std::exp(x));
        case ORC_ACT_SIGMOID: return 1.0f / (1.0f + std::exp(-x));
        case ORC_ACT_SILU: return x / (1.0f + std::exp(-x));
        default: return x;
    }
}

struct Cursor { uint32_t batch, token, len; };
// Packed form: src/tensor/mod.rs:53-60 and e.g. time_mix_v6.wgsl:49-56 (8-bit batch, 16-bit
// token, 8-bit len: a 256-token run wraps to len 0).  Wide form: three u32 per token.
inline Cursor cursor_at(const uint32_t* cursors, int wide, uint32_t t) {
    Cursor c;
    if (wide) {
        c.batch = cursors[3 * t]; c.token = cursors[3 * t + 1]; c.len = cursors[3 * t + 2];
    } else {
        uint32_t x = cursors[t];
        c.batch = x & 0xffu; c.token = (x >> 8) & 0xffffu; c.len = (x >> 24) & 0xffu;
    }
    return c;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------------
// Int8 quantizer.  src/shaders/quant_mat_int8.wgsl:24-59, src/tensor/ops.rs:2393-2486.
// Flat blocks of 128 f16 values: (min, max) stored as an f16 pair; each value becomes
// floor(0.5 + 255 * clamp((v - min) / (max - min), 0, 1)) with every f32 operation rounded
// separately.  A degenerate block (max == min → 0/0) maps to 0 (dequantizes to min exactly).
// ---------------------------------------------------------------------------------------
void orc_quantize_mat_int8(const uint16_t* input, uint64_t len, uint16_t* minmax, uint8_t* output) {
    const uint64_t nblk = (len + 127) / 128;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < (int64_t)nblk; ++b) {
        const uint64_t s = (uint64_t)b * 128, e = std::min<uint64_t>(s + 128, len);
        float mn = 65504.0f, mx = -65504.0f;
        for (uint64_t i = s; i < e; ++i) {
            float v = h2f(input[i]);
            mn = std::min(v, mn);
            mx = std::max(v, mx);
        }
        minmax[2 * b] = f2h(mn);
        minmax[2 * b + 1] = f2h(mx);
        const float range = mx - mn;
        for (uint64_t i = s; i < e; ++i) {
            float v = h2f(input[i]);
            float x = (v - mn) / range;
            if (!(x > 0.0f)) x = 0.0f;  // also catches NaN
            if (x > 1.0f) x = 1.0f;
            float q = std::floor(0.5f + 255.0f * x);
            output[i] = (uint8_t)q;
        }
    }
}

// ---------------------------------------------------------------------------------------
// NF4 quantizer.  src/shaders/quant_mat_nf4.wgsl:24-81, src/tensor/ops.rs:2488-2589.
// Flat blocks of 64: absmax (exact, stored f16); a = 1/absmax (f32 division), x = v * a;
// index = last j with |table[j] - x| <= running minimum, starting from (1.0, index 0).
// Element i of an 8-group occupies bits 4i..4i+3 of a little-endian u32, i.e. even flat
// elements sit in the low nibble of byte e/2.
// ---------------------------------------------------------------------------------------
void orc_quantize_mat_nf4(const uint16_t* input, uint64_t len, const float* table, uint16_t* absmax,
                          uint8_t* output) {
    const uint64_t nblk = (len + 63) / 64;
    std::memset(output, 0, (len + 1) / 2);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < (int64_t)nblk; ++b) {
        const uint64_t s = (uint64_t)b * 64, e = std::min<uint64_t>(s + 64, len);
        float mx = 0.0f;
        for (uint64_t i = s; i < e; ++i) mx = std::max(std::fabs(h2f(input[i])), mx);
        absmax[b] = f2h(mx);
        const float a = 1.0f / mx;
        for (uint64_t i = s; i < e; ++i) {
            const float x = h2f(input[i]) * a;
            float min_err = 1.0f;
            uint32_t min_index = 0;
            for (uint32_t j = 0; j < 16; ++j) {
                const float err = std::fabs(table[j] - x);
                if (err <= min_err) { min_err = err; min_index = j; }
            }
            output[i >> 1] |= (uint8_t)(min_index << ((i & 1) * 4));
        }
    }
}

// ---------------------------------------------------------------------------------------
// Matrix-vector / matrix-matrix product with fp16, Int8 or NF4 weights.
//   vec: src/shaders/matmul_vec_{fp16,int8,nf4}.wgsl (128 strided partial sums + tree reduce)
//   mat: src/shaders/matmul_mat_{fp16,int8,nf4}.wgsl (sequential accumulation along K)
// matrix: [K, M, B] (NF4: K/2 bytes per row); input view [K, N, B]; output view [M, N, B].
// scale: Int8 → f16 (min, max) pairs per 128 flat elements; NF4 → f16 absmax per 64.
// Dequant: Int8 fma(q/255, max-min, min) (matmul_vec_int8.wgsl:89); NF4 table[nib]*absmax.
// mode 0 = vec arithmetic order, 1 = mat arithmetic order.
// ---------------------------------------------------------------------------------------
int orc_matmul(int kind, int mode, const void* matrix, const uint16_t* scale, const float* table,
               uint32_t K, uint32_t M, uint32_t B, const orc_view* input, const orc_view* output, int act) {
    const uint32_t N = output->shape[1];
    if (input->shape[0] != K || output->shape[0] != M || input->shape[1] != N || input->shape[2] != B ||
        output->shape[2] != B)
        return -5;
    for (uint32_t b = 0; b < B; ++b) {
        std::vector<float> xf((size_t)N * K);
#pragma omp parallel for schedule(static)
        for (int64_t n = 0; n < (int64_t)N; ++n)
            for (uint32_t k = 0; k < K; ++k)
                xf[(size_t)n * K + k] = vload(*input, vindex(*input, k, (uint32_t)n, b));
#pragma omp parallel
        {
            std::vector<float> w(K);
#pragma omp for schedule(static)
            for (int64_t m = 0; m < (int64_t)M; ++m) {
                const size_t row = ((size_t)b * M + m) * K;  // flat element index of (b, m, 0)
                if (kind == ORC_MAT_FP16) {
                    const uint16_t* p = (const uint16_t*)matrix + row;
                    for (uint32_t k = 0; k < K; ++k) w[k] = h2f(p[k]);
                } else if (kind == ORC_MAT_INT8) {
                    const uint8_t* p = (const uint8_t*)matrix + row;
                    for (uint32_t k = 0; k < K; ++k) {
                        const size_t blk = (row + k) / 128;
                        const float mn = h2f(scale[2 * blk]), mx = h2f(scale[2 * blk + 1]);
                        w[k] = std::fmaf((float)p[k] / 255.0f, mx - mn, mn);
                    }
                } else {
                    const uint8_t* p = (const uint8_t*)matrix + row / 2;
                    for (uint32_t k = 0; k < K; ++k) {
                        const uint32_t nib = (p[k >> 1] >> ((k & 1) * 4)) & 15u;
                        w[k] = table[nib];  // absmax applied below, in the order each shader uses
                    }
                }
                for (uint32_t n = 0; n < N; ++n) {
                    const float* x = xf.data() + (size_t)n * K;
                    float acc;
                    if (mode == 0) {
                        // 128 lanes, lane i takes 4-groups (NF4: 8-groups) i, i+128, ...; tree reduce.
                        float lane[128];
                        const uint32_t g = kind == ORC_MAT_NF4 ? 8 : 4;
                        const uint32_t ngroup = K / g;
                        for (uint32_t i = 0; i < 128; ++i) {
                            float s = 0.0f;
                            for (uint32_t q = i; q < ngroup; q += 128) {
                                if (kind == ORC_MAT_NF4) {
                                    const float a = h2f(scale[(row + q * 8) / 64]);
                                    for (uint32_t hh = 0; hh < 2; ++hh) {
                                        const uint32_t k0 = q * 8 + hh * 4;
                                        float d = w[k0] * x[k0];
                                        d += w[k0 + 1] * x[k0 + 1];
                                        d += w[k0 + 2] * x[k0 + 2];
                                        d += w[k0 + 3] * x[k0 + 3];
                                        s = std::fmaf(d, a, s);  // matmul_vec_nf4.wgsl:138,149
                                    }
                                } else {
                                    const uint32_t k0 = q * 4;
                                    float d = w[k0] * x[k0];
                                    d += w[k0 + 1] * x[k0 + 1];
                                    d += w[k0 + 2] * x[k0 + 2];
                                    d += w[k0 + 3] * x[k0 + 3];
                                    s += d;
                                }
                            }
                            lane[i] = s;
                        }
                        for (uint32_t st = 64; st > 0; st >>= 1)
                            for (uint32_t i = 0; i < st; ++i) lane[i] += lane[i + st];
                        acc = lane[0];
                    } else {
                        acc = 0.0f;
                        for (uint32_t k0 = 0; k0 < K; k0 += 4) {
                            float a = 1.0f;
                            if (kind == ORC_MAT_NF4) a = h2f(scale[(row + k0) / 64]);
                            float d;
                            if (kind == ORC_MAT_NF4) {  // (absmax * table) * x: matmul_mat_nf4.wgsl:154-159
                                d = (a * w[k0]) * x[k0];
                                d += (a * w[k0 + 1]) * x[k0 + 1];
                                d += (a * w[k0 + 2]) * x[k0 + 2];
                                d += (a * w[k0 + 3]) * x[k0 + 3];
                            } else {
                                d = w[k0] * x[k0];
                                d += w[k0 + 1] * x[k0 + 1];
                                d += w[k0 + 2] * x[k0 + 2];
                                d += w[k0 + 3] * x[k0 + 3];
                            }
                            acc += d;
                        }
                    }
                    vstore(*output, vindex(*output, (uint32_t)m, n, b), activate(act, acc));
                }
            }
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------------------
// WKV v5 / v6.  src/shaders/time_mix_v5.wgsl:82-157, time_mix_v6.wgsl:82-157.
//   k, v, r, x: [S, H, T] (x's dtype for all four); time_decay: f32 [S, H] (v5, per_token = 0)
//   or [S, H, T] (v6, per_token = 1), already activated; time_first: f32 [S, H];
//   state view: f32 [S*H, S+1, B]: row 0 = token-shift carry, row 1+i = key index i.
// Per token t (sequence b = cursor.batch), head h, value column j:
//   y_j = sum_i r_i * fma(u_i, k_i * v_j, S_ij);   S_ij <- fma(w_i, S_ij, k_i * v_j)
// and, at the last token of the sequence's run, state row 0 <- x_in[t] before x[t] <- y.
// ---------------------------------------------------------------------------------------
int orc_time_mix_v56(int per_token_decay, const uint32_t* cursors, int wide, const float* time_decay,
                     const float* time_first, const orc_view* state, int dtype, const void* k, const void* v,
                     const void* r, void* x, uint32_t S, uint32_t H, uint32_t T) {
    const uint32_t C = S * H;
    orc_view kv = {const_cast<void*>(k), dtype, {C, T, 1, 1}, {C, T, 1, 1}, {0, 0, 0, 0}};
    orc_view vv = kv, rv = kv, xv = kv;
    vv.data = const_cast<void*>(v); rv.data = const_cast<void*>(r); xv.data = x;
    float* st = (float*)state->data;
    for (uint32_t t = 0; t < T; ++t) {
        const Cursor cur = cursor_at(cursors, wide, t);
        if (t - cur.token + 1u == cur.len) {
            const uint32_t src = cur.token + cur.len - 1u;
            for (uint32_t c = 0; c < C; ++c)
                st[vindex(*state, c, 0, cur.batch)] = vload(xv, (size_t)src * C + c);
        }
#pragma omp parallel for schedule(static)
        for (int64_t c = 0; c < (int64_t)C; ++c) {
            const uint32_t h = (uint32_t)c / S;
            const float vj = vload(vv, (size_t)t * C + c);
            float y = 0.0f;
            for (uint32_t i = 0; i < S; ++i) {
                const size_t hi = (size_t)h * S + i;
                const float kk = vload(kv, (size_t)t * C + hi);
                const float rr = vload(rv, (size_t)t * C + hi);
                const float uu = time_first[hi];
                const float ww = per_token_decay ? time_decay[(size_t)t * C + hi] : time_decay[hi];
                const size_t si = vindex(*state, (uint32_t)c, i + 1, cur.batch);
                const float ss = st[si];
                const float kvp = kk * vj;
                y += rr * std::fmaf(uu, kvp, ss);
                st[si] = std::fmaf(ww, ss, kvp);
            }
            // all reads of x[t] for the carry happened above, before this store
            vstore(xv, (size_t)t * C + c, y);
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------------------
// WKV v7.  src/shaders/time_mix_v7.wgsl:143-221.
//   r, w, x: [S, H, T]; n: [S, H, T, 4] = stacked k, v, a, kk; state as above.
//   w_i = exp(-0.606531 * sigmoid(w_raw_i));  sa_j = sum_i S_ij * (-kk_i);
//   S_ij <- S_ij * w_i + k_i * v_j + sa_j * (kk_i * a_i);  y_j = sum_i r_i * S_ij (new S).
// ---------------------------------------------------------------------------------------
int orc_time_mix_v7(const uint32_t* cursors, int wide, const orc_view* state, int dtype, const void* r,
                    const void* w, const void* n, void* x, uint32_t S, uint32_t H, uint32_t T) {
    const uint32_t C = S * H;
    orc_view rv = {const_cast<void*>(r), dtype, {C, T, 1, 1}, {C, T, 1, 1}, {0, 0, 0, 0}};
    orc_view wv = rv, nv = rv, xv = rv;
    wv.data = const_cast<void*>(w); nv.data = const_cast<void*>(n); xv.data = x;
    const size_t plane = (size_t)T * C;
    float* st = (float*)state->data;
    std::vector<float> rr(C), ww(C), kk(C), aa(C), bb(C);
    for (uint32_t t = 0; t < T; ++t) {
        const Cursor cur = cursor_at(cursors, wide, t);
        if (t - cur.token + 1u == cur.len) {
            const uint32_t src = cur.token + cur.len - 1u;
            for (uint32_t c = 0; c < C; ++c)
                st[vindex(*state, c, 0, cur.batch)] = vload(xv, (size_t)src * C + c);
        }
        for (uint32_t c = 0; c < C; ++c) {
            const size_t ti = (size_t)t * C + c;
            rr[c] = vload(rv, ti);
            const float wr = vload(wv, ti);
            ww[c] = std::exp(-0.606531f * (1.0f / (1.0f + std::exp(-wr))));
            kk[c] = vload(nv, ti);
            const float a = vload(nv, ti + 2 * plane);
            const float kkk = vload(nv, ti + 3 * plane);
            aa[c] = -kkk;
            bb[c] = kkk * a;
        }
#pragma omp parallel for schedule(static)
        for (int64_t c = 0; c < (int64_t)C; ++c) {
            const uint32_t h = (uint32_t)c / S;
            float sa = 0.0f;
            for (uint32_t i = 0; i < S; ++i)
                sa += st[vindex(*state, (uint32_t)c, i + 1, cur.batch)] * aa[h * S + i];
            const float vj = vload(nv, (size_t)t * C + c + plane);
            float y = 0.0f;
            for (uint32_t i = 0; i < S; ++i) {
                const size_t hi = (size_t)h * S + i;
                const size_t si = vindex(*state, (uint32_t)c, i + 1, cur.batch);
                float ss = st[si];
                ss = ss * ww[hi] + kk[hi] * vj + sa * bb[hi];
                y += rr[hi] * ss;
                st[si] = ss;
            }
            vstore(xv, (size_t)t * C + c, y);
        }
    }
    return 0;
}

// time_first_v7: src/shaders/time_mix_v7.wgsl:223-262.  x_j += (sum_i u_i k_i r_i) * v_j per head.
int orc_time_first_v7(const uint16_t* u, int dtype, const void* r, const void* n, void* x, uint32_t S,
                      uint32_t H, uint32_t T) {
    const uint32_t C = S * H;
    orc_view rv = {const_cast<void*>(r), dtype, {C, T, 1, 1}, {C, T, 1, 1}, {0, 0, 0, 0}};
    orc_view nv = rv, xv = rv;
    nv.data = const_cast<void*>(n); xv.data = x;
    const size_t plane = (size_t)T * C;
    for (uint32_t t = 0; t < T; ++t)
        for (uint32_t h = 0; h < H; ++h) {
            // the shader reduces vec4 partials with a halving tree, then dots with (1,1,1,1)
            float part[64][4];
            const uint32_t groups = S / 4;
            for (uint32_t g = 0; g < groups; ++g)
                for (uint32_t e = 0; e < 4; ++e) {
                    const size_t i = (size_t)t * C + h * S + g * 4 + e;
                    part[g][e] = h2f(u[h * S + g * 4 + e]) * vload(nv, i) * vload(rv, i);
                }
            for (uint32_t step = groups >> 1; step > 0; step >>= 1)
                for (uint32_t g = 0; g < step; ++g)
                    for (uint32_t e = 0; e < 4; ++e) part[g][e] += part[g + step][e];
            const float xx = part[0][0] + part[0][1] + part[0][2] + part[0][3];
            for (uint32_t j = 0; j < S; ++j) {
                const size_t i = (size_t)t * C + h * S + j;
                vstore(xv, i, vload(xv, i) + xx * vload(nv, i + plane));
            }
        }
    return 0;
}

// ---------------------------------------------------------------------------------------
// Supporting ops needed to produce logits (not individually performance-graded).
// ---------------------------------------------------------------------------------------

// layer_norm / group_norm: src/shaders/layer_norm.wgsl:62-121, ops.rs:407-508.
// x: [C, T, B] with one statistic per (t, b); for group norm x is [S, H, T] and the
// statistic is per (head, token) with w, b indexed [S, H].  Mean and variance in f32
// (Welford), result fma((x - mean) * rsqrt(var + eps), w, b).
int orc_layer_norm(const uint16_t* w, const uint16_t* b, int dtype, void* x, uint32_t C, uint32_t rows,
                   uint32_t wrows, float eps) {
    orc_view xv = {x, dtype, {C, rows, 1, 1}, {C, rows, 1, 1}, {0, 0, 0, 0}};
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; ++row) {
        float mu = 0.0f, m2 = 0.0f;
        for (uint32_t c = 0; c < C; ++c) {
            const float val = vload(xv, (size_t)row * C + c);
            const float d = val - mu;
            mu += d / (float)(c + 1);
            m2 += d * (val - mu);
        }
        const float var = m2 / (float)C + eps;
        const float dev = 1.0f / std::sqrt(var);
        const size_t wb = (size_t)((uint32_t)row % wrows) * C;
        for (uint32_t c = 0; c < C; ++c) {
            const size_t i = (size_t)row * C + c;
            const float val = (vload(xv, i) - mu) * dev;
            vstore(xv, i, std::fmaf(val, h2f(w[wb + c]), h2f(b[wb + c])));
        }
    }
    return 0;
}

// time_mix_v4: src/shaders/time_mix_v4.wgsl:62-124.  State view [C, 4, B]: row 0 = token-shift carry, rows 1..3 =
// (aa, bb, pp).  Every token rewrites row 0 from the input x of its sequence's last token of the job (read before
// that slot of x is overwritten), then x_t = sigmoid(r) (e1 aa + e2 v) / (e1 bb + e2) and the (aa, bb, pp) update.
int orc_time_mix_v4(const uint32_t* cursors, int wide, const float* time_decay, const float* time_first,
                    const orc_view* state, int dtype, const void* k, const void* v, const void* r, void* x, uint32_t C,
                    uint32_t T) {
    orc_view kv = {const_cast<void*>(k), dtype, {C, T, 1, 1}, {C, T, 1, 1}, {0, 0, 0, 0}};
    orc_view vv_ = kv, rv = kv, xv = kv;
    vv_.data = const_cast<void*>(v);
    rv.data = const_cast<void*>(r);
    xv.data = x;
    float* st = (float*)state->data;
    for (uint32_t c = 0; c < C; ++c) {
        const float u = time_first[c], w = time_decay[c];
        for (uint32_t t = 0; t < T; ++t) {
            uint32_t batch, token, len;
            if (wide) {
                batch = cursors[3 * t], token = cursors[3 * t + 1], len = cursors[3 * t + 2];
            } else {
                batch = cursors[t] & 0xffu, token = (cursors[t] >> 8) & 0xffffu, len = (cursors[t] >> 24) & 0xffu;
            }
            const size_t ai = vindex(*state, c, 1, batch), bi = vindex(*state, c, 2, batch), pi = vindex(*state, c, 3, batch);
            float aa = st[ai], bb = st[bi], pp = st[pi];
            const uint32_t last = token + len - 1u;
            if (last < T) st[vindex(*state, c, 0, batch)] = vload(xv, (size_t)last * C + c);
            const size_t ti = (size_t)t * C + c;
            const float kk = vload(kv, ti), vv = vload(vv_, ti);
            const float rr = 1.0f / (1.0f + std::exp(-vload(rv, ti)));
            float ww = u + kk;
            float q = std::max(pp, ww);
            float e1 = std::exp(pp - q), e2 = std::exp(ww - q);
            vstore(xv, ti, rr * (e1 * aa + e2 * vv) / (e1 * bb + e2));
            ww = w + pp;
            q = std::max(ww, kk);
            e1 = std::exp(ww - q);
            e2 = std::exp(kk - q);
            st[ai] = e1 * aa + e2 * vv;
            st[bi] = e1 * bb + e2;
            st[pi] = q;
        }
    }
    return 0;
}

// softmax: src/shaders/softmax.wgsl:52-106.  x <- exp(x - max) / sum exp(x - max) per row of C, f32 math.
int orc_softmax(int dtype, void* x, uint32_t C, uint32_t rows) {
    orc_view xv = {x, dtype, {C, rows, 1, 1}, {C, rows, 1, 1}, {0, 0, 0, 0}};
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; ++row) {
        float mx = -1.0e30f;
        for (uint32_t c = 0; c < C; ++c) mx = std::max(mx, vload(xv, (size_t)row * C + c));
        float sum = 0.0f;
        for (uint32_t c = 0; c < C; ++c) sum += std::exp(vload(xv, (size_t)row * C + c) - mx);
        for (uint32_t c = 0; c < C; ++c) {
            const size_t i = (size_t)row * C + c;
            vstore(xv, i, std::exp(vload(xv, i) - mx) / sum);
        }
    }
    return 0;
}

// recenter: src/shaders/normalize.wgsl:46-80.  x -= mean(x) per row of C.
int orc_recenter(int dtype, void* x, uint32_t C, uint32_t rows) {
    orc_view xv = {x, dtype, {C, rows, 1, 1}, {C, rows, 1, 1}, {0, 0, 0, 0}};
    for (uint32_t row = 0; row < rows; ++row) {
        float s = 0.0f;
        for (uint32_t c = 0; c < C; ++c) s += vload(xv, (size_t)row * C + c);
        const float mean = s / (float)C;
        for (uint32_t c = 0; c < C; ++c) {
            const size_t i = (size_t)row * C + c;
            vstore(xv, i, vload(xv, i) - mean);
        }
    }
    return 0;
}

// rms_norm: src/shaders/normalize.wgsl:82-118.  x = fma(x * rsqrt(mean x^2 + eps), w, b) per row of C.
int orc_rms_norm(const uint16_t* w, const uint16_t* b, int dtype, void* x, uint32_t C, uint32_t rows, float eps) {
    orc_view xv = {x, dtype, {C, rows, 1, 1}, {C, rows, 1, 1}, {0, 0, 0, 0}};
    for (uint32_t row = 0; row < rows; ++row) {
        float s = 0.0f;
        for (uint32_t c = 0; c < C; ++c) {
            const float val = vload(xv, (size_t)row * C + c);
            s += val * val;
        }
        const float norm = 1.0f / std::sqrt(s / (float)C + eps);
        for (uint32_t c = 0; c < C; ++c) {
            const size_t i = (size_t)row * C + c;
            vstore(xv, i, std::fma(vload(xv, i) * norm, h2f(w[c]), h2f(b[c])));
        }
    }
    return 0;
}

// embed: src/shaders/embed.wgsl:21-41.  output[:, row] = input[:, tokens[row]] for row = b * T + t.
int orc_embed(const uint32_t* tokens, const uint16_t* input, int dtype, void* output, uint32_t C, uint32_t rows) {
    orc_view ov = {output, dtype, {C, rows, 1, 1}, {C, rows, 1, 1}, {0, 0, 0, 0}};
    for (uint32_t row = 0; row < rows; ++row)
        for (uint32_t c = 0; c < C; ++c) vstore(ov, (size_t)row * C + c, h2f(input[(size_t)tokens[row] * C + c]));
    return 0;
}

// broadcast: src/shaders/reshape.wgsl:35-57.  output[c, t, b] = input[c, t % in.T, b % in.B].
int orc_broadcast(const orc_view* input, const orc_view* output) {
    for (uint32_t b = 0; b < output->shape[2]; ++b)
        for (uint32_t t = 0; t < output->shape[1]; ++t)
            for (uint32_t c = 0; c < output->shape[0]; ++c)
                vstore(*output, vindex(*output, c, t, b),
                       vload(*input, vindex(*input, c, t % input->shape[1], b % input->shape[2])));
    return 0;
}

// blend: src/shaders/blend.wgsl:38-60.  output = factor.x * input + factor.y * output.
int orc_blend(const float* factor, const orc_view* input, const orc_view* output) {
    for (uint32_t b = 0; b < output->shape[2]; ++b)
        for (uint32_t t = 0; t < output->shape[1]; ++t)
            for (uint32_t c = 0; c < output->shape[0]; ++c) {
                const size_t o = vindex(*output, c, t, b);
                vstore(*output, o, factor[0] * vload(*input, vindex(*input, c, t, b)) + factor[1] * vload(*output, o));
            }
    return 0;
}

// blend_lora: src/shaders/blend_lora.wgsl:44-108.  output[m, n, b] = factor.x * sum_k xa[k, m, b] * xb[k, n, b] +
// factor.y * output[m, n, b]; the sum runs over min(K_a, K_b) / 4 groups of four, in f32.
int orc_blend_lora(const float* factor, const orc_view* xa, const orc_view* xb, const orc_view* output) {
    const uint32_t K = std::min(xa->shape[0] / 4, xb->shape[0] / 4) * 4;
    for (uint32_t b = 0; b < output->shape[2]; ++b)
        for (uint32_t n = 0; n < output->shape[1]; ++n)
            for (uint32_t m = 0; m < output->shape[0]; ++m) {
                float sum = 0.0f;
                for (uint32_t k = 0; k < K; ++k)
                    sum += vload(*xa, vindex(*xa, k, m, b)) * vload(*xb, vindex(*xb, k, n, b));
                const size_t o = vindex(*output, m, n, b);
                vstore(*output, o, factor[0] * sum + factor[1] * vload(*output, o));
            }
    return 0;
}

// l2_norm: src/shaders/normalize.wgsl:120-152.  x *= rsqrt(sum x^2 + eps) per row of C.
int orc_l2_norm(int dtype, void* x, uint32_t C, uint32_t rows, float eps) {
    orc_view xv = {x, dtype, {C, rows, 1, 1}, {C, rows, 1, 1}, {0, 0, 0, 0}};
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; ++row) {
        float s = 0.0f;
        for (uint32_t c = 0; c < C; ++c) {
            const float val = vload(xv, (size_t)row * C + c);
            s += val * val;
        }
        const float norm = 1.0f / std::sqrt(s + eps);
        for (uint32_t c = 0; c < C; ++c) {
            const size_t i = (size_t)row * C + c;
            vstore(xv, i, vload(xv, i) * norm);
        }
    }
    return 0;
}

// token_shift: src/shaders/token_shift.wgsl:85-117, ops.rs:1393-1461.
// time_mix view [C, T or 1, count]; state view [C, rows, B] (row 0 used); input [C, T] (contiguous);
// output [C, T, count].  reversed: out = mix(x_t, prev, f) = x_t + (prev - x_t) * f.
int orc_token_shift(const uint32_t* cursors, int wide, const orc_view* time_mix, const orc_view* state,
                    int in_dtype, const void* input, const orc_view* output, int reversed) {
    const uint32_t C = output->shape[0], T = output->shape[1], count = output->shape[2];
    orc_view xin = {const_cast<void*>(input), in_dtype, {C, T, 1, 1}, {C, T, 1, 1}, {0, 0, 0, 0}};
    for (uint32_t z = 0; z < count; ++z)
        for (uint32_t t = 0; t < T; ++t) {
            const Cursor cur = cursor_at(cursors, wide, t);
            const uint32_t tok = t - cur.token;
            for (uint32_t c = 0; c < C; ++c) {
                const float f = vload(*time_mix, vindex(*time_mix, c, time_mix->shape[1] == 1 ? 0 : t, z));
                const float cur_x = vload(xin, (size_t)t * C + c);
                const float prev = tok == 0 ? ((const float*)state->data)[vindex(*state, c, 0, cur.batch)]
                                            : vload(xin, (size_t)(t - 1) * C + c);
                // WGSL mix(a, b, f) = a * (1 - f) + b * f
                const float a = reversed ? cur_x : prev, bb = reversed ? prev : cur_x;
                vstore(*output, vindex(*output, c, t, z), a * (1.0f - f) + bb * f);
            }
        }
    return 0;
}

// channel_mix / channel_mix_v7: src/shaders/channel_mix.wgsl:83-108, ops.rs:1860-1971.
// At a sequence's last token the FFN carry row <- x_in[t]; then x = sigmoid(r) * v (v7: x = v).
int orc_channel_mix(const uint32_t* cursors, int wide, const orc_view* state, int dtype, const void* r,
                    const void* v, void* x, uint32_t C, uint32_t T, int v7) {
    orc_view xv = {x, dtype, {C, T, 1, 1}, {C, T, 1, 1}, {0, 0, 0, 0}};
    orc_view rv = xv, vv = xv;
    rv.data = const_cast<void*>(r); vv.data = const_cast<void*>(v);
    for (uint32_t t = 0; t < T; ++t) {
        const Cursor cur = cursor_at(cursors, wide, t);
        const uint32_t tok = t - cur.token;
        for (uint32_t c = 0; c < C; ++c) {
            const size_t i = (size_t)t * C + c;
            if (tok + 1u == cur.len) ((float*)state->data)[vindex(*state, c, 0, cur.batch)] = vload(xv, i);
            if (v7) vstore(xv, i, vload(vv, i));
            else vstore(xv, i, (1.0f / (1.0f + std::exp(-vload(rv, i)))) * vload(vv, i));
        }
    }
    return 0;
}

// add_activate / mul_activate: src/shaders/binary.wgsl:37-78, ops.rs:1227-1391.
// out = ACT_OUT(ACT_X(in) op ACT_Y(out)); input broadcasts along token and/or batch when its extent is 1.
int orc_binary(int is_mul, const orc_view* input, const orc_view* output, int act_x, int act_y, int act_out) {
    const uint32_t C = output->shape[0], T = output->shape[1], B = output->shape[2];
    for (uint32_t b = 0; b < B; ++b)
        for (uint32_t t = 0; t < T; ++t)
            for (uint32_t c = 0; c < C; ++c) {
                const float xi = vload(*input, vindex(*input, c, input->shape[1] == 1 ? 0 : t,
                                                      input->shape[2] == 1 ? 0 : b));
                const size_t o = vindex(*output, c, t, b);
                const float yo = vload(*output, o);
                const float ax = activate(act_x, xi), ay = activate(act_y, yo);
                vstore(*output, o, activate(act_out, is_mul ? ax * ay : ax + ay));
            }
    return 0;
}

// activate: src/shaders/activation.wgsl:30-46.
int orc_activate(const orc_view* x, int act) {
    for (uint32_t b = 0; b < x->shape[2]; ++b)
        for (uint32_t t = 0; t < x->shape[1]; ++t)
            for (uint32_t c = 0; c < x->shape[0]; ++c) {
                const size_t i = vindex(*x, c, t, b);
                vstore(*x, i, activate(act, vload(*x, i)));
            }
    return 0;
}

// blit (transpose = 0): src/shaders/blit.wgsl:34-54; transpose of token and batch axes
// (transpose = 1): src/shaders/reshape.wgsl:59-78.  Loop extents are the input's.
int orc_blit(const orc_view* input, const orc_view* output, int transpose) {
    for (uint32_t b = 0; b < input->shape[2]; ++b)
        for (uint32_t t = 0; t < input->shape[1]; ++t)
            for (uint32_t c = 0; c < input->shape[0]; ++c) {
                const float val = vload(*input, vindex(*input, c, t, b));
                vstore(*output, transpose ? vindex(*output, c, b, t) : vindex(*output, c, t, b), val);
            }
    return 0;
}

// lerp: src/shaders/lerp.wgsl:72-93.  y = mix(x, y, f) (reversed: mix(y, x, f)); f broadcasts.
int orc_lerp(const orc_view* input, const orc_view* output, const orc_view* factor, int reversed) {
    const uint32_t C = output->shape[0], T = output->shape[1], B = output->shape[2];
    for (uint32_t b = 0; b < B; ++b)
        for (uint32_t t = 0; t < T; ++t)
            for (uint32_t c = 0; c < C; ++c) {
                const float f = vload(*factor, vindex(*factor, c, factor->shape[1] == 1 ? 0 : t,
                                                      factor->shape[2] == 1 ? 0 : b));
                const float xi = vload(*input, vindex(*input, c, t, b));
                const size_t o = vindex(*output, c, t, b);
                const float yo = vload(*output, o);
                const float a = reversed ? yo : xi, bb = reversed ? xi : yo;
                vstore(*output, o, a * (1.0f - f) + bb * f);
            }
    return 0;
}

// affine: src/shaders/affine.wgsl:16-31.  x = scale * x + bias.
int orc_affine(int dtype, void* x, uint64_t len, float scale, float bias) {
    orc_view xv = {x, dtype, {1, 1, 1, 1}, {1, 1, 1, 1}, {0, 0, 0, 0}};
    for (uint64_t i = 0; i < len; ++i) vstore(xv, i, scale * vload(xv, i) + bias);
    return 0;
}

// control_k_v7: src/shaders/control_k_v7.wgsl:61-75.  k = k * (1 + (a - 1) * p), p: f16 [C].
int orc_control_k_v7(const uint16_t* p, const orc_view* a, const orc_view* k) {
    for (uint32_t b = 0; b < k->shape[2]; ++b)
        for (uint32_t t = 0; t < k->shape[1]; ++t)
            for (uint32_t c = 0; c < k->shape[0]; ++c) {
                const float pp = h2f(p[c]);
                const float av = vload(*a, vindex(*a, c, t, b));
                const size_t o = vindex(*k, c, t, b);
                vstore(*k, o, vload(*k, o) * (1.0f + (av - 1.0f) * pp));
            }
    return 0;
}

// f16 <-> f32 helpers for the Python side (round-to-nearest-even).
void orc_f32_to_f16(const float* in, uint16_t* out, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = f2h(in[i]);
}
// Load-time discount: f16(discount * f32(x)), src/runtime/loader.rs:660-661.
void orc_discount_f16(const uint16_t* in, uint16_t* out, uint64_t n, float discount) {
    for (uint64_t i = 0; i < n; ++i) out[i] = f2h(discount * h2f(in[i]));
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
