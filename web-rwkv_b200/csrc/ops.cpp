// Op builders: the `TensorOp::*` constructors of src/tensor/ops.rs restated over CUDA launches.
// Each builder performs the reference's shape checks, returns the same error kinds, and yields a
// deferred op; nothing runs until the op is submitted.
#include <cmath>

#include "common.h"
#include "kernels/decode.cuh"
#include "kernels/kernels.h"

using namespace wrk;

namespace {

inline int cursors_wide(const wrk_tensor* cursors, uint32_t T) {
    // packed: one u32 per token ([T]); wide: three u32 per token ([3, T] or [3 * T])
    return cursors->len() == (size_t)3 * T && T != 0 ? 1 : 0;
}

int32_t check_cursors(const wrk_tensor* cursors, uint32_t T) {
    WRK_REQUIRE(cursors->dtype == WRK_U32, WRK_ERR_TYPE, "data type mismatch: cursors must be u32");
    WRK_REQUIRE(cursors->len() == T || cursors->len() == (size_t)3 * T, WRK_ERR_SHAPE,
                "tensor shape not match (cursors): %zu entries for %u tokens", cursors->len(), T);
    return WRK_OK;
}

#define REQ_FLOAT(t, what) \
    WRK_REQUIRE(is_float((t)->dtype), WRK_ERR_TYPE, "data type mismatch: %s must be f32 or f16", what)
#define REQ_DTYPE(t, dt, what) \
    WRK_REQUIRE((t)->dtype == (dt), WRK_ERR_TYPE, "data type mismatch: %s has dtype %d, expected %d", what, (t)->dtype, (int)(dt))
#define REQ_NN(...)                                                                      \
    do {                                                                                 \
        const void* _p[] = {__VA_ARGS__};                                                \
        for (auto q : _p) WRK_REQUIRE(q, WRK_ERR_INVALID_ARGUMENT, "null argument");     \
    } while (0)

// Checks the operands of out = act(W x) and fills the kernels' argument block.
int32_t matmul_args(int kind, wrk_tensor* matrix, wrk_tensor* scale, wrk_tensor* quant, const wrk_view* input,
                    const wrk_view* output, int32_t act, k::MatmulArgs* args) {
    REQ_NN(matrix, input, output, input->tensor, output->tensor);
    REQ_FLOAT(input->tensor, "input");
    REQ_FLOAT(output->tensor, "output");
    WRK_REQUIRE(act >= WRK_ACT_NONE && act <= WRK_ACT_SILU, WRK_ERR_INVALID_ARGUMENT, "unknown activation %d", act);
    const uint32_t m = output->shape[0], n = output->shape[1], b = output->shape[2];
    const uint32_t k = input->shape[0];
    if (kind == k::MAT_FP16) {
        REQ_DTYPE(matrix, WRK_F16, "matrix");
        WRK_TRY(check_shape("matrix", matrix->shape, k, m, b, 1));
    } else if (kind == k::MAT_INT8) {
        REQ_NN(scale);
        REQ_DTYPE(matrix, WRK_U8, "matrix");
        REQ_DTYPE(scale, WRK_F16, "minmax");
        const size_t len = matrix->len();
        WRK_TRY(check_shape("minmax", scale->shape, (uint32_t)(((len << 1) + 127) / 128), 1, 1, 1));
        WRK_TRY(check_shape("matrix", matrix->shape, k, m, b, 1));
    } else {
        REQ_NN(scale, quant);
        REQ_DTYPE(matrix, WRK_U8, "matrix");
        REQ_DTYPE(scale, WRK_F16, "absmax");
        REQ_DTYPE(quant, WRK_F32, "quant");
        WRK_TRY(check_shape("quant", quant->shape, 16, 1, 1, 1));
        const size_t len = matrix->len() << 1;
        WRK_TRY(check_shape("absmax", scale->shape, (uint32_t)((len + 63) / 64), 1, 1, 1));
        WRK_TRY(check_shape("matrix", matrix->shape, k >> 1, m, b, 1));
    }
    WRK_TRY(check_view("input", input, k, n, b, 1));
    WRK_TRY(check_view("output", output, m, n, b, 1));

    k::MatmulArgs& a = *args;
    a = k::MatmulArgs{};
    a.kind = kind;
    a.matrix = matrix->ptr();
    a.scale = scale ? static_cast<const __half*>(scale->ptr()) : nullptr;
    a.table = quant ? static_cast<const float*>(quant->ptr()) : nullptr;
    a.K = k;
    a.M = m;
    a.B = b;
    a.N = n;
    a.in = make_dview(*input);
    a.out = make_dview(*output);
    a.act = act;
    a.status = matrix->ctx->device_status;
    return WRK_OK;
}

int32_t matmul_common(const char* name, int kind, wrk_tensor* matrix, wrk_tensor* scale, wrk_tensor* quant,
                      const wrk_view* input, const wrk_view* output, int32_t act, wrk_op** out) {
    REQ_NN(out);
    k::MatmulArgs a;
    WRK_TRY(matmul_args(kind, matrix, scale, quant, input, output, act, &a));
    const uint32_t m = a.M, n = a.N, b = a.B, k = a.K;
    (void)m;
    const int sms = matrix->ctx->num_sms;
    // few tokens, fp16 activations, whole rows: the weight-streaming kernel of the decode path
    const uint32_t need = kind == k::MAT_FP16 ? 32 : 128;
    const size_t in_row0 = a.in.index(0, 0, 0), out_row0 = a.out.index(0, 0, 0);
    const bool stream_ok = b == 1 && n >= 1 && n <= (uint32_t)k::kDecodeMaxTokens && a.in.dtype == WRK_F16 &&
                           k % need == 0 && in_row0 % 8 == 0 && a.in.stride[0] % 8 == 0 &&
                           k::fused_gemv_smem(n, k, k, k::PRO_NONE, 2) <= 200 * 1024;
    if (stream_ok) {
        k::FusedGemvArgs f{};
        f.T = n;
        f.C = k;
        f.prologue = k::PRO_NONE;
        f.epilogue = k::EPI_STORE;
        f.table = a.table;
        f.status = matrix->ctx->device_status;
        f.rescale = 1.0f;
        f.num_problems = 1;
        k::GemvProblem& p = f.p[0];
        p.w = static_cast<const uint8_t*>(a.matrix);
        p.scale = a.scale;
        p.kind = kind;
        p.K = k;
        p.M = m;
        p.x = static_cast<const __half*>(a.in.base) + in_row0;
        p.x_stride = a.in.stride[0];
        p.out = a.out.dtype == WRK_F16 ? static_cast<void*>(static_cast<__half*>(a.out.base) + out_row0)
                                       : static_cast<void*>(static_cast<float*>(a.out.base) + out_row0);
        p.out_stride = a.out.stride[0];
        p.out_dtype = a.out.dtype;
        p.act = act;
        std::vector<k::GemvSegment> table;
        if (k::fused_gemv_partition(f, sms, table)) {
            const uint32_t tshape[4] = {(uint32_t)(table.size() * 4), 1, 1, 1};
            wrk_tensor* tt = nullptr;
            WRK_TRY(wrk_tensor_from_data(matrix->ctx, WRK_U32, tshape, table.data(),
                                         table.size() * sizeof(k::GemvSegment), &tt));
            f.segments = static_cast<const k::GemvSegment*>(tt->ptr());
            k::fused_gemv_inline_partition(f, sms, table);
            *out = new_atom(name, [f, sms](cudaStream_t s) { return k::fused_gemv(f, sms, s); },
                            {matrix, scale, quant, input->tensor, output->tensor, tt});
            wrk_tensor_release(tt);  // the atom keeps the buffer alive
            return WRK_OK;
        }
    }
    *out = new_atom(name, [a, sms](cudaStream_t s) { return k::matmul(a, sms, s); },
                    {matrix, scale, quant, input->tensor, output->tensor});
    return WRK_OK;
}

int32_t time_mix_v56(const char* name, int per_token, wrk_tensor* cursors, wrk_tensor* time_decay,
                     wrk_tensor* time_first, const wrk_view* state, wrk_tensor* k, wrk_tensor* v, wrk_tensor* r,
                     wrk_tensor* x, wrk_op** out, bool blocks = false) {
    REQ_NN(cursors, time_decay, time_first, state, state->tensor, k, v, r, x, out);
    REQ_FLOAT(x, "x");
    REQ_DTYPE(k, x->dtype, "k");
    REQ_DTYPE(v, x->dtype, "v");
    REQ_DTYPE(r, x->dtype, "r");
    REQ_DTYPE(time_decay, WRK_F32, "time_decay");
    REQ_DTYPE(time_first, WRK_F32, "time_first");
    REQ_DTYPE(state->tensor, WRK_F32, "state");
    const Shape4 sh = x->shape;
    const uint32_t S = sh[0], H = sh[1], T = sh[2], stride = S * H;
    WRK_TRY(check_shape("x", sh, S, H, T, 1));
    WRK_TRY(check_shape("k", k->shape, S, H, T, 1));
    WRK_TRY(check_shape("v", v->shape, S, H, T, 1));
    WRK_TRY(check_shape("r", r->shape, S, H, T, 1));
    if (per_token) WRK_TRY(check_shape("time_decay", time_decay->shape, S, H, T, 1));
    else WRK_TRY(check_shape("time_decay", time_decay->shape, S, H, 1, 1));
    WRK_TRY(check_shape("time_first", time_first->shape, S, H, 1, 1));
    WRK_TRY(check_view("state", state, stride, S + 1, state->shape[2], 1));
    WRK_TRY(check_cursors(cursors, T));
    WRK_REQUIRE(S == 32 || S == 64 || S == 128, WRK_ERR_UNSUPPORTED, "head size %u not built (32, 64, 128)", S);

    k::WkvArgs a{};
    a.cursors = static_cast<const uint32_t*>(cursors->ptr());
    a.wide = cursors_wide(cursors, T);
    a.state = make_dview(*state);
    a.S = S; a.H = H; a.T = T; a.B = state->shape[2];
    a.dtype = x->dtype;
    a.time_decay = static_cast<const float*>(time_decay->ptr());
    a.time_first = static_cast<const float*>(time_first->ptr());
    a.per_token_decay = per_token;
    a.k = k->ptr(); a.v = v->ptr(); a.r = r->ptr(); a.x = x->ptr();
    a.status = x->ctx->device_status;
    if (blocks) {
        WRK_REQUIRE(k::time_mix_v56_chunked_supported(a), WRK_ERR_UNSUPPORTED, "time_mix_blocks takes heads of 64 channels");
        *out = new_atom(name, [a](cudaStream_t s) { return k::time_mix_v56_chunked(a, s); },
                        {cursors, time_decay, time_first, state->tensor, k, v, r, x});
        return WRK_OK;
    }
    *out = new_atom(name, [a](cudaStream_t s) { return k::time_mix_v56(a, s); },
                    {cursors, time_decay, time_first, state->tensor, k, v, r, x});
    return WRK_OK;
}

}  // namespace

namespace {

// Regularized incomplete beta function I_x(a, b): continued fraction evaluated with the modified Lentz method.
double beta_cf(double a, double b, double x) {
    const double tiny = 1e-300, eps = 1e-16;
    const double qab = a + b, qap = a + 1.0, qam = a - 1.0;
    double c = 1.0, d = 1.0 - qab * x / qap;
    if (std::fabs(d) < tiny) d = tiny;
    d = 1.0 / d;
    double h = d;
    for (int m = 1; m <= 500; ++m) {
        const int m2 = 2 * m;
        double aa = m * (b - m) * x / ((qam + m2) * (a + m2));
        d = 1.0 + aa * d;
        if (std::fabs(d) < tiny) d = tiny;
        c = 1.0 + aa / c;
        if (std::fabs(c) < tiny) c = tiny;
        d = 1.0 / d;
        h *= d * c;
        aa = -(a + m) * (qab + m) * x / ((a + m2) * (qap + m2));
        d = 1.0 + aa * d;
        if (std::fabs(d) < tiny) d = tiny;
        c = 1.0 + aa / c;
        if (std::fabs(c) < tiny) c = tiny;
        d = 1.0 / d;
        const double del = d * c;
        h *= del;
        if (std::fabs(del - 1.0) < eps) break;
    }
    return h;
}
double reg_inc_beta(double a, double b, double x) {
    if (x <= 0.0) return 0.0;
    if (x >= 1.0) return 1.0;
    const double front = std::exp(std::lgamma(a + b) - std::lgamma(a) - std::lgamma(b) + a * std::log(x) + b * std::log1p(-x));
    if (x < (a + 1.0) / (a + b + 2.0)) return front * beta_cf(a, b, x) / a;
    return 1.0 - front * beta_cf(b, a, 1.0 - x) / b;
}
// Distribution function of Student's t with nu degrees of freedom, and its inverse by bisection (monotone, 200
// halvings of a bracket that doubles until it contains the root: exact to the last bit of a double).
double student_cdf(double t, double nu) {
    const double tail = 0.5 * reg_inc_beta(0.5 * nu, 0.5, nu / (nu + t * t));
    return t >= 0.0 ? 1.0 - tail : tail;
}
double student_quantile(double p, double nu) {
    if (p == 0.5) return 0.0;
    double lo = -1.0, hi = 1.0;
    while (student_cdf(lo, nu) > p) lo *= 2.0;
    while (student_cdf(hi, nu) < p) hi *= 2.0;
    for (int i = 0; i < 200; ++i) {
        const double mid = 0.5 * (lo + hi);
        if (student_cdf(mid, nu) < p) lo = mid;
        else hi = mid;
    }
    return 0.5 * (lo + hi);
}

}  // namespace

extern "C" {

int32_t wrk_nf4_table(float table[16]) {
    // Float4Quant::new, src/tensor/matrix.rs:48-70 (the NormalFloat4 code book)
    static const float q[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
    WRK_REQUIRE(table, WRK_ERR_INVALID_ARGUMENT, "null argument");
    for (int i = 0; i < 16; ++i) table[i] = q[i];
    return WRK_OK;
}

int32_t wrk_sf4_table(double nu, float table[16]) {
    // quantile_student, src/tensor/matrix.rs:29-44: 16 probabilities (7 steps from delta up to 1/2, 9 from 1/2 to
    // 1 - delta), the Student-t quantile of each, divided by the largest.  The reference takes the quantile from
    // the statrs crate (0.18, StudentsT::inverse_cdf); here it is the root of the distribution function, which
    // is written with the regularized incomplete beta function (continued fraction, modified Lentz).
    WRK_REQUIRE(table, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(nu > 0.0 && std::isfinite(nu), WRK_ERR_INVALID_ARGUMENT, "nu must be positive");
    const double delta = (1.0 / 32.0 + 1.0 / 30.0) / 2.0;
    double prob[16];
    const double step_lo = (0.5 - delta) / 7.0, step_hi = (1.0 - delta - 0.5) / 8.0;
    for (int i = 0; i < 7; ++i) prob[i] = delta + step_lo * i;
    for (int i = 0; i < 9; ++i) prob[7 + i] = 0.5 + step_hi * i;
    double q[16], largest = 0.0;
    for (int i = 0; i < 16; ++i) {
        q[i] = student_quantile(prob[i], nu);
        largest = std::max(largest, q[i]);
    }
    for (int i = 0; i < 16; ++i) table[i] = (float)(q[i] / largest);
    return WRK_OK;
}

int32_t wrk_op_quantize_mat_int8(wrk_tensor* input, wrk_tensor* minmax, wrk_tensor* output, wrk_op** out) {
    REQ_NN(input, minmax, output, out);
    REQ_DTYPE(input, WRK_F16, "input");
    REQ_DTYPE(minmax, WRK_F16, "minmax");
    REQ_DTYPE(output, WRK_U8, "output");
    const Shape4 sh = output->shape;
    const size_t minmax_len = (sh.len() + 127) / 128;
    WRK_TRY(check_shape("input", input->shape, sh[0], sh[1], sh[2], sh[3]));
    WRK_TRY(check_shape("minmax", minmax->shape, (uint32_t)(minmax_len << 1), 1, 1, 1));
    const __half* in = static_cast<const __half*>(input->ptr());
    __half* mm = static_cast<__half*>(minmax->ptr());
    uint8_t* o = static_cast<uint8_t*>(output->ptr());
    const size_t len = sh.len();
    const int sms = output->ctx->num_sms;
    *out = new_atom("quantize_mat_int8", [=](cudaStream_t s) { return k::quantize_int8(in, len, mm, o, sms, s); },
                    {input, minmax, output});
    return WRK_OK;
}

int32_t wrk_op_quantize_mat_nf4(wrk_tensor* input, wrk_tensor* quant, wrk_tensor* absmax, wrk_tensor* output,
                                wrk_op** out) {
    REQ_NN(input, quant, absmax, output, out);
    REQ_DTYPE(input, WRK_F16, "input");
    REQ_DTYPE(quant, WRK_F32, "quant");
    REQ_DTYPE(absmax, WRK_F16, "absmax");
    REQ_DTYPE(output, WRK_U8, "output");
    const Shape4 sh = output->shape;
    const size_t in_len = sh.len() << 1;
    WRK_TRY(check_shape("input", input->shape, sh[0] << 1, sh[1], sh[2], sh[3]));
    WRK_TRY(check_shape("absmax", absmax->shape, (uint32_t)((in_len + 63) / 64), 1, 1, 1));
    WRK_TRY(check_shape("quant", quant->shape, 16, 1, 1, 1));
    // The bracketing search needs a strictly ascending code book with sane gaps; otherwise the
    // kernel runs the reference's 16-way scan.  Reading the table back is a one-off at load time.
    float table[16];
    WRK_TRY(wrk_tensor_back(quant, table, sizeof table));
    bool sorted = true;
    for (int i = 0; i + 1 < 16; ++i)
        if (!(table[i + 1] - table[i] > 1e-4f)) sorted = false;
    const __half* in = static_cast<const __half*>(input->ptr());
    const float* q = static_cast<const float*>(quant->ptr());
    __half* am = static_cast<__half*>(absmax->ptr());
    uint8_t* o = static_cast<uint8_t*>(output->ptr());
    const int sms = output->ctx->num_sms;
    *out = new_atom("quantize_mat_nf4",
                    [=](cudaStream_t s) { return k::quantize_nf4(in, in_len, q, sorted, am, o, sms, s); },
                    {input, quant, absmax, output});
    return WRK_OK;
}

int32_t wrk_op_matmul_vec_fp16(wrk_tensor* matrix, const wrk_view* input, const wrk_view* output, int32_t act,
                               int32_t sparse, wrk_op** out) {
    (void)sparse;  // skipping all-zero input groups never changes the result (matmul_vec_fp16.wgsl)
    return matmul_common("matmul_vec_fp16", k::MAT_FP16, matrix, nullptr, nullptr, input, output, act, out);
}

int32_t wrk_op_matmul_vec_int8(wrk_tensor* matrix, wrk_tensor* minmax, const wrk_view* input, const wrk_view* output,
                               int32_t act, int32_t sparse, wrk_op** out) {
    (void)sparse;
    return matmul_common("matmul_vec_int8", k::MAT_INT8, matrix, minmax, nullptr, input, output, act, out);
}

int32_t wrk_op_matmul_vec_nf4(wrk_tensor* matrix, wrk_tensor* quant, wrk_tensor* absmax, const wrk_view* input,
                              const wrk_view* output, int32_t act, int32_t sparse, wrk_op** out) {
    (void)sparse;
    return matmul_common("matmul_vec_nf4", k::MAT_NF4, matrix, absmax, quant, input, output, act, out);
}

static int32_t whole_matrix(const wrk_view* matrix, wrk_tensor** t) {
    REQ_NN(matrix, matrix->tensor);
    // the reference's matrix-matrix kernels index the scales with the unsliced row stride
    // (matmul_mat_int8.wgsl:99-104): only whole-tensor views are meaningful
    for (int i = 0; i < 4; ++i)
        WRK_REQUIRE(matrix->offset[i] == 0 && matrix->shape[i] == matrix->tensor->shape.v[i] &&
                        matrix->stride[i] == matrix->tensor->shape.v[i],
                    WRK_ERR_SLICE_INVALID, "slice not contiguous: matrix views must cover the whole tensor");
    *t = matrix->tensor;
    return WRK_OK;
}

int32_t wrk_op_matmul_mat_fp16(const wrk_view* matrix, const wrk_view* input, const wrk_view* output, int32_t act,
                               wrk_op** out) {
    wrk_tensor* m = nullptr;
    WRK_TRY(whole_matrix(matrix, &m));
    return matmul_common("matmul_mat_fp16", k::MAT_FP16, m, nullptr, nullptr, input, output, act, out);
}

int32_t wrk_op_matmul_mat_int8(const wrk_view* matrix, wrk_tensor* minmax, const wrk_view* input,
                               const wrk_view* output, int32_t act, wrk_op** out) {
    wrk_tensor* m = nullptr;
    WRK_TRY(whole_matrix(matrix, &m));
    return matmul_common("matmul_mat_int8", k::MAT_INT8, m, minmax, nullptr, input, output, act, out);
}

int32_t wrk_op_matmul_mat_nf4(const wrk_view* matrix, wrk_tensor* quant, wrk_tensor* absmax, const wrk_view* input,
                              const wrk_view* output, int32_t act, wrk_op** out) {
    wrk_tensor* m = nullptr;
    WRK_TRY(whole_matrix(matrix, &m));
    return matmul_common("matmul_mat_nf4", k::MAT_NF4, m, absmax, quant, input, output, act, out);
}

int32_t wrk_op_time_mix_v4(wrk_tensor* cursors, wrk_tensor* time_decay, wrk_tensor* time_first, const wrk_view* state,
                           wrk_tensor* k, wrk_tensor* v, wrk_tensor* r, wrk_tensor* x, wrk_op** out) {
    REQ_NN(cursors, time_decay, time_first, state, state->tensor, k, v, r, x, out);
    REQ_FLOAT(x, "x");
    REQ_DTYPE(k, x->dtype, "k");
    REQ_DTYPE(v, x->dtype, "v");
    REQ_DTYPE(r, x->dtype, "r");
    REQ_DTYPE(time_decay, WRK_F32, "time_decay");
    REQ_DTYPE(time_first, WRK_F32, "time_first");
    REQ_DTYPE(state->tensor, WRK_F32, "state");
    const Shape4 sh = x->shape;
    const uint32_t C = sh[0], T = sh[1];
    WRK_TRY(check_shape("x", sh, C, T, 1, 1));
    WRK_TRY(check_shape("k", k->shape, C, T, 1, 1));
    WRK_TRY(check_shape("v", v->shape, C, T, 1, 1));
    WRK_TRY(check_shape("r", r->shape, C, T, 1, 1));
    WRK_TRY(check_shape("time_decay", time_decay->shape, C, 1, 1, 1));
    WRK_TRY(check_shape("time_first", time_first->shape, C, 1, 1, 1));
    WRK_TRY(check_view("state", state, C, 4, state->shape[2], 1));
    WRK_TRY(check_cursors(cursors, T));
    const uint32_t* cp = static_cast<const uint32_t*>(cursors->ptr());
    const int wide = cursors_wide(cursors, T);
    const float* td = static_cast<const float*>(time_decay->ptr());
    const float* tf = static_cast<const float*>(time_first->ptr());
    DView sv = make_dview(*state);
    const int dt = x->dtype;
    const void *kp = k->ptr(), *vp = v->ptr(), *rp = r->ptr();
    void* xp = x->ptr();
    *out = new_atom("time_mix_v4",
                    [=](cudaStream_t s) { return k::time_mix_v4(cp, wide, td, tf, sv, dt, kp, vp, rp, xp, C, T, s); },
                    {cursors, time_decay, time_first, state->tensor, k, v, r, x});
    return WRK_OK;
}

int32_t wrk_op_time_mix_v5(wrk_tensor* cursors, wrk_tensor* time_decay, wrk_tensor* time_first, const wrk_view* state,
                           wrk_tensor* k, wrk_tensor* v, wrk_tensor* r, wrk_tensor* x, wrk_op** out) {
    return time_mix_v56("time_mix_v5", 0, cursors, time_decay, time_first, state, k, v, r, x, out);
}

int32_t wrk_op_time_mix_v6(wrk_tensor* cursors, wrk_tensor* time_decay, wrk_tensor* time_first, const wrk_view* state,
                           wrk_tensor* k, wrk_tensor* v, wrk_tensor* r, wrk_tensor* x, wrk_op** out) {
    return time_mix_v56("time_mix_v6", 1, cursors, time_decay, time_first, state, k, v, r, x, out);
}

int32_t wrk_op_time_mix_blocks(int32_t per_token_decay, wrk_tensor* cursors, wrk_tensor* time_decay, wrk_tensor* time_first,
                               const wrk_view* state, wrk_tensor* k, wrk_tensor* v, wrk_tensor* r, wrk_tensor* x, wrk_op** out) {
    return time_mix_v56("time_mix_blocks", per_token_decay ? 1 : 0, cursors, time_decay, time_first, state, k, v, r, x, out, true);
}

int32_t wrk_op_time_mix_v7(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* r, wrk_tensor* w, wrk_tensor* n,
                           wrk_tensor* x, wrk_op** out) {
    REQ_NN(cursors, state, state->tensor, r, w, n, x, out);
    REQ_FLOAT(x, "x");
    REQ_DTYPE(r, x->dtype, "r");
    REQ_DTYPE(w, x->dtype, "w");
    REQ_DTYPE(n, x->dtype, "n");
    REQ_DTYPE(state->tensor, WRK_F32, "state");
    const Shape4 sh = x->shape;
    const uint32_t S = sh[0], H = sh[1], T = sh[2], stride = S * H;
    WRK_TRY(check_shape("x", sh, S, H, T, 1));
    WRK_TRY(check_shape("r", r->shape, S, H, T, 1));
    WRK_TRY(check_shape("w", w->shape, S, H, T, 1));
    WRK_TRY(check_shape("n", n->shape, S, H, T, 4));
    WRK_TRY(check_view("state", state, stride, S + 1, state->shape[2], 1));
    WRK_TRY(check_cursors(cursors, T));
    WRK_REQUIRE(S == 32 || S == 64 || S == 128, WRK_ERR_UNSUPPORTED, "head size %u not built (32, 64, 128)", S);
    k::WkvArgs a{};
    a.cursors = static_cast<const uint32_t*>(cursors->ptr());
    a.wide = cursors_wide(cursors, T);
    a.state = make_dview(*state);
    a.S = S; a.H = H; a.T = T; a.B = state->shape[2];
    a.dtype = x->dtype;
    a.r = r->ptr(); a.w = w->ptr(); a.n = n->ptr(); a.x = x->ptr();
    a.status = x->ctx->device_status;
    *out = new_atom("time_mix_v7", [a](cudaStream_t s) { return k::time_mix_v7(a, s); },
                    {cursors, state->tensor, r, w, n, x});
    return WRK_OK;
}

int32_t wrk_op_time_first_v7(wrk_tensor* u, wrk_tensor* r, wrk_tensor* n, wrk_tensor* x, wrk_op** out) {
    REQ_NN(u, r, n, x, out);
    REQ_FLOAT(x, "x");
    REQ_DTYPE(u, WRK_F16, "u");
    REQ_DTYPE(r, x->dtype, "r");
    REQ_DTYPE(n, x->dtype, "n");
    const Shape4 sh = x->shape;
    const uint32_t S = sh[0], H = sh[1], T = sh[2];
    WRK_TRY(check_shape("x", sh, S, H, T, 1));
    WRK_TRY(check_shape("r", r->shape, S, H, T, 1));
    WRK_TRY(check_shape("u", u->shape, S, H, 1, 1));
    WRK_TRY(check_shape("n", n->shape, S, H, T, 4));
    const __half* up = static_cast<const __half*>(u->ptr());
    const void *rp = r->ptr(), *np = n->ptr();
    void* xp = x->ptr();
    const int dt = x->dtype;
    *out = new_atom("time_first_v7", [=](cudaStream_t s) { return k::time_first_v7(up, dt, rp, np, xp, S, H, T, s); },
                    {u, r, n, x});
    return WRK_OK;
}

// ---- supporting ops ----------------------------------------------------------------------

static int32_t norm_common(const char* name, bool group, wrk_tensor* w, wrk_tensor* b, wrk_tensor* x, float eps,
                           wrk_op** out) {
    REQ_NN(w, b, x, out);
    REQ_FLOAT(x, "x");
    REQ_DTYPE(w, WRK_F16, "w");
    REQ_DTYPE(b, WRK_F16, "b");
    const Shape4 sh = x->shape;
    WRK_TRY(check_shape("x", sh, sh[0], sh[1], sh[2], 1));
    uint32_t rows, wrows;
    if (group) {
        WRK_TRY(check_shape("w", w->shape, sh[0], sh[1], 1, 1));
        WRK_TRY(check_shape("b", b->shape, sh[0], sh[1], 1, 1));
        rows = sh[1] * sh[2];
        wrows = sh[1];
    } else {
        WRK_TRY(check_shape("w", w->shape, sh[0], 1, 1, 1));
        WRK_TRY(check_shape("b", b->shape, sh[0], 1, 1, 1));
        rows = sh[1] * sh[2];
        wrows = 1;
    }
    const __half* wp = static_cast<const __half*>(w->ptr());
    const __half* bp = static_cast<const __half*>(b->ptr());
    void* xp = x->ptr();
    const int dt = x->dtype;
    const uint32_t C = sh[0];
    *out = new_atom(name, [=](cudaStream_t s) { return k::layer_norm(wp, bp, dt, xp, C, rows, wrows, eps, s); },
                    {w, b, x});
    return WRK_OK;
}

int32_t wrk_op_layer_norm(wrk_tensor* w, wrk_tensor* b, wrk_tensor* x, float eps, wrk_op** out) {
    return norm_common("layer_norm", false, w, b, x, eps, out);
}

int32_t wrk_op_layer_norm_copy(wrk_tensor* w, wrk_tensor* b, wrk_tensor* delta, wrk_tensor* src, wrk_tensor* dst, float eps,
                               wrk_op** out) {
    REQ_NN(w, b, src, dst, out);
    REQ_FLOAT(dst, "dst");
    REQ_DTYPE(src, dst->dtype, "src");
    REQ_DTYPE(w, WRK_F16, "w");
    REQ_DTYPE(b, WRK_F16, "b");
    const Shape4 sh = dst->shape;
    WRK_TRY(check_shape("dst", sh, sh[0], sh[1], sh[2], 1));
    WRK_TRY(check_shape("src", src->shape, sh[0], sh[1], sh[2], 1));
    WRK_TRY(check_shape("w", w->shape, sh[0], 1, 1, 1));
    WRK_TRY(check_shape("b", b->shape, sh[0], 1, 1, 1));
    if (delta) {
        REQ_DTYPE(delta, dst->dtype, "delta");
        WRK_TRY(check_shape("delta", delta->shape, sh[0], sh[1], sh[2], 1));
        WRK_REQUIRE(delta->ptr() != src->ptr() && src->ptr() != dst->ptr(), WRK_ERR_INVALID_ARGUMENT,
                    "delta, src and dst must be three tensors");
    }
    const __half* wp = static_cast<const __half*>(w->ptr());
    const __half* bp = static_cast<const __half*>(b->ptr());
    const void* ap = delta ? delta->ptr() : nullptr;
    void* sp = src->ptr();
    void* dp = dst->ptr();
    const int dt = dst->dtype;
    const uint32_t C = sh[0], rows = sh[1] * sh[2];
    *out = new_atom("layer_norm_copy", [=](cudaStream_t s) { return k::layer_norm_copy(wp, bp, dt, ap, sp, dp, C, rows, 1, eps, s); },
                    {w, b, src, dst});
    if (delta) (*out)->keep.push_back(delta->buf);
    return WRK_OK;
}

int32_t wrk_op_token_shift_multi(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* input, uint32_t count,
                                 wrk_tensor* const* time_mix, wrk_tensor* const* outputs, int32_t reversed, wrk_op** out) {
    REQ_NN(cursors, state, state->tensor, input, time_mix, outputs, out);
    WRK_REQUIRE(count >= 1 && count <= k::kShiftMultiMax, WRK_ERR_INVALID_ARGUMENT, "%u shifts: 1 to %u", count, k::kShiftMultiMax);
    REQ_DTYPE(input, WRK_F16, "input");
    REQ_DTYPE(state->tensor, WRK_F32, "state");
    const Shape4 sh = input->shape;
    const uint32_t C = sh[0], T = sh[1];
    WRK_TRY(check_shape("input", sh, C, T, 1, 1));
    WRK_TRY(check_view("state", state, C, state->shape[1], state->shape[2], 1));
    WRK_TRY(check_cursors(cursors, T));
    k::ShiftMultiArgs a{};
    a.cursors = static_cast<const uint32_t*>(cursors->ptr());
    a.wide = cursors_wide(cursors, T);
    a.state = make_dview(*state);
    a.in = static_cast<const __half*>(input->ptr());
    a.C = C;
    a.T = T;
    a.count = count;
    a.reversed = reversed;
    wrk_op* op = new_atom("token_shift_multi", nullptr, {cursors, state->tensor, input});
    for (uint32_t i = 0; i < count; ++i) {
        const int32_t s1 = time_mix[i] && outputs[i] ? WRK_OK : set_error(WRK_ERR_INVALID_ARGUMENT, "null argument");
        int32_t s2 = s1;
        if (s2 == WRK_OK && (time_mix[i]->dtype != WRK_F16 || outputs[i]->dtype != WRK_F16)) s2 = set_error(WRK_ERR_TYPE, "data type mismatch: f16 mixes and outputs");
        if (s2 == WRK_OK) s2 = check_shape("time_mix", time_mix[i]->shape, C, 1, 1, 1);
        if (s2 == WRK_OK) s2 = check_shape("output", outputs[i]->shape, C, T, 1, 1);
        if (s2 != WRK_OK) {
            wrk_op_release(op);
            return s2;
        }
        a.mix[i] = static_cast<const __half*>(time_mix[i]->ptr());
        a.out[i] = static_cast<__half*>(outputs[i]->ptr());
        op->keep.push_back(time_mix[i]->buf);
        op->keep.push_back(outputs[i]->buf);
    }
    op->launch = [a](cudaStream_t s) { return k::token_shift_multi(a, s); };
    *out = op;
    return WRK_OK;
}

int32_t wrk_op_pack_v7(wrk_tensor* k_k, wrk_tensor* k_a, wrk_tensor* k, wrk_tensor* v, wrk_tensor* a, wrk_tensor* kk, wrk_tensor* n,
                       float eps, wrk_op** out) {
    REQ_NN(k_k, k_a, k, v, a, kk, n, out);
    const Shape4 sh = k->shape;  // [S, H, T]
    const uint32_t S = sh[0], H = sh[1], T = sh[2];
    for (wrk_tensor* t : {k_k, k_a, k, v, a, kk, n}) REQ_DTYPE(t, WRK_F16, "tensor");
    WRK_TRY(check_shape("k", sh, S, H, T, 1));
    WRK_TRY(check_shape("v", v->shape, S, H, T, 1));
    WRK_TRY(check_shape("a", a->shape, S, H, T, 1));
    WRK_TRY(check_shape("kk", kk->shape, S, H, T, 1));
    WRK_TRY(check_shape("n", n->shape, S, H, T, 4));
    WRK_REQUIRE(k_k->len() == (size_t)S * H && k_a->len() == (size_t)S * H, WRK_ERR_SHAPE, "k_k and k_a hold %u values", S * H);
    k::PackV7Args p{};
    p.k_k = static_cast<const __half*>(k_k->ptr());
    p.k_a = static_cast<const __half*>(k_a->ptr());
    p.k = static_cast<__half*>(k->ptr());
    p.kk = static_cast<__half*>(kk->ptr());
    p.n = static_cast<__half*>(n->ptr());
    p.v = static_cast<const __half*>(v->ptr());
    p.a = static_cast<const __half*>(a->ptr());
    p.S = S;
    p.H = H;
    p.rows = H * T;
    p.eps = eps;
    *out = new_atom("pack_v7", [p](cudaStream_t s) { return k::pack_v7(p, s); }, {k_k, k_a, k, v, a, kk, n});
    return WRK_OK;
}

int32_t wrk_op_group_norm(wrk_tensor* w, wrk_tensor* b, wrk_tensor* x, float eps, wrk_op** out) {
    return norm_common("group_norm", true, w, b, x, eps, out);
}

int32_t wrk_op_softmax(wrk_tensor* x, wrk_op** out) {
    REQ_NN(x, out);
    REQ_FLOAT(x, "x");
    const Shape4 sh = x->shape;
    void* xp = x->ptr();
    const int dt = x->dtype;
    const uint32_t C = sh[0], rows = sh[1] * sh[2] * sh[3];
    *out = new_atom("softmax", [=](cudaStream_t s) { return k::softmax(dt, xp, C, rows, s); }, {x});
    return WRK_OK;
}

int32_t wrk_op_recenter(wrk_tensor* x, wrk_op** out) {
    REQ_NN(x, out);
    REQ_FLOAT(x, "x");
    const Shape4 sh = x->shape;
    void* xp = x->ptr();
    const int dt = x->dtype;
    const uint32_t C = sh[0], rows = sh[1] * sh[2];
    *out = new_atom("recenter", [=](cudaStream_t s) { return k::recenter(dt, xp, C, rows, s); }, {x});
    return WRK_OK;
}

int32_t wrk_op_rms_norm(wrk_tensor* w, wrk_tensor* b, wrk_tensor* x, float eps, wrk_op** out) {
    REQ_NN(w, b, x, out);
    REQ_FLOAT(x, "x");
    REQ_DTYPE(w, WRK_F16, "w");
    REQ_DTYPE(b, WRK_F16, "b");
    const Shape4 sh = x->shape;
    WRK_TRY(check_shape("x", sh, sh[0], sh[1], sh[2], 1));
    WRK_TRY(check_shape("w", w->shape, sh[0], 1, 1, 1));
    WRK_TRY(check_shape("b", b->shape, sh[0], 1, 1, 1));
    const __half* wp = static_cast<const __half*>(w->ptr());
    const __half* bp = static_cast<const __half*>(b->ptr());
    void* xp = x->ptr();
    const int dt = x->dtype;
    const uint32_t C = sh[0], rows = sh[1] * sh[2];
    *out = new_atom("rms_norm", [=](cudaStream_t s) { return k::rms_norm(wp, bp, dt, xp, C, rows, eps, s); }, {w, b, x});
    return WRK_OK;
}

int32_t wrk_op_embed(wrk_tensor* tokens, wrk_tensor* input, wrk_tensor* output, wrk_op** out) {
    REQ_NN(tokens, input, output, out);
    REQ_DTYPE(tokens, WRK_U32, "tokens");
    REQ_DTYPE(input, WRK_F16, "input");
    REQ_FLOAT(output, "output");
    const Shape4 sh = output->shape;
    WRK_TRY(check_shape("tokens", tokens->shape, sh[1], sh[2], 1, 1));
    WRK_TRY(check_shape("input", input->shape, sh[0], input->shape[1], 1, 1));
    WRK_TRY(check_shape("output", sh, sh[0], sh[1], sh[2], 1));
    const uint32_t* tp = static_cast<const uint32_t*>(tokens->ptr());
    const __half* ip = static_cast<const __half*>(input->ptr());
    void* op = output->ptr();
    const int dt = output->dtype;
    const uint32_t C = sh[0], rows = sh[1] * sh[2], vocab = input->shape[1];
    int32_t* status = output->ctx->device_status;
    *out = new_atom("embed", [=](cudaStream_t s) { return k::embed(tp, ip, dt, op, C, rows, vocab, status, s); },
                    {tokens, input, output});
    return WRK_OK;
}

int32_t wrk_op_l2_norm(wrk_tensor* x, float eps, wrk_op** out) {
    REQ_NN(x, out);
    REQ_FLOAT(x, "x");
    const Shape4 sh = x->shape;
    void* xp = x->ptr();
    const int dt = x->dtype;
    const uint32_t C = sh[0], rows = sh[1] * sh[2];
    *out = new_atom("l2_norm", [=](cudaStream_t s) { return k::l2_norm(dt, xp, C, rows, eps, s); }, {x});
    return WRK_OK;
}

int32_t wrk_op_token_shift(wrk_tensor* cursors, const wrk_view* time_mix, const wrk_view* state, wrk_tensor* input,
                           wrk_tensor* output, int32_t reversed, wrk_op** out) {
    REQ_NN(cursors, time_mix, time_mix->tensor, state, state->tensor, input, output, out);
    REQ_FLOAT(time_mix->tensor, "time_mix");
    REQ_FLOAT(input, "input");
    REQ_FLOAT(output, "output");
    REQ_DTYPE(state->tensor, WRK_F32, "state");
    const Shape4 sh = output->shape;
    const uint32_t C = sh[0], T = sh[1], count = sh[2];
    if (!(input->shape == Shape4{{C, T, count, 1}}) && !(input->shape == Shape4{{C, T, 1, 1}}))
        return check_shape("input", input->shape, C, T, 1, 1);
    if (!view_is(*time_mix, C, T, count, 1) && !view_is(*time_mix, C, 1, 1, 1))
        return check_view("time_mix", time_mix, C, 1, 1, 1);
    WRK_TRY(check_view("state", state, C, state->shape[1], state->shape[2], 1));
    WRK_TRY(check_cursors(cursors, T));
    const uint32_t* cp = static_cast<const uint32_t*>(cursors->ptr());
    const int wide = cursors_wide(cursors, T);
    DView tm = make_dview(*time_mix), st = make_dview(*state), in = make_dview(input), o = make_dview(output);
    *out = new_atom("token_shift", [=](cudaStream_t s) { return k::token_shift(cp, wide, tm, st, in, o, reversed, s); },
                    {cursors, time_mix->tensor, state->tensor, input, output});
    return WRK_OK;
}

int32_t wrk_op_token_shift_lora(wrk_tensor* cursors, const wrk_view* time_mix, const wrk_view* bias, const wrk_view* state,
                                wrk_tensor* input, wrk_tensor* output, int32_t reversed, wrk_op** out) {
    REQ_NN(cursors, time_mix, time_mix->tensor, bias, bias->tensor, state, state->tensor, input, output, out);
    REQ_DTYPE(state->tensor, WRK_F32, "state");
    const Shape4 sh = output->shape;
    const uint32_t C = sh[0], T = sh[1], count = sh[2];
    WRK_TRY(check_shape("input", input->shape, C, T, 1, 1));
    WRK_TRY(check_view("time_mix", time_mix, C, T, count, 1));
    WRK_TRY(check_view("bias", bias, C, 1, count, 1));
    WRK_TRY(check_view("state", state, C, state->shape[1], state->shape[2], 1));
    WRK_TRY(check_cursors(cursors, T));
    const uint32_t* cp = static_cast<const uint32_t*>(cursors->ptr());
    const int wide = cursors_wide(cursors, T);
    const DView tm = make_dview(*time_mix), bs = make_dview(*bias), st = make_dview(*state), in = make_dview(input),
                o = make_dview(output);
    WRK_REQUIRE(k::token_shift_vec_fits(tm, &bs, st, in, o), WRK_ERR_UNSUPPORTED,
                "token_shift_lora takes dense f16 tensors of a multiple of 8 channels and at most %u planes", k::kShiftMultiMax);
    *out = new_atom("token_shift_lora",
                    [=](cudaStream_t s) {
                        return k::token_shift_vec(cp, wide, tm, &bs, st, in, o, reversed, s) ? cudaGetLastError() : cudaErrorInvalidValue;
                    },
                    {cursors, time_mix->tensor, bias->tensor, state->tensor, input, output});
    return WRK_OK;
}

int32_t wrk_op_group_norm_gate(wrk_tensor* w, wrk_tensor* b, wrk_tensor* x, wrk_tensor* gate, wrk_tensor* output, float eps,
                               int32_t gate_act, wrk_op** out) {
    REQ_NN(w, b, x, gate, output, out);
    REQ_FLOAT(x, "x");
    REQ_DTYPE(w, WRK_F16, "w");
    REQ_DTYPE(b, WRK_F16, "b");
    REQ_DTYPE(gate, WRK_F16, "gate");
    REQ_DTYPE(output, WRK_F16, "output");
    const Shape4 sh = x->shape;  // [S, H, T]
    WRK_TRY(check_shape("x", sh, sh[0], sh[1], sh[2], 1));
    WRK_TRY(check_shape("w", w->shape, sh[0], sh[1], 1, 1));
    WRK_TRY(check_shape("b", b->shape, sh[0], sh[1], 1, 1));
    WRK_REQUIRE(gate->len() == x->len() && output->len() == x->len(), WRK_ERR_SHAPE, "gate and output hold x's %zu values", x->len());
    const __half* wp = static_cast<const __half*>(w->ptr());
    const __half* bp = static_cast<const __half*>(b->ptr());
    const __half* gp = static_cast<const __half*>(gate->ptr());
    __half* op = static_cast<__half*>(output->ptr());
    void* xp = x->ptr();
    const int dt = x->dtype;
    const uint32_t C = sh[0], rows = sh[1] * sh[2], wrows = sh[1];
    WRK_REQUIRE(k::group_norm_gate_supported(wp, bp, xp, gp, op, C), WRK_ERR_UNSUPPORTED,
                "group_norm_gate takes heads of 8, 16, ... 256 channels");
    *out = new_atom("group_norm_gate",
                    [=](cudaStream_t s) { return k::group_norm_gate(wp, bp, dt, xp, C, rows, wrows, eps, gp, op, gate_act, s); },
                    {w, b, x, gate, output});
    return WRK_OK;
}

int32_t wrk_op_channel_mix_add(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* r, wrk_tensor* v, wrk_tensor* x,
                               wrk_tensor* residual, int32_t v7, wrk_op** out) {
    REQ_NN(cursors, state, state->tensor, v, x, residual, out);
    REQ_FLOAT(x, "x");
    REQ_DTYPE(v, x->dtype, "v");
    REQ_DTYPE(residual, x->dtype, "residual");
    REQ_DTYPE(state->tensor, WRK_F32, "state");
    const Shape4 sh = x->shape;
    WRK_TRY(check_shape("x", sh, sh[0], sh[1], 1, 1));
    WRK_TRY(check_shape("v", v->shape, sh[0], sh[1], 1, 1));
    WRK_TRY(check_shape("residual", residual->shape, sh[0], sh[1], 1, 1));
    if (!v7) {
        REQ_NN(r);
        REQ_DTYPE(r, x->dtype, "r");
        WRK_TRY(check_shape("r", r->shape, sh[0], sh[1], 1, 1));
    }
    WRK_TRY(check_view("state", state, sh[0], 1, state->shape[2], 1));
    WRK_TRY(check_cursors(cursors, sh[1]));
    WRK_REQUIRE(sh[0] % 8 == 0, WRK_ERR_UNSUPPORTED, "channel_mix_add takes a multiple of 8 channels");
    const uint32_t* cp = static_cast<const uint32_t*>(cursors->ptr());
    const int wide = cursors_wide(cursors, sh[1]);
    DView st = make_dview(*state);
    const void* rp = r ? r->ptr() : nullptr;
    const void* vp = v->ptr();
    void* xp = x->ptr();
    void* res = residual->ptr();
    const int dt = x->dtype;
    const uint32_t C = sh[0], T = sh[1];
    *out = new_atom("channel_mix_add",
                    [=](cudaStream_t s) {
                        return k::channel_mix_vec(cp, wide, st, dt, rp, vp, xp, res, C, T, v7, s) ? cudaGetLastError() : cudaErrorInvalidValue;
                    },
                    {cursors, state->tensor, r, v, x, residual});
    return WRK_OK;
}

static int32_t channel_mix_common(const char* name, int v7, wrk_tensor* cursors, const wrk_view* state, wrk_tensor* r,
                                  wrk_tensor* v, wrk_tensor* x, wrk_op** out) {
    REQ_NN(cursors, state, state->tensor, v, x, out);
    REQ_FLOAT(x, "x");
    REQ_DTYPE(v, x->dtype, "v");
    REQ_DTYPE(state->tensor, WRK_F32, "state");
    const Shape4 sh = x->shape;
    WRK_TRY(check_shape("x", sh, sh[0], sh[1], 1, 1));
    WRK_TRY(check_shape("v", v->shape, sh[0], sh[1], 1, 1));
    if (!v7) {
        REQ_NN(r);
        REQ_DTYPE(r, x->dtype, "r");
        WRK_TRY(check_shape("r", r->shape, sh[0], sh[1], 1, 1));
    }
    WRK_TRY(check_view("state", state, sh[0], 1, state->shape[2], 1));
    WRK_TRY(check_cursors(cursors, sh[1]));
    const uint32_t* cp = static_cast<const uint32_t*>(cursors->ptr());
    const int wide = cursors_wide(cursors, sh[1]);
    DView st = make_dview(*state);
    const void* rp = r ? r->ptr() : nullptr;
    const void* vp = v->ptr();
    void* xp = x->ptr();
    const int dt = x->dtype;
    const uint32_t C = sh[0], T = sh[1];
    *out = new_atom(name, [=](cudaStream_t s) { return k::channel_mix(cp, wide, st, dt, rp, vp, xp, C, T, v7, s); },
                    {cursors, state->tensor, r, v, x});
    return WRK_OK;
}

int32_t wrk_op_shift_carry(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* x, wrk_op** out) {
    REQ_NN(cursors, state, state->tensor, x, out);
    REQ_FLOAT(x, "x");
    REQ_DTYPE(state->tensor, WRK_F32, "state");
    const Shape4 sh = x->shape;
    WRK_TRY(check_shape("x", sh, sh[0], sh[1], 1, 1));
    WRK_TRY(check_view("state", state, sh[0], 1, state->shape[2], 1));
    WRK_TRY(check_cursors(cursors, sh[1]));
    const uint32_t* cp = static_cast<const uint32_t*>(cursors->ptr());
    const int wide = cursors_wide(cursors, sh[1]);
    DView st = make_dview(*state);
    const void* xp = x->ptr();
    const int dt = x->dtype;
    const uint32_t C = sh[0], T = sh[1];
    *out = new_atom("shift_carry", [=](cudaStream_t s) { return k::shift_carry(cp, wide, st, dt, xp, C, T, s); },
                    {cursors, state->tensor, x});
    return WRK_OK;
}

int32_t wrk_op_channel_mix(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* r, wrk_tensor* v, wrk_tensor* x,
                           wrk_op** out) {
    return channel_mix_common("channel_mix", 0, cursors, state, r, v, x, out);
}

int32_t wrk_op_channel_mix_v7(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* v, wrk_tensor* x, wrk_op** out) {
    return channel_mix_common("channel_mix_v7", 1, cursors, state, nullptr, v, x, out);
}

static int32_t binary_common(const char* name, int is_mul, const wrk_view* input, const wrk_view* output, int32_t act_x,
                             int32_t act_y, int32_t act_out, wrk_op** out) {
    REQ_NN(input, input->tensor, output, output->tensor, out);
    REQ_FLOAT(input->tensor, "input");
    REQ_FLOAT(output->tensor, "output");
    const uint32_t C = output->shape[0], T = output->shape[1], B = output->shape[2];
    if (!view_is(*input, C, T, B, 1) && !view_is(*input, C, 1, B, 1) && !view_is(*input, C, T, 1, 1) &&
        !view_is(*input, C, 1, 1, 1))
        return check_view("input", input, C, T, B, 1);
    WRK_TRY(check_view("output", output, C, T, B, 1));
    DView in = make_dview(*input), o = make_dview(*output);
    *out = new_atom(name, [=](cudaStream_t s) { return k::binary(is_mul, in, o, act_x, act_y, act_out, s); },
                    {input->tensor, output->tensor});
    return WRK_OK;
}

int32_t wrk_op_add_activate(const wrk_view* input, const wrk_view* output, int32_t act_x, int32_t act_y,
                            int32_t act_out, wrk_op** out) {
    return binary_common("add", 0, input, output, act_x, act_y, act_out, out);
}

int32_t wrk_op_mul_activate(const wrk_view* input, const wrk_view* output, int32_t act_x, int32_t act_y,
                            int32_t act_out, wrk_op** out) {
    return binary_common("mul", 1, input, output, act_x, act_y, act_out, out);
}

int32_t wrk_op_activate(const wrk_view* x, int32_t act, wrk_op** out) {
    REQ_NN(x, x->tensor, out);
    REQ_FLOAT(x->tensor, "x");
    DView xv = make_dview(*x);
    *out = new_atom("activate", [=](cudaStream_t s) { return k::activate(xv, act, s); }, {x->tensor});
    return WRK_OK;
}

int32_t wrk_op_blit(const wrk_view* input, const wrk_view* output, wrk_op** out) {
    REQ_NN(input, input->tensor, output, output->tensor, out);
    REQ_FLOAT(input->tensor, "input");
    REQ_FLOAT(output->tensor, "output");
    WRK_TRY(check_view("input", input, output->shape[0], output->shape[1], output->shape[2], output->shape[3]));
    DView in = make_dview(*input), o = make_dview(*output);
    *out = new_atom("blit", [=](cudaStream_t s) { return k::blit(in, o, 0, s); }, {input->tensor, output->tensor});
    return WRK_OK;
}

int32_t wrk_op_broadcast(const wrk_view* input, const wrk_view* output, wrk_op** out) {
    REQ_NN(input, input->tensor, output, output->tensor, out);
    REQ_FLOAT(input->tensor, "input");
    REQ_FLOAT(output->tensor, "output");
    WRK_TRY(check_view("input", input, output->shape[0], input->shape[1], input->shape[2], 1));
    WRK_REQUIRE(input->shape[1] > 0 && input->shape[2] > 0, WRK_ERR_EMPTY, "input is empty");
    DView in = make_dview(*input), o = make_dview(*output);
    *out = new_atom("broadcast", [=](cudaStream_t s) { return k::broadcast(in, o, s); }, {input->tensor, output->tensor});
    return WRK_OK;
}

int32_t wrk_op_blend(wrk_tensor* factor, wrk_tensor* input, wrk_tensor* output, wrk_op** out) {
    REQ_NN(factor, input, output, out);
    REQ_DTYPE(factor, WRK_F32, "factor");
    REQ_FLOAT(input, "input");
    REQ_FLOAT(output, "output");
    const Shape4 sh = output->shape;
    WRK_TRY(check_shape("input", input->shape, sh[0], sh[1], sh[2], sh[3]));
    WRK_TRY(check_shape("factor", factor->shape, 4, 1, 1, 1));
    wrk_view iv, ov;
    WRK_TRY(wrk_tensor_as_view(input, &iv));
    WRK_TRY(wrk_tensor_as_view(output, &ov));
    DView in = make_dview(iv), o = make_dview(ov);
    const float* fp = static_cast<const float*>(factor->ptr());
    *out = new_atom("blend", [=](cudaStream_t s) { return k::blend(fp, in, o, s); }, {factor, input, output});
    return WRK_OK;
}

int32_t wrk_op_blend_lora(wrk_tensor* factor, const wrk_view* xa, const wrk_view* xb, const wrk_view* output,
                          wrk_op** out) {
    REQ_NN(factor, xa, xa->tensor, xb, xb->tensor, output, output->tensor, out);
    REQ_DTYPE(factor, WRK_F32, "factor");
    REQ_DTYPE(xa->tensor, WRK_F16, "xa");
    REQ_DTYPE(xb->tensor, WRK_F16, "xb");
    REQ_DTYPE(output->tensor, WRK_F16, "output");
    WRK_TRY(check_shape("factor", factor->shape, 4, 1, 1, 1));
    WRK_TRY(check_view("xa", xa, xa->shape[0], output->shape[0], output->shape[2], 1));
    WRK_TRY(check_view("xb", xb, xb->shape[0], output->shape[1], output->shape[2], 1));
    // the shader sums over min(K_a, K_b) / 4 groups of four
    const uint32_t K = std::min(xa->shape[0] / 4, xb->shape[0] / 4) * 4;
    DView a = make_dview(*xa), b = make_dview(*xb), o = make_dview(*output);
    const float* fp = static_cast<const float*>(factor->ptr());
    *out = new_atom("blend_lora", [=](cudaStream_t s) { return k::blend_lora(fp, a, b, o, K, s); },
                    {factor, xa->tensor, xb->tensor, output->tensor});
    return WRK_OK;
}

int32_t wrk_op_transpose(const wrk_view* input, const wrk_view* output, wrk_op** out) {
    REQ_NN(input, input->tensor, output, output->tensor, out);
    REQ_FLOAT(input->tensor, "input");
    REQ_FLOAT(output->tensor, "output");
    WRK_TRY(check_view("input", input, input->shape[0], input->shape[1], input->shape[2], 1));
    WRK_TRY(check_view("output", output, input->shape[0], input->shape[2], input->shape[1], 1));
    DView in = make_dview(*input), o = make_dview(*output);
    *out = new_atom("transpose", [=](cudaStream_t s) { return k::blit(in, o, 1, s); }, {input->tensor, output->tensor});
    return WRK_OK;
}

int32_t wrk_op_lerp(const wrk_view* input, const wrk_view* output, const wrk_view* factor, int32_t reversed,
                    wrk_op** out) {
    REQ_NN(input, input->tensor, output, output->tensor, factor, factor->tensor, out);
    REQ_FLOAT(input->tensor, "input");
    REQ_FLOAT(output->tensor, "output");
    REQ_FLOAT(factor->tensor, "factor");
    const uint32_t C = output->shape[0], T = output->shape[1], B = output->shape[2];
    if (!view_is(*factor, C, T, B, 1) && !view_is(*factor, C, 1, B, 1) && !view_is(*factor, C, T, 1, 1) &&
        !view_is(*factor, C, 1, 1, 1))
        return check_view("factor", factor, C, T, B, 1);
    WRK_TRY(check_view("input", input, C, T, B, 1));
    WRK_TRY(check_view("output", output, C, T, B, 1));
    DView in = make_dview(*input), o = make_dview(*output), f = make_dview(*factor);
    *out = new_atom("lerp", [=](cudaStream_t s) { return k::lerp(in, o, f, reversed, s); },
                    {input->tensor, output->tensor, factor->tensor});
    return WRK_OK;
}

int32_t wrk_op_affine(wrk_tensor* x, float scale, float bias, wrk_op** out) {
    REQ_NN(x, out);
    REQ_FLOAT(x, "x");
    void* xp = x->ptr();
    const int dt = x->dtype;
    const size_t len = x->len();
    *out = new_atom("affine", [=](cudaStream_t s) { return k::affine(dt, xp, len, scale, bias, s); }, {x});
    return WRK_OK;
}

int32_t wrk_op_control_k_v7(wrk_tensor* p, const wrk_view* a, const wrk_view* k, wrk_op** out) {
    REQ_NN(p, a, a->tensor, k, k->tensor, out);
    REQ_DTYPE(p, WRK_F16, "p");
    REQ_FLOAT(a->tensor, "a");
    REQ_FLOAT(k->tensor, "k");
    const uint32_t C = k->shape[0], T = k->shape[1], B = k->shape[2];
    WRK_TRY(check_view("a", a, C, T, B, 1));
    WRK_TRY(check_shape("p", p->shape, C, 1, 1, 1));
    const __half* pp = static_cast<const __half*>(p->ptr());
    DView av = make_dview(*a), kv = make_dview(*k);
    *out = new_atom("control_k_v7", [=](cudaStream_t s) { return k::control_k_v7(pp, av, kv, s); },
                    {p, a->tensor, k->tensor});
    return WRK_OK;
}

// ---- Matrix ---------------------------------------------------------------------------------

int32_t wrk_matrix_fp16(wrk_tensor* w, wrk_matrix** out) {
    REQ_NN(w, out);
    REQ_DTYPE(w, WRK_F16, "matrix");
    auto m = new wrk_matrix();
    m->kind = 0;
    wrk_tensor_retain(w);
    m->w = w;
    *out = m;
    return WRK_OK;
}

int32_t wrk_matrix_quant_u8(wrk_tensor* matrix, wrk_matrix** out) {
    REQ_NN(matrix, out);
    REQ_DTYPE(matrix, WRK_F16, "matrix");
    wrk_context* ctx = matrix->ctx;
    const Shape4 sh = matrix->shape;
    wrk_tensor *w = nullptr, *m = nullptr;
    WRK_TRY(tensor_alloc(ctx, WRK_U8, sh.v, false, &w));
    const uint32_t ms[4] = {(uint32_t)(((sh.len() << 1) + 127) / 128), 1, 1, 1};
    int32_t s = tensor_alloc(ctx, WRK_F16, ms, false, &m);
    wrk_op* op = nullptr;
    if (s == WRK_OK) s = wrk_op_quantize_mat_int8(matrix, m, w, &op);
    if (s == WRK_OK) s = wrk_run(ctx, op);
    wrk_op_release(op);
    if (s != WRK_OK) {
        wrk_tensor_release(w);
        wrk_tensor_release(m);
        return s;
    }
    auto mat = new wrk_matrix();
    mat->kind = 1;
    mat->w = w;
    mat->m = m;
    *out = mat;
    return WRK_OK;
}

int32_t wrk_matrix_quant_fp4(wrk_tensor* matrix, const float table[16], wrk_matrix** out) {
    REQ_NN(matrix, table, out);
    REQ_DTYPE(matrix, WRK_F16, "matrix");
    wrk_context* ctx = matrix->ctx;
    const Shape4 sh = matrix->shape;
    WRK_REQUIRE(sh[0] % 2 == 0, WRK_ERR_SHAPE, "tensor shape not match: NF4 needs an even row length, got %u", sh[0]);
    wrk_tensor *w = nullptr, *m = nullptr, *q = nullptr;
    const uint32_t ws[4] = {sh[0] / 2, sh[1], sh[2], sh[3]};
    const uint32_t ms[4] = {(uint32_t)((sh.len() + 63) / 64), 1, 1, 1};
    const uint32_t qs[4] = {16, 1, 1, 1};
    int32_t s = tensor_alloc(ctx, WRK_U8, ws, false, &w);
    if (s == WRK_OK) s = tensor_alloc(ctx, WRK_F16, ms, false, &m);
    if (s == WRK_OK) s = wrk_tensor_from_data(ctx, WRK_F32, qs, table, 16 * sizeof(float), &q);
    wrk_op* op = nullptr;
    if (s == WRK_OK) s = wrk_op_quantize_mat_nf4(matrix, q, m, w, &op);
    if (s == WRK_OK) s = wrk_run(ctx, op);
    wrk_op_release(op);
    if (s != WRK_OK) {
        wrk_tensor_release(w);
        wrk_tensor_release(m);
        wrk_tensor_release(q);
        return s;
    }
    auto mat = new wrk_matrix();
    mat->kind = 2;
    mat->w = w;
    mat->m = m;
    mat->q = q;
    *out = mat;
    return WRK_OK;
}

int32_t wrk_matrix_quant_nf4(wrk_tensor* matrix, wrk_matrix** out) {
    float table[16];
    wrk_nf4_table(table);
    return wrk_matrix_quant_fp4(matrix, table, out);
}

int32_t wrk_matrix_quant_sf4(wrk_tensor* matrix, double nu, wrk_matrix** out) {
    float table[16];
    WRK_TRY(wrk_sf4_table(nu, table));
    return wrk_matrix_quant_fp4(matrix, table, out);
}

int32_t wrk_matrix_release(wrk_matrix* m) {
    if (!m) return WRK_OK;
    if (m->refs.fetch_sub(1) == 1) delete m;
    return WRK_OK;
}

int32_t wrk_matrix_parts(wrk_matrix* mat, int32_t* kind, wrk_tensor** w, wrk_tensor** m, wrk_tensor** q) {
    REQ_NN(mat);
    if (kind) *kind = mat->kind;
    if (w) *w = mat->w;
    if (m) *m = mat->m;
    if (q) *q = mat->q;
    return WRK_OK;
}

static int32_t matrix_matmul(wrk_matrix* m, const wrk_view* input, const wrk_view* output, int32_t act, int32_t turbo,
                             int32_t sparse, wrk_op** out) {
    REQ_NN(m, input, output, out);
    wrk_view mv;
    WRK_TRY(wrk_tensor_as_view(m->w, &mv));
    switch (m->kind) {
        case 0:
            return turbo ? wrk_op_matmul_mat_fp16(&mv, input, output, act, out)
                         : wrk_op_matmul_vec_fp16(m->w, input, output, act, sparse, out);
        case 1:
            return turbo ? wrk_op_matmul_mat_int8(&mv, m->m, input, output, act, out)
                         : wrk_op_matmul_vec_int8(m->w, m->m, input, output, act, sparse, out);
        default:
            return turbo ? wrk_op_matmul_mat_nf4(&mv, m->q, m->m, input, output, act, out)
                         : wrk_op_matmul_vec_nf4(m->w, m->q, m->m, input, output, act, sparse, out);
    }
}

int32_t wrk_matrix_matmul_op(wrk_matrix* m, const wrk_view* input, const wrk_view* output, int32_t act, int32_t turbo,
                             wrk_op** out) {
    return matrix_matmul(m, input, output, act, turbo, 0, out);
}

int32_t wrk_matrix_matmul_op_sparse(wrk_matrix* m, const wrk_view* input, const wrk_view* output, int32_t act,
                                    int32_t turbo, wrk_op** out) {
    return matrix_matmul(m, input, output, act, turbo, 1, out);
}

int32_t wrk_matrix_matmul_group_op(wrk_matrix* const* matrices, const wrk_view* inputs, const wrk_view* outputs, const int32_t* acts,
                                   uint32_t count, int32_t turbo, wrk_op** out) {
    REQ_NN(matrices, inputs, outputs, acts, out);
    WRK_REQUIRE(count >= 1 && count <= 4, WRK_ERR_INVALID_ARGUMENT, "a group holds 1 to 4 matrices, not %u", count);
    k::MatmulArgs args[4];
    bool one_launch = turbo != 0;
    for (uint32_t i = 0; i < count && one_launch; ++i) {
        wrk_matrix* m = matrices[i];
        REQ_NN(m);
        const int kind = m->kind == 0 ? k::MAT_FP16 : m->kind == 1 ? k::MAT_INT8 : k::MAT_NF4;
        WRK_TRY(matmul_args(kind, m->w, m->m, m->q, &inputs[i], &outputs[i], acts[i], &args[i]));
    }
    one_launch = one_launch && k::matmul_umma_group_supported(args, (int)count);
    if (one_launch) {
        std::vector<k::MatmulArgs> all(args, args + count);
        int32_t* status = args[0].status;
        wrk_op* op = new_atom("matmul_group", [all, status](cudaStream_t s) { return k::matmul_umma_group(all.data(), (int)all.size(), status, s); },
                              {});
        for (uint32_t i = 0; i < count; ++i) {
            for (wrk_tensor* t : {matrices[i]->w, matrices[i]->m, matrices[i]->q, inputs[i].tensor, outputs[i].tensor})
                if (t != nullptr && t->buf) op->keep.push_back(t->buf);
        }
        *out = op;
        return WRK_OK;
    }
    // shapes the grouped kernel does not take: the same work as a list of single matmuls
    std::vector<wrk_op*> ops;
    int32_t status = WRK_OK;
    for (uint32_t i = 0; i < count && status == WRK_OK; ++i) {
        wrk_op* o = nullptr;
        status = matrix_matmul(matrices[i], &inputs[i], &outputs[i], acts[i], turbo, 0, &o);
        if (status == WRK_OK) ops.push_back(o);
    }
    if (status == WRK_OK) status = wrk_op_list(ops.data(), ops.size(), out);
    for (wrk_op* o : ops) wrk_op_release(o);
    return status;
}

}  // extern "C"

// ---- no counterpart in the reference: Int8 GEMV that never allocates ----
extern "C" int32_t wrk_gemv_int8_static(int32_t device, void* cuda_stream, const void* matrix, const void* minmax,
                                        const void* x, void* y, uint32_t k, uint32_t m, uint32_t t, int32_t act,
                                        uint32_t num_ctas) {
    WRK_REQUIRE(matrix && minmax && x && y, WRK_ERR_INVALID_ARGUMENT, "null device pointer");
    WRK_REQUIRE((reinterpret_cast<uintptr_t>(matrix) | reinterpret_cast<uintptr_t>(x)) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(minmax) % 4 == 0 && reinterpret_cast<uintptr_t>(y) % 4 == 0,
                WRK_ERR_INVALID_ARGUMENT, "matrix and x must be 16-byte aligned, minmax and y 4-byte aligned");
    WRK_REQUIRE(act >= 0 && act <= 7, WRK_ERR_INVALID_ARGUMENT, "unknown activation %d", act);
    cudaError_t ce = cudaSuccess;
    const int r = wrk::k::gemv_int8_static(device, static_cast<cudaStream_t>(cuda_stream), static_cast<const uint8_t*>(matrix),
                                           static_cast<const __half*>(minmax), static_cast<const __half*>(x),
                                           static_cast<float*>(y), k, m, t, act, num_ctas, &ce);
    switch (r) {
        case wrk::k::SG_OK: return WRK_OK;
        case wrk::k::SG_TOO_MANY_CTAS:
            return wrk::set_error(WRK_ERR_SIZE,
                                  "the static row-range table holds %d CTAs; %u requested (0 = one per SM of the device)",
                                  wrk::k::kStaticGemvMaxCtas, num_ctas);
        case wrk::k::SG_BAD_SHAPE:
            return wrk::set_error(WRK_ERR_SHAPE,
                                  "unsupported size k = %u, m = %u, t = %u: k must be a non-zero multiple of 128 whose "
                                  "staged activations fit in shared memory, m >= 1, 1 <= t <= %d",
                                  k, m, t, wrk::k::kDecodeMaxTokens);
        case wrk::k::SG_BAD_DEVICE:
            return wrk::set_error(WRK_ERR_INVALID_ARGUMENT, "device %d must be the current CUDA device (and below %d)", device,
                                  wrk::k::kStaticGemvMaxDevices);
        default:
            return wrk::set_error(WRK_ERR_CUDA, "static Int8 GEMV failed: %s", cudaGetErrorString(ce));
    }
}
