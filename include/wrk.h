/* wrk.h — C ABI of the B200-native quantized-matmul + WKV inference path of web-rwkv.
 *
 * Every entry point returns an int32 status (0 = ok, negative = error, see wrk_status) and
 * never aborts or throws across the boundary; wrk_last_error_message() gives the text of the
 * calling thread's most recent failure.  Handles are opaque and reference counted.
 *
 * Tensor shapes follow the reference crate: [x, y, z, w] with x the fastest-moving axis
 * (src/tensor/shape.rs:96-99); a weight [K, M] is M rows of K contiguous elements.
 * Each declaration cites the reference interface (path:line inside cryscan/web-rwkv) that a
 * Rust `-sys` crate would bind it to.
 */
#ifndef WRK_H
#define WRK_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: TensorErrorKind (src/tensor/mod.rs:127-155) + device error classes ---- */
typedef enum {
    WRK_OK = 0,
    WRK_ERR_EMPTY = -1,              /* TensorErrorKind::Empty */
    WRK_ERR_TYPE = -2,               /* TensorErrorKind::Type */
    WRK_ERR_SIZE = -3,               /* TensorErrorKind::Size */
    WRK_ERR_BATCH = -4,              /* TensorErrorKind::Batch */
    WRK_ERR_SHAPE = -5,              /* TensorErrorKind::Shape */
    WRK_ERR_DEDUCE = -6,             /* TensorErrorKind::Deduce */
    WRK_ERR_BATCH_OUT_OF_RANGE = -7, /* TensorErrorKind::BatchOutOfRange */
    WRK_ERR_SLICE_OUT_OF_RANGE = -8, /* TensorErrorKind::SliceOutOfRange */
    WRK_ERR_SLICE_INVALID = -9,      /* TensorErrorKind::SliceInvalid */
    WRK_ERR_SPLIT_INVALID = -10,     /* TensorErrorKind::SplitInvalid */
    WRK_ERR_ANY = -11,               /* TensorErrorKind::Any */
    WRK_ERR_INVALID_VERSION = -20,   /* LoaderError::InvalidVersion (src/runtime/loader.rs:27-39) */
    WRK_ERR_MISSING_TENSOR = -21,    /* LoaderError::SafeTensor(TensorNotFound) */
    WRK_ERR_INPUT_EXHAUSTED = -30,   /* RuntimeError::InputExhausted (src/runtime/mod.rs:68-79) */
    WRK_ERR_CUDA = -100,             /* a CUDA runtime/driver call failed */
    WRK_ERR_NCCL = -101,             /* an NCCL call failed */
    WRK_ERR_TIMEOUT = -102,          /* a bounded device-side wait gave up */
    WRK_ERR_INVALID_ARGUMENT = -103, /* null handle, bad enum value, ... */
    WRK_ERR_UNSUPPORTED = -104,      /* valid in the reference, not built here */
    WRK_ERR_NO_DEVICE = -105         /* no CUDA device / library built without device code */
} wrk_status;

/* Element types: the `Scalar` implementors of src/num.rs:82-96. */
typedef enum { WRK_F32 = 0, WRK_F16 = 1, WRK_U8 = 2, WRK_U16 = 3, WRK_U32 = 4 } wrk_dtype;

/* `Activation`, src/tensor/ops.rs:146-160. */
typedef enum {
    WRK_ACT_NONE = 0,
    WRK_ACT_SQUARED_RELU = 1,
    WRK_ACT_TANH = 2,
    WRK_ACT_STABLE_EXP = 3,
    WRK_ACT_OPPOSITE_EXP = 4,
    WRK_ACT_SOFTPLUS = 5,
    WRK_ACT_SIGMOID = 6,
    WRK_ACT_SILU = 7
} wrk_activation;

/* `Quant`, src/runtime/model.rs:125-135. */
typedef enum { WRK_QUANT_NONE = 0, WRK_QUANT_INT8 = 1, WRK_QUANT_NF4 = 2, WRK_QUANT_SF4 = 3 } wrk_quant;

/* `RnnOption`, src/runtime/infer/rnn.rs:136-144; WRK_RNN_NONE is the `None` of Option<RnnOption>. */
typedef enum { WRK_RNN_LAST = 0, WRK_RNN_FULL = 1, WRK_RNN_NONE = 2 } wrk_rnn_option;

#define WRK_INT8_BLOCK_SIZE 128u /* TensorOp::INT8_BLOCK_SIZE, src/tensor/ops.rs:292 */
#define WRK_NF4_BLOCK_SIZE 64u   /* TensorOp::NF4_BLOCK_SIZE,  src/tensor/ops.rs:291 */
#define WRK_MIN_TOKEN_CHUNK_SIZE 32u /* src/runtime/infer/rnn.rs:10 */
#define WRK_DIM_AUTO 0xffffffffu /* TensorDimension::Auto in wrk_tensor_reshape */

typedef struct wrk_context wrk_context;   /* replaces `Context`, src/context.rs:53-84 */
typedef struct wrk_tensor wrk_tensor;     /* `TensorGpu<T, K>`, src/tensor/mod.rs:294-299 */
typedef struct wrk_op wrk_op;             /* `TensorOp`, src/tensor/ops.rs:280-288 */
typedef struct wrk_commands wrk_commands; /* the Vec<CommandBuffer> of Context::encode, ops.rs:78-144 */
typedef struct wrk_matrix wrk_matrix;     /* `Matrix`, src/tensor/matrix.rs:82-94 */

/* `TensorGpuView` = tensor + `View {shape, stride, offset}`, src/tensor/mod.rs:28-32, 546-569. */
typedef struct {
    wrk_tensor* tensor;
    uint32_t shape[4];
    uint32_t stride[4];
    uint32_t offset[4];
} wrk_view;

const char* wrk_last_error_message(void);
/* Names of this build's device architecture, e.g. "sm_100a". */
const char* wrk_build_arch(void);

/* ---- context: CUDA device + stream + device/pinned allocators (src/context.rs:86-186) ---- */
int32_t wrk_context_create(int32_t device, wrk_context** out);
int32_t wrk_context_destroy(wrk_context* ctx);
int32_t wrk_context_synchronize(wrk_context* ctx);            /* device.poll(Wait) */
int32_t wrk_context_stream(wrk_context* ctx, void** cuda_stream);
int32_t wrk_context_device(wrk_context* ctx, int32_t* device);
/* Device-side status word written by kernels whose bounded waits or bounds checks fail. */
int32_t wrk_context_device_status(wrk_context* ctx, int32_t* status);
/* Pinned host staging memory (the read-back/upload buffers of src/context.rs:343-394). */
int32_t wrk_pinned_alloc(wrk_context* ctx, size_t bytes, void** out);
int32_t wrk_pinned_free(wrk_context* ctx, void* ptr);
/* CUDA-event timer on the context's stream. */
int32_t wrk_timer_start(wrk_context* ctx);
int32_t wrk_timer_stop(wrk_context* ctx, float* milliseconds);
/* Number of kernels launched on this context since creation (graph replays count their nodes). */
int32_t wrk_context_launch_count(wrk_context* ctx, uint64_t* count);

/* ---- tensors (src/tensor/mod.rs:572-606, 671-714, 774-795, 1121-1157) ---- */
int32_t wrk_tensor_create(wrk_context* ctx, wrk_dtype dtype, const uint32_t shape[4], wrk_tensor** out); /* tensor_init */
int32_t wrk_tensor_zeros(wrk_context* ctx, wrk_dtype dtype, const uint32_t shape[4], wrk_tensor** out);  /* Context::zeros */
int32_t wrk_tensor_from_data(wrk_context* ctx, wrk_dtype dtype, const uint32_t shape[4], const void* host,
                             size_t bytes, wrk_tensor** out);                                           /* tensor_from_data */
int32_t wrk_tensor_load(wrk_tensor* t, const void* host, size_t bytes);  /* TensorGpu::load (H2D, stream ordered) */
int32_t wrk_tensor_back(wrk_tensor* t, void* host, size_t bytes);        /* TensorGpu::back (D2H + wait) */
int32_t wrk_tensor_retain(wrk_tensor* t);                                /* Clone (aliases the buffer) */
int32_t wrk_tensor_release(wrk_tensor* t);                               /* Drop */
int32_t wrk_tensor_deep_clone(wrk_tensor* t, wrk_tensor** out);          /* DeepClone */
int32_t wrk_tensor_shape(const wrk_tensor* t, uint32_t shape[4]);
int32_t wrk_tensor_dtype(const wrk_tensor* t, int32_t* dtype);
int32_t wrk_tensor_device_ptr(const wrk_tensor* t, void** ptr);
/* TensorReshape::reshape; one dimension may be WRK_DIM_AUTO. Aliases the buffer. */
int32_t wrk_tensor_reshape(wrk_tensor* t, const uint32_t shape[4], wrk_tensor** out);
/* TensorGpu::view(x, y, z, w) with half-open ranges [start, end). */
int32_t wrk_tensor_view(wrk_tensor* t, const uint32_t start[4], const uint32_t end[4], wrk_view* out);
/* The whole tensor as a view (`impl From<&TensorGpu> for TensorGpuView`). */
int32_t wrk_tensor_as_view(wrk_tensor* t, wrk_view* out);

/* ---- deferred ops: build → encode → submit (src/tensor/ops.rs:78-144, 280-288) ---- */
int32_t wrk_op_list(wrk_op* const* ops, size_t count, wrk_op** out); /* TensorOp::List (takes references) */
int32_t wrk_op_sep(wrk_op** out);                                    /* TensorOp::Sep */
int32_t wrk_op_release(wrk_op* op);
int32_t wrk_op_num_atoms(const wrk_op* op, uint64_t* count);
/* Context::encode: flatten the op tree into a launch list; with use_graph != 0 the list is also
 * captured into a CUDA graph so that submit is a single graph launch. */
int32_t wrk_encode(wrk_context* ctx, wrk_op* op, int32_t use_graph, wrk_commands** out);
int32_t wrk_submit(wrk_context* ctx, wrk_commands* commands);        /* queue.submit(commands) */
int32_t wrk_commands_release(wrk_commands* commands);
int32_t wrk_run(wrk_context* ctx, wrk_op* op);                       /* submit(encode(op)) */

/* -- the hot path -- */
/* TensorOp::quantize_mat_int8(input, minmax, output), src/tensor/ops.rs:2393-2486 */
int32_t wrk_op_quantize_mat_int8(wrk_tensor* input, wrk_tensor* minmax, wrk_tensor* output, wrk_op** out);
/* TensorOp::quantize_mat_nf4(input, quant, absmax, output), src/tensor/ops.rs:2488-2589 */
int32_t wrk_op_quantize_mat_nf4(wrk_tensor* input, wrk_tensor* quant, wrk_tensor* absmax, wrk_tensor* output,
                                wrk_op** out);
/* TensorOp::matmul_vec_fp16(matrix, input, output, act, sparse), src/tensor/ops.rs:697-784 */
int32_t wrk_op_matmul_vec_fp16(wrk_tensor* matrix, const wrk_view* input, const wrk_view* output, int32_t act,
                               int32_t sparse, wrk_op** out);
/* TensorOp::matmul_vec_int8(matrix, minmax, input, output, act, sparse), src/tensor/ops.rs:791-886 */
int32_t wrk_op_matmul_vec_int8(wrk_tensor* matrix, wrk_tensor* minmax, const wrk_view* input,
                               const wrk_view* output, int32_t act, int32_t sparse, wrk_op** out);
/* TensorOp::matmul_vec_nf4(matrix, quant, absmax, input, output, act, sparse), src/tensor/ops.rs:892-991 */
int32_t wrk_op_matmul_vec_nf4(wrk_tensor* matrix, wrk_tensor* quant, wrk_tensor* absmax, const wrk_view* input,
                              const wrk_view* output, int32_t act, int32_t sparse, wrk_op** out);
/* TensorOp::matmul_mat_fp16(matrix, input, output, act), src/tensor/ops.rs:999-1061 */
int32_t wrk_op_matmul_mat_fp16(const wrk_view* matrix, const wrk_view* input, const wrk_view* output,
                               int32_t act, wrk_op** out);
/* TensorOp::matmul_mat_int8(matrix, minmax, input, output, act), src/tensor/ops.rs:1072-1140 */
int32_t wrk_op_matmul_mat_int8(const wrk_view* matrix, wrk_tensor* minmax, const wrk_view* input,
                               const wrk_view* output, int32_t act, wrk_op** out);
/* TensorOp::matmul_mat_nf4(matrix, quant, absmax, input, output, act), src/tensor/ops.rs:1150-1221 */
int32_t wrk_op_matmul_mat_nf4(const wrk_view* matrix, wrk_tensor* quant, wrk_tensor* absmax,
                              const wrk_view* input, const wrk_view* output, int32_t act, wrk_op** out);
/* TensorOp::time_mix_v4(cursors, time_decay, time_first, state, k, v, r, x), src/tensor/ops.rs:1464-1528 (shader
 * src/shaders/time_mix_v4.wgsl): k, v, r, x [C, T]; time_decay, time_first f32 [C]; state view f32 [C, 4, B] (rows: shift
 * carry, aa, bb, pp). */
int32_t wrk_op_time_mix_v4(wrk_tensor* cursors, wrk_tensor* time_decay, wrk_tensor* time_first, const wrk_view* state,
                           wrk_tensor* k, wrk_tensor* v, wrk_tensor* r, wrk_tensor* x, wrk_op** out);
/* TensorOp::time_mix_v5(cursors, time_decay, time_first, state, k, v, r, x), src/tensor/ops.rs:1530-1598 */
int32_t wrk_op_time_mix_v5(wrk_tensor* cursors, wrk_tensor* time_decay, wrk_tensor* time_first,
                           const wrk_view* state, wrk_tensor* k, wrk_tensor* v, wrk_tensor* r, wrk_tensor* x,
                           wrk_op** out);
/* TensorOp::time_mix_v6(cursors, time_decay, time_first, state, k, v, r, x), src/tensor/ops.rs:1601-1669 */
int32_t wrk_op_time_mix_v6(wrk_tensor* cursors, wrk_tensor* time_decay, wrk_tensor* time_first,
                           const wrk_view* state, wrk_tensor* k, wrk_tensor* v, wrk_tensor* r, wrk_tensor* x,
                           wrk_op** out);
/* No counterpart in the reference: time_mix_v5 (per_token_decay == 0) or time_mix_v6 (!= 0) with the same arguments and
 * the same result up to fp32 summation order, computed in blocks of 16 tokens (the recurrence unrolled into three small
 * matrix products per block, so that the tokens of a block do not wait for one another).  Heads of 64 channels;
 * WRK_ERR_UNSUPPORTED otherwise.  The runtime uses it for jobs of more than 8 tokens outside strict mode. */
int32_t wrk_op_time_mix_blocks(int32_t per_token_decay, wrk_tensor* cursors, wrk_tensor* time_decay, wrk_tensor* time_first,
                               const wrk_view* state, wrk_tensor* k, wrk_tensor* v, wrk_tensor* r, wrk_tensor* x, wrk_op** out);
/* TensorOp::time_mix_v7(cursors, state, r, w, n, x), src/tensor/ops.rs:1679-1741 */
int32_t wrk_op_time_mix_v7(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* r, wrk_tensor* w,
                           wrk_tensor* n, wrk_tensor* x, wrk_op** out);
/* TensorOp::time_first_v7(u, r, n, x), src/tensor/ops.rs:1743-1798 */
int32_t wrk_op_time_first_v7(wrk_tensor* u, wrk_tensor* r, wrk_tensor* n, wrk_tensor* x, wrk_op** out);

/* -- supporting ops the v5/v6/v7 jobs need to reach logits -- */
/* TensorOp::layer_norm(w, b, x, eps), src/tensor/ops.rs:407-452 */
int32_t wrk_op_layer_norm(wrk_tensor* w, wrk_tensor* b, wrk_tensor* x, float eps, wrk_op** out);
/* TensorOp::group_norm(w, b, x, eps), src/tensor/ops.rs:454-508 */
int32_t wrk_op_group_norm(wrk_tensor* w, wrk_tensor* b, wrk_tensor* x, float eps, wrk_op** out);
/* TensorOp::softmax(x), src/tensor/ops.rs:299-352 (shader src/shaders/softmax.wgsl): in place over every row of
 * x.shape[0] elements; the device-side half of the logits hand-off of src/runtime/softmax.rs. */
int32_t wrk_op_softmax(wrk_tensor* x, wrk_op** out);
/* TensorOp::embed(tokens, input, output), src/tensor/ops.rs:346-400 (shader src/shaders/embed.wgsl): the device-side
 * embedding gather.  tokens u32 [T, B], input f16 [C, V], output [C, T, B].  A token id >= V leaves its row
 * untouched and records WRK_ERR_BATCH_OUT_OF_RANGE in the context's device status. */
int32_t wrk_op_embed(wrk_tensor* tokens, wrk_tensor* input, wrk_tensor* output, wrk_op** out);
/* TensorOp::recenter(x), src/tensor/ops.rs:511-560 (shader src/shaders/normalize.wgsl:46-80) */
int32_t wrk_op_recenter(wrk_tensor* x, wrk_op** out);
/* TensorOp::rms_norm(w, b, x, eps), src/tensor/ops.rs:566-640 (shader src/shaders/normalize.wgsl:82-118) */
int32_t wrk_op_rms_norm(wrk_tensor* w, wrk_tensor* b, wrk_tensor* x, float eps, wrk_op** out);
/* TensorOp::l2_norm(x, eps), src/tensor/ops.rs:642-691 */
int32_t wrk_op_l2_norm(wrk_tensor* x, float eps, wrk_op** out);
/* TensorOp::token_shift(cursors, time_mix, state, input, output, reversed), src/tensor/ops.rs:1393-1461 */
int32_t wrk_op_token_shift(wrk_tensor* cursors, const wrk_view* time_mix, const wrk_view* state,
                           wrk_tensor* input, wrk_tensor* output, int32_t reversed, wrk_op** out);
/* No counterpart in the reference: runs of its ops as one launch each, with the same arithmetic and the same roundings
 * per element, so that results are bit-identical to the separate ops.  The runtime uses them where no hook sits between
 * the ops they replace.
 *   layer_norm_copy: src <- src + delta when delta is not NULL (TensorOp::add, src/tensor/ops.rs:1656); dst <-
 *     layer_norm(src) (TensorOp::blit + TensorOp::layer_norm, src/tensor/ops.rs:2015, 407).  Three distinct tensors of
 *     one shape [C, T, B] and data type.
 *   token_shift_multi: up to six TensorOp::token_shift (src/tensor/ops.rs:1393-1462) of one f16 input [C, T] with f16
 *     mixes [C] into f16 outputs [C, T].
 *   pack_v7: on f16 tensors [S, H, T] of one layer of v7: kk <- l2_norm(k * k_k) per head (blit + mul + l2_norm,
 *     src/runtime/v7.rs:888-890), k <- control_k(k_a, a, k) (TensorOp::control_k_v7), n[S, H, T, 4] <- k, v, a, kk
 *     (the four blits of src/runtime/v7.rs:925-928).
 *   token_shift_lora: TensorOp::add of the static factors [C, 1, Z] to the adapter's output [C, T, Z] (the sum rounded
 *     to f16) + the TensorOp::token_shift that uses it (src/runtime/v6.rs:794-804); the adapter's output is left as
 *     it was.  Dense f16 tensors, C a multiple of 8, Z <= 6.
 *   group_norm_gate: TensorOp::group_norm of x [S, H, T] + TensorOp::blit into an f16 tensor + TensorOp::mul_activate
 *     with act(gate) (src/runtime/v6.rs:862-879): output <- act(gate) * f16(group_norm(x)); x is left as it was.
 *   channel_mix_add: TensorOp::channel_mix (v7 != 0: channel_mix_v7, r may be NULL) + TensorOp::add of its result to
 *     the residual stream (src/runtime/v6.rs:941-949). */
int32_t wrk_op_layer_norm_copy(wrk_tensor* w, wrk_tensor* b, wrk_tensor* delta, wrk_tensor* src, wrk_tensor* dst, float eps,
                               wrk_op** out);
int32_t wrk_op_token_shift_lora(wrk_tensor* cursors, const wrk_view* time_mix, const wrk_view* bias, const wrk_view* state,
                                wrk_tensor* input, wrk_tensor* output, int32_t reversed, wrk_op** out);
int32_t wrk_op_group_norm_gate(wrk_tensor* w, wrk_tensor* b, wrk_tensor* x, wrk_tensor* gate, wrk_tensor* output, float eps,
                               int32_t gate_act, wrk_op** out);
int32_t wrk_op_channel_mix_add(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* r, wrk_tensor* v, wrk_tensor* x,
                               wrk_tensor* residual, int32_t v7, wrk_op** out);
int32_t wrk_op_token_shift_multi(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* input, uint32_t count,
                                 wrk_tensor* const* time_mix, wrk_tensor* const* outputs, int32_t reversed, wrk_op** out);
int32_t wrk_op_pack_v7(wrk_tensor* k_k, wrk_tensor* k_a, wrk_tensor* k, wrk_tensor* v, wrk_tensor* a, wrk_tensor* kk, wrk_tensor* n,
                       float eps, wrk_op** out);
/* No counterpart in the reference, where the time-mix and channel-mix shaders store this row themselves
 * (src/shaders/time_mix_v6.wgsl:100, channel_mix.wgsl:98): state row 0 of every sequence with tokens in the job <- x at
 * that sequence's last token.  A rank of a split model uses it for the channels its time-mix op does not own. */
int32_t wrk_op_shift_carry(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* x, wrk_op** out);
/* TensorOp::channel_mix(cursors, state, r, v, x), src/tensor/ops.rs:1860-1915 */
int32_t wrk_op_channel_mix(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* r, wrk_tensor* v,
                           wrk_tensor* x, wrk_op** out);
/* TensorOp::channel_mix_v7(cursors, state, v, x), src/tensor/ops.rs:1917-1971 */
int32_t wrk_op_channel_mix_v7(wrk_tensor* cursors, const wrk_view* state, wrk_tensor* v, wrk_tensor* x,
                              wrk_op** out);
/* TensorOp::add_activate / add, src/tensor/ops.rs:1227-1305 */
int32_t wrk_op_add_activate(const wrk_view* input, const wrk_view* output, int32_t act_x, int32_t act_y,
                            int32_t act_out, wrk_op** out);
/* TensorOp::mul_activate / mul, src/tensor/ops.rs:1312-1391 */
int32_t wrk_op_mul_activate(const wrk_view* input, const wrk_view* output, int32_t act_x, int32_t act_y,
                            int32_t act_out, wrk_op** out);
/* TensorOp::activate(x, act), src/tensor/ops.rs:1973-2013 */
int32_t wrk_op_activate(const wrk_view* x, int32_t act, wrk_op** out);
/* TensorOp::blit(input, output), src/tensor/ops.rs:2015-2068 */
int32_t wrk_op_blit(const wrk_view* input, const wrk_view* output, wrk_op** out);
/* TensorOp::broadcast(input, output), src/tensor/ops.rs:2069-2118: input repeats along the token and batch axes */
int32_t wrk_op_broadcast(const wrk_view* input, const wrk_view* output, wrk_op** out);
/* TensorOp::blend(factor, input, output), src/tensor/ops.rs:2171-2223: output = factor[0] * input + factor[1] * output;
 * factor is an f32 tensor of 4 entries (the reference's uniform). */
int32_t wrk_op_blend(wrk_tensor* factor, wrk_tensor* input, wrk_tensor* output, wrk_op** out);
/* TensorOp::blend_lora(factor, xa, xb, output), src/tensor/ops.rs:2226-2282 (shader src/shaders/blend_lora.wgsl):
 * output[m, n, b] = factor[0] * sum_k xa[k, m, b] * xb[k, n, b] + factor[1] * output[m, n, b]; all f16, f32 sum. */
int32_t wrk_op_blend_lora(wrk_tensor* factor, const wrk_view* xa, const wrk_view* xb, const wrk_view* output,
                          wrk_op** out);
/* TensorOp::transpose(input, output), src/tensor/ops.rs:2121-2169 */
int32_t wrk_op_transpose(const wrk_view* input, const wrk_view* output, wrk_op** out);
/* TensorOp::lerp(input, output, factor, reversed), src/tensor/ops.rs:2284-2350 */
int32_t wrk_op_lerp(const wrk_view* input, const wrk_view* output, const wrk_view* factor, int32_t reversed,
                    wrk_op** out);
/* TensorOp::affine(x, scale, bias), src/tensor/ops.rs:2352-2391 */
int32_t wrk_op_affine(wrk_tensor* x, float scale, float bias, wrk_op** out);
/* TensorOp::control_k_v7(p, a, k), src/tensor/ops.rs:1800-1858 */
int32_t wrk_op_control_k_v7(wrk_tensor* p, const wrk_view* a, const wrk_view* k, wrk_op** out);

/* ---- Matrix (src/tensor/matrix.rs:82-222) ---- */
int32_t wrk_matrix_fp16(wrk_tensor* w, wrk_matrix** out);          /* Matrix::Fp16 */
int32_t wrk_matrix_quant_u8(wrk_tensor* matrix, wrk_matrix** out);  /* Matrix::quant_u8, matrix.rs:162-178 */
int32_t wrk_matrix_quant_nf4(wrk_tensor* matrix, wrk_matrix** out); /* Matrix::quant_nf4, matrix.rs:180-200 */
/* Matrix::quant_sf4 with a caller-supplied 16-entry table (matrix.rs:202-222; the Student-t table
 * itself comes from a third-party crate and is not generated here). */
int32_t wrk_matrix_quant_fp4(wrk_tensor* matrix, const float table[16], wrk_matrix** out);
int32_t wrk_matrix_release(wrk_matrix* m);
/* kind: 0 = Fp16, 1 = Int8, 2 = Fp4; w = weights, m = minmax/absmax (null for Fp16), q = table (Fp4 only).
 * Returned tensors are borrowed (retain them to keep them). */
int32_t wrk_matrix_parts(wrk_matrix* mat, int32_t* kind, wrk_tensor** w, wrk_tensor** m, wrk_tensor** q);
/* Matrix::matmul_op(input, output, act, turbo), matrix.rs:136-147 */
int32_t wrk_matrix_matmul_op(wrk_matrix* m, const wrk_view* input, const wrk_view* output, int32_t act,
                             int32_t turbo, wrk_op** out);
/* Matrix::matmul_op_sparse(input, output, act, turbo), matrix.rs:149-160 */
int32_t wrk_matrix_matmul_op_sparse(wrk_matrix* m, const wrk_view* input, const wrk_view* output, int32_t act,
                                    int32_t turbo, wrk_op** out);
/* No counterpart in the reference: up to four Matrix::matmul_op of one point of a layer (e.g. key / value / receptance /
 * gate, each with its own input, output and activation) as one op.  Matrices of one format, input width and token count
 * with 16 or more tokens run as the row tiles of a single tensor-core launch, which fills the SMs without splitting K;
 * anything else becomes the list of the single ops.  Results are those of the single ops up to the order of the fp32
 * sums over K (a single op may split K over CTAs where the group does not). */
int32_t wrk_matrix_matmul_group_op(wrk_matrix* const* matrices, const wrk_view* inputs, const wrk_view* outputs, const int32_t* acts,
                                   uint32_t count, int32_t turbo, wrk_op** out);
/* The default NF4 table of Float4Quant::new, matrix.rs:48-70. */
int32_t wrk_nf4_table(float table[16]);
/* Float4Quant::new_student(nu) / quantile_student, matrix.rs:29-44 and 72-77: the SF4 code book.  The Student-t
 * quantile the reference takes from the statrs crate (0.18) is computed here from the regularized incomplete
 * beta function. */
int32_t wrk_sf4_table(double nu, float table[16]);
/* Matrix::quant_sf4(matrix, nu), matrix.rs:202-222 */
int32_t wrk_matrix_quant_sf4(wrk_tensor* matrix, double nu, wrk_matrix** out);

/* ---- Tensor-parallel plumbing (the reference is single-GPU; no counterpart) ----
 * One process per GPU.  Rank 0 makes an id, every rank (rank 0 included) creates its communicator from the
 * same 128 bytes; the collectives are deferred ops on the context's stream like any other op. */
typedef struct wrk_comm wrk_comm;
int32_t wrk_comm_unique_id(uint8_t id[128]);
int32_t wrk_comm_create(wrk_context* ctx, const uint8_t id[128], int32_t rank, int32_t world, wrk_comm** out);
int32_t wrk_comm_retain(wrk_comm* comm);
int32_t wrk_comm_release(wrk_comm* comm);
/* The host-side wait of a rank of a split job: waits for everything submitted to the communicator's context, polling
 * ncclCommGetAsyncError; after timeout_ms, or on an asynchronous NCCL error, aborts the communicator (its kernels leave
 * the device, the context stays usable) and returns WRK_ERR_TIMEOUT / WRK_ERR_NCCL. */
int32_t wrk_comm_wait(wrk_comm* comm, uint32_t timeout_ms);
/* The loop under wrk_comm_wait with its two questions passed in: ends WRK_OK when done(user) is non-zero, WRK_ERR_NCCL
 * when failure(user) is (may be null), WRK_ERR_TIMEOUT after timeout_ms; polls every poll_us microseconds. */
int32_t wrk_watchdog_wait(int32_t (*done)(void*), int32_t (*failure)(void*), void* user, uint32_t timeout_ms, uint32_t poll_us);
int32_t wrk_comm_rank(const wrk_comm* comm, int32_t* rank, int32_t* world);
/* One-shot all-reduce over peer memory.  wrk_comm_enable_peer_reduce is itself a collective (every rank calls it at the
 * same point, outside any graph capture): each rank allocates two slots of `slot_bytes` and a flag word per rank, the CUDA
 * IPC handles travel through an NCCL all-gather, every rank maps every other rank's region.  wrk_comm_peer_slot returns a
 * tensor over one of this rank's slots (a matmul's f32 output goes there directly); wrk_op_peer_all_reduce makes every
 * rank signal its slot, wait (bounded; WRK_ERR_TIMEOUT in the device status word on expiry) for all ranks' signals and
 * add the ranks' slots in rank order with plain loads over NVLink into `dst` (f16 or f32).  Consecutive reduces on a
 * communicator alternate between slot 0 and slot 1. */
int32_t wrk_comm_enable_peer_reduce(wrk_comm* comm, size_t slot_bytes);
int32_t wrk_comm_peer_slot_bytes(const wrk_comm* comm, size_t* slot_bytes); /* 0 before wrk_comm_enable_peer_reduce */
int32_t wrk_comm_peer_slot(wrk_comm* comm, uint32_t slot, int32_t dtype, const uint32_t shape[4], wrk_tensor** out);
int32_t wrk_op_peer_all_reduce(wrk_comm* comm, uint32_t slot, size_t count, wrk_tensor* dst, wrk_op** out);
/* x <- sum over ranks of x, in place (f16 or f32). */
int32_t wrk_op_all_reduce(wrk_comm* comm, wrk_tensor* x, wrk_op** out);
/* output (world x len(input) elements) <- every rank's input, in rank order. */
int32_t wrk_op_all_gather(wrk_comm* comm, wrk_tensor* input, wrk_tensor* output, wrk_op** out);

/* ---- No counterpart in the reference ----
 * y[t][m] = act(W[m][:] . x[t][:]) for an Int8 matrix (the layout quantize_mat_int8 produces: u8 W[m][k], f16
 * (min, max) per 128-weight block), f16 x[t][k], f32 y[t][m], all raw device pointers, launched on `cuda_stream`
 * of `device`, which must be the current device.  The call allocates nothing, on the device or through any
 * library: the only scratch the kernel needs, its table of row ranges per CTA, lives in a static device array
 * of 512 ranges (24 KB).  It is for callers that must not allocate where they stand: inside a region the
 * application has fenced off from the allocator (all device memory handed to its own arena up front, so a
 * cudaMalloc would fail or stall every stream of the process), or on a latency-critical thread that may not
 * take the allocator's locks.
 *   - The first call on a device also looks up the array's address and the device's SM count; make that call
 *     once at start-up, before any stream capture.  Later calls only launch kernels.
 *   - num_ctas = 0 uses one CTA per SM; more than 512 is refused with WRK_ERR_SIZE.  k must be a multiple of
 *     128 small enough for t rows of x to be staged in shared memory, 1 <= t <= 8; else WRK_ERR_SHAPE.
 *   - Every call on a device rewrites the same array (nothing in it has to be zero beforehand): two calls
 *     that can run at the same time, from two streams or two threads, race.  Order them on one stream.
 * matrix and x must be 16-byte aligned. */
int32_t wrk_gemv_int8_static(int32_t device, void* cuda_stream, const void* matrix, const void* minmax, const void* x,
                             void* y, uint32_t k, uint32_t m, uint32_t t, int32_t act, uint32_t num_ctas);

#ifdef __cplusplus
}
#endif
#endif /* WRK_H */
