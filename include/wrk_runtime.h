/* wrk_runtime.h — C ABI of the v5/v6/v7 `run()` jobs: model building with per-layer
 * quantization, recurrent state, token chunking (`token_chunk_size`, `num_batch`) and the
 * dispatch → load → submit → back job protocol of the reference crate.
 *
 * Status codes, tensors and ops are those of wrk.h.  Citations are path:line inside
 * cryscan/web-rwkv.
 */
#ifndef WRK_RUNTIME_H
#define WRK_RUNTIME_H

#include "wrk.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct wrk_model_builder wrk_model_builder; /* `ModelBuilder<R>`, src/runtime/model.rs:137-185 */
typedef struct wrk_model wrk_model;                 /* `v5::Model` / `v6::Model` / `v7::Model` */
typedef struct wrk_bundle wrk_bundle;               /* `Bundle<f16>` + its `State`, src/runtime/v6.rs:489-521 */
typedef struct wrk_rnn_input wrk_rnn_input;         /* `RnnInput`, src/runtime/infer/rnn.rs:194-228 */
typedef struct wrk_rnn_iter wrk_rnn_iter;           /* `RnnIter`, src/runtime/infer/rnn.rs:274-335 */
typedef struct wrk_job wrk_job;                     /* `RnnJob`, src/runtime/v6.rs:408-477 */

/* `ModelInfo`, src/runtime/model.rs:24-76 (+ `ModelCustomInfo`: v6 {time_mix, time_decay},
 * v7 {w, a, g, v}). version is 4, 5, 6 or 7 (v4 counts one head: src/runtime/loader.rs:290-294). */
typedef struct {
    uint32_t version;
    uint32_t num_layer;
    uint32_t num_emb;
    uint32_t num_hidden;
    uint32_t num_vocab;
    uint32_t num_head;
    uint32_t custom[4];
} wrk_model_info;

/* ---- ModelBuilder: the `Reader` trait (src/runtime/loader.rs:44-74) is fed tensor by tensor ---- */
int32_t wrk_model_builder_create(wrk_context* ctx, wrk_model_builder** out); /* ModelBuilder::new */
int32_t wrk_model_builder_destroy(wrk_model_builder* b);
/* One safetensors entry: fp16 data, shape outermost-first as stored in the file (a weight of M rows
 * and K columns is {M, K}).  The bytes are copied. */
int32_t wrk_model_builder_add_tensor(wrk_model_builder* b, const char* name, const uint64_t* shape, uint32_t ndim,
                                     const void* data_f16, size_t bytes);
/* ModelBuilder::lora (src/runtime/model.rs:176-179) with a `Lora` (src/runtime/loader.rs:104-171) fed piece by piece:
 * `_lora` opens one and returns its index, `_lora_tensor` adds a named fp16 tensor of the LoRA file (a vector or
 * matrix named like the model's, or "<matrix name without .weight>.lora.0 / .lora.1"), `_lora_blend` appends a
 * LoraBlendPattern (regex searched in the tensor name, factor alpha; the last matching pattern of a LoRA counts).
 * LoraBlend::full(alpha) = blend(".+", 1.0) then
 * blend("blocks\.([0-9]+)\.(att|ffn)\.(key|value|receptance|gate|output)\.weight", alpha).
 * Applied at build time as in src/runtime/loader.rs:393-686: vectors alpha * lora + (1 - alpha) * model in f32,
 * matrices += discount * alpha / rank * lora.0 x lora.1 (TensorOp::blend_lora) before quantization. */
int32_t wrk_model_builder_lora(wrk_model_builder* b, uint32_t* index);
int32_t wrk_model_builder_lora_tensor(wrk_model_builder* b, uint32_t index, const char* name, const uint64_t* shape,
                                      uint32_t ndim, const void* data_f16, size_t bytes);
int32_t wrk_model_builder_lora_blend(wrk_model_builder* b, uint32_t index, const char* pattern, float alpha);
/* No counterpart in the reference (one GPU).  Makes the builder keep one rank's part of a model split `world` ways:
 * call before the first tensor; every tensor is cut as it is added.  Time-mix channels are split by whole heads
 * (key / value / receptance / gate and the per-channel adapters' second matrices keep the rank's rows, `output` the
 * matching columns), ffn `key` by rows and `value` by the matching columns, the head by vocabulary rows; everything
 * else is held whole.  Splits of a K dimension fall on multiples of `block` (128 when any layer is Int8, 64 for
 * NF4 / SF4, 1 for fp16), so a rank's packed bytes and scales equal the matching slice of the whole model's.
 * wrk_shard_range is the rule: `world` contiguous ranges of whole `align` units, sizes within one unit, larger first. */
int32_t wrk_model_builder_shard(wrk_model_builder* b, uint32_t rank, uint32_t world, uint32_t head_size, uint32_t block);
int32_t wrk_shard_range(uint32_t total, uint32_t align, uint32_t world, uint32_t rank, uint32_t* begin, uint32_t* end);
int32_t wrk_model_builder_quant(wrk_model_builder* b, uint32_t layer, int32_t quant); /* ModelBuilder::quant */
int32_t wrk_model_builder_rescale(wrk_model_builder* b, uint32_t value);             /* ModelBuilder::rescale */
int32_t wrk_model_builder_sep(wrk_model_builder* b, uint32_t value);                 /* ModelBuilder::sep */
/* read_state (src/runtime/v6.rs:1175-1208, same in v5.rs / v7.rs): the pre-trained initial state stored in the file as
 * blocks.N.att.time_state, as the f32 [C, S + 2, L] tensor that State::load (wrk_state_load) takes for a batch slot. */
int32_t wrk_model_builder_read_state(wrk_model_builder* b, float* host, size_t bytes);
/* Loader::info (src/runtime/loader.rs:208-324) on the tensors added so far. */
int32_t wrk_model_builder_info(wrk_model_builder* b, wrk_model_info* info);
/* ModelBuilder::build_v4 / build_v5 / build_v6 / build_v7 (src/runtime/v4.rs:829-960, v5.rs:922-1082, v6.rs:995-1172,
 * v7.rs:1038-1226), chosen by the version Loader::info finds. */
int32_t wrk_model_builder_build(wrk_model_builder* b, wrk_model** out);

/* The built model (packed weights, block scales, code tables; no fp16 originals of quantized matrices) written to
 * one file and restored from it: the reference derives Serialize for its `Model` (every `TensorGpu` is read back as a
 * `TensorBlob {shape, data}`, src/tensor/serialization.rs:11-75), restores through `Seed<Context, Model>`
 * (src/tensor/serialization.rs:96-159) and round-trips through CBOR in examples/serde.rs:218-268.  The file is that
 * CBOR tree: maps keyed by the reference's field names, `Matrix` as `Fp16` / `Int8 {w, m}` / `Fp4 {q, w, m}`. */
int32_t wrk_model_save(wrk_model* m, const char* path);
int32_t wrk_model_load(wrk_context* ctx, const char* path, wrk_model** out);

int32_t wrk_model_info_get(const wrk_model* m, wrk_model_info* info);
int32_t wrk_model_retain(wrk_model* m);
int32_t wrk_model_release(wrk_model* m);
/* A layer's matrix by field name ("att.w_k", "att.w_v", "att.w_r", "att.w_g", "att.w_o", "ffn.w_k",
 * "ffn.w_v", "ffn.w_r"; layer = UINT32_MAX with "head.w").  Borrowed: valid while the model lives. */
int32_t wrk_model_matrix(wrk_model* m, uint32_t layer, const char* name, wrk_matrix** out);

/* ---- Bundle + State (src/runtime/model.rs:78-120, src/runtime/v6.rs:142-266, 499-521) ---- */
int32_t wrk_bundle_create(wrk_model* model, uint32_t num_batch, wrk_bundle** out); /* Bundle::<f16>::new */
/* The bundle of one rank of a split model (wrk_model_builder_shard): the op list of the reference's dispatch_layer
 * (src/runtime/v5.rs:656-885, v6.rs:701-958, v7.rs:716-1007) with the time-mix ops on the rank's heads, `output` and
 * ffn `value` producing f32 partial sums that one all-reduce per sub-block adds across the ranks, and the rank's
 * vocabulary rows gathered into full logits.  Every rank submits the same jobs in the same order.  State rows of
 * heads the rank does not own stay zero (wrk_state_back returns them so). */
int32_t wrk_bundle_create_sharded(wrk_model* model, uint32_t num_batch, wrk_comm* comm, wrk_bundle** out);
/* How the partial sums of a sharded bundle meet: 1 = the one-shot reduce over peer memory (wrk_op_peer_all_reduce; the
 * matmuls write into the exchange slots, no copy), the default where wrk_bundle_create_sharded could set the exchange
 * region up (jobs of up to 256 tokens; larger ones use NCCL); 0 = NCCL all-reduce.  Every rank sets the same value. */
int32_t wrk_bundle_set_peer_reduce(wrk_bundle* b, int32_t on);
int32_t wrk_bundle_peer_reduce(const wrk_bundle* b, int32_t* on);
int32_t wrk_bundle_release(wrk_bundle* b);
/* Cursor format uploaded with every job: 0 (default) = three u32 per token, exact for any run length;
 * 1 = the reference's packed u32 (8-bit batch, 16-bit token, 8-bit len: src/tensor/mod.rs:53-60). */
int32_t wrk_bundle_set_packed_cursors(wrk_bundle* b, int32_t packed);
/* Build jobs as CUDA graphs (default 1) or as plain launch lists (0). */
int32_t wrk_bundle_set_use_graph(wrk_bundle* b, int32_t use_graph);
/* 2 (default): jobs may use fused kernels in place of runs of reference ops, one launch per phase (seven per v6
 * layer, chained by programmatic dependent launch inside a CUDA graph); 1: a v6 job of at most 8 tokens runs as
 * one persistent kernel instead (all layers and the head; the CTAs meet at a grid barrier between phases; Int8 and
 * fp16 matrices with one or two tokens are multiplied by tcgen05.mma from shared memory, anything else by cp.async
 * rings and mma.sync); 3: as 1 but always the mma.sync kernel; 0: one launch per reference op, every intermediate
 * tensor materialised with the reference's dtypes.  No counterpart in the reference, whose jobs are always one
 * pass per op (src/runtime/v6.rs:560-900). */
int32_t wrk_bundle_set_fused(wrk_bundle* b, int32_t fused);

/* ---- Hooks (`Hook` and `HookMap` of each version: src/runtime/v4.rs:304-330, v5.rs:330-358, v6.rs:366-406,
 * v7.rs:385-425; called through `hook_op`, src/runtime/v6.rs:572-581) ----
 * A hook is a callback that, while a job is being built, may return one op to insert at its point of the layer's op
 * list (or leave *op null: TensorOp::empty()).  It sees the job's `Frame` (src/runtime/v6.rs:479-487): runtime buffers
 * by the reference's field name ("x", "att_x", "att_k", "ffn_k", ... of `Runtime`, src/runtime/v6.rs:305-345; "head_x",
 * "head_o" of `Header`), and the state through wrk_state_layer.  The enum is the union of the four versions' hooks; a
 * point a version does not have is never reached.  `layer` is ignored for the embed / head hooks.  While a bundle
 * has any hook, its jobs are built one launch per reference op (the fused kernels have no such points); setting or
 * clearing a hook drops the cached jobs.  fn == NULL clears the hook. */
typedef enum {
    WRK_HOOK_POST_EMBED_LOADED = 0, WRK_HOOK_POST_EMBED_LAYER_NORM,
    WRK_HOOK_PRE_ATT, WRK_HOOK_POST_ATT_LAYER_NORM, WRK_HOOK_PRE_ATT_TOKEN_SHIFT, WRK_HOOK_POST_ATT_TOKEN_SHIFT,
    WRK_HOOK_PRE_ATT_TOKEN_SHIFT_ADAPT, WRK_HOOK_POST_ATT_TOKEN_SHIFT_ADAPT_ACTIVATE, WRK_HOOK_POST_ATT_TOKEN_SHIFT_ADAPT,
    WRK_HOOK_PRE_ATT_GATED_TOKEN_SHIFT, WRK_HOOK_POST_ATT_GATED_TOKEN_SHIFT,
    WRK_HOOK_PRE_ATT_LINEAR, WRK_HOOK_POST_ATT_LINEAR,
    WRK_HOOK_PRE_ATT_TIME_DECAY_ADAPT, WRK_HOOK_POST_ATT_TIME_DECAY_ADAPT_ACTIVATE, WRK_HOOK_POST_ATT_TIME_DECAY_ADAPT,
    WRK_HOOK_PRE_ATT_TIME_DECAY_ACTIVATE, WRK_HOOK_POST_ATT_TIME_DECAY_ACTIVATE,
    WRK_HOOK_PRE_ATT_ADAPT, WRK_HOOK_POST_ATT_ADAPT, WRK_HOOK_PRE_ATT_CONTROL, WRK_HOOK_POST_ATT_CONTROL,
    WRK_HOOK_PRE_ATT_VALUE_RESIDUAL, WRK_HOOK_POST_ATT_VALUE_RESIDUAL,
    WRK_HOOK_PRE_ATT_TIME_MIX, WRK_HOOK_POST_ATT_TIME_MIX, WRK_HOOK_PRE_ATT_GATE, WRK_HOOK_POST_ATT_GATE,
    WRK_HOOK_PRE_ATT_OUT, WRK_HOOK_POST_ATT_OUT, WRK_HOOK_POST_ATT,
    WRK_HOOK_PRE_FFN, WRK_HOOK_POST_FFN_LAYER_NORM, WRK_HOOK_PRE_FFN_TOKEN_SHIFT, WRK_HOOK_POST_FFN_TOKEN_SHIFT,
    WRK_HOOK_PRE_FFN_LINEAR, WRK_HOOK_POST_FFN_ACTIVATE, WRK_HOOK_POST_FFN_LINEAR,
    WRK_HOOK_PRE_FFN_CHANNEL_MIX, WRK_HOOK_POST_FFN_CHANNEL_MIX, WRK_HOOK_POST_FFN,
    WRK_HOOK_PRE_HEAD, WRK_HOOK_POST_HEAD_LAYER_NORM, WRK_HOOK_POST_HEAD,
    WRK_HOOK_COUNT
} wrk_hook;
typedef struct wrk_frame wrk_frame; /* `Frame`, src/runtime/v6.rs:479-487: valid only inside the callback */
typedef int32_t (*wrk_hook_fn)(void* user, const wrk_frame* frame, wrk_op** op);
int32_t wrk_bundle_set_hook(wrk_bundle* b, int32_t hook, uint32_t layer, wrk_hook_fn fn, void* user);
int32_t wrk_frame_bundle(const wrk_frame* frame, wrk_bundle** bundle);               /* Frame::state lives in the bundle */
int32_t wrk_frame_num_token(const wrk_frame* frame, uint32_t* num_token, uint32_t* num_header);
/* A buffer of the frame by field name; borrowed: valid while the job lives (ops built on it keep it alive). */
int32_t wrk_frame_buffer(const wrk_frame* frame, const char* name, wrk_tensor** out);
/* No counterpart in the reference (its profiler hooks are wgpu timestamp queries, commented out in
 * src/tensor/ops.rs:2600).  Makes the persistent decode kernel record the device's nanosecond timer when each CTA
 * starts (after the grid barrier) and ends every phase; max_phases = 0 switches it off.  Jobs built afterwards with
 * at most max_phases phases record; wrk_job_phase_timeline copies the stamps of the job's last run to the host
 * as [2 * num_phases][num_ctas] u64 (phase start rows even, phase end rows odd). */
int32_t wrk_bundle_set_phase_timeline(wrk_bundle* b, uint32_t max_phases);
int32_t wrk_job_phase_timeline(wrk_job* job, uint64_t* stamps, size_t capacity, uint32_t* num_phases, uint32_t* num_ctas);
int32_t wrk_state_num_batch(wrk_bundle* b, uint32_t* num_batch);                 /* State::num_batch */
/* State::init_shape as [C, rows, L, 1] with rows = S + 2 (v5 / v6 / v7: src/runtime/v6.rs:163-168) or 5 (v4, whose
 * reference shape [C, 5 L] is the same memory: src/runtime/v4.rs:158-161).  A new v4 bundle holds State::init's f32::MIN
 * in the running-maximum row (src/runtime/v4.rs:163-180). */
int32_t wrk_state_init_shape(wrk_bundle* b, uint32_t shape[4]);
int32_t wrk_state_load(wrk_bundle* b, const float* host, size_t bytes, uint32_t batch); /* State::load */
int32_t wrk_state_back(wrk_bundle* b, uint32_t batch, float* host, size_t bytes);       /* State::back */
/* State::write / State::read (src/runtime/model.rs:98-100; v6: src/runtime/v6.rs:223-258): a batch slot from / to a
 * device tensor f32 [C, S + 2, L], ordered on the context's stream (no host wait); `read` returns a new tensor. */
int32_t wrk_state_write(wrk_bundle* b, wrk_tensor* tensor, uint32_t batch);
int32_t wrk_state_read(wrk_bundle* b, uint32_t batch, wrk_tensor** out);
/* State::embed (src/runtime/model.rs:102; v6: src/runtime/v6.rs:260-262): row 0 of layer `layer` of a state read back
 * with wrk_state_back, C floats. */
int32_t wrk_state_embed(wrk_bundle* b, uint32_t layer, const float* backed, size_t bytes, float* embed, size_t embed_bytes);
/* The per-layer state tensor [C, S + 2, num_batch] (borrowed), as State::att / State::ffn slice it. */
int32_t wrk_state_layer(wrk_bundle* b, uint32_t layer, wrk_tensor** out);

/* ---- RnnInput / RnnIter / RnnInfo::redirect (src/runtime/infer/rnn.rs) ---- */
int32_t wrk_rnn_input_create(uint32_t num_batch, uint32_t token_chunk_size, wrk_rnn_input** out); /* RnnInput::new */
int32_t wrk_rnn_input_destroy(wrk_rnn_input* in);
int32_t wrk_rnn_input_set_option(wrk_rnn_input* in, uint32_t batch, int32_t option);
int32_t wrk_rnn_input_append(wrk_rnn_input* in, uint32_t batch, const uint32_t* tokens, size_t count); /* RnnInputBatch::append */
int32_t wrk_rnn_input_token_chunk_size(const wrk_rnn_input* in, uint32_t* size);
int32_t wrk_rnn_input_num_token(const wrk_rnn_input* in, uint64_t* count);
int32_t wrk_rnn_input_remaining(const wrk_rnn_input* in, uint32_t batch, uint64_t* count);
int32_t wrk_rnn_input_step(wrk_rnn_input* in);                                   /* JobInput::step */
/* `(&input).into_iter()` and `RnnIter::next`: per batch the token count of the next job and its
 * Option<RnnOption> (WRK_RNN_NONE = None). */
int32_t wrk_rnn_iter_create(const wrk_rnn_input* in, wrk_rnn_iter** out);
int32_t wrk_rnn_iter_next(wrk_rnn_iter* it, uint32_t* lens, int32_t* options);
int32_t wrk_rnn_iter_destroy(wrk_rnn_iter* it);
/* RnnInfo::redirect: headers (capacity = total tokens), and per batch the [start, end) ranges in the
 * input and output tensors (2 * num_batch entries each). */
int32_t wrk_rnn_redirect(const uint32_t* lens, const int32_t* options, uint32_t num_batch, uint32_t* headers,
                         uint32_t* num_headers, uint32_t* inputs, uint32_t* outputs);

/* ---- Dispatcher / Job (src/runtime/mod.rs:36-58, src/runtime/v6.rs:408-477, 583-697) ---- */
int32_t wrk_bundle_dispatch(wrk_bundle* b, const uint32_t* lens, const int32_t* options, wrk_job** out);
/* Job::load: the chunk's tokens, batch after batch (sum(lens) entries). */
int32_t wrk_job_load(wrk_job* job, const uint32_t* tokens, size_t count);
/* Job::load for `Token::Embed` inputs (src/runtime/infer/mod.rs:21-25) that already live on the device:
 * rows [row0, row0 + num_token) of `embeds` ([num_emb, rows] fp16) become the job's input; cursors are
 * uploaded as in wrk_job_load.  Stream ordered, no host synchronisation. */
int32_t wrk_job_load_embed(wrk_job* job, wrk_tensor* embeds, uint32_t row0);
int32_t wrk_job_submit(wrk_job* job);
/* Job::back: waits, copies the [num_vocab_padded, num_header] f32 logits to `logits` (capacity in
 * floats) and reports per batch the [start, end) header rows (2 * num_batch entries). */
int32_t wrk_job_back(wrk_job* job, float* logits, size_t capacity, uint32_t* outputs, uint32_t* num_headers);
/* The job's logits tensor [num_vocab_padded, num_header] f32 on the device (borrowed). */
int32_t wrk_job_output(wrk_job* job, wrk_tensor** out);
int32_t wrk_job_num_kernels(const wrk_job* job, uint64_t* count);
int32_t wrk_job_release(wrk_job* job);

/* SimpleRuntime::infer (src/runtime/mod.rs:237-262): next chunk → dispatch → load → submit → back →
 * step.  Returns WRK_ERR_INPUT_EXHAUSTED when no token is left. */
int32_t wrk_runtime_infer(wrk_bundle* b, wrk_rnn_input* in, float* logits, size_t capacity, uint32_t* outputs,
                          uint32_t* num_headers);
#ifdef __cplusplus
}
#endif
#endif /* WRK_RUNTIME_H */
