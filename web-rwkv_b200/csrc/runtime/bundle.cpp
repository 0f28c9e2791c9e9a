// Bundle, State and the dispatch → load → submit → back job protocol of the v5/v6/v7 runtimes.
//
// dispatch() builds, per job shape, the same operator list the reference builds in
// dispatch_layer / dispatch_header (src/runtime/v5.rs:656-920, v6.rs:701-992, v7.rs:716-1036) with the
// same buffer dtypes (Bundle<f16>), encodes it once (optionally as a CUDA graph: the analogue of the
// reference's pre-encoded command buffers) and caches it by (num_token, header rows).  load() gathers
// the embeddings on the host like the reference (v6.rs:423-459) into pinned memory and uploads them
// with the cursors; back() reads the [vocab, num_header] fp32 logits into the caller's buffer.
// Hooks (v6.rs:366-406) are not built.
#include <cstring>
#include <limits>
#include <list>

#include "../kernels/decode.cuh"
#include "runtime.h"

using namespace wrk;
using namespace wrk::rt;

namespace {

constexpr float LN_EPS = 1.0e-5f, GN_EPS = 64.0e-5f, L2_EPS = 1.0e-12f;

struct Buffers {
    std::unordered_map<std::string, TensorH> t;
    std::vector<uint32_t> cursor_lens;  // per-batch lens of the cursors currently held in t["cursors"]
    wrk_tensor* operator[](const char* name) const { return t.at(name).p; }
};

struct CachedJob {
    std::shared_ptr<Buffers> buffer, header;
    RnnRedirect redirect;
    wrk_commands* commands = nullptr;
    uint32_t num_token = 0, num_header = 0;
    uint64_t tick = 0;
    std::vector<TensorH> tables;  // row partitions, phase lists and work lists of the fused paths
    uint32_t num_phases = 0;      // phases of the step kernel (0: the job runs as a list of launches)
    ~CachedJob() {
        if (commands) wrk_commands_release(commands);
    }
};

}  // namespace

struct wrk_bundle {
    std::atomic<int> refs{1};
    wrk_model* model = nullptr;
    uint32_t num_batch = 0;
    std::vector<TensorH> state;  // per layer f32 [C, S + 2, num_batch]
    struct HookEntry {
        wrk_hook_fn fn;
        void* user;
    };
    std::map<std::pair<int32_t, uint32_t>, HookEntry> hooks;  // (hook, layer; 0 for the embed / head hooks)
    const Buffers* building_header = nullptr;  // of the job being built (for the hooks' frame)
    uint32_t building_tokens = 0, building_headers = 0;
    bool peer_reduce = false;  // partial sums meet through the communicator's exchange region instead of NCCL
    wrk_comm* comm = nullptr;  // a rank of a split model: sums of partial products cross this communicator
    bool packed_cursors = false, use_graph = true, fused = true;
    bool step_kernel = false;  // fused jobs of at most 8 tokens run as one persistent kernel where the job shape allows it
    int step_engine = 1;      // 1: tensor-core kernel where the matrices allow it; 3: always the mma.sync kernel
    TensorH timeline;         // optional globaltimer stamps of the step kernel: [2 * timeline_phases][num_sms] u64
    size_t timeline_phases = 0;
    std::map<uint32_t, std::shared_ptr<Buffers>> buffers, headers;
    std::map<std::vector<uint32_t>, std::shared_ptr<CachedJob>> jobs;
    uint64_t tick = 0;
    // pinned staging
    uint16_t* stage_input = nullptr;
    uint32_t* stage_cursors = nullptr;
    size_t stage_tokens = 0;
    std::mutex mutex;
    ~wrk_bundle() {
        jobs.clear();
        if (stage_input) cudaFreeHost(stage_input);
        if (stage_cursors) cudaFreeHost(stage_cursors);
        state.clear();
        if (model) wrk_model_release(model);
        if (comm) wrk_comm_release(comm);
    }
};

struct wrk_job {
    wrk_bundle* bundle = nullptr;
    std::shared_ptr<CachedJob> job;
    RnnInfo info;
    RnnRedirect redirect;  // this dispatch's per-batch output ranges (jobs of one structure share a CachedJob)
};

namespace {

struct OpList {
    std::vector<wrk_op*> ops;
    ~OpList() {
        for (auto o : ops) wrk_op_release(o);
    }
};

#define ADD(call)                   \
    do {                            \
        wrk_op* _o = nullptr;       \
        WRK_TRY(call);              \
        ops.ops.push_back(_o);      \
    } while (0)

wrk_view V(wrk_tensor* t) {
    wrk_view v;
    wrk_tensor_as_view(t, &v);
    return v;
}
wrk_view Vz(wrk_tensor* t, uint32_t z) {  // t.view(.., .., z, ..)
    wrk_view v = V(t);
    v.shape[2] = 1;
    v.offset[2] = z;
    return v;
}
wrk_view Vy(wrk_tensor* t, uint32_t y0, uint32_t y1) {  // t.view(.., y0..y1, .., ..)
    wrk_view v = V(t);
    v.shape[1] = y1 - y0;
    v.offset[1] = y0;
    return v;
}

wrk_view Vx(wrk_tensor* t, uint32_t x0, uint32_t x1) {  // t.view(x0..x1, .., .., ..)
    wrk_view v = V(t);
    v.shape[0] = x1 - x0;
    v.offset[0] = x0;
    return v;
}

int32_t reshape(wrk_tensor* t, uint32_t x, uint32_t y, uint32_t z, uint32_t w, TensorH* out) {
    const uint32_t s[4] = {x, y, z, w};
    wrk_tensor* r = nullptr;
    WRK_TRY(wrk_tensor_reshape(t, s, &r));
    *out = TensorH(r);
    return WRK_OK;
}

int32_t alloc(wrk_context* ctx, Buffers& b, const char* name, int dtype, uint32_t x, uint32_t y, uint32_t z = 1) {
    const uint32_t s[4] = {x, y, z, 1};
    wrk_tensor* t = nullptr;
    WRK_TRY(wrk_tensor_create(ctx, (wrk_dtype)dtype, s, &t));
    b.t[name] = TensorH(t);
    return WRK_OK;
}

// Rows of a layer's state per batch slot: S + 2 (v5 / v6 / v7: v6.rs:163-168), 5 for v4 (v4.rs:158-161).
uint32_t state_rows(const wrk_model_info& info) { return info.version == 4 ? 5u : info.num_emb / info.num_head + 2; }

// Runtime<f16>::new of each version (v5.rs:258-315, v6.rs:268-345, v7.rs:279-363)
int32_t make_runtime(wrk_bundle* bd, uint32_t T, std::shared_ptr<Buffers>* out) {
    const wrk_model_info& info = bd->model->info;
    wrk_context* ctx = bd->model->ctx;
    auto b = std::make_shared<Buffers>();
    const uint32_t C = info.num_emb;
    // a rank of a split model keeps its own time-mix channels (Cl of C) and FFN columns (F of num_hidden); the
    // residual stream, the token shifts and the sums after `output` / ffn `value` span all C channels
    const Shard& sh = bd->model->shard;
    const uint32_t Cl = sh.on() ? sh.c1 - sh.c0 : C, F = sh.on() ? sh.f1 - sh.f0 : info.num_hidden;
    const int H16 = WRK_F16, F32 = WRK_F32;
    WRK_TRY(alloc(ctx, *b, "cursors", WRK_U32, bd->packed_cursors ? T : 3 * T, 1));
    WRK_TRY(alloc(ctx, *b, "input", H16, C, T));
    WRK_TRY(alloc(ctx, *b, "x", H16, C, T));
    if (sh.on()) {
        WRK_TRY(alloc(ctx, *b, "att_xl", H16, Cl, T));
        size_t slot_bytes = 0;
        if (bd->peer_reduce) WRK_TRY(wrk_comm_peer_slot_bytes(bd->comm, &slot_bytes));
        if ((size_t)C * T * 4 <= slot_bytes) {
            // the partial sums of `output` (slot 0) and ffn `value` (slot 1) are written where the peers read them
            const uint32_t shape[4] = {C, T, 1, 1};
            for (uint32_t slot = 0; slot < 2; ++slot) {
                wrk_tensor* t = nullptr;
                WRK_TRY(wrk_comm_peer_slot(bd->comm, slot, WRK_F32, shape, &t));
                b->t[slot == 0 ? "partial0" : "partial1"] = TensorH(t);
            }
        } else {
            WRK_TRY(alloc(ctx, *b, "partial", F32, C, T));
        }
    }
    if (info.version == 7) {
        for (auto n : {"att_x", "att_rx", "att_wx", "att_kx", "att_vx", "att_ax", "att_gx", "att_o", "ffn_x", "ffn_kx", "ffn_v"})
            WRK_TRY(alloc(ctx, *b, n, H16, C, T));
        for (auto n : {"att_v0", "att_r", "att_w", "att_k", "att_v", "att_a", "att_g", "att_kk", "att_vv"})
            WRK_TRY(alloc(ctx, *b, n, H16, Cl, T));
        WRK_TRY(alloc(ctx, *b, "att_n", H16, Cl, T, 4));
        WRK_TRY(alloc(ctx, *b, "aux_w", H16, info.custom[0], T));
        WRK_TRY(alloc(ctx, *b, "aux_a", H16, info.custom[1], T));
        WRK_TRY(alloc(ctx, *b, "aux_g", H16, info.custom[2], T));
        WRK_TRY(alloc(ctx, *b, "aux_v", H16, info.custom[3], T));
        WRK_TRY(alloc(ctx, *b, "ffn_k", H16, F, T));
    } else if (info.version == 4) {
        // Runtime<f16>::new, v4.rs:258-282
        WRK_TRY(alloc(ctx, *b, "aux_x", F32, C, T));
        for (auto n : {"att_x", "att_kx", "att_vx", "att_rx", "att_o", "ffn_x", "ffn_kx", "ffn_rx", "ffn_v", "ffn_r"})
            WRK_TRY(alloc(ctx, *b, n, H16, C, T));
        for (auto n : {"att_k", "att_v", "att_r"}) WRK_TRY(alloc(ctx, *b, n, F32, C, T));
        WRK_TRY(alloc(ctx, *b, "ffn_k", H16, F, T));
    } else {
        WRK_TRY(alloc(ctx, *b, "aux_x", F32, Cl, T));
        for (auto n : {"att_x", "att_o", "ffn_x", "ffn_kx", "ffn_rx", "ffn_v", "ffn_r"})
            WRK_TRY(alloc(ctx, *b, n, H16, C, T));
        WRK_TRY(alloc(ctx, *b, "att_g", H16, Cl, T));
        for (auto n : {"att_k", "att_v", "att_r"}) WRK_TRY(alloc(ctx, *b, n, F32, Cl, T));
        WRK_TRY(alloc(ctx, *b, "ffn_k", H16, F, T));
        if (info.version == 6) {
            WRK_TRY(alloc(ctx, *b, "att_xx", H16, C, T));
            WRK_TRY(alloc(ctx, *b, "att_sx", H16, C, T, 5));
            WRK_TRY(alloc(ctx, *b, "att_w", H16, info.custom[1], T));
            WRK_TRY(alloc(ctx, *b, "time_mix_x", H16, info.custom[0], 5, T));
            WRK_TRY(alloc(ctx, *b, "time_mix_t", H16, info.custom[0], T, 5));
            WRK_TRY(alloc(ctx, *b, "time_mix", H16, C, T, 5));
            WRK_TRY(alloc(ctx, *b, "time_decay", F32, Cl, T));
        } else {
            for (auto n : {"att_kx", "att_vx", "att_rx", "att_gx"}) WRK_TRY(alloc(ctx, *b, n, H16, C, T));
        }
    }
    *out = b;
    return WRK_OK;
}

int32_t make_header(wrk_bundle* bd, uint32_t num_header, std::shared_ptr<Buffers>* out) {
    const wrk_model_info& info = bd->model->info;
    auto b = std::make_shared<Buffers>();
    WRK_TRY(alloc(bd->model->ctx, *b, "head_x", WRK_F16, info.num_emb, num_header));
    uint32_t vocab = 0;
    {
        uint32_t s[4];
        wrk_tensor* w = nullptr;
        wrk_matrix_parts(bd->model->head_w, nullptr, &w, nullptr, nullptr);
        wrk_tensor_shape(w, s);
        vocab = s[1];
    }
    const Shard& sh = bd->model->shard;
    if (sh.on()) {
        // the rank's slice of the vocabulary, every rank's slice (gathered), and the rows put in order
        WRK_TRY(alloc(bd->model->ctx, *b, "head_l", WRK_F32, vocab, num_header));
        WRK_TRY(alloc(bd->model->ctx, *b, "head_all", WRK_F32, vocab, num_header, sh.world));
        vocab *= sh.world;
    }
    WRK_TRY(alloc(bd->model->ctx, *b, "head_o", WRK_F32, vocab, num_header));
    *out = b;
    return WRK_OK;
}

int32_t matmul(OpList& ops, wrk_matrix* m, wrk_view in, wrk_view out, int32_t act, bool turbo, bool sparse = false) {
    wrk_op* _o = nullptr;
    if (sparse) WRK_TRY(wrk_matrix_matmul_op_sparse(m, &in, &out, act, turbo, &_o));
    else WRK_TRY(wrk_matrix_matmul_op(m, &in, &out, act, turbo, &_o));
    ops.ops.push_back(_o);
    return WRK_OK;
}

struct GroupItem {
    wrk_matrix* m;
    wrk_view in, out;
    int32_t act;
};
int32_t matmul_group(OpList& ops, std::initializer_list<GroupItem> items, bool turbo) {
    wrk_matrix* ms[4];
    wrk_view ins[4], outs[4];
    int32_t acts[4];
    uint32_t n = 0;
    for (const GroupItem& it : items) {
        if (n == 4) return set_error(WRK_ERR_INVALID_ARGUMENT, "a group holds at most 4 matrices");
        ms[n] = it.m, ins[n] = it.in, outs[n] = it.out, acts[n] = it.act;
        ++n;
    }
    ADD(wrk_matrix_matmul_group_op(ms, ins, outs, acts, n, turbo, &_o));
    return WRK_OK;
}

int32_t token_shift(OpList& ops, wrk_tensor* cursors, wrk_view mix, wrk_view state, wrk_tensor* in, wrk_tensor* out,
                    bool reversed) {
    ADD(wrk_op_token_shift(cursors, &mix, &state, in, out, reversed, &_o));
    return WRK_OK;
}

int32_t blit(OpList& ops, wrk_view in, wrk_view out) {
    ADD(wrk_op_blit(&in, &out, &_o));
    return WRK_OK;
}

int32_t add(OpList& ops, wrk_view in, wrk_view out, int32_t act_out = WRK_ACT_NONE) {
    ADD(wrk_op_add_activate(&in, &out, WRK_ACT_NONE, WRK_ACT_NONE, act_out, &_o));
    return WRK_OK;
}

}  // namespace

struct wrk_frame {
    wrk_bundle* bundle;
    const Buffers* buffer;
    const Buffers* header;
    uint32_t num_token, num_header;
};

namespace {

// hook_op, v6.rs:572-581: the op a registered callback returns for this point of the job, if any
int32_t hook(wrk_bundle* bd, OpList& ops, const Buffers& B, int32_t kind, uint32_t layer) {
    if (bd->hooks.empty()) return WRK_OK;
    const bool global = kind <= WRK_HOOK_POST_EMBED_LAYER_NORM || kind >= WRK_HOOK_PRE_HEAD;
    auto it = bd->hooks.find({kind, global ? 0u : layer});
    if (it == bd->hooks.end()) return WRK_OK;
    wrk_frame frame{bd, &B, bd->building_header, bd->building_tokens, bd->building_headers};
    wrk_op* op = nullptr;
    const int32_t s = it->second.fn(it->second.user, &frame, &op);
    if (s != WRK_OK) {
        if (op) wrk_op_release(op);
        return s;
    }
    if (op) ops.ops.push_back(op);
    return WRK_OK;
}
#define HOOK(kind) WRK_TRY(hook(bd, ops, B, WRK_HOOK_##kind, index))

// State::att / State::ffn, v6.rs:187-197
wrk_view state_att(wrk_bundle* bd, uint32_t layer, uint32_t S) { return Vy(bd->state[layer], 0, S + 1); }
wrk_view state_ffn(wrk_bundle* bd, uint32_t layer, uint32_t S) { return Vy(bd->state[layer], S + 1, S + 2); }

// dispatch_layer of v4 (v4.rs:630-795); the layer's state is [C, 5, B]: rows 0-3 for the time mix (shift row, the two
// running sums and the running maximum), row 4 the ffn shift row (v4.rs:182-192)
int32_t layer_v4(wrk_bundle* bd, OpList& ops, const Buffers& B, uint32_t index, uint32_t T) {
    const Layer& L = bd->model->layers[index];
    const bool turbo = T % WRK_MIN_TOKEN_CHUNK_SIZE == 0;
    wrk_tensor* cursors = B["cursors"];
    const wrk_view sa = Vy(bd->state[index], 0, 4), sf = Vy(bd->state[index], 4, 5);
    WRK_TRY(blit(ops, V(B["x"]), V(B["att_x"])));
    HOOK(PRE_ATT);
    ADD(wrk_op_layer_norm(L.att_ln.w, L.att_ln.b, B["att_x"], LN_EPS, &_o));
    HOOK(POST_ATT_LAYER_NORM);
    HOOK(PRE_ATT_TOKEN_SHIFT);
    WRK_TRY(token_shift(ops, cursors, V(L.time_mix_k), sa, B["att_x"], B["att_kx"], false));
    WRK_TRY(token_shift(ops, cursors, V(L.time_mix_v), sa, B["att_x"], B["att_vx"], false));
    WRK_TRY(token_shift(ops, cursors, V(L.time_mix_r), sa, B["att_x"], B["att_rx"], false));
    HOOK(POST_ATT_TOKEN_SHIFT);
    HOOK(PRE_ATT_LINEAR);
    WRK_TRY(matmul(ops, L.att_w_k, V(B["att_kx"]), V(B["att_k"]), WRK_ACT_NONE, turbo));
    WRK_TRY(matmul(ops, L.att_w_v, V(B["att_vx"]), V(B["att_v"]), WRK_ACT_NONE, turbo));
    WRK_TRY(matmul(ops, L.att_w_r, V(B["att_rx"]), V(B["att_r"]), WRK_ACT_NONE, turbo));
    HOOK(POST_ATT_LINEAR);
    HOOK(PRE_ATT_TIME_MIX);
    WRK_TRY(blit(ops, V(B["att_x"]), V(B["aux_x"])));
    ADD(wrk_op_time_mix_v4(cursors, L.time_decay, L.time_first, &sa, B["att_k"], B["att_v"], B["att_r"], B["aux_x"], &_o));
    WRK_TRY(blit(ops, V(B["aux_x"]), V(B["att_x"])));
    HOOK(POST_ATT_TIME_MIX);
    HOOK(PRE_ATT_OUT);
    WRK_TRY(matmul(ops, L.att_w_o, V(B["att_x"]), V(B["att_o"]), WRK_ACT_NONE, turbo));
    HOOK(POST_ATT_OUT);
    WRK_TRY(add(ops, V(B["att_o"]), V(B["x"])));
    HOOK(POST_ATT);

    WRK_TRY(blit(ops, V(B["x"]), V(B["ffn_x"])));
    HOOK(PRE_FFN);
    ADD(wrk_op_layer_norm(L.ffn_ln.w, L.ffn_ln.b, B["ffn_x"], LN_EPS, &_o));
    HOOK(POST_FFN_LAYER_NORM);
    HOOK(PRE_FFN_TOKEN_SHIFT);
    WRK_TRY(token_shift(ops, cursors, V(L.ffn_time_mix_k), sf, B["ffn_x"], B["ffn_kx"], false));
    WRK_TRY(token_shift(ops, cursors, V(L.ffn_time_mix_r), sf, B["ffn_x"], B["ffn_rx"], false));
    HOOK(POST_FFN_TOKEN_SHIFT);
    HOOK(PRE_FFN_LINEAR);
    WRK_TRY(matmul(ops, L.ffn_w_k, V(B["ffn_kx"]), V(B["ffn_k"]), WRK_ACT_SQUARED_RELU, turbo));
    HOOK(POST_FFN_ACTIVATE);
    WRK_TRY(matmul(ops, L.ffn_w_v, V(B["ffn_k"]), V(B["ffn_v"]), WRK_ACT_NONE, turbo, true));
    WRK_TRY(matmul(ops, L.ffn_w_r, V(B["ffn_rx"]), V(B["ffn_r"]), WRK_ACT_NONE, turbo));
    HOOK(POST_FFN_LINEAR);
    HOOK(PRE_FFN_CHANNEL_MIX);
    ADD(wrk_op_channel_mix(cursors, &sf, B["ffn_r"], B["ffn_v"], B["ffn_x"], &_o));
    HOOK(POST_FFN_CHANNEL_MIX);
    WRK_TRY(add(ops, V(B["ffn_x"]), V(B["x"])));
    HOOK(POST_FFN);
    if ((index + 1) % bd->model->rescale == 0) ADD(wrk_op_affine(B["x"], 0.5f, 0.0f, &_o));
    return WRK_OK;
}

// ---- a rank of a split model (no counterpart in the reference, which runs on one GPU) ----
// The layer functions below serve both: with the whole model on this GPU the local channel range is all of C and
// they emit the reference's op list; on a rank of a split model the time-mix ops between the token shifts and
// `output` run on the rank's channels, `output` and ffn `value` multiply the rank's slice of K into an f32 partial
// sum over all C channels, and one all-reduce per sub-block turns it into the sum the residual needs.
struct Split {
    bool on;
    uint32_t c0, Cl;
};
Split split_of(const wrk_bundle* bd) {
    const Shard& sh = bd->model->shard;
    return {sh.on(), sh.on() ? sh.c0 : 0u, sh.on() ? sh.c1 - sh.c0 : bd->model->info.num_emb};
}
// The state rows a time-mix op touches (the shift row and the S rows of the recurrence), for the rank's channels.
wrk_view state_wkv(wrk_bundle* bd, uint32_t layer, uint32_t S, const Split& sp) {
    wrk_view v = state_att(bd, layer, S);
    if (sp.on) {
        v.shape[0] = sp.Cl;
        v.offset[0] = sp.c0;
    }
    return v;
}
// Where `output` (which = 0) / ffn `value` (which = 1) write this rank's share of their product over all C channels.
wrk_tensor* partial_of(const Buffers& B, uint32_t which) {
    if (B.t.count("partial")) return B["partial"];
    return B[which == 0 ? "partial0" : "partial1"];
}
// Sum over the ranks, round to fp16 once: NCCL all-reduce in place + a copy, or the one-shot reduce over peer memory,
// whose two slots the two reduces of a layer use in turn.
int32_t reduce_partial(wrk_bundle* bd, OpList& ops, const Buffers& B, wrk_tensor* out, uint32_t which) {
    if (B.t.count("partial")) {
        ADD(wrk_op_all_reduce(bd->comm, B["partial"], &_o));
        return blit(ops, V(B["partial"]), V(out));
    }
    ADD(wrk_op_peer_all_reduce(bd->comm, which, out->len(), out, &_o));
    return WRK_OK;
}
// The time-mix op has written the shift row (the normalised input of every sequence's last token) for the rank's
// channels only; the next job's token shifts read all of them.
int32_t carry_all_channels(wrk_bundle* bd, OpList& ops, const Buffers& B, uint32_t index, uint32_t S) {
    (void)S;
    const wrk_view row0 = Vy(bd->state[index], 0, 1);
    ADD(wrk_op_shift_carry(B["cursors"], &row0, B["att_x"], &_o));
    return WRK_OK;
}

// dispatch_layer of v5 (v5.rs:656-885) and v6 (v6.rs:701-958)
int32_t layer_v56(wrk_bundle* bd, OpList& ops, const Buffers& B, uint32_t index, uint32_t T) {
    const wrk_model_info& info = bd->model->info;
    const Layer& L = bd->model->layers[index];
    const uint32_t C = info.num_emb, S = C / info.num_head;
    const bool turbo = T % WRK_MIN_TOKEN_CHUNK_SIZE == 0;
    const bool v6 = info.version == 6;
    wrk_tensor* cursors = B["cursors"];
    const Split sp = split_of(bd);
    wrk_tensor* att_loc = sp.on ? B["att_xl"] : B["att_x"];  // the gated WKV output, `output`'s input

    TensorH time_first, time_decay, aux_x, att_k, att_v, att_r;
    WRK_TRY(reshape(L.time_first, S, WRK_DIM_AUTO, 1, 1, &time_first));
    if (v6) WRK_TRY(reshape(B["time_decay"], S, WRK_DIM_AUTO, T, 1, &time_decay));
    else WRK_TRY(reshape(L.time_decay, S, WRK_DIM_AUTO, 1, 1, &time_decay));
    WRK_TRY(reshape(B["aux_x"], S, WRK_DIM_AUTO, T, 1, &aux_x));
    WRK_TRY(reshape(B["att_k"], S, WRK_DIM_AUTO, T, 1, &att_k));
    WRK_TRY(reshape(B["att_v"], S, WRK_DIM_AUTO, T, 1, &att_v));
    WRK_TRY(reshape(B["att_r"], S, WRK_DIM_AUTO, T, 1, &att_r));

    // Runs of elementwise ops as one launch each (bit-identical results) unless the op list is to be the reference's,
    // op for op: with hooks, which sit between those ops, or in strict mode.
    const bool merged = bd->fused && bd->hooks.empty();
    const bool merged8 = merged && C % 8 == 0 && (!sp.on || sp.Cl % 8 == 0);  // ops that take eight channels per thread
    if (merged) {
        ADD(wrk_op_layer_norm_copy(L.att_ln.w, L.att_ln.b, nullptr, B["x"], B["att_x"], LN_EPS, &_o));
    } else {
        WRK_TRY(blit(ops, V(B["x"]), V(B["att_x"])));
        HOOK(PRE_ATT);
        ADD(wrk_op_layer_norm(L.att_ln.w, L.att_ln.b, B["att_x"], LN_EPS, &_o));
    }
    HOOK(POST_ATT_LAYER_NORM);
    HOOK(PRE_ATT_TOKEN_SHIFT);
    if (v6) {
        TensorH time_mix_x;
        WRK_TRY(reshape(B["time_mix_x"], WRK_DIM_AUTO, T, 1, 1, &time_mix_x));
        WRK_TRY(token_shift(ops, cursors, V(L.time_mix_x), state_att(bd, index, S), B["att_x"], B["att_xx"], true));
        HOOK(POST_ATT_TOKEN_SHIFT);
        HOOK(PRE_ATT_TOKEN_SHIFT_ADAPT);
        WRK_TRY(matmul(ops, L.time_mix_w1, V(B["att_xx"]), V(time_mix_x), WRK_ACT_TANH, turbo));
        {
            const wrk_view in = V(B["time_mix_x"]), out = V(B["time_mix_t"]);
            ADD(wrk_op_transpose(&in, &out, &_o));
        }
        HOOK(POST_ATT_TOKEN_SHIFT_ADAPT_ACTIVATE);
        WRK_TRY(matmul(ops, L.time_mix_w2, V(B["time_mix_t"]), V(B["time_mix"]), WRK_ACT_NONE, turbo));
        HOOK(POST_ATT_TOKEN_SHIFT_ADAPT);
        if (merged8) {
            const wrk_view tm = V(B["time_mix"]), bias = V(L.time_mix), st = state_att(bd, index, S);
            ADD(wrk_op_token_shift_lora(cursors, &tm, &bias, &st, B["att_x"], B["att_sx"], true, &_o));
        } else {
            WRK_TRY(add(ops, V(L.time_mix), V(B["time_mix"])));
            HOOK(PRE_ATT_GATED_TOKEN_SHIFT);
            WRK_TRY(token_shift(ops, cursors, V(B["time_mix"]), state_att(bd, index, S), B["att_x"], B["att_sx"], true));
        }
        HOOK(POST_ATT_GATED_TOKEN_SHIFT);
        HOOK(PRE_ATT_LINEAR);
        if (merged) {  // the four matrices as the row tiles of one launch
            WRK_TRY(matmul_group(ops, {{L.att_w_k, Vz(B["att_sx"], 1), V(B["att_k"]), WRK_ACT_NONE},
                                       {L.att_w_v, Vz(B["att_sx"], 2), V(B["att_v"]), WRK_ACT_NONE},
                                       {L.att_w_r, Vz(B["att_sx"], 3), V(B["att_r"]), WRK_ACT_NONE},
                                       {L.att_w_g, Vz(B["att_sx"], 4), V(B["att_g"]), WRK_ACT_NONE}}, turbo));
        } else {
            WRK_TRY(matmul(ops, L.att_w_k, Vz(B["att_sx"], 1), V(B["att_k"]), WRK_ACT_NONE, turbo));
            WRK_TRY(matmul(ops, L.att_w_v, Vz(B["att_sx"], 2), V(B["att_v"]), WRK_ACT_NONE, turbo));
            WRK_TRY(matmul(ops, L.att_w_r, Vz(B["att_sx"], 3), V(B["att_r"]), WRK_ACT_NONE, turbo));
            WRK_TRY(matmul(ops, L.att_w_g, Vz(B["att_sx"], 4), V(B["att_g"]), WRK_ACT_NONE, turbo));
        }
        HOOK(POST_ATT_LINEAR);
        HOOK(PRE_ATT_TIME_DECAY_ADAPT);
        WRK_TRY(matmul(ops, L.time_decay_w1, Vz(B["att_sx"], 0), V(B["att_w"]), WRK_ACT_TANH, turbo));
        HOOK(POST_ATT_TIME_DECAY_ADAPT_ACTIVATE);
        WRK_TRY(matmul(ops, L.time_decay_w2, V(B["att_w"]), V(B["time_decay"]), WRK_ACT_NONE, turbo));
        HOOK(POST_ATT_TIME_DECAY_ADAPT);
        if (merged) {  // the sum stays f32 between the two ops: one op with the activation on its output is the same
            WRK_TRY(add(ops, V(L.time_decay), V(B["time_decay"]), WRK_ACT_STABLE_EXP));
        } else {
            WRK_TRY(add(ops, V(L.time_decay), V(B["time_decay"])));
            HOOK(PRE_ATT_TIME_DECAY_ACTIVATE);
            const wrk_view td = V(B["time_decay"]);
            ADD(wrk_op_activate(&td, WRK_ACT_STABLE_EXP, &_o));
        }
        HOOK(POST_ATT_TIME_DECAY_ACTIVATE);
    } else if (merged) {
        const wrk_view sa = state_att(bd, index, S);
        wrk_tensor* const mixes[4] = {L.time_mix_k, L.time_mix_v, L.time_mix_r, L.time_mix_g};
        wrk_tensor* const outs[4] = {B["att_kx"], B["att_vx"], B["att_rx"], B["att_gx"]};
        ADD(wrk_op_token_shift_multi(cursors, &sa, B["att_x"], 4, mixes, outs, false, &_o));
        WRK_TRY(matmul_group(ops, {{L.att_w_k, V(B["att_kx"]), V(B["att_k"]), WRK_ACT_NONE},
                                   {L.att_w_v, V(B["att_vx"]), V(B["att_v"]), WRK_ACT_NONE},
                                   {L.att_w_r, V(B["att_rx"]), V(B["att_r"]), WRK_ACT_NONE},
                                   {L.att_w_g, V(B["att_gx"]), V(B["att_g"]), WRK_ACT_NONE}}, turbo));
    } else {
        WRK_TRY(token_shift(ops, cursors, V(L.time_mix_k), state_att(bd, index, S), B["att_x"], B["att_kx"], false));
        WRK_TRY(token_shift(ops, cursors, V(L.time_mix_v), state_att(bd, index, S), B["att_x"], B["att_vx"], false));
        WRK_TRY(token_shift(ops, cursors, V(L.time_mix_r), state_att(bd, index, S), B["att_x"], B["att_rx"], false));
        WRK_TRY(token_shift(ops, cursors, V(L.time_mix_g), state_att(bd, index, S), B["att_x"], B["att_gx"], false));
        HOOK(POST_ATT_TOKEN_SHIFT);
        HOOK(PRE_ATT_LINEAR);
        WRK_TRY(matmul(ops, L.att_w_k, V(B["att_kx"]), V(B["att_k"]), WRK_ACT_NONE, turbo));
        WRK_TRY(matmul(ops, L.att_w_v, V(B["att_vx"]), V(B["att_v"]), WRK_ACT_NONE, turbo));
        WRK_TRY(matmul(ops, L.att_w_r, V(B["att_rx"]), V(B["att_r"]), WRK_ACT_NONE, turbo));
        WRK_TRY(matmul(ops, L.att_w_g, V(B["att_gx"]), V(B["att_g"]), WRK_ACT_NONE, turbo));
        HOOK(POST_ATT_LINEAR);
    }
    HOOK(PRE_ATT_TIME_MIX);
    WRK_TRY(blit(ops, Vx(B["att_x"], sp.c0, sp.c0 + sp.Cl), V(B["aux_x"])));
    {
        const wrk_view st = state_wkv(bd, index, S, sp);
        // blocks of 16 tokens where there are tokens to block; the serial kernel for short jobs and in strict mode
        if (merged && S == 64 && T > 8) ADD(wrk_op_time_mix_blocks(v6, cursors, time_decay, time_first, &st, att_k, att_v, att_r, aux_x, &_o));
        else if (v6) ADD(wrk_op_time_mix_v6(cursors, time_decay, time_first, &st, att_k, att_v, att_r, aux_x, &_o));
        else ADD(wrk_op_time_mix_v5(cursors, time_decay, time_first, &st, att_k, att_v, att_r, aux_x, &_o));
    }
    if (merged8 && S % 8 == 0 && S <= 256 && (S & (S - 1)) == 0) {
        ADD(wrk_op_group_norm_gate(L.gn.w, L.gn.b, aux_x, B["att_g"], att_loc, GN_EPS, WRK_ACT_SILU, &_o));
    } else {
        ADD(wrk_op_group_norm(L.gn.w, L.gn.b, aux_x, GN_EPS, &_o));
        WRK_TRY(blit(ops, V(B["aux_x"]), V(att_loc)));
        HOOK(POST_ATT_TIME_MIX);
        HOOK(PRE_ATT_GATE);
        const wrk_view g = V(B["att_g"]), x = V(att_loc);
        ADD(wrk_op_mul_activate(&g, &x, WRK_ACT_SILU, WRK_ACT_NONE, WRK_ACT_NONE, &_o));
    }
    HOOK(POST_ATT_GATE);
    HOOK(PRE_ATT_OUT);
    WRK_TRY(matmul(ops, L.att_w_o, V(att_loc), V(sp.on ? partial_of(B, 0) : B["att_o"]), WRK_ACT_NONE, turbo));
    if (sp.on) {
        WRK_TRY(reduce_partial(bd, ops, B, B["att_o"], 0));
        WRK_TRY(carry_all_channels(bd, ops, B, index, S));
    }
    HOOK(POST_ATT_OUT);
    if (merged) {
        ADD(wrk_op_layer_norm_copy(L.ffn_ln.w, L.ffn_ln.b, B["att_o"], B["x"], B["ffn_x"], LN_EPS, &_o));
        const wrk_view sf = state_ffn(bd, index, S);
        wrk_tensor* const mixes[2] = {L.ffn_time_mix_k, L.ffn_time_mix_r};
        wrk_tensor* const outs[2] = {B["ffn_kx"], B["ffn_rx"]};
        ADD(wrk_op_token_shift_multi(cursors, &sf, B["ffn_x"], 2, mixes, outs, v6, &_o));
    } else {
        WRK_TRY(add(ops, V(B["att_o"]), V(B["x"])));
        HOOK(POST_ATT);
        WRK_TRY(blit(ops, V(B["x"]), V(B["ffn_x"])));
        HOOK(PRE_FFN);
        ADD(wrk_op_layer_norm(L.ffn_ln.w, L.ffn_ln.b, B["ffn_x"], LN_EPS, &_o));
        HOOK(POST_FFN_LAYER_NORM);
        HOOK(PRE_FFN_TOKEN_SHIFT);
        WRK_TRY(token_shift(ops, cursors, V(L.ffn_time_mix_k), state_ffn(bd, index, S), B["ffn_x"], B["ffn_kx"], v6));
        WRK_TRY(token_shift(ops, cursors, V(L.ffn_time_mix_r), state_ffn(bd, index, S), B["ffn_x"], B["ffn_rx"], v6));
    }
    HOOK(POST_FFN_TOKEN_SHIFT);
    HOOK(PRE_FFN_LINEAR);
    if (merged) {  // key and receptance read different shifts of one input: one launch; value follows
        WRK_TRY(matmul_group(ops, {{L.ffn_w_k, V(B["ffn_kx"]), V(B["ffn_k"]), WRK_ACT_SQUARED_RELU},
                                   {L.ffn_w_r, V(B["ffn_rx"]), V(B["ffn_r"]), WRK_ACT_NONE}}, turbo));
    } else {
        WRK_TRY(matmul(ops, L.ffn_w_k, V(B["ffn_kx"]), V(B["ffn_k"]), WRK_ACT_SQUARED_RELU, turbo));
        HOOK(POST_FFN_ACTIVATE);
    }
    WRK_TRY(matmul(ops, L.ffn_w_v, V(B["ffn_k"]), V(sp.on ? partial_of(B, 1) : B["ffn_v"]), WRK_ACT_NONE, turbo, true));
    if (sp.on) WRK_TRY(reduce_partial(bd, ops, B, B["ffn_v"], 1));
    if (!merged) WRK_TRY(matmul(ops, L.ffn_w_r, V(B["ffn_rx"]), V(B["ffn_r"]), WRK_ACT_NONE, turbo));
    HOOK(POST_FFN_LINEAR);
    HOOK(PRE_FFN_CHANNEL_MIX);
    {
        const wrk_view st = state_ffn(bd, index, S);
        if (merged8) {
            ADD(wrk_op_channel_mix_add(cursors, &st, B["ffn_r"], B["ffn_v"], B["ffn_x"], B["x"], 0, &_o));
        } else {
            ADD(wrk_op_channel_mix(cursors, &st, B["ffn_r"], B["ffn_v"], B["ffn_x"], &_o));
            HOOK(POST_FFN_CHANNEL_MIX);
            WRK_TRY(add(ops, V(B["ffn_x"]), V(B["x"])));
        }
    }
    HOOK(POST_FFN);
    if ((index + 1) % bd->model->rescale == 0) ADD(wrk_op_affine(B["x"], 0.5f, 0.0f, &_o));
    return WRK_OK;
}

// dispatch_layer of v7 (v7.rs:716-1007)
int32_t layer_v7(wrk_bundle* bd, OpList& ops, const Buffers& B, uint32_t index, uint32_t T) {
    const wrk_model_info& info = bd->model->info;
    const Layer& L = bd->model->layers[index];
    const uint32_t C = info.num_emb, S = C / info.num_head;
    const bool turbo = T % WRK_MIN_TOKEN_CHUNK_SIZE == 0;
    wrk_tensor* cursors = B["cursors"];
    const Split sp = split_of(bd);
    wrk_tensor* att_loc = sp.on ? B["att_xl"] : B["att_x"];  // the time-mix op's input (shift source) and output

    TensorH att_kk, att_x, att_r, att_w, att_n;
    WRK_TRY(reshape(B["att_kk"], S, WRK_DIM_AUTO, T, 1, &att_kk));
    WRK_TRY(reshape(att_loc, S, WRK_DIM_AUTO, T, 1, &att_x));
    WRK_TRY(reshape(B["att_r"], S, WRK_DIM_AUTO, T, 1, &att_r));
    WRK_TRY(reshape(B["att_w"], S, WRK_DIM_AUTO, T, 1, &att_w));
    WRK_TRY(reshape(B["att_n"], S, WRK_DIM_AUTO, T, 4, &att_n));

    // Runs of elementwise ops as one launch each (bit-identical results) unless the op list is to be the reference's,
    // op for op: with hooks, which sit between those ops, or in strict mode.
    const bool merged = bd->fused && bd->hooks.empty();
    const wrk_view sa = state_att(bd, index, S);
    if (merged) {
        ADD(wrk_op_layer_norm_copy(L.att_ln.w, L.att_ln.b, nullptr, B["x"], B["att_x"], LN_EPS, &_o));
        wrk_tensor* const mixes[6] = {L.x_r, L.x_w, L.x_k, L.x_v, L.x_a, L.x_g};
        wrk_tensor* const outs[6] = {B["att_rx"], B["att_wx"], B["att_kx"], B["att_vx"], B["att_ax"], B["att_gx"]};
        ADD(wrk_op_token_shift_multi(cursors, &sa, B["att_x"], 6, mixes, outs, true, &_o));
    } else {
        WRK_TRY(blit(ops, V(B["x"]), V(B["att_x"])));
        HOOK(PRE_ATT);
        ADD(wrk_op_layer_norm(L.att_ln.w, L.att_ln.b, B["att_x"], LN_EPS, &_o));
        HOOK(POST_ATT_LAYER_NORM);
        HOOK(PRE_ATT_TOKEN_SHIFT);
        WRK_TRY(token_shift(ops, cursors, V(L.x_r), sa, B["att_x"], B["att_rx"], true));
        WRK_TRY(token_shift(ops, cursors, V(L.x_w), sa, B["att_x"], B["att_wx"], true));
        WRK_TRY(token_shift(ops, cursors, V(L.x_k), sa, B["att_x"], B["att_kx"], true));
        WRK_TRY(token_shift(ops, cursors, V(L.x_v), sa, B["att_x"], B["att_vx"], true));
        WRK_TRY(token_shift(ops, cursors, V(L.x_a), sa, B["att_x"], B["att_ax"], true));
        WRK_TRY(token_shift(ops, cursors, V(L.x_g), sa, B["att_x"], B["att_gx"], true));
    }
    HOOK(POST_ATT_TOKEN_SHIFT);
    HOOK(PRE_ATT_LINEAR);
    if (merged) {
        WRK_TRY(matmul_group(ops, {{L.att_w_r, V(B["att_rx"]), V(B["att_r"]), WRK_ACT_NONE},
                                   {L.att_w_k, V(B["att_kx"]), V(B["att_k"]), WRK_ACT_NONE},
                                   {L.att_w_v, V(B["att_vx"]), V(B["att_v"]), WRK_ACT_NONE}}, turbo));
    } else {
        WRK_TRY(matmul(ops, L.att_w_r, V(B["att_rx"]), V(B["att_r"]), WRK_ACT_NONE, turbo));
        WRK_TRY(matmul(ops, L.att_w_k, V(B["att_kx"]), V(B["att_k"]), WRK_ACT_NONE, turbo));
        WRK_TRY(matmul(ops, L.att_w_v, V(B["att_vx"]), V(B["att_v"]), WRK_ACT_NONE, turbo));
    }
    HOOK(POST_ATT_LINEAR);
    HOOK(PRE_ATT_ADAPT);
    WRK_TRY(matmul(ops, L.w1, V(B["att_wx"]), V(B["aux_w"]), WRK_ACT_TANH, turbo));
    WRK_TRY(matmul(ops, L.w2, V(B["aux_w"]), V(B["att_w"]), WRK_ACT_NONE, turbo));
    WRK_TRY(add(ops, V(L.w0), V(B["att_w"])));
    WRK_TRY(matmul(ops, L.a1, V(B["att_ax"]), V(B["aux_a"]), WRK_ACT_NONE, turbo));
    WRK_TRY(matmul(ops, L.a2, V(B["aux_a"]), V(B["att_a"]), WRK_ACT_NONE, turbo));
    WRK_TRY(add(ops, V(L.a0), V(B["att_a"]), WRK_ACT_SIGMOID));
    WRK_TRY(matmul(ops, L.g1, V(B["att_gx"]), V(B["aux_g"]), WRK_ACT_SIGMOID, turbo));
    WRK_TRY(matmul(ops, L.g2, V(B["aux_g"]), V(B["att_g"]), WRK_ACT_NONE, turbo));
    HOOK(POST_ATT_ADAPT);
    HOOK(PRE_ATT_CONTROL);
    if (!merged) {
        WRK_TRY(blit(ops, V(B["att_k"]), V(B["att_kk"])));
        {
            const wrk_view kk = V(L.k_k), o = V(B["att_kk"]);
            ADD(wrk_op_mul_activate(&kk, &o, WRK_ACT_NONE, WRK_ACT_NONE, WRK_ACT_NONE, &_o));
        }
        ADD(wrk_op_l2_norm(att_kk, L2_EPS, &_o));
        {
            const wrk_view a = V(B["att_a"]), k = V(B["att_k"]);
            ADD(wrk_op_control_k_v7(L.k_a, &a, &k, &_o));
        }
    }
    HOOK(POST_ATT_CONTROL);
    HOOK(PRE_ATT_VALUE_RESIDUAL);
    if (index == 0) {
        WRK_TRY(blit(ops, V(B["att_v"]), V(B["att_v0"])));
    } else {
        WRK_TRY(matmul(ops, L.v1, V(B["att_vx"]), V(B["aux_v"]), WRK_ACT_NONE, turbo));
        WRK_TRY(matmul(ops, L.v2, V(B["aux_v"]), V(B["att_vv"]), WRK_ACT_NONE, turbo));
        WRK_TRY(add(ops, V(L.v0), V(B["att_vv"]), WRK_ACT_SIGMOID));
        const wrk_view in = V(B["att_v0"]), out = V(B["att_v"]), f = V(B["att_vv"]);
        ADD(wrk_op_lerp(&in, &out, &f, 1, &_o));
    }
    HOOK(POST_ATT_VALUE_RESIDUAL);
    HOOK(PRE_ATT_TIME_MIX);
    if (merged) {  // kk, the controlled k and the four planes of the time-mix operand (k and kk do not depend on v)
        TensorH k3, v3, a3;
        WRK_TRY(reshape(B["att_k"], S, WRK_DIM_AUTO, T, 1, &k3));
        WRK_TRY(reshape(B["att_v"], S, WRK_DIM_AUTO, T, 1, &v3));
        WRK_TRY(reshape(B["att_a"], S, WRK_DIM_AUTO, T, 1, &a3));
        ADD(wrk_op_pack_v7(L.k_k, L.k_a, k3, v3, a3, att_kk, att_n, L2_EPS, &_o));
    } else {
        WRK_TRY(blit(ops, V(B["att_k"]), Vz(B["att_n"], 0)));
        WRK_TRY(blit(ops, V(B["att_v"]), Vz(B["att_n"], 1)));
        WRK_TRY(blit(ops, V(B["att_a"]), Vz(B["att_n"], 2)));
        WRK_TRY(blit(ops, V(B["att_kk"]), Vz(B["att_n"], 3)));
    }
    if (sp.on) WRK_TRY(blit(ops, Vx(B["att_x"], sp.c0, sp.c0 + sp.Cl), V(att_loc)));
    {
        const wrk_view st = state_wkv(bd, index, S, sp);
        ADD(wrk_op_time_mix_v7(cursors, &st, att_r, att_w, att_n, att_x, &_o));
    }
    ADD(wrk_op_group_norm(L.gn.w, L.gn.b, att_x, GN_EPS, &_o));
    ADD(wrk_op_time_first_v7(L.r_k, att_r, att_n, att_x, &_o));
    HOOK(POST_ATT_TIME_MIX);
    HOOK(PRE_ATT_GATE);
    {
        const wrk_view g = V(B["att_g"]), x = V(att_loc);
        ADD(wrk_op_mul_activate(&g, &x, WRK_ACT_NONE, WRK_ACT_NONE, WRK_ACT_NONE, &_o));
    }
    HOOK(POST_ATT_GATE);
    HOOK(PRE_ATT_OUT);
    WRK_TRY(matmul(ops, L.att_w_o, V(att_loc), V(sp.on ? partial_of(B, 0) : B["att_o"]), WRK_ACT_NONE, turbo));
    if (sp.on) {
        WRK_TRY(reduce_partial(bd, ops, B, B["att_o"], 0));
        WRK_TRY(carry_all_channels(bd, ops, B, index, S));
    }
    HOOK(POST_ATT_OUT);
    if (merged) {
        ADD(wrk_op_layer_norm_copy(L.ffn_ln.w, L.ffn_ln.b, B["att_o"], B["x"], B["ffn_x"], LN_EPS, &_o));
    } else {
        WRK_TRY(add(ops, V(B["att_o"]), V(B["x"])));
        HOOK(POST_ATT);
        WRK_TRY(blit(ops, V(B["x"]), V(B["ffn_x"])));
        HOOK(PRE_FFN);
        ADD(wrk_op_layer_norm(L.ffn_ln.w, L.ffn_ln.b, B["ffn_x"], LN_EPS, &_o));
    }
    HOOK(POST_FFN_LAYER_NORM);
    HOOK(PRE_FFN_TOKEN_SHIFT);
    WRK_TRY(token_shift(ops, cursors, V(L.ffn_x_k), state_ffn(bd, index, S), B["ffn_x"], B["ffn_kx"], true));
    HOOK(POST_FFN_TOKEN_SHIFT);
    HOOK(PRE_FFN_LINEAR);
    WRK_TRY(matmul(ops, L.ffn_w_k, V(B["ffn_kx"]), V(B["ffn_k"]), WRK_ACT_SQUARED_RELU, turbo));
    HOOK(POST_FFN_ACTIVATE);
    WRK_TRY(matmul(ops, L.ffn_w_v, V(B["ffn_k"]), V(sp.on ? partial_of(B, 1) : B["ffn_v"]), WRK_ACT_NONE, turbo, true));
    if (sp.on) WRK_TRY(reduce_partial(bd, ops, B, B["ffn_v"], 1));
    HOOK(POST_FFN_LINEAR);
    HOOK(PRE_FFN_CHANNEL_MIX);
    {
        const wrk_view st = state_ffn(bd, index, S);
        if (merged && C % 8 == 0) {
            ADD(wrk_op_channel_mix_add(cursors, &st, nullptr, B["ffn_v"], B["ffn_x"], B["x"], 1, &_o));
        } else {
            ADD(wrk_op_channel_mix_v7(cursors, &st, B["ffn_v"], B["ffn_x"], &_o));
            HOOK(POST_FFN_CHANNEL_MIX);
            WRK_TRY(add(ops, V(B["ffn_x"]), V(B["x"])));
        }
    }
    HOOK(POST_FFN);
    if ((index + 1) % bd->model->rescale == 0) ADD(wrk_op_affine(B["x"], 0.5f, 0.0f, &_o));
    return WRK_OK;
}


// ---------------------------------------------------------------------------------------------
// Fused v6 job for a few tokens (decode): seven weight-streaming launches per layer, chained with
// programmatic dependent launch.  Same arithmetic and fp16 rounding points as the op-by-op list.
// ---------------------------------------------------------------------------------------------

struct MatInfo {
    int kind;
    const uint8_t* w;
    const __half* scale;
    const float* table;
    uint32_t K, M;
};

MatInfo mat_info(wrk_matrix* m) {
    MatInfo r{};
    r.kind = m->kind == 0 ? k::MAT_FP16 : m->kind == 1 ? k::MAT_INT8 : k::MAT_NF4;
    r.w = static_cast<const uint8_t*>(m->w->ptr());
    r.scale = m->m ? static_cast<const __half*>(m->m->ptr()) : nullptr;
    r.table = m->q ? static_cast<const float*>(m->q->ptr()) : nullptr;
    r.K = m->kind == 2 ? m->w->shape[0] * 2 : m->w->shape[0];
    r.M = m->w->shape[1];
    return r;
}

bool mat_fusable(const MatInfo& m) {
    const uint32_t need = m.kind == k::MAT_FP16 ? 32 : 128;
    return m.K % need == 0 && m.K % 8 == 0;
}

k::GemvProblem problem(const MatInfo& m, const __half* x, int x_sel, void* out, int out_dtype, int act) {
    k::GemvProblem p{};
    p.w = m.w;
    p.scale = m.scale;
    p.kind = m.kind;
    p.K = m.K;
    p.M = m.M;
    p.x = x;
    p.x_sel = x_sel;
    p.x_stride = m.K;
    p.out = out;
    p.out_stride = m.M;
    p.out_dtype = out_dtype;
    p.act = act;
    return p;
}

// Row partition of a fused launch, uploaded once when the job is built.
int32_t make_partition(wrk_context* ctx, k::FusedGemvArgs& a, int grid, CachedJob* job) {
    std::vector<k::GemvSegment> table;
    WRK_REQUIRE(k::fused_gemv_partition(a, grid, table), WRK_ERR_UNSUPPORTED,
                "row partition overflow: too many small matrices per CTA");
    const uint32_t shape[4] = {(uint32_t)(table.size() * 4), 1, 1, 1};
    wrk_tensor* t = nullptr;
    WRK_TRY(wrk_tensor_from_data(ctx, WRK_U32, shape, table.data(), table.size() * sizeof(k::GemvSegment), &t));
    job->tables.emplace_back(t);
    a.segments = static_cast<const k::GemvSegment*>(t->ptr());
    k::fused_gemv_inline_partition(a, grid, table);
    return WRK_OK;
}

int32_t add_fused_gemv(wrk_context* ctx, OpList& ops, CachedJob* job, k::FusedGemvArgs a, const char* name,
                       std::initializer_list<const wrk_tensor*> keep) {
    const int grid = ctx->num_sms;
    a.status = ctx->device_status;
    for (int i = 0; i < a.num_problems; ++i)
        if (a.p[i].kind == k::MAT_NF4 && a.table == nullptr)
            return set_error(WRK_ERR_INVALID_ARGUMENT, "NF4 problem without a code book");
    WRK_TRY(make_partition(ctx, a, grid, job));
    ops.ops.push_back(new_atom(name, [a, grid](cudaStream_t s) { return k::fused_gemv(a, grid, s); }, keep));
    return WRK_OK;
}

const __half* H(wrk_tensor* t) { return static_cast<const __half*>(t->ptr()); }
__half* Hm(wrk_tensor* t) { return static_cast<__half*>(t->ptr()); }

bool fused_v6_supported(wrk_bundle* bd, uint32_t T) {
    const wrk_model_info& info = bd->model->info;
    if (!bd->fused || info.version != 6 || T == 0 || T > (uint32_t)k::kDecodeMaxTokens) return false;
    if (!bd->hooks.empty()) return false;     // hooks sit between reference ops
    if (bd->model->shard.on()) return false;  // the fused phases end in residual adds; a split model sums across ranks first
    if (info.num_emb / info.num_head != 64 || info.num_emb % 128 || info.custom[0] % 8 || info.custom[0] > 64 ||
        info.custom[1] % 32 || info.custom[1] > 128)
        return false;
    for (auto& L : bd->model->layers)
        for (wrk_matrix* m : {L.att_w_k.p, L.att_w_v.p, L.att_w_r.p, L.att_w_g.p, L.att_w_o.p, L.ffn_w_k.p, L.ffn_w_v.p,
                              L.ffn_w_r.p, L.time_mix_w1.p, L.time_decay_w1.p})
            if (!mat_fusable(mat_info(m))) return false;
    if (!mat_fusable(mat_info(bd->model->head_w))) return false;
    const uint32_t kmax = std::max(info.num_emb, info.num_hidden);
    return k::fused_gemv_smem(T, kmax, info.num_emb, k::PRO_NONE, 2) <= 200 * 1024 &&
           k::fused_gemv_smem(T, info.num_emb, info.num_emb, k::PRO_LN_SHIFT2, 2) <= 200 * 1024 && info.num_emb <= 8192;
}

// The phases of a job that runs as one persistent kernel (kernels/decode_step.cu), collected while the
// fused layers are emitted.
struct StepRange {
    const uint8_t* w;
    const __half* scale;
    int32_t r0, r1;
    uint32_t K, M;
    int16_t kind, problem;
};
struct StepBuilder {
    std::vector<k::StepPhase> phases;
    std::vector<std::vector<StepRange>> work;  // [gemv phase][cta]
    uint32_t kmax = 0, kmax_int8 = 0, kmax_fp16 = 0;
    bool any_prologue = false, has_nf4 = false, umma_shapes = true;
    const float* table = nullptr;
};

// Where the fused layers go: a list of launches (one per phase, chained with programmatic dependent launch) or
// the phase list of the step kernel.
struct FusedSink {
    wrk_context* ctx;
    OpList* ops;
    CachedJob* job;
    StepBuilder* step;  // null: one launch per phase
};

int32_t emit_gemv(FusedSink& sink, k::FusedGemvArgs a, const char* name, std::initializer_list<const wrk_tensor*> keep) {
    if (sink.step == nullptr) return add_fused_gemv(sink.ctx, *sink.ops, sink.job, a, name, keep);
    StepBuilder& sb = *sink.step;
    const int grid = sink.ctx->num_sms;
    a.status = sink.ctx->device_status;
    uint32_t kmax = 0;
    for (int i = 0; i < a.num_problems; ++i) {
        kmax = std::max(kmax, a.p[i].K);
        if (a.p[i].kind == k::MAT_NF4 && a.table == nullptr)
            return set_error(WRK_ERR_INVALID_ARGUMENT, "NF4 problem without a code book");
    }
    a.kmax = kmax;
    sb.kmax = std::max(sb.kmax, kmax);
    if (a.table) sb.table = a.table;
    if (a.prologue != k::PRO_NONE) sb.any_prologue = true;
    k::StepPhase ph{};
    ph.type = k::PH_GEMV;
    ph.gemv_index = -1;
    if (a.num_problems > 0) {
        std::vector<k::GemvSegment> table;
        WRK_REQUIRE(k::fused_gemv_partition(a, grid, table), WRK_ERR_UNSUPPORTED,
                    "row partition overflow: too many small matrices per CTA");
        std::vector<StepRange> work(grid);
        for (int c = 0; c < grid; ++c) {
            StepRange wk{};
            int used = 0;
            for (int i = 0; i < k::kSegmentsPerCta; ++i) {
                const k::GemvSegment& sg = table[(size_t)c * k::kSegmentsPerCta + i];
                if (sg.row1 <= sg.row0) continue;
                const k::GemvProblem& p = a.p[sg.problem];
                wk.w = p.w;
                wk.scale = p.scale;
                wk.r0 = sg.row0;
                wk.r1 = sg.row1;
                wk.K = p.K;
                wk.M = p.M;
                wk.kind = (int16_t)p.kind;
                wk.problem = (int16_t)sg.problem;
                ++used;
            }
            WRK_REQUIRE(used <= 1, WRK_ERR_UNSUPPORTED, "a CTA of the step kernel takes one row range per phase");
            work[c] = wk;
        }
        for (int i = 0; i < a.num_problems; ++i) {
            const k::GemvProblem& p = a.p[i];
            if (p.kind == k::MAT_NF4) sb.has_nf4 = true;
            if (p.kind == k::MAT_INT8) sb.kmax_int8 = std::max(sb.kmax_int8, p.K);
            if (p.kind == k::MAT_FP16) sb.kmax_fp16 = std::max(sb.kmax_fp16, p.K);
            // tensor-core path: whole 128-byte blocks per row (fp16: four per stage of a packed tile), 16-byte
            // aligned rows and inputs
            const uint32_t unit = p.kind == k::MAT_INT8 ? 128 : 256;
            if (p.K % unit != 0 || reinterpret_cast<uintptr_t>(p.w) % 16 != 0 || (p.x != nullptr && (p.x_stride % 8 != 0 || reinterpret_cast<uintptr_t>(p.x) % 16 != 0)))
                sb.umma_shapes = false;
        }
        ph.gemv_index = (int32_t)sb.work.size();
        sb.work.push_back(std::move(work));
    }
    ph.gemv = static_cast<const k::GemvCore&>(a);
    sb.phases.push_back(ph);
    return WRK_OK;
}

int32_t layer_v6_fused(wrk_bundle* bd, FusedSink& sink, const Buffers& B, uint32_t index, uint32_t T) {
    const wrk_model_info& info = bd->model->info;
    OpList& ops = *sink.ops;
    const Layer& L = bd->model->layers[index];
    const uint32_t C = info.num_emb, S = 64, F = info.num_hidden;
    const uint32_t* cursors = static_cast<const uint32_t*>(B["cursors"]->ptr());
    const int wide = bd->packed_cursors ? 0 : 1;
    const DView st_att = make_dview(state_att(bd, index, S)), st_ffn = make_dview(state_ffn(bd, index, S));
    const float* table = nullptr;
    for (wrk_matrix* m : {L.att_w_k.p, L.att_w_o.p, L.ffn_w_k.p})
        if (m->q) table = static_cast<const float*>(m->q->ptr());

    // A: layer norm + shift(time_mix_x) -> adapter W1 (tanh)
    {
        k::FusedGemvArgs a{};
        a.T = T;
        a.C = C;
        a.prologue = k::PRO_LN_SHIFT1;
        a.ln_x = H(B["x"]);
        a.ln_w = H(L.att_ln.w);
        a.ln_b = H(L.att_ln.b);
        a.ln_eps = LN_EPS;
        a.cursors = cursors;
        a.wide = wide;
        a.state = st_att;
        a.mix0 = H(L.time_mix_x);
        a.reversed = 1;
        a.ln_out = Hm(B["att_x"]);
        a.num_problems = 1;
        a.p[0] = problem(mat_info(L.time_mix_w1), nullptr, 0, B["time_mix_x"]->ptr(), WRK_F16, WRK_ACT_TANH);
        a.epilogue = k::EPI_STORE;
        a.rescale = 1.0f;
        WRK_TRY(emit_gemv(sink, a, "fused_ln_shift_adapter", {B["x"], B["att_x"], B["time_mix_x"], L.time_mix_w1.p->w}));
    }
    // B: adapter W2 + static mixes + five-way token shift
    {
        k::TmixArgs a{};
        a.w2 = H(L.time_mix_w2.p->w);
        a.tmx = H(B["time_mix_x"]);
        a.mix = H(L.time_mix);
        a.att_x = H(B["att_x"]);
        a.cursors = cursors;
        a.wide = wide;
        a.state = st_att;
        a.sx = Hm(B["att_sx"]);
        a.C = C;
        a.D = info.custom[0];
        a.T = T;
        if (sink.step) {
            k::StepPhase ph{};
            ph.type = k::PH_TMIX;
            ph.gemv_index = -1;
            ph.tmix = a;
            sink.step->phases.push_back(ph);
        } else {
            ops.ops.push_back(new_atom("fused_tmix_shift", [a](cudaStream_t s) { return k::tmix_shift_v6(a, s); },
                                       {B["time_mix_x"], B["att_x"], B["att_sx"], L.time_mix_w2.p->w, L.time_mix.p}));
        }
    }
    // C: key / value / receptance / gate + decay adapter W1 in one launch
    {
        const __half* sx = H(B["att_sx"]);
        const size_t plane = (size_t)T * C;
        k::FusedGemvArgs a{};
        a.T = T;
        a.C = C;
        a.prologue = k::PRO_NONE;
        a.table = table;
        a.num_problems = 5;
        a.p[0] = problem(mat_info(L.att_w_k), sx + 1 * plane, 0, B["att_k"]->ptr(), WRK_F32, WRK_ACT_NONE);
        a.p[1] = problem(mat_info(L.att_w_v), sx + 2 * plane, 0, B["att_v"]->ptr(), WRK_F32, WRK_ACT_NONE);
        a.p[2] = problem(mat_info(L.att_w_r), sx + 3 * plane, 0, B["att_r"]->ptr(), WRK_F32, WRK_ACT_NONE);
        a.p[3] = problem(mat_info(L.att_w_g), sx + 4 * plane, 0, B["att_g"]->ptr(), WRK_F16, WRK_ACT_NONE);
        a.p[4] = problem(mat_info(L.time_decay_w1), sx, 0, B["att_w"]->ptr(), WRK_F16, WRK_ACT_TANH);
        a.epilogue = k::EPI_STORE;
        a.rescale = 1.0f;
        WRK_TRY(emit_gemv(sink, a, "fused_att_linear",
                               {B["att_sx"], B["att_k"], B["att_v"], B["att_r"], B["att_g"], B["att_w"]}));
    }
    // D: decay adapter W2 + WKV + group norm + gate
    {
        k::Wkv6Args a{};
        a.cursors = cursors;
        a.wide = wide;
        a.state = st_att;
        a.H = info.num_head;
        a.T = T;
        a.B = bd->num_batch;
        a.per_token_decay = 1;
        a.tdw = H(B["att_w"]);
        a.td_w2 = H(L.time_decay_w2.p->w);
        a.td0 = H(L.time_decay);
        a.D = info.custom[1];
        a.time_first = static_cast<const float*>(L.time_first.p->ptr());
        a.k = static_cast<const float*>(B["att_k"]->ptr());
        a.v = static_cast<const float*>(B["att_v"]->ptr());
        a.r = static_cast<const float*>(B["att_r"]->ptr());
        a.g = H(B["att_g"]);
        a.att_x = H(B["att_x"]);
        a.gn_w = H(L.gn.w);
        a.gn_b = H(L.gn.b);
        a.gn_eps = GN_EPS;
        a.out = Hm(B["att_xx"]);
        if (sink.step) {
            k::StepPhase ph{};
            ph.type = k::PH_WKV;
            ph.gemv_index = -1;
            ph.wkv = a;
            sink.step->phases.push_back(ph);
        } else {
            ops.ops.push_back(new_atom("fused_wkv6", [a](cudaStream_t s) { return k::wkv56_fused(a, s); },
                                       {B["att_w"], B["att_k"], B["att_v"], B["att_r"], B["att_g"], B["att_x"], B["att_xx"],
                                        bd->state[index].p}));
        }
    }
    // E: output projection + residual
    {
        k::FusedGemvArgs a{};
        a.T = T;
        a.C = C;
        a.prologue = k::PRO_NONE;
        a.table = table;
        a.num_problems = 1;
        a.p[0] = problem(mat_info(L.att_w_o), H(B["att_xx"]), 0, nullptr, WRK_F16, WRK_ACT_NONE);
        a.epilogue = k::EPI_RESIDUAL;
        a.xres = Hm(B["x"]);
        a.rescale = 1.0f;
        WRK_TRY(emit_gemv(sink, a, "fused_att_out", {B["att_xx"], B["x"]}));
    }
    // F: layer norm + two shifts -> ffn key (squared ReLU) and receptance
    {
        k::FusedGemvArgs a{};
        a.T = T;
        a.C = C;
        a.prologue = k::PRO_LN_SHIFT2;
        a.table = table;
        a.ln_x = H(B["x"]);
        a.ln_w = H(L.ffn_ln.w);
        a.ln_b = H(L.ffn_ln.b);
        a.ln_eps = LN_EPS;
        a.cursors = cursors;
        a.wide = wide;
        a.state = st_ffn;
        a.mix0 = H(L.ffn_time_mix_k);
        a.mix1 = H(L.ffn_time_mix_r);
        a.reversed = 1;
        a.ln_out = Hm(B["ffn_x"]);
        a.num_problems = 2;
        a.p[0] = problem(mat_info(L.ffn_w_k), nullptr, 0, B["ffn_k"]->ptr(), WRK_F16, WRK_ACT_SQUARED_RELU);
        a.p[1] = problem(mat_info(L.ffn_w_r), nullptr, 1, B["ffn_r"]->ptr(), WRK_F16, WRK_ACT_NONE);
        a.epilogue = k::EPI_STORE;
        a.rescale = 1.0f;
        WRK_TRY(emit_gemv(sink, a, "fused_ffn_in", {B["x"], B["ffn_x"], B["ffn_k"], B["ffn_r"]}));
    }
    // G: ffn value + channel mix + residual (+ rescale)
    {
        k::FusedGemvArgs a{};
        a.T = T;
        a.C = C;
        a.prologue = k::PRO_NONE;
        a.table = table;
        a.cursors = cursors;
        a.wide = wide;
        a.num_problems = 1;
        a.p[0] = problem(mat_info(L.ffn_w_v), H(B["ffn_k"]), 0, nullptr, WRK_F16, WRK_ACT_NONE);
        a.epilogue = k::EPI_CHANNEL_MIX;
        a.xres = Hm(B["x"]);
        a.cm_r = H(B["ffn_r"]);
        a.cm_x = H(B["ffn_x"]);
        a.cm_state = st_ffn;
        a.rescale = (index + 1) % bd->model->rescale == 0 ? 0.5f : 1.0f;
        WRK_TRY(emit_gemv(sink, a, "fused_ffn_out", {B["ffn_k"], B["ffn_r"], B["ffn_x"], B["x"], bd->state[index].p}));
    }
    (void)F;
    return WRK_OK;
}

// The job as one persistent kernel: embedding layer norm, the fused layers and (when rows need logits) the head.
// Returns WRK_ERR_UNSUPPORTED when the job shape does not fit the kernel (the caller then builds launches).
int32_t build_step_job(wrk_bundle* bd, CachedJob* job, OpList& ops) {
    wrk_model* m = bd->model;
    wrk_context* ctx = m->ctx;
    const uint32_t T = job->num_token, NH = job->num_header, C = m->info.num_emb;
    const Buffers& B = *job->buffer;
    const Buffers& Hd = *job->header;
    const int grid = ctx->num_sms;
    WRK_REQUIRE((5 * C + grid - 1) / grid <= 512, WRK_ERR_UNSUPPORTED, "token-shift phase wider than a CTA");
    StepBuilder sb;
    OpList unused;
    FusedSink sink{ctx, &unused, job, &sb};
    // embed: layer norm of the uploaded rows into x (a phase without matrices; CTA 0 writes the rows)
    {
        k::FusedGemvArgs a{};
        a.T = T;
        a.C = C;
        a.prologue = k::PRO_LN;
        a.ln_x = H(B["input"]);
        a.ln_w = H(m->embed_ln.w);
        a.ln_b = H(m->embed_ln.b);
        a.ln_eps = LN_EPS;
        a.ln_out = Hm(B["x"]);
        a.num_problems = 0;
        a.epilogue = k::EPI_STORE;
        a.rescale = 1.0f;
        WRK_TRY(emit_gemv(sink, a, "step_embed", {}));
    }
    for (uint32_t i = 0; i < m->info.num_layer; ++i) WRK_TRY(layer_v6_fused(bd, sink, B, i, T));
    if (NH > 0) {
        k::FusedGemvArgs a{};
        a.T = NH;
        a.C = C;
        a.prologue = k::PRO_LN;
        a.ln_x = H(B["x"]);
        // RnnRedirect::op (rnn.rs:102-133): head row h normalises row headers[h] of x
        for (uint32_t h = 0; h < NH; ++h) a.ln_row_off[h] = (int32_t)job->redirect.headers[h] - (int32_t)h;
        a.ln_w = H(m->head_ln.w);
        a.ln_b = H(m->head_ln.b);
        a.ln_eps = LN_EPS;
        a.num_problems = 1;
        a.p[0] = problem(mat_info(m->head_w), nullptr, 0, Hd["head_o"]->ptr(), WRK_F32, WRK_ACT_NONE);
        a.epilogue = k::EPI_STORE;
        a.rescale = 1.0f;
        WRK_TRY(emit_gemv(sink, a, "step_head", {}));
    }
    auto upload = [&](const void* data, size_t bytes, wrk_tensor** out) -> int32_t {
        const uint32_t shape[4] = {(uint32_t)((bytes + 3) / 4), 1, 1, 1};
        WRK_TRY(wrk_tensor_from_data(ctx, WRK_U32, shape, data, bytes, out));
        job->tables.emplace_back(*out);
        return WRK_OK;
    };
    wrk_tensor *t_phases = nullptr, *t_work = nullptr, *t_bar = nullptr;
    WRK_TRY(upload(sb.phases.data(), sb.phases.size() * sizeof(k::StepPhase), &t_phases));
    const uint32_t zero[4] = {0, 0, 0, 0};
    WRK_TRY(upload(zero, sizeof zero, &t_bar));
    unsigned long long* timeline = nullptr;
    if (bd->timeline_phases >= sb.phases.size() && bd->timeline.p != nullptr)
        timeline = static_cast<unsigned long long*>(bd->timeline.p->ptr());
    job->num_phases = (uint32_t)sb.phases.size();
    const size_t ng = sb.work.size();

    // Int8 / fp16 matrices and at most two tokens: the tensor-core kernel (TMA boxes + tcgen05)
    if (bd->step_engine != 3 && !sb.has_nf4 && sb.umma_shapes && T <= 2) {
        k::UmmaStepArgs u{};
        u.num_phases = (int32_t)sb.phases.size();
        u.num_gemv = (int32_t)ng;
        u.T = T;
        u.C = C;
        u.status = ctx->device_status;
        // the activation operand of a phase sits in front of the prologue's rows (T normalised, up to 2 T shifted,
        // one of bias; pitch C + 8), which only phases with a prologue use
        const uint32_t x_bytes = sb.any_prologue ? (uint32_t)(((size_t)(3 * T + 1) * (C + 8) * 2 + 127) / 128 * 128) : 0;
        uint32_t operand = 0;
        for (const auto& ph : sb.phases) {
            if (ph.type != k::PH_GEMV || ph.gemv_index < 0) continue;
            const uint32_t tail = ph.gemv.prologue != k::PRO_NONE ? x_bytes : 0;
            for (int c = 0; c < grid; ++c) {
                const StepRange& r = sb.work[ph.gemv_index][c];
                operand = std::max(operand, k::umma_operand_bytes(r.r1 - r.r0, r.kind, r.K, ph.gemv.T) + tail);
            }
        }
        operand = std::max(operand, x_bytes);
        if (k::decode_step_umma_prepare(u, operand, x_bytes, sb.kmax_int8) != 0) {
            // phases whose prologue the kernel runs in registers (one token, a row of at most 4096 values): ranges of
            // one or two rows of an fp16 matrix are multiplied there as well and never staged
            std::vector<bool> direct_phase(ng, false);
            for (const auto& ph : sb.phases)
                if (ph.type == k::PH_GEMV && ph.gemv_index >= 0 && ph.gemv.prologue != k::PRO_NONE && ph.gemv.T == 1 && C % 128 == 0 && C <= 4096)
                    direct_phase[ph.gemv_index] = true;
            std::vector<k::UmmaWork> flat((size_t)grid * ng);
            for (size_t g = 0; g < ng; ++g)
                for (int c = 0; c < grid; ++c) {
                    const StepRange& r = sb.work[g][c];
                    k::UmmaWork& wk = flat[(size_t)c * ng + g];
                    std::memset(&wk, 0, sizeof wk);
                    wk.direct = direct_phase[g] && r.kind == k::MAT_FP16 && r.K == C && r.r1 - r.r0 >= 1 && r.r1 - r.r0 <= 2 ? 1 : 0;
                    wk.w = r.w;
                    wk.scale = r.scale;
                    wk.r0 = r.r0;
                    wk.r1 = r.r1;
                    wk.K = r.K;
                    wk.kind = r.kind;
                    wk.problem = r.problem;
                }
            WRK_TRY(upload(flat.data(), std::max<size_t>(flat.size(), 1) * sizeof(k::UmmaWork), &t_work));
            u.phases = static_cast<const k::StepPhase*>(t_phases->ptr());
            u.work = static_cast<const k::UmmaWork*>(t_work->ptr());
            u.barrier = static_cast<uint32_t*>(t_bar->ptr());
            u.timeline = timeline;
            ops.ops.push_back(new_atom("decode_step_umma", [u, grid](cudaStream_t st) { return k::decode_step_umma(u, grid, st); },
                                       {B["input"], B["x"], t_phases, t_work, t_bar}));
            return WRK_OK;
        }
    }

    k::StepArgs s{};
    s.num_phases = (int32_t)sb.phases.size();
    s.num_gemv = (int32_t)ng;
    s.T = T;
    s.kmax = std::max(sb.kmax, C);
    s.C = C;
    s.table = sb.table;
    s.status = ctx->device_status;
    WRK_REQUIRE(k::decode_step_prepare(s, sb.any_prologue) != 0, WRK_ERR_UNSUPPORTED,
                "job of %u tokens does not fit the step kernel's shared memory", T);
    // work lists ([cta][phase]) live as long as the job
    std::vector<k::StepWork> flat((size_t)grid * ng);
    for (size_t g = 0; g < ng; ++g)
        for (int c = 0; c < grid; ++c) {
            const StepRange& r = sb.work[g][c];
            k::StepWork& wk = flat[(size_t)c * ng + g];
            wk.w = r.w;
            wk.scale = r.scale;
            wk.r0 = r.r0;
            wk.r1 = r.r1;
            wk.K = r.K;
            wk.kind = r.kind;
            wk.problem = r.problem;
        }
    WRK_TRY(upload(flat.data(), std::max<size_t>(flat.size(), 1) * sizeof(k::StepWork), &t_work));
    s.phases = static_cast<const k::StepPhase*>(t_phases->ptr());
    s.work = static_cast<const k::StepWork*>(t_work->ptr());
    s.barrier = static_cast<uint32_t*>(t_bar->ptr());
    s.timeline = timeline;
    ops.ops.push_back(new_atom("decode_step", [s, grid](cudaStream_t st) { return k::decode_step(s, grid, st); },
                               {B["input"], B["x"], t_phases, t_work, t_bar}));
    return WRK_OK;
}

// Bundle::dispatch body (v6.rs:586-697) for a job with at least one token.
int32_t build_job(wrk_bundle* bd, const RnnInfo& info, CachedJob* job) {
    wrk_model* m = bd->model;
    const uint32_t T = job->num_token, NH = job->num_header;
    const Buffers& B = *job->buffer;
    const Buffers& Hd = *job->header;
    OpList ops;
    const bool fused = fused_v6_supported(bd, T);
    bd->building_header = &Hd;
    bd->building_tokens = T;
    bd->building_headers = NH;
    const uint32_t index = 0;  // the embed / head hooks take no layer
    // the whole job as one persistent kernel (launched eagerly: a memset of the barrier word and one cooperative
    // launch per job need no graph)
    if (fused && bd->step_kernel && NH <= (uint32_t)k::kDecodeMaxTokens) {
        const int32_t st = build_step_job(bd, job, ops);
        if (st == WRK_OK) {
            wrk_op* list = nullptr;
            WRK_TRY(wrk_op_list(ops.ops.data(), ops.ops.size(), &list));
            const int32_t s = wrk_encode(m->ctx, list, 0, &job->commands);
            wrk_op_release(list);
            return s;
        }
        if (st != WRK_ERR_UNSUPPORTED) return st;
        job->tables.clear();
        job->num_phases = 0;
    }

    // embed: layer norm on the uploaded rows, then copy into x
    HOOK(POST_EMBED_LOADED);
    ADD(wrk_op_layer_norm(m->embed_ln.w, m->embed_ln.b, B["input"], LN_EPS, &_o));
    WRK_TRY(blit(ops, V(B["input"]), V(B["x"])));
    HOOK(POST_EMBED_LAYER_NORM);
    FusedSink sink{m->ctx, &ops, job, nullptr};
    for (uint32_t i = 0; i < m->info.num_layer; ++i) {
        if (fused) WRK_TRY(layer_v6_fused(bd, sink, B, i, T));
        else if (m->info.version == 7) WRK_TRY(layer_v7(bd, ops, B, i, T));
        else if (m->info.version == 4) WRK_TRY(layer_v4(bd, ops, B, i, T));
        else WRK_TRY(layer_v56(bd, ops, B, i, T));
        if ((i + 1) % m->sep == 0) ADD(wrk_op_sep(&_o));
    }
    // RnnRedirect::op (rnn.rs:102-133): gather the rows that need logits into head_x
    wrk_tensor* head_x = nullptr;
    if (T == 1 || T == NH) {
        head_x = B["x"];
    } else {
        head_x = Hd["head_x"];
        const auto& h = job->redirect.headers;
        size_t start = 0, end = 1;
        while (end <= h.size()) {
            if (end == h.size() || h[end - 1] + 1 != h[end]) {
                const uint32_t first = h[start], last = h[end - 1];
                WRK_TRY(blit(ops, Vy(B["x"], first, last + 1), Vy(Hd["head_x"], (uint32_t)start, (uint32_t)end)));
                start = end;
            }
            ++end;
        }
    }
    if (NH > 0 && fused && NH <= (uint32_t)k::kDecodeMaxTokens) {
        // layer norm as the prologue of the (fp16) head's weight-streaming launch
        k::FusedGemvArgs a{};
        a.T = NH;
        a.C = m->info.num_emb;
        a.prologue = k::PRO_LN;
        a.ln_x = H(head_x);
        a.ln_w = H(m->head_ln.w);
        a.ln_b = H(m->head_ln.b);
        a.ln_eps = LN_EPS;
        a.num_problems = 1;
        a.p[0] = problem(mat_info(m->head_w), nullptr, 0, Hd["head_o"]->ptr(), WRK_F32, WRK_ACT_NONE);
        a.epilogue = k::EPI_STORE;
        a.rescale = 1.0f;
        WRK_TRY(add_fused_gemv(m->ctx, ops, job, a, "fused_head", {head_x, Hd["head_o"]}));
    } else if (NH > 0 && m->shard.on()) {
        // every rank multiplies its slice of the vocabulary; the slices are gathered and put in order
        HOOK(PRE_HEAD);
        ADD(wrk_op_layer_norm(m->head_ln.w, m->head_ln.b, head_x, LN_EPS, &_o));
        HOOK(POST_HEAD_LAYER_NORM);
        WRK_TRY(matmul(ops, m->head_w, V(head_x), V(Hd["head_l"]), WRK_ACT_NONE, NH % WRK_MIN_TOKEN_CHUNK_SIZE == 0));
        ADD(wrk_op_all_gather(bd->comm, Hd["head_l"], Hd["head_all"], &_o));
        const uint32_t Vl = m->shard.v1 - m->shard.v0;
        for (uint32_t r = 0; r < m->shard.world; ++r) WRK_TRY(blit(ops, Vz(Hd["head_all"], r), Vx(Hd["head_o"], r * Vl, (r + 1) * Vl)));
        HOOK(POST_HEAD);
    } else if (NH > 0) {
        HOOK(PRE_HEAD);
        ADD(wrk_op_layer_norm(m->head_ln.w, m->head_ln.b, head_x, LN_EPS, &_o));
        HOOK(POST_HEAD_LAYER_NORM);
        WRK_TRY(matmul(ops, m->head_w, V(head_x), V(Hd["head_o"]), WRK_ACT_NONE, NH % WRK_MIN_TOKEN_CHUNK_SIZE == 0));
        HOOK(POST_HEAD);
    }
    wrk_op* list = nullptr;
    WRK_TRY(wrk_op_list(ops.ops.data(), ops.ops.size(), &list));
    int32_t s = wrk_encode(m->ctx, list, bd->use_graph ? 1 : 0, &job->commands);
    wrk_op_release(list);
    return s;
}

int32_t ensure_staging(wrk_bundle* bd, size_t tokens) {
    if (tokens <= bd->stage_tokens) return WRK_OK;
    wrk_context* ctx = bd->model->ctx;
    WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    if (bd->stage_input) cudaFreeHost(bd->stage_input);
    if (bd->stage_cursors) cudaFreeHost(bd->stage_cursors);
    bd->stage_input = nullptr;
    bd->stage_cursors = nullptr;
    size_t cap = 64;
    while (cap < tokens) cap *= 2;
    WRK_CUDA(cudaMallocHost(&bd->stage_input, cap * bd->model->info.num_emb * 2));
    WRK_CUDA(cudaMallocHost(&bd->stage_cursors, cap * 3 * sizeof(uint32_t)));
    bd->stage_tokens = cap;
    return WRK_OK;
}

}  // namespace

extern "C" {

static int32_t bundle_create(wrk_model* model, uint32_t num_batch, wrk_comm* comm, wrk_bundle** out);
static void drop_caches(wrk_bundle* b);

int32_t wrk_bundle_create(wrk_model* model, uint32_t num_batch, wrk_bundle** out) {
    WRK_REQUIRE(model && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(!model->shard.on(), WRK_ERR_INVALID_ARGUMENT, "rank %u of a model split %u ways needs wrk_bundle_create_sharded", model->shard.rank,
                model->shard.world);
    return bundle_create(model, num_batch, nullptr, out);
}

int32_t wrk_bundle_create_sharded(wrk_model* model, uint32_t num_batch, wrk_comm* comm, wrk_bundle** out) {
    WRK_REQUIRE(model && comm && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    int32_t rank = 0, world = 1;
    WRK_TRY(wrk_comm_rank(comm, &rank, &world));
    WRK_REQUIRE((uint32_t)world == model->shard.world && (uint32_t)rank == model->shard.rank, WRK_ERR_INVALID_ARGUMENT,
                "the model is rank %u of %u, the communicator rank %d of %d", model->shard.rank, model->shard.world, rank, world);
    if (world == 1) return bundle_create(model, num_batch, nullptr, out);
    WRK_TRY(bundle_create(model, num_batch, comm, out));
    // slots for jobs of up to 256 tokens; larger jobs, or a node without peer access, use NCCL
    const size_t slot = ((size_t)model->info.num_emb * 256 * 4 + 255) / 256 * 256;
    (*out)->peer_reduce = wrk_comm_enable_peer_reduce(comm, slot) == WRK_OK;
    return WRK_OK;
}

int32_t wrk_bundle_set_peer_reduce(wrk_bundle* b, int32_t on) {
    WRK_REQUIRE(b, WRK_ERR_INVALID_ARGUMENT, "null argument");
    if (on) {
        size_t bytes = 0;
        WRK_REQUIRE(b->comm, WRK_ERR_INVALID_ARGUMENT, "the bundle is not a rank of a split model");
        WRK_TRY(wrk_comm_peer_slot_bytes(b->comm, &bytes));
        WRK_REQUIRE(bytes != 0, WRK_ERR_UNSUPPORTED, "the communicator has no exchange region (peer access unavailable)");
    }
    drop_caches(b);
    b->peer_reduce = on != 0;
    return WRK_OK;
}

int32_t wrk_bundle_peer_reduce(const wrk_bundle* b, int32_t* on) {
    WRK_REQUIRE(b && on, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *on = b->peer_reduce ? 1 : 0;
    return WRK_OK;
}

static int32_t bundle_create(wrk_model* model, uint32_t num_batch, wrk_comm* comm, wrk_bundle** out) {
    WRK_REQUIRE(num_batch >= 1, WRK_ERR_INVALID_ARGUMENT, "num_batch must be at least 1");
    auto b = new wrk_bundle();
    if (comm) {
        wrk_comm_retain(comm);
        b->comm = comm;
    }
    wrk_model_retain(model);
    b->model = model;
    b->num_batch = num_batch;
    const wrk_model_info& info = model->info;
    const uint32_t shape[4] = {info.num_emb, state_rows(info), num_batch, 1};
    // v4: State::init puts f32::MIN in the running-maximum row (v4.rs:163-180)
    std::vector<float> init;
    if (info.version == 4) {
        init.assign((size_t)shape[0] * shape[1] * num_batch, 0.0f);
        for (uint32_t batch = 0; batch < num_batch; ++batch)
            std::fill_n(init.begin() + ((size_t)batch * 5 + 3) * info.num_emb, info.num_emb, std::numeric_limits<float>::lowest());
    }
    for (uint32_t l = 0; l < info.num_layer; ++l) {
        wrk_tensor* t = nullptr;
        int32_t s = wrk_tensor_zeros(model->ctx, WRK_F32, shape, &t);
        if (s == WRK_OK && !init.empty()) s = wrk_tensor_load(t, init.data(), init.size() * sizeof(float));
        if (s != WRK_OK) {
            if (t) wrk_tensor_release(t);
            delete b;
            return s;
        }
        b->state.emplace_back(t);
    }
    *out = b;
    return WRK_OK;
}

int32_t wrk_bundle_release(wrk_bundle* b) {
    if (!b) return WRK_OK;
    if (b->refs.fetch_sub(1) == 1) {
        cudaStreamSynchronize(b->model->ctx->stream);
        delete b;
    }
    return WRK_OK;
}

static void drop_caches(wrk_bundle* b) {
    cudaStreamSynchronize(b->model->ctx->stream);
    b->jobs.clear();
    b->buffers.clear();
    b->headers.clear();
}

int32_t wrk_bundle_set_packed_cursors(wrk_bundle* b, int32_t packed) {
    WRK_REQUIRE(b, WRK_ERR_INVALID_ARGUMENT, "null argument");
    if (b->packed_cursors != (packed != 0)) drop_caches(b);
    b->packed_cursors = packed != 0;
    return WRK_OK;
}

int32_t wrk_bundle_set_use_graph(wrk_bundle* b, int32_t use_graph) {
    WRK_REQUIRE(b, WRK_ERR_INVALID_ARGUMENT, "null argument");
    if (b->use_graph != (use_graph != 0)) drop_caches(b);
    b->use_graph = use_graph != 0;
    return WRK_OK;
}

int32_t wrk_bundle_set_fused(wrk_bundle* b, int32_t fused) {
    WRK_REQUIRE(b, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(fused >= 0 && fused <= 3, WRK_ERR_INVALID_ARGUMENT, "fused mode %d: 0, 1, 2 or 3", fused);
    drop_caches(b);
    b->fused = fused != 0;
    b->step_kernel = fused == 1 || fused == 3;
    b->step_engine = fused == 3 ? 3 : 1;
    return WRK_OK;
}

int32_t wrk_bundle_set_hook(wrk_bundle* b, int32_t hook, uint32_t layer, wrk_hook_fn fn, void* user) {
    WRK_REQUIRE(b, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(hook >= 0 && hook < WRK_HOOK_COUNT, WRK_ERR_INVALID_ARGUMENT, "unknown hook %d", hook);
    const bool global = hook <= WRK_HOOK_POST_EMBED_LAYER_NORM || hook >= WRK_HOOK_PRE_HEAD;
    WRK_REQUIRE(global || layer < b->model->info.num_layer, WRK_ERR_INVALID_ARGUMENT, "layer %u out of range", layer);
    drop_caches(b);
    const std::pair<int32_t, uint32_t> key{hook, global ? 0u : layer};
    if (fn) b->hooks[key] = {fn, user};
    else b->hooks.erase(key);
    return WRK_OK;
}

int32_t wrk_frame_bundle(const wrk_frame* frame, wrk_bundle** bundle) {
    WRK_REQUIRE(frame && bundle, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *bundle = frame->bundle;
    return WRK_OK;
}

int32_t wrk_frame_num_token(const wrk_frame* frame, uint32_t* num_token, uint32_t* num_header) {
    WRK_REQUIRE(frame && num_token && num_header, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *num_token = frame->num_token;
    *num_header = frame->num_header;
    return WRK_OK;
}

int32_t wrk_frame_buffer(const wrk_frame* frame, const char* name, wrk_tensor** out) {
    WRK_REQUIRE(frame && name && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    for (const Buffers* b : {frame->buffer, frame->header}) {
        if (!b) continue;
        auto it = b->t.find(name);
        if (it != b->t.end()) {
            *out = it->second;
            return WRK_OK;
        }
    }
    return set_error(WRK_ERR_INVALID_ARGUMENT, "the job has no buffer named %s", name);
}

int32_t wrk_bundle_set_phase_timeline(wrk_bundle* b, uint32_t max_phases) {
    WRK_REQUIRE(b, WRK_ERR_INVALID_ARGUMENT, "null argument");
    drop_caches(b);
    b->timeline = TensorH();
    b->timeline_phases = 0;
    if (max_phases == 0) return WRK_OK;
    wrk_context* ctx = b->model->ctx;
    const uint32_t shape[4] = {2u * (uint32_t)ctx->num_sms * 2u, max_phases, 1, 1};  // u64 as pairs of u32
    wrk_tensor* t = nullptr;
    WRK_TRY(wrk_tensor_zeros(ctx, WRK_U32, shape, &t));
    b->timeline = TensorH(t);
    b->timeline_phases = max_phases;
    return WRK_OK;
}

int32_t wrk_job_phase_timeline(wrk_job* job, uint64_t* stamps, size_t capacity, uint32_t* num_phases, uint32_t* num_ctas) {
    WRK_REQUIRE(job && num_phases && num_ctas, WRK_ERR_INVALID_ARGUMENT, "null argument");
    wrk_bundle* b = job->bundle;
    wrk_context* ctx = b->model->ctx;
    *num_phases = job->job->num_phases;
    *num_ctas = (uint32_t)ctx->num_sms;
    WRK_REQUIRE(b->timeline.p != nullptr && job->job->num_phases > 0 && job->job->num_phases <= b->timeline_phases,
                WRK_ERR_EMPTY, "list must not be empty: the job records no phase timeline");
    const size_t need = (size_t)2 * job->job->num_phases * ctx->num_sms;
    WRK_REQUIRE(stamps && capacity >= need, WRK_ERR_SIZE, "data size not match: %zu vs. %zu", capacity, need);
    WRK_CUDA(cudaMemcpyAsync(stamps, b->timeline.p->ptr(), need * sizeof(uint64_t), cudaMemcpyDeviceToHost, ctx->stream));
    WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    return WRK_OK;
}

int32_t wrk_state_num_batch(wrk_bundle* b, uint32_t* num_batch) {
    WRK_REQUIRE(b && num_batch, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *num_batch = b->num_batch;
    return WRK_OK;
}

int32_t wrk_state_init_shape(wrk_bundle* b, uint32_t shape[4]) {
    WRK_REQUIRE(b && shape, WRK_ERR_INVALID_ARGUMENT, "null argument");
    const wrk_model_info& info = b->model->info;
    shape[0] = info.num_emb;
    shape[1] = state_rows(info);
    shape[2] = info.num_layer;
    shape[3] = 1;
    return WRK_OK;
}

// State::load, v6.rs:199-206: host tensor [C, S + 2, L] → slot `batch` of every layer
int32_t wrk_state_load(wrk_bundle* b, const float* host, size_t bytes, uint32_t batch) {
    WRK_REQUIRE(b && host, WRK_ERR_INVALID_ARGUMENT, "null argument");
    const wrk_model_info& info = b->model->info;
    const size_t per_layer = (size_t)info.num_emb * state_rows(info);
    WRK_REQUIRE(bytes == per_layer * info.num_layer * 4, WRK_ERR_SIZE, "data size not match: %zu vs. %zu", bytes,
                per_layer * info.num_layer * 4);
    if (batch >= b->num_batch)
        return set_error(WRK_ERR_BATCH_OUT_OF_RANGE, "batch %u out of range of max %u", batch, b->num_batch);
    wrk_context* ctx = b->model->ctx;
    for (uint32_t l = 0; l < info.num_layer; ++l)
        WRK_CUDA(cudaMemcpyAsync(static_cast<float*>(b->state[l].p->ptr()) + batch * per_layer, host + l * per_layer,
                                 per_layer * 4, cudaMemcpyHostToDevice, ctx->stream));
    WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    return WRK_OK;
}

// State::back, v6.rs:141-159
int32_t wrk_state_back(wrk_bundle* b, uint32_t batch, float* host, size_t bytes) {
    WRK_REQUIRE(b && host, WRK_ERR_INVALID_ARGUMENT, "null argument");
    const wrk_model_info& info = b->model->info;
    const size_t per_layer = (size_t)info.num_emb * state_rows(info);
    WRK_REQUIRE(bytes == per_layer * info.num_layer * 4, WRK_ERR_SIZE, "data size not match: %zu vs. %zu", bytes,
                per_layer * info.num_layer * 4);
    if (batch >= b->num_batch)
        return set_error(WRK_ERR_BATCH_OUT_OF_RANGE, "batch %u out of range of max %u", batch, b->num_batch);
    wrk_context* ctx = b->model->ctx;
    for (uint32_t l = 0; l < info.num_layer; ++l)
        WRK_CUDA(cudaMemcpyAsync(host + l * per_layer, static_cast<float*>(b->state[l].p->ptr()) + batch * per_layer,
                                 per_layer * 4, cudaMemcpyDeviceToHost, ctx->stream));
    WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    return WRK_OK;
}

// State::write, v6.rs:223-239: a device tensor [C, S + 2, L] into one batch slot, stream-ordered (no host wait)
int32_t wrk_state_write(wrk_bundle* b, wrk_tensor* tensor, uint32_t batch) {
    WRK_REQUIRE(b && tensor, WRK_ERR_INVALID_ARGUMENT, "null argument");
    const wrk_model_info& info = b->model->info;
    const uint32_t rows = state_rows(info);
    WRK_REQUIRE(tensor->dtype == WRK_F32, WRK_ERR_TYPE, "data type mismatch: the state is f32");
    WRK_TRY(check_shape("state", tensor->shape, info.num_emb, rows, info.num_layer, 1));
    WRK_REQUIRE(tensor->ctx == b->model->ctx, WRK_ERR_INVALID_ARGUMENT, "tensor and bundle belong to different contexts");
    if (batch >= b->num_batch)
        return set_error(WRK_ERR_BATCH_OUT_OF_RANGE, "batch %u out of range of max %u", batch, b->num_batch);
    const size_t per_layer = (size_t)info.num_emb * rows;
    wrk_context* ctx = b->model->ctx;
    for (uint32_t l = 0; l < info.num_layer; ++l)
        WRK_CUDA(cudaMemcpyAsync(static_cast<float*>(b->state[l].p->ptr()) + batch * per_layer,
                                 static_cast<const float*>(tensor->ptr()) + l * per_layer, per_layer * 4, cudaMemcpyDeviceToDevice,
                                 ctx->stream));
    return WRK_OK;
}

// State::read, v6.rs:241-258: one batch slot as a new device tensor [C, S + 2, L]
int32_t wrk_state_read(wrk_bundle* b, uint32_t batch, wrk_tensor** out) {
    WRK_REQUIRE(b && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    const wrk_model_info& info = b->model->info;
    const uint32_t rows = state_rows(info);
    if (batch >= b->num_batch)
        return set_error(WRK_ERR_BATCH_OUT_OF_RANGE, "batch %u out of range of max %u", batch, b->num_batch);
    const uint32_t shape[4] = {info.num_emb, rows, info.num_layer, 1};
    wrk_tensor* t = nullptr;
    WRK_TRY(wrk_tensor_create(b->model->ctx, WRK_F32, shape, &t));
    const size_t per_layer = (size_t)info.num_emb * rows;
    wrk_context* ctx = b->model->ctx;
    for (uint32_t l = 0; l < info.num_layer; ++l) {
        const cudaError_t e = cudaMemcpyAsync(static_cast<float*>(t->ptr()) + l * per_layer,
                                              static_cast<const float*>(b->state[l].p->ptr()) + batch * per_layer, per_layer * 4,
                                              cudaMemcpyDeviceToDevice, ctx->stream);
        if (e != cudaSuccess) {
            wrk_tensor_release(t);
            return set_error(WRK_ERR_CUDA, "cudaMemcpyAsync failed: %s", cudaGetErrorString(e));
        }
    }
    *out = t;
    return WRK_OK;
}

// State::embed, v6.rs:260-262: row 0 (the time-mix shift row) of one layer of a backed state
int32_t wrk_state_embed(wrk_bundle* b, uint32_t layer, const float* backed, size_t bytes, float* embed, size_t embed_bytes) {
    WRK_REQUIRE(b && backed && embed, WRK_ERR_INVALID_ARGUMENT, "null argument");
    const wrk_model_info& info = b->model->info;
    const size_t per_layer = (size_t)info.num_emb * state_rows(info);
    WRK_REQUIRE(bytes == per_layer * info.num_layer * 4, WRK_ERR_SIZE, "data size not match: %zu vs. %zu", bytes,
                per_layer * info.num_layer * 4);
    WRK_REQUIRE(embed_bytes == (size_t)info.num_emb * 4, WRK_ERR_SIZE, "data size not match: %zu vs. %zu", embed_bytes,
                (size_t)info.num_emb * 4);
    if (layer >= info.num_layer) return set_error(WRK_ERR_SLICE_OUT_OF_RANGE, "layer %u out of range of %u", layer, info.num_layer);
    std::memcpy(embed, backed + layer * per_layer, embed_bytes);
    return WRK_OK;
}

int32_t wrk_state_layer(wrk_bundle* b, uint32_t layer, wrk_tensor** out) {
    WRK_REQUIRE(b && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(layer < b->state.size(), WRK_ERR_INVALID_ARGUMENT, "layer %u out of range", layer);
    *out = b->state[layer];
    return WRK_OK;
}

int32_t wrk_bundle_dispatch(wrk_bundle* b, const uint32_t* lens, const int32_t* options, wrk_job** out) {
    WRK_REQUIRE(b && lens && options && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    std::lock_guard<std::mutex> lock(b->mutex);
    auto job = new wrk_job();
    job->bundle = b;
    job->info.lens.assign(lens, lens + b->num_batch);
    job->info.options.assign(options, options + b->num_batch);
    const uint32_t T = job->info.num_token();
    RnnRedirect rd = redirect(job->info);

    // cache key: the job's structure depends only on num_token and on which rows need logits
    std::vector<uint32_t> key;
    key.push_back(T);
    key.insert(key.end(), rd.headers.begin(), rd.headers.end());
    auto it = b->jobs.find(key);
    std::shared_ptr<CachedJob> cj;
    if (it != b->jobs.end()) {
        cj = it->second;
    } else {
        cj = std::make_shared<CachedJob>();
        cj->num_token = T;
        cj->num_header = (uint32_t)rd.headers.size();
        cj->redirect = rd;
        int32_t s = WRK_OK;
        if (T > 0) {
            auto& rb = b->buffers[T];
            if (!rb) s = make_runtime(b, T, &rb);
            cj->buffer = rb;
            if (s == WRK_OK) {
                auto& hb = b->headers[cj->num_header];
                if (!hb) s = make_header(b, cj->num_header, &hb);
                cj->header = hb;
            }
            if (s == WRK_OK) s = build_job(b, job->info, cj.get());
        }
        if (s != WRK_OK) {
            delete job;
            return s;
        }
        // bounded cache, least recently used first (ResourceCache, src/tensor/cache.rs:21-117)
        if (b->jobs.size() >= 64) {
            auto victim = b->jobs.begin();
            for (auto j = b->jobs.begin(); j != b->jobs.end(); ++j)
                if (j->second->tick < victim->second->tick) victim = j;
            cudaStreamSynchronize(b->model->ctx->stream);
            b->jobs.erase(victim);
        }
        b->jobs[key] = cj;
    }
    cj->tick = ++b->tick;
    job->redirect = std::move(rd);  // per-batch ranges differ between jobs that share a structure
    job->job = cj;
    *out = job;
    return WRK_OK;
}

// cursors: one record per token, identical for all tokens of a sequence (tensor/mod.rs:47-85).
// Jobs of the same shape carry the same cursors, so the upload is skipped when nothing changed.
static int32_t upload_cursors(wrk_job* job) {
    wrk_bundle* b = job->bundle;
    wrk_context* ctx = b->model->ctx;
    const uint32_t T = job->info.num_token();
    CachedJob& cj = *job->job;
    if (cj.buffer->cursor_lens == job->info.lens) return WRK_OK;
    WRK_TRY(ensure_staging(b, T));
    WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    uint32_t p = 0;
    for (uint32_t batch = 0; batch < b->num_batch; ++batch) {
        const uint32_t len = job->info.lens[batch];
        for (uint32_t i = 0; i < len; ++i) {
            if (b->packed_cursors) {
                b->stage_cursors[p + i] = (batch & 0xffu) | ((p & 0xffffu) << 8) | ((len & 0xffu) << 24);
            } else {
                b->stage_cursors[3 * (p + i)] = batch;
                b->stage_cursors[3 * (p + i) + 1] = p;
                b->stage_cursors[3 * (p + i) + 2] = len;
            }
        }
        p += len;
    }
    const Buffers& B = *cj.buffer;
    WRK_CUDA(cudaMemcpyAsync(B["cursors"]->ptr(), b->stage_cursors, (b->packed_cursors ? T : 3 * T) * sizeof(uint32_t),
                             cudaMemcpyHostToDevice, ctx->stream));
    WRK_CUDA(cudaStreamSynchronize(ctx->stream));  // the staging buffer is reused by the next job
    cj.buffer->cursor_lens = job->info.lens;
    return WRK_OK;
}

int32_t wrk_job_load_embed(wrk_job* job, wrk_tensor* embeds, uint32_t row0) {
    WRK_REQUIRE(job && embeds, WRK_ERR_INVALID_ARGUMENT, "null argument");
    wrk_bundle* b = job->bundle;
    const uint32_t T = job->info.num_token();
    if (T == 0) return WRK_OK;
    std::lock_guard<std::mutex> lock(b->mutex);
    wrk_model* m = b->model;
    const uint32_t C = m->info.num_emb;
    WRK_REQUIRE(embeds->dtype == WRK_F16, WRK_ERR_TYPE, "data type mismatch: embeds must be f16");
    WRK_REQUIRE(embeds->shape[0] == C, WRK_ERR_SHAPE, "tensor shape not match (embeds): row length %u vs. %u",
                embeds->shape[0], C);
    if ((size_t)row0 + T > embeds->len() / C)
        return set_error(WRK_ERR_SLICE_OUT_OF_RANGE, "slice %u..%u out of range for dimension size %zu", row0, row0 + T,
                         embeds->len() / C);
    WRK_TRY(upload_cursors(job));
    const Buffers& B = *job->job->buffer;
    WRK_CUDA(cudaMemcpyAsync(B["input"]->ptr(), static_cast<const uint16_t*>(embeds->ptr()) + (size_t)row0 * C,
                             (size_t)T * C * 2, cudaMemcpyDeviceToDevice, m->ctx->stream));
    return WRK_OK;
}

int32_t wrk_job_output(wrk_job* job, wrk_tensor** out) {
    WRK_REQUIRE(job && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(job->job->header, WRK_ERR_EMPTY, "list must not be empty: the job has no output");
    *out = (*job->job->header)["head_o"];
    return WRK_OK;
}

// Job::load, v6.rs:423-459
int32_t wrk_job_load(wrk_job* job, const uint32_t* tokens, size_t count) {
    WRK_REQUIRE(job && (tokens || count == 0), WRK_ERR_INVALID_ARGUMENT, "null argument");
    wrk_bundle* b = job->bundle;
    const uint32_t T = job->info.num_token();
    WRK_REQUIRE(count == T, WRK_ERR_SIZE, "data size not match: %zu vs. %u", count, T);
    if (T == 0) return WRK_OK;
    std::lock_guard<std::mutex> lock(b->mutex);
    wrk_model* m = b->model;
    wrk_context* ctx = m->ctx;
    const uint32_t C = m->info.num_emb;
    WRK_TRY(ensure_staging(b, T));
    WRK_TRY(upload_cursors(job));
    // the previous upload from the staging buffers must have been consumed
    WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    for (uint32_t t = 0; t < T; ++t) {
        const uint32_t tok = tokens[t];
        WRK_REQUIRE(tok < m->num_vocab_padded, WRK_ERR_INVALID_ARGUMENT, "token %u out of vocabulary %u", tok,
                    m->num_vocab_padded);
        std::memcpy(b->stage_input + (size_t)t * C, m->embed_host + (size_t)tok * C, (size_t)C * 2);
    }
    const Buffers& B = *job->job->buffer;
    WRK_CUDA(cudaMemcpyAsync(B["input"]->ptr(), b->stage_input, (size_t)T * C * 2, cudaMemcpyHostToDevice, ctx->stream));
    return WRK_OK;
}

int32_t wrk_job_submit(wrk_job* job) {
    WRK_REQUIRE(job, WRK_ERR_INVALID_ARGUMENT, "null argument");
    if (!job->job->commands) return WRK_OK;
    return wrk_submit(job->bundle->model->ctx, job->job->commands);
}

// Job::back, v6.rs:466-476
int32_t wrk_job_back(wrk_job* job, float* logits, size_t capacity, uint32_t* outputs, uint32_t* num_headers) {
    WRK_REQUIRE(job, WRK_ERR_INVALID_ARGUMENT, "null argument");
    wrk_bundle* b = job->bundle;
    wrk_context* ctx = b->model->ctx;
    const CachedJob& cj = *job->job;
    if (num_headers) *num_headers = cj.num_header;
    if (outputs)
        for (uint32_t i = 0; i < b->num_batch; ++i) {
            outputs[2 * i] = job->redirect.outputs[i].first;
            outputs[2 * i + 1] = job->redirect.outputs[i].second;
        }
    if (cj.num_token == 0 || cj.num_header == 0) {
        WRK_CUDA(cudaStreamSynchronize(ctx->stream));
        return WRK_OK;
    }
    wrk_tensor* head_o = (*cj.header)["head_o"];
    WRK_REQUIRE(logits && capacity >= head_o->len(), WRK_ERR_SIZE, "data size not match: %zu vs. %zu", capacity,
                head_o->len());
    WRK_CUDA(cudaMemcpyAsync(logits, head_o->ptr(), head_o->bytes(), cudaMemcpyDeviceToHost, ctx->stream));
    WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    return WRK_OK;
}

int32_t wrk_job_num_kernels(const wrk_job* job, uint64_t* count) {
    WRK_REQUIRE(job && count, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *count = job->job->commands ? job->job->commands->num_kernels : 0;
    return WRK_OK;
}

int32_t wrk_job_release(wrk_job* job) {
    delete job;
    return WRK_OK;
}

// SimpleRuntime::infer, src/runtime/mod.rs:237-262
int32_t wrk_runtime_infer(wrk_bundle* b, wrk_rnn_input* in, float* logits, size_t capacity, uint32_t* outputs,
                          uint32_t* num_headers) {
    WRK_REQUIRE(b && in, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(in->batches.size() == b->num_batch, WRK_ERR_BATCH, "batch size not match: %zu vs. %u",
                in->batches.size(), b->num_batch);
    RnnIter it = make_iter(*in);
    RnnInfo info = it.next();
    if (info.num_token() == 0) return set_error(WRK_ERR_INPUT_EXHAUSTED, "input iterator exhausted");
    std::vector<uint32_t> chunk;
    for (uint32_t i = 0; i < b->num_batch; ++i)
        chunk.insert(chunk.end(), in->batches[i].tokens.begin(), in->batches[i].tokens.begin() + info.lens[i]);
    wrk_job* job = nullptr;
    WRK_TRY(wrk_bundle_dispatch(b, info.lens.data(), info.options.data(), &job));
    int32_t s = wrk_job_load(job, chunk.data(), chunk.size());
    if (s == WRK_OK) s = wrk_job_submit(job);
    if (s == WRK_OK) s = wrk_job_back(job, logits, capacity, outputs, num_headers);
    wrk_job_release(job);
    if (s == WRK_OK) s = wrk_rnn_input_step(in);
    return s;
}

}  // extern "C"
