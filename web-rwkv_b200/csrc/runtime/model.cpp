// Model building: Loader::info, load-time transforms, per-layer quantization.
// Restates src/runtime/loader.rs (version sniffing, vector/matrix loaders, discount, padding) and
// ModelBuilder::build_v5 / build_v6 / build_v7 over the C ABI of wrk.h.  LoRA merging is not built.
#include <cmath>
#include <cstring>

#include "runtime.h"

using namespace wrk;
using namespace wrk::rt;

wrk_model::~wrk_model() {
    if (embed_host) cudaFreeHost(embed_host);
}

namespace wrk {
namespace rt {
int32_t shard_range(const char* what, uint32_t total, uint32_t align, uint32_t world, uint32_t rank, uint32_t* begin, uint32_t* end) {
    WRK_REQUIRE(align >= 1 && world >= 1 && rank < world, WRK_ERR_INVALID_ARGUMENT, "%s: unit %u, rank %u of %u", what, align, rank, world);
    WRK_REQUIRE(total % align == 0, WRK_ERR_SHAPE, "%s: %u is not a multiple of the unit %u", what, total, align);
    const uint32_t units = total / align;
    WRK_REQUIRE(units >= world, WRK_ERR_SHAPE, "%s: %u units of %u cannot be split %u ways", what, units, align, world);
    const uint32_t base = units / world, extra = units % world;
    const uint32_t first = rank * base + std::min(rank, extra);
    *begin = first * align;
    *end = (first + base + (rank < extra ? 1u : 0u)) * align;
    return WRK_OK;
}
}  // namespace rt
}  // namespace wrk

namespace {

struct Loader {
    wrk_model_builder* b;
    wrk_context* ctx;

    const wrk_model_builder::Entry* find(const std::string& name) const {
        auto it = b->tensors.find(name);
        return it == b->tensors.end() ? nullptr : &it->second;
    }
    bool contains(const std::string& name) const { return find(name) != nullptr; }

    int32_t entry(const std::string& name, const wrk_model_builder::Entry** e) const {
        *e = find(name);
        if (!*e) return set_error(WRK_ERR_MISSING_TENSOR, "tensor %s not found", name.c_str());
        return WRK_OK;
    }

    // Shape::from_slice_rev, src/tensor/shape.rs:113-124
    static int32_t rev_shape(const std::vector<uint64_t>& s, uint32_t out[4]) {
        out[0] = out[1] = out[2] = out[3] = 1;
        WRK_REQUIRE(s.size() >= 1 && s.size() <= 4, WRK_ERR_DEDUCE, "cannot deduce dimension");
        for (size_t i = 0; i < s.size(); ++i) out[i] = (uint32_t)s[s.size() - 1 - i];
        return WRK_OK;
    }

    // In each LoRA only the last pattern that matches the name counts (rfind, src/runtime/loader.rs:333-341).
    static const float* lora_alpha(const wrk_model_builder::Lora& lora, const std::string& name) {
        for (auto it = lora.blend.rbegin(); it != lora.blend.rend(); ++it)
            if (std::regex_search(name, it->first)) return &it->second;
        return nullptr;
    }

    int32_t upload_f16(const wrk_model_builder::Entry& e, TensorH* out) const {
        uint32_t shape[4];
        WRK_TRY(rev_shape(e.shape, shape));
        wrk_tensor* t = nullptr;
        WRK_TRY(wrk_tensor_from_data(ctx, WRK_F16, shape, e.data.data(), e.data.size() * 2, &t));
        *out = TensorH(t);
        return WRK_OK;
    }

    int32_t factor_tensor(float x, float y, TensorH* out) const {
        const float f[4] = {x, y, 0.0f, 0.0f};
        const uint32_t shape[4] = {4, 1, 1, 1};
        wrk_tensor* t = nullptr;
        WRK_TRY(wrk_tensor_from_data(ctx, WRK_F32, shape, f, sizeof f, &t));
        *out = TensorH(t);
        return WRK_OK;
    }

    int32_t run_and_release(wrk_op* op) const {
        const int32_t s = wrk_run(ctx, op);
        wrk_op_release(op);
        return s;
    }

    // lora_vectors (src/runtime/loader.rs:326-352) applied as TensorOp::blend with factor (fx * alpha, keep): the
    // LoRA holds a tensor of the same name; `target` is viewed with that tensor's shape.
    int32_t blend_named(const std::string& name, wrk_tensor* target, float fx, bool replace) const {
        for (const auto& lora : b->loras) {
            const float* alpha = lora_alpha(lora, name);
            if (!alpha) continue;
            auto it = lora.tensors.find(name);
            if (it == lora.tensors.end()) continue;
            TensorH lt, factor;
            WRK_TRY(upload_f16(it->second, &lt));
            WRK_TRY(factor_tensor(fx * *alpha, replace ? 1.0f - *alpha : 1.0f, &factor));
            wrk_tensor* shaped = nullptr;
            WRK_TRY(wrk_tensor_reshape(target, lt.p->shape.v, &shaped));
            TensorH sh(shaped);
            wrk_op* op = nullptr;
            WRK_TRY(wrk_op_blend(factor, lt, sh, &op));
            WRK_TRY(run_and_release(op));
        }
        return WRK_OK;
    }

    bool has_named(const std::string& name) const {
        for (const auto& lora : b->loras)
            if (lora_alpha(lora, name) && lora.tensors.count(name)) return true;
        return false;
    }

    // lora_matrices (src/runtime/loader.rs:354-385) applied as TensorOp::blend_lora with factor
    // (discount * alpha / rank, 1): tensors "<name without its weight component>.lora.0" and ".lora.1".
    int32_t blend_matrices(const std::string& name, wrk_tensor* target, float discount) const {
        std::string base;
        size_t pos = 0;
        while (pos <= name.size()) {
            const size_t dot = std::min(name.find('.', pos), name.size());
            const std::string part = name.substr(pos, dot - pos);
            if (part.find("weight") == std::string::npos) base += (base.empty() ? "" : ".") + part;
            pos = dot + 1;
        }
        for (const auto& lora : b->loras) {
            const float* alpha = lora_alpha(lora, name);
            if (!alpha) continue;
            auto ix = lora.tensors.find(base + ".lora.0"), iy = lora.tensors.find(base + ".lora.1");
            if (ix == lora.tensors.end() || iy == lora.tensors.end()) continue;
            WRK_REQUIRE(ix->second.shape.size() == 2, WRK_ERR_SHAPE, "tensor shape not match (%s.lora.0)", base.c_str());
            const float rank = (float)ix->second.shape[1];
            TensorH x, y, factor;
            WRK_TRY(upload_f16(ix->second, &x));
            WRK_TRY(upload_f16(iy->second, &y));
            WRK_TRY(factor_tensor(discount * *alpha / rank, 1.0f, &factor));
            wrk_view vx, vy, vo;
            WRK_TRY(wrk_tensor_as_view(x, &vx));
            WRK_TRY(wrk_tensor_as_view(y, &vy));
            WRK_TRY(wrk_tensor_as_view(target, &vo));
            wrk_op* op = nullptr;
            WRK_TRY(wrk_op_blend_lora(factor, &vx, &vy, &vo, &op));
            WRK_TRY(run_and_release(op));
        }
        return WRK_OK;
    }

    // load_vector_f16, src/runtime/loader.rs:514-565: flattened to [n, 1, 1, 1]; with a LoRA vector the blend runs
    // in f32 and the result is rounded to fp16 once
    int32_t vector_f16(const std::string& name, TensorH* out) const {
        const wrk_model_builder::Entry* e;
        WRK_TRY(entry(name, &e));
        const uint32_t shape[4] = {(uint32_t)e->data.size(), 1, 1, 1};
        wrk_tensor* t = nullptr;
        if (has_named(name)) {
            TensorH f32;
            WRK_TRY(vector_f32(name, &f32));
            WRK_TRY(wrk_tensor_create(ctx, WRK_F16, shape, &t));
            *out = TensorH(t);
            wrk_view vi, vo;
            WRK_TRY(wrk_tensor_as_view(f32, &vi));
            WRK_TRY(wrk_tensor_as_view(t, &vo));
            wrk_op* op = nullptr;
            WRK_TRY(wrk_op_blit(&vi, &vo, &op));
            return run_and_release(op);
        }
        WRK_TRY(wrk_tensor_from_data(ctx, WRK_F16, shape, e->data.data(), e->data.size() * 2, &t));
        *out = TensorH(t);
        return WRK_OK;
    }

    // load_vector_f32, src/runtime/loader.rs:393-426: f16 → f32 on the host
    int32_t vector_f32(const std::string& name, TensorH* out) const {
        const wrk_model_builder::Entry* e;
        WRK_TRY(entry(name, &e));
        std::vector<float> f(e->data.size());
        for (size_t i = 0; i < f.size(); ++i) f[i] = __half2float(__ushort_as_half(e->data[i]));
        const uint32_t shape[4] = {(uint32_t)f.size(), 1, 1, 1};
        wrk_tensor* t = nullptr;
        WRK_TRY(wrk_tensor_from_data(ctx, WRK_F32, shape, f.data(), f.size() * 4, &t));
        *out = TensorH(t);
        return blend_named(name, t, 1.0f, true);  // factor (alpha, 1 - alpha), src/runtime/loader.rs:410-425
    }

    // load_vector_exp_exp_f32, src/runtime/loader.rs:472-512: f32 vector, then StableExp on the device
    int32_t vector_exp_exp_f32(const std::string& name, TensorH* out) const {
        WRK_TRY(vector_f32(name, out));
        wrk_view v;
        WRK_TRY(wrk_tensor_as_view(*out, &v));
        wrk_op* op = nullptr;
        WRK_TRY(wrk_op_activate(&v, WRK_ACT_STABLE_EXP, &op));
        int32_t s = wrk_run(ctx, op);
        wrk_op_release(op);
        return s;
    }

    // load_vector_exp_f32, src/runtime/loader.rs:431-470: f32 vector, then OppositeExp (-exp(x)) on the device
    int32_t vector_exp_f32(const std::string& name, TensorH* out) const {
        WRK_TRY(vector_f32(name, out));
        wrk_view v;
        WRK_TRY(wrk_tensor_as_view(*out, &v));
        wrk_op* op = nullptr;
        WRK_TRY(wrk_op_activate(&v, WRK_ACT_OPPOSITE_EXP, &op));
        return run_and_release(op);
    }

    // load_matrix_f16, src/runtime/loader.rs:567-592 (optionally padded to multiples of 8: :688-707)
    int32_t matrix_f16(const std::string& name, bool padded, float discount, TensorH* out) const {
        const wrk_model_builder::Entry* e;
        WRK_TRY(entry(name, &e));
        uint32_t shape[4];
        WRK_TRY(rev_shape(e->shape, shape));
        const uint16_t* src = e->data.data();
        std::vector<uint16_t> tmp;
        if (discount != 1.0f) {
            // f16(discount * f32(x)) on the host, src/runtime/loader.rs:660-661
            tmp.resize(e->data.size());
            for (size_t i = 0; i < tmp.size(); ++i)
                tmp[i] = __half_as_ushort(__float2half_rn(discount * __half2float(__ushort_as_half(e->data[i]))));
            src = tmp.data();
        }
        std::vector<uint16_t> pad;
        if (padded && (shape[0] % 8 || shape[1] % 8)) {
            const uint32_t px = (shape[0] + 7) / 8 * 8, py = (shape[1] + 7) / 8 * 8;
            pad.assign((size_t)px * py * shape[2] * shape[3], 0);
            for (size_t z = 0; z < (size_t)shape[2] * shape[3]; ++z)
                for (uint32_t y = 0; y < shape[1]; ++y)
                    std::memcpy(&pad[(z * py + y) * px], &src[(z * shape[1] + y) * shape[0]], shape[0] * 2);
            shape[0] = px;
            shape[1] = py;
            src = pad.data();
        }
        const size_t n = (size_t)shape[0] * shape[1] * shape[2] * shape[3];
        wrk_tensor* t = nullptr;
        WRK_TRY(wrk_tensor_from_data(ctx, WRK_F16, shape, src, n * 2, &t));
        *out = TensorH(t);
        if (padded || b->loras.empty()) return WRK_OK;  // load_matrix_f16_padded_cpu takes no LoRA
        // blend_lora, then blend of a same-named tensor, src/runtime/loader.rs:577-588 and 606-617
        WRK_TRY(blend_matrices(name, t, discount));
        return blend_named(name, t, discount, false);
    }

    int32_t matrix_fp16(const std::string& name, MatrixH* out) const {
        TensorH t;
        WRK_TRY(matrix_f16(name, false, 1.0f, &t));
        wrk_matrix* m = nullptr;
        WRK_TRY(wrk_matrix_fp16(t, &m));
        *out = MatrixH(m);
        return WRK_OK;
    }

    // load_matrix / load_matrix_discount, src/runtime/loader.rs:709-762
    int32_t matrix(const std::string& name, int32_t quant, float discount, MatrixH* out) const {
        TensorH t;
        WRK_TRY(matrix_f16(name, false, discount, &t));
        wrk_matrix* m = nullptr;
        switch (quant) {
            case WRK_QUANT_NONE: WRK_TRY(wrk_matrix_fp16(t, &m)); break;
            case WRK_QUANT_INT8: WRK_TRY(wrk_matrix_quant_u8(t, &m)); break;
            case WRK_QUANT_NF4: WRK_TRY(wrk_matrix_quant_nf4(t, &m)); break;
            case WRK_QUANT_SF4: WRK_TRY(wrk_matrix_quant_sf4(t, 5.0, &m)); break;  // Quant::SF4: nu = 5 (model.rs:133-134)
            default: return set_error(WRK_ERR_INVALID_ARGUMENT, "unknown quant %d", quant);
        }
        *out = MatrixH(m);
        // the fp16 staging tensor is released here; the stream orders its reuse after the quantizer
        return WRK_OK;
    }

    int32_t layer_norm(const std::string& prefix, LayerNorm* ln) const {
        WRK_TRY(vector_f16(prefix + ".weight", &ln->w));
        WRK_TRY(vector_f16(prefix + ".bias", &ln->b));
        return WRK_OK;
    }

    int32_t group_norm(const std::string& prefix, uint32_t num_head, LayerNorm* ln) const {
        TensorH w, b;
        WRK_TRY(vector_f16(prefix + ".weight", &w));
        WRK_TRY(vector_f16(prefix + ".bias", &b));
        const uint32_t shape[4] = {WRK_DIM_AUTO, num_head, 1, 1};
        wrk_tensor *rw = nullptr, *rb = nullptr;
        WRK_TRY(wrk_tensor_reshape(w, shape, &rw));
        ln->w = TensorH(rw);
        WRK_TRY(wrk_tensor_reshape(b, shape, &rb));
        ln->b = TensorH(rb);
        return WRK_OK;
    }
};

// A dimension of the tensor as the file holds it (a sharded builder keeps the rank's slice and this record).
uint32_t file_dim(const wrk_model_builder::Entry* e, size_t i) { return (uint32_t)(e->full.empty() ? e->shape[i] : e->full[i]); }

// Which slice of a tensor a rank of a sharded model keeps, by the tensor's name.  Time-mix channels go by whole
// heads: key / value / receptance / gate and the second matrices of the per-channel adapters keep the rows of the
// rank's channels, `output` the matching columns (a split of its K), per-channel vectors their slice; ffn `key` keeps
// a slice of rows, `value` the matching columns; the head keeps a slice of the vocabulary.  Everything else (layer
// norms, token-shift mixes, the adapters' first matrices, ffn `receptance`, the embedding) is held whole by every rank.
enum class Cut { None, RowsC, ColsC, FlatC, RowsF, ColsF, RowsV };
Cut cut_of(const std::string& name) {
    if (name == "head.weight") return Cut::RowsV;
    if (name.rfind("blocks.", 0) != 0) return Cut::None;
    const size_t dot = name.find('.', 7);
    if (dot == std::string::npos) return Cut::None;
    const std::string leaf = name.substr(dot + 1);
    for (auto n : {"att.key.weight", "att.value.weight", "att.receptance.weight", "att.gate.weight", "att.time_decay_w2", "att.w2",
                   "att.a2", "att.g2", "att.v2"})
        if (leaf == n) return Cut::RowsC;
    if (leaf == "att.output.weight") return Cut::ColsC;
    for (auto n : {"att.time_decay", "att.time_first", "att.ln_x.weight", "att.ln_x.bias", "att.w0", "att.a0", "att.v0", "att.k_k",
                   "att.k_a", "att.r_k"})
        if (leaf == n) return Cut::FlatC;
    if (leaf == "ffn.key.weight") return Cut::RowsF;
    if (leaf == "ffn.value.weight") return Cut::ColsF;
    return Cut::None;
}

int32_t cut_entry(const wrk_model_builder* b, const std::string& name, wrk_model_builder::Entry& e) {
    const Cut cut = cut_of(name);
    if (cut == Cut::None) return WRK_OK;
    const uint32_t S = b->shard_head_size, blk = b->shard_block;
    const uint32_t align_c = std::max(S, blk), align_f = std::max(blk, 8u);
    size_t n = 1;
    for (auto d : e.shape) n *= d;
    uint32_t b0 = 0, b1 = 0;
    const std::vector<uint64_t> full = e.shape;
    if (cut == Cut::FlatC) {
        WRK_TRY(shard_range(name.c_str(), (uint32_t)n, align_c, b->shard_world, b->shard_rank, &b0, &b1));
        std::memmove(e.data.data(), e.data.data() + b0, (size_t)(b1 - b0) * 2);
        e.data.resize(b1 - b0);
        // (heads, head size) stays two-dimensional; everything else becomes a vector
        if (full.size() == 2 && full[1] == S && full[0] * S == n) e.shape = {(b1 - b0) / S, S};
        else e.shape = {b1 - b0};
        e.full = full;
        return WRK_OK;
    }
    WRK_REQUIRE(e.shape.size() == 2, WRK_ERR_SHAPE, "tensor shape not match: %s is not a matrix", name.c_str());
    const uint32_t M = (uint32_t)e.shape[0], K = (uint32_t)e.shape[1];
    const bool rows = cut == Cut::RowsC || cut == Cut::RowsF || cut == Cut::RowsV;
    uint32_t align = cut == Cut::RowsC || cut == Cut::ColsC ? align_c : align_f;
    if (cut == Cut::RowsV) {
        WRK_REQUIRE(M % (8 * b->shard_world) == 0, WRK_ERR_SHAPE, "a vocabulary of %u rows does not split into %u slices of whole 8-row groups",
                    M, b->shard_world);
        align = M / b->shard_world;
    }
    WRK_TRY(shard_range(name.c_str(), rows ? M : K, align, b->shard_world, b->shard_rank, &b0, &b1));
    if (rows) {
        std::memmove(e.data.data(), e.data.data() + (size_t)b0 * K, (size_t)(b1 - b0) * K * 2);
        e.data.resize((size_t)(b1 - b0) * K);
        e.shape = {b1 - b0, K};
    } else {
        const uint32_t Kl = b1 - b0;
        for (uint32_t m = 0; m < M; ++m) std::memmove(e.data.data() + (size_t)m * Kl, e.data.data() + (size_t)m * K + b0, (size_t)Kl * 2);
        e.data.resize((size_t)M * Kl);
        e.shape = {M, Kl};
    }
    e.data.shrink_to_fit();
    e.full = full;
    return WRK_OK;
}

// Loader::info, src/runtime/loader.rs:208-324.
int32_t sniff_info(const wrk_model_builder* b, wrk_model_info* info) {
    Loader ld{const_cast<wrk_model_builder*>(b), b->ctx};
    uint32_t num_layer = 0;
    for (auto& kv : b->tensors) {
        const std::string& n = kv.first;
        if (n.rfind("blocks.", 0) == 0) {
            const size_t dot = n.find('.', 7);
            if (dot == std::string::npos) continue;
            num_layer = std::max<uint32_t>(num_layer, (uint32_t)std::stoul(n.substr(7, dot - 7)));
        }
    }
    num_layer += 1;
    auto all = [&](std::initializer_list<const char*> names) {
        for (auto n : names)
            if (!ld.contains(n)) return false;
        return true;
    };
    const bool v4 = all({"blocks.0.att.time_decay", "blocks.0.att.time_first", "blocks.0.att.time_mix_k",
                         "blocks.0.att.time_mix_v", "blocks.0.att.time_mix_r"});
    const bool v5 = all({"blocks.0.att.gate.weight", "blocks.0.att.ln_x.weight", "blocks.0.att.ln_x.bias"});
    const bool v6 = all({"blocks.0.att.time_mix_x", "blocks.0.att.time_mix_w", "blocks.0.att.time_mix_k",
                         "blocks.0.att.time_mix_v", "blocks.0.att.time_mix_r", "blocks.0.att.time_mix_g",
                         "blocks.0.att.time_mix_w1", "blocks.0.att.time_mix_w2", "blocks.0.att.time_decay_w1",
                         "blocks.0.att.time_decay_w2", "blocks.0.ffn.time_mix_k", "blocks.0.ffn.time_mix_r"});
    const bool v7 = all({"blocks.0.att.x_r", "blocks.0.att.x_w", "blocks.0.att.x_k", "blocks.0.att.x_v",
                         "blocks.0.att.x_a", "blocks.0.att.x_g", "blocks.0.att.w0", "blocks.0.att.w1",
                         "blocks.0.att.w2", "blocks.0.att.a0", "blocks.0.att.a1", "blocks.0.att.a2",
                         "blocks.0.att.g1", "blocks.0.att.g2", "blocks.0.att.r_k", "blocks.0.att.k_k",
                         "blocks.0.att.k_a"});
    uint32_t version;
    if (v7) version = 7;
    else if (v6) version = 6;
    else if (v5) version = 5;
    else if (v4) version = 4;
    else
        return set_error(WRK_ERR_INVALID_VERSION, "invalid model version");

    const wrk_model_builder::Entry *embed, *ffn;
    WRK_TRY(ld.entry("emb.weight", &embed));
    WRK_TRY(ld.entry("blocks.0.ffn.key.weight", &ffn));
    WRK_REQUIRE(embed->shape.size() == 2 && ffn->shape.size() == 2, WRK_ERR_SHAPE, "tensor shape not match: emb/ffn");
    std::memset(info, 0, sizeof *info);
    info->version = version;
    info->num_layer = num_layer;
    info->num_emb = file_dim(embed, 1);
    info->num_hidden = file_dim(ffn, 0);
    info->num_vocab = file_dim(embed, 0);
    const wrk_model_builder::Entry* e;
    if (version == 7) {
        WRK_TRY(ld.entry("blocks.0.att.r_k", &e));
        info->num_head = file_dim(e, 0);
        WRK_TRY(ld.entry("blocks.0.att.w1", &e));
        info->custom[0] = (uint32_t)e->shape[0];
        WRK_TRY(ld.entry("blocks.0.att.a1", &e));
        info->custom[1] = (uint32_t)e->shape[0];
        WRK_TRY(ld.entry("blocks.0.att.g1", &e));
        info->custom[2] = (uint32_t)e->shape[0];
        WRK_TRY(ld.entry("blocks.1.att.v1", &e));
        info->custom[3] = (uint32_t)e->shape[0];
    } else if (version == 4) {
        info->num_head = 1;  // src/runtime/loader.rs:290-294
    } else {
        WRK_TRY(ld.entry("blocks.0.att.time_first", &e));
        info->num_head = file_dim(e, 0);
        if (version == 6) {
            WRK_TRY(ld.entry("blocks.0.att.time_mix_w1", &e));
            info->custom[0] = (uint32_t)e->shape[0] / 5;
            WRK_TRY(ld.entry("blocks.0.att.time_decay_w1", &e));
            info->custom[1] = (uint32_t)e->shape[0];
        }
    }
    return WRK_OK;
}

int32_t build_common(const Loader& ld, wrk_model* m) {
    const wrk_model_info& info = m->info;
    WRK_TRY(ld.layer_norm("blocks.0.ln0", &m->embed_ln));
    WRK_TRY(ld.layer_norm("ln_out", &m->head_ln));
    // embedding table stays on the host, padded to a multiple of 8 rows (load_matrix_f16_padded_cpu)
    const wrk_model_builder::Entry* e;
    WRK_TRY(ld.entry("emb.weight", &e));
    m->num_vocab_padded = (info.num_vocab + 7) / 8 * 8;
    const size_t bytes = (size_t)m->num_vocab_padded * info.num_emb * 2;
    WRK_CUDA(cudaMallocHost(&m->embed_host, bytes));
    std::memset(m->embed_host, 0, bytes);
    std::memcpy(m->embed_host, e->data.data(), e->data.size() * 2);
    // head: never quantized; v6 / v7 pad it, v5 does not (v5.rs:956, v6.rs:1029, v7.rs:1073)
    TensorH head;
    WRK_TRY(ld.matrix_f16("head.weight", info.version >= 6, 1.0f, &head));  // v4: src/runtime/v4.rs:861
    wrk_matrix* hm = nullptr;
    WRK_TRY(wrk_matrix_fp16(head, &hm));
    m->head_w = MatrixH(hm);
    return WRK_OK;
}

// The rank's ranges, from the whole model's dimensions with the rules cut_entry applied tensor by tensor.
int32_t plan_shard(const wrk_model_builder* b, wrk_model* m) {
    const wrk_model_info& info = m->info;
    const uint32_t S = info.num_emb / info.num_head;
    WRK_REQUIRE(S == b->shard_head_size, WRK_ERR_SHAPE, "the model's heads have %u channels, the split was set up for %u", S,
                b->shard_head_size);
    uint32_t blk = 1;
    for (uint32_t layer = 0; layer < info.num_layer; ++layer) {
        auto it = b->quant.find(layer);
        const int32_t q = it == b->quant.end() ? WRK_QUANT_NONE : it->second;
        blk = std::max(blk, q == WRK_QUANT_INT8 ? 128u : q == WRK_QUANT_NONE ? 1u : 64u);
    }
    WRK_REQUIRE(b->shard_block % blk == 0, WRK_ERR_INVALID_ARGUMENT,
                "the split was set up for quantization blocks of %u values, the layers' quantization needs %u", b->shard_block, blk);
    Shard& sh = m->shard;
    sh.rank = b->shard_rank;
    sh.world = b->shard_world;
    WRK_TRY(shard_range("channels", info.num_emb, std::max(S, b->shard_block), sh.world, sh.rank, &sh.c0, &sh.c1));
    WRK_TRY(shard_range("ffn columns", info.num_hidden, std::max(b->shard_block, 8u), sh.world, sh.rank, &sh.f0, &sh.f1));
    WRK_REQUIRE(info.num_vocab % (8 * sh.world) == 0, WRK_ERR_SHAPE, "a vocabulary of %u rows does not split into %u slices of whole 8-row groups",
                info.num_vocab, sh.world);
    WRK_TRY(shard_range("vocabulary", info.num_vocab, info.num_vocab / sh.world, sh.world, sh.rank, &sh.v0, &sh.v1));
    return WRK_OK;
}

uint32_t local_heads(const wrk_model* m) {
    const uint32_t S = m->info.num_emb / m->info.num_head;
    return m->shard.on() ? (m->shard.c1 - m->shard.c0) / S : m->info.num_head;
}

int32_t quant_of(const wrk_model_builder* b, uint32_t layer) {
    auto it = b->quant.find(layer);
    return it == b->quant.end() ? WRK_QUANT_NONE : it->second;
}

// ModelBuilder::build_v5 (src/runtime/v5.rs:922-1082) and build_v6 (src/runtime/v6.rs:995-1172)
int32_t build_v56(const Loader& ld, wrk_model* m) {
    const wrk_model_info& info = m->info;
    wrk_context* ctx = m->ctx;
    m->layers.resize(info.num_layer);
    for (uint32_t layer = 0; layer < info.num_layer; ++layer) {
        Layer& L = m->layers[layer];
        const int32_t quant = quant_of(ld.b, layer);
        const float discount = std::ldexp(1.0f, -(int)(layer / m->rescale));
        const std::string blk = "blocks." + std::to_string(layer);
        const std::string att = blk + ".att", ffn = blk + ".ffn";
        WRK_TRY(ld.layer_norm(blk + ".ln1", &L.att_ln));
        WRK_TRY(ld.vector_f32(att + ".time_first", &L.time_first));
        if (info.version == 5) {
            WRK_TRY(ld.vector_exp_exp_f32(att + ".time_decay", &L.time_decay));
            WRK_TRY(ld.vector_f16(att + ".time_mix_k", &L.time_mix_k));
            WRK_TRY(ld.vector_f16(att + ".time_mix_v", &L.time_mix_v));
            WRK_TRY(ld.vector_f16(att + ".time_mix_r", &L.time_mix_r));
            WRK_TRY(ld.vector_f16(att + ".time_mix_g", &L.time_mix_g));
        } else {
            WRK_TRY(ld.vector_f16(att + ".time_decay", &L.time_decay));
            WRK_TRY(ld.vector_f16(att + ".time_mix_x", &L.time_mix_x));
            // five static mixes stacked as [C, 1, 5] in the order w, k, v, r, g (v6.rs:1063-1080)
            const uint32_t shape[4] = {info.num_emb, 1, 5, 1};
            wrk_tensor* tm = nullptr;
            WRK_TRY(wrk_tensor_zeros(ctx, WRK_F16, shape, &tm));
            L.time_mix = TensorH(tm);
            const char* names[5] = {".time_mix_w", ".time_mix_k", ".time_mix_v", ".time_mix_r", ".time_mix_g"};
            for (uint32_t i = 0; i < 5; ++i) {
                const wrk_model_builder::Entry* e;
                WRK_TRY(ld.entry(att + names[i], &e));
                WRK_REQUIRE(e->data.size() == info.num_emb, WRK_ERR_SHAPE, "tensor shape not match: %s",
                            (att + names[i]).c_str());
                WRK_CUDA(cudaMemcpyAsync(static_cast<uint16_t*>(tm->ptr()) + (size_t)i * info.num_emb, e->data.data(),
                                         (size_t)info.num_emb * 2, cudaMemcpyHostToDevice, ctx->stream));
            }
            WRK_CUDA(cudaStreamSynchronize(ctx->stream));
            WRK_TRY(ld.matrix_fp16(att + ".time_decay_w1", &L.time_decay_w1));
            WRK_TRY(ld.matrix_fp16(att + ".time_decay_w2", &L.time_decay_w2));
            WRK_TRY(ld.matrix_fp16(att + ".time_mix_w1", &L.time_mix_w1));
            WRK_TRY(ld.matrix_fp16(att + ".time_mix_w2", &L.time_mix_w2));
        }
        WRK_TRY(ld.group_norm(att + ".ln_x", local_heads(m), &L.gn));
        WRK_TRY(ld.matrix(att + ".key.weight", quant, 1.0f, &L.att_w_k));
        WRK_TRY(ld.matrix(att + ".value.weight", quant, 1.0f, &L.att_w_v));
        WRK_TRY(ld.matrix(att + ".receptance.weight", quant, 1.0f, &L.att_w_r));
        WRK_TRY(ld.matrix(att + ".gate.weight", quant, 1.0f, &L.att_w_g));
        WRK_TRY(ld.matrix(att + ".output.weight", quant, discount, &L.att_w_o));
        WRK_TRY(ld.layer_norm(blk + ".ln2", &L.ffn_ln));
        WRK_TRY(ld.vector_f16(ffn + ".time_mix_k", &L.ffn_time_mix_k));
        WRK_TRY(ld.vector_f16(ffn + ".time_mix_r", &L.ffn_time_mix_r));
        WRK_TRY(ld.matrix(ffn + ".receptance.weight", quant, 1.0f, &L.ffn_w_r));
        WRK_TRY(ld.matrix(ffn + ".key.weight", quant, 1.0f, &L.ffn_w_k));
        WRK_TRY(ld.matrix(ffn + ".value.weight", quant, discount, &L.ffn_w_v));
        WRK_CUDA(cudaStreamSynchronize(ctx->stream));  // frees the fp16 staging of this layer (v6.rs:1135-1139)
    }
    return WRK_OK;
}

// ModelBuilder::build_v4, src/runtime/v4.rs:829-960
int32_t build_v4(const Loader& ld, wrk_model* m) {
    const wrk_model_info& info = m->info;
    wrk_context* ctx = m->ctx;
    m->layers.resize(info.num_layer);
    for (uint32_t layer = 0; layer < info.num_layer; ++layer) {
        Layer& L = m->layers[layer];
        const int32_t quant = quant_of(ld.b, layer);
        const float discount = std::ldexp(1.0f, -(int)(layer / m->rescale));
        const std::string blk = "blocks." + std::to_string(layer);
        const std::string att = blk + ".att", ffn = blk + ".ffn";
        WRK_TRY(ld.layer_norm(blk + ".ln1", &L.att_ln));
        WRK_TRY(ld.vector_exp_f32(att + ".time_decay", &L.time_decay));
        WRK_TRY(ld.vector_f32(att + ".time_first", &L.time_first));
        WRK_TRY(ld.vector_f16(att + ".time_mix_k", &L.time_mix_k));
        WRK_TRY(ld.vector_f16(att + ".time_mix_v", &L.time_mix_v));
        WRK_TRY(ld.vector_f16(att + ".time_mix_r", &L.time_mix_r));
        WRK_TRY(ld.matrix(att + ".key.weight", quant, 1.0f, &L.att_w_k));
        WRK_TRY(ld.matrix(att + ".value.weight", quant, 1.0f, &L.att_w_v));
        WRK_TRY(ld.matrix(att + ".receptance.weight", quant, 1.0f, &L.att_w_r));
        WRK_TRY(ld.matrix(att + ".output.weight", quant, discount, &L.att_w_o));
        WRK_TRY(ld.layer_norm(blk + ".ln2", &L.ffn_ln));
        WRK_TRY(ld.vector_f16(ffn + ".time_mix_k", &L.ffn_time_mix_k));
        WRK_TRY(ld.vector_f16(ffn + ".time_mix_r", &L.ffn_time_mix_r));
        WRK_TRY(ld.matrix(ffn + ".receptance.weight", quant, 1.0f, &L.ffn_w_r));
        WRK_TRY(ld.matrix(ffn + ".key.weight", quant, 1.0f, &L.ffn_w_k));
        WRK_TRY(ld.matrix(ffn + ".value.weight", quant, discount, &L.ffn_w_v));
        WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    return WRK_OK;
}

// ModelBuilder::build_v7, src/runtime/v7.rs:1038-1226
int32_t build_v7(const Loader& ld, wrk_model* m) {
    const wrk_model_info& info = m->info;
    wrk_context* ctx = m->ctx;
    m->layers.resize(info.num_layer);
    for (uint32_t layer = 0; layer < info.num_layer; ++layer) {
        Layer& L = m->layers[layer];
        const int32_t quant = quant_of(ld.b, layer);
        const float discount = std::ldexp(1.0f, -(int)(layer / m->rescale));
        const std::string blk = "blocks." + std::to_string(layer);
        const std::string att = blk + ".att", ffn = blk + ".ffn";
        WRK_TRY(ld.layer_norm(blk + ".ln1", &L.att_ln));
        WRK_TRY(ld.vector_f16(att + ".x_r", &L.x_r));
        WRK_TRY(ld.vector_f16(att + ".x_w", &L.x_w));
        WRK_TRY(ld.vector_f16(att + ".x_k", &L.x_k));
        WRK_TRY(ld.vector_f16(att + ".x_v", &L.x_v));
        WRK_TRY(ld.vector_f16(att + ".x_a", &L.x_a));
        WRK_TRY(ld.vector_f16(att + ".x_g", &L.x_g));
        WRK_TRY(ld.vector_f16(att + ".w0", &L.w0));
        WRK_TRY(ld.vector_f16(att + ".a0", &L.a0));
        WRK_TRY(ld.matrix_fp16(att + ".w1", &L.w1));
        WRK_TRY(ld.matrix_fp16(att + ".w2", &L.w2));
        WRK_TRY(ld.matrix_fp16(att + ".a1", &L.a1));
        WRK_TRY(ld.matrix_fp16(att + ".a2", &L.a2));
        WRK_TRY(ld.matrix_fp16(att + ".g1", &L.g1));
        WRK_TRY(ld.matrix_fp16(att + ".g2", &L.g2));
        if (layer == 0) {  // placeholders, never used (v7.rs:1114-1121)
            L.v0 = L.a0;
            L.v1 = L.a1;
            L.v2 = L.a2;
        } else {
            WRK_TRY(ld.vector_f16(att + ".v0", &L.v0));
            WRK_TRY(ld.matrix_fp16(att + ".v1", &L.v1));
            WRK_TRY(ld.matrix_fp16(att + ".v2", &L.v2));
        }
        WRK_TRY(ld.matrix_f16(att + ".r_k", false, 1.0f, &L.r_k));
        WRK_TRY(ld.vector_f16(att + ".k_k", &L.k_k));
        WRK_TRY(ld.vector_f16(att + ".k_a", &L.k_a));
        WRK_TRY(ld.group_norm(att + ".ln_x", local_heads(m), &L.gn));
        WRK_TRY(ld.matrix(att + ".key.weight", quant, 1.0f, &L.att_w_k));
        WRK_TRY(ld.matrix(att + ".value.weight", quant, 1.0f, &L.att_w_v));
        WRK_TRY(ld.matrix(att + ".receptance.weight", quant, 1.0f, &L.att_w_r));
        WRK_TRY(ld.matrix(att + ".output.weight", quant, discount, &L.att_w_o));
        WRK_TRY(ld.layer_norm(blk + ".ln2", &L.ffn_ln));
        WRK_TRY(ld.vector_f16(ffn + ".x_k", &L.ffn_x_k));
        WRK_TRY(ld.matrix(ffn + ".key.weight", quant, 1.0f, &L.ffn_w_k));
        WRK_TRY(ld.matrix(ffn + ".value.weight", quant, discount, &L.ffn_w_v));
        WRK_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    return WRK_OK;
}

}  // namespace

extern "C" {

int32_t wrk_model_builder_create(wrk_context* ctx, wrk_model_builder** out) {
    WRK_REQUIRE(ctx && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    auto b = new wrk_model_builder();
    b->ctx = ctx;
    *out = b;
    return WRK_OK;
}

int32_t wrk_model_builder_destroy(wrk_model_builder* b) {
    delete b;
    return WRK_OK;
}

int32_t wrk_model_builder_add_tensor(wrk_model_builder* b, const char* name, const uint64_t* shape, uint32_t ndim,
                                     const void* data_f16, size_t bytes) {
    WRK_REQUIRE(b && name && shape && (data_f16 || bytes == 0), WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(ndim >= 1 && ndim <= 4, WRK_ERR_DEDUCE, "cannot deduce dimension");
    size_t n = 1;
    for (uint32_t i = 0; i < ndim; ++i) n *= shape[i];
    WRK_REQUIRE(n * 2 == bytes, WRK_ERR_SIZE, "data size not match: %zu vs. %zu", n * 2, bytes);
    auto& e = b->tensors[name];
    e.shape.assign(shape, shape + ndim);
    e.full.clear();
    e.data.resize(n);
    std::memcpy(e.data.data(), data_f16, bytes);
    if (b->shard_world > 1) {
        const int32_t s = cut_entry(b, name, e);
        if (s != WRK_OK) b->tensors.erase(name);
        return s;
    }
    return WRK_OK;
}

int32_t wrk_model_builder_shard(wrk_model_builder* b, uint32_t rank, uint32_t world, uint32_t head_size, uint32_t block) {
    WRK_REQUIRE(b, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(world >= 1 && rank < world, WRK_ERR_INVALID_ARGUMENT, "rank %u of %u", rank, world);
    WRK_REQUIRE(head_size >= 1 && block >= 1, WRK_ERR_INVALID_ARGUMENT, "head size %u, block %u", head_size, block);
    WRK_REQUIRE(b->tensors.empty() && b->loras.empty(), WRK_ERR_INVALID_ARGUMENT,
                "the split is chosen before the first tensor is added (tensors are cut as they arrive)");
    b->shard_rank = rank;
    b->shard_world = world;
    b->shard_head_size = head_size;
    b->shard_block = block;
    return WRK_OK;
}

int32_t wrk_shard_range(uint32_t total, uint32_t align, uint32_t world, uint32_t rank, uint32_t* begin, uint32_t* end) {
    WRK_REQUIRE(begin && end, WRK_ERR_INVALID_ARGUMENT, "null argument");
    return shard_range("range", total, align, world, rank, begin, end);
}

int32_t wrk_model_builder_quant(wrk_model_builder* b, uint32_t layer, int32_t quant) {
    WRK_REQUIRE(b, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(quant >= WRK_QUANT_NONE && quant <= WRK_QUANT_SF4, WRK_ERR_INVALID_ARGUMENT, "unknown quant %d", quant);
    b->quant[layer] = quant;
    return WRK_OK;
}

int32_t wrk_model_builder_lora(wrk_model_builder* b, uint32_t* index) {
    WRK_REQUIRE(b && index, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(b->shard_world == 1, WRK_ERR_UNSUPPORTED, "LoRA blending is not built for split models: merge first, then split");
    b->loras.emplace_back();
    *index = (uint32_t)b->loras.size() - 1;
    return WRK_OK;
}

int32_t wrk_model_builder_lora_tensor(wrk_model_builder* b, uint32_t index, const char* name, const uint64_t* shape,
                                      uint32_t ndim, const void* data_f16, size_t bytes) {
    WRK_REQUIRE(b && name && shape && data_f16, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(index < b->loras.size(), WRK_ERR_INVALID_ARGUMENT, "no LoRA %u", index);
    WRK_REQUIRE(ndim >= 1 && ndim <= 4, WRK_ERR_DEDUCE, "cannot deduce dimension");
    size_t n = 1;
    for (uint32_t i = 0; i < ndim; ++i) n *= shape[i];
    WRK_REQUIRE(n * 2 == bytes, WRK_ERR_SIZE, "tensor %s: %zu bytes for %zu fp16 elements", name, bytes, n);
    wrk_model_builder::Entry e;
    e.shape.assign(shape, shape + ndim);
    e.data.resize(n);
    std::memcpy(e.data.data(), data_f16, bytes);
    b->loras[index].tensors[name] = std::move(e);
    return WRK_OK;
}

int32_t wrk_model_builder_lora_blend(wrk_model_builder* b, uint32_t index, const char* pattern, float alpha) {
    WRK_REQUIRE(b && pattern, WRK_ERR_INVALID_ARGUMENT, "null argument");
    WRK_REQUIRE(index < b->loras.size(), WRK_ERR_INVALID_ARGUMENT, "no LoRA %u", index);
    try {
        b->loras[index].blend.emplace_back(std::regex(pattern, std::regex::ECMAScript), alpha);
    } catch (const std::regex_error& err) {
        return set_error(WRK_ERR_INVALID_ARGUMENT, "bad blend pattern %s: %s", pattern, err.what());
    }
    return WRK_OK;
}

int32_t wrk_model_builder_rescale(wrk_model_builder* b, uint32_t value) {
    WRK_REQUIRE(b, WRK_ERR_INVALID_ARGUMENT, "null argument");
    b->rescale = value == 0 ? SIZE_MAX : value;  // ModelBuilder::rescale: 0 disables (model.rs:160-166)
    return WRK_OK;
}

int32_t wrk_model_builder_sep(wrk_model_builder* b, uint32_t value) {
    WRK_REQUIRE(b, WRK_ERR_INVALID_ARGUMENT, "null argument");
    b->sep = value == 0 ? SIZE_MAX : value;
    return WRK_OK;
}

int32_t wrk_model_builder_read_state(wrk_model_builder* b, float* host, size_t bytes) {
    // read_state, src/runtime/v5.rs / v6.rs:1175-1208 / v7.rs: per layer the matrix blocks.N.att.time_state
    // (H x S x S in the file) is transposed to [S, H, S], viewed as [C, S] and copied into rows 1..S of an f32
    // [C, S + 2, L] tensor of zeros, which State::load takes for one batch slot.
    WRK_REQUIRE(b && host, WRK_ERR_INVALID_ARGUMENT, "null argument");
    wrk_model_info info{};
    WRK_TRY(sniff_info(b, &info));
    const uint32_t C = info.num_emb, H = info.num_head, L = info.num_layer;
    WRK_REQUIRE(H > 0 && C % H == 0, WRK_ERR_SHAPE, "num_emb %u is not a multiple of num_head %u", C, H);
    const uint32_t S = C / H;
    WRK_REQUIRE(bytes == (size_t)C * (S + 2) * L * sizeof(float), WRK_ERR_SIZE, "state of %zu bytes expected",
                (size_t)C * (S + 2) * L * sizeof(float));
    Loader ld{b, b->ctx};
    const uint32_t data_shape[4] = {C, S + 2, L, 1};
    wrk_tensor* data_raw = nullptr;
    WRK_TRY(wrk_tensor_zeros(b->ctx, WRK_F32, data_shape, &data_raw));
    TensorH data(data_raw);
    for (uint32_t layer = 0; layer < L; ++layer) {
        TensorH matrix;
        WRK_TRY(ld.matrix_f16("blocks." + std::to_string(layer) + ".att.time_state", false, 1.0f, &matrix));
        WRK_TRY(check_shape("time_state", matrix.p->shape, S, S, H, 1));
        const uint32_t state_shape[4] = {S, H, S, 1}, flat_shape[4] = {C, S, 1, WRK_DIM_AUTO};
        wrk_tensor *state_raw = nullptr, *flat_raw = nullptr;
        WRK_TRY(wrk_tensor_create(b->ctx, WRK_F16, state_shape, &state_raw));
        TensorH state(state_raw);
        WRK_TRY(wrk_tensor_reshape(state, flat_shape, &flat_raw));
        TensorH flat(flat_raw);
        wrk_view vm, vs, vf, vd;
        WRK_TRY(wrk_tensor_as_view(matrix, &vm));
        WRK_TRY(wrk_tensor_as_view(state, &vs));
        WRK_TRY(wrk_tensor_as_view(flat, &vf));
        const uint32_t start[4] = {0, 1, layer, 0}, end[4] = {C, S + 1, layer + 1, 1};
        WRK_TRY(wrk_tensor_view(data, start, end, &vd));
        wrk_op* op = nullptr;
        WRK_TRY(wrk_op_transpose(&vm, &vs, &op));
        WRK_TRY(ld.run_and_release(op));
        WRK_TRY(wrk_op_blit(&vf, &vd, &op));
        WRK_TRY(ld.run_and_release(op));
    }
    return wrk_tensor_back(data, host, bytes);
}

int32_t wrk_model_builder_info(wrk_model_builder* b, wrk_model_info* info) {
    WRK_REQUIRE(b && info, WRK_ERR_INVALID_ARGUMENT, "null argument");
    return sniff_info(b, info);
}

int32_t wrk_model_builder_build(wrk_model_builder* b, wrk_model** out) {
    WRK_REQUIRE(b && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    auto m = new wrk_model();
    m->ctx = b->ctx;
    int32_t s = sniff_info(b, &m->info);
    if (s == WRK_OK) {
        const size_t def_rescale = m->info.version == 7 ? 1024 : 6;  // Model::DEFAULT_RESCALE
        m->rescale = b->rescale ? b->rescale : def_rescale;
        m->sep = b->sep ? b->sep : 1024;
        if (m->info.num_emb % m->info.num_head != 0)
            s = set_error(WRK_ERR_SHAPE, "num_emb %u not divisible by num_head %u", m->info.num_emb, m->info.num_head);
        if (s == WRK_OK && b->shard_world > 1) s = plan_shard(b, m);
        Loader ld{b, b->ctx};
        if (s == WRK_OK) s = build_common(ld, m);
        if (s == WRK_OK && m->info.version == 4 && b->shard_world > 1)
            s = set_error(WRK_ERR_UNSUPPORTED, "v4 models are not split across GPUs (their time-mix has no heads)");
        if (s == WRK_OK) s = m->info.version == 7 ? build_v7(ld, m) : m->info.version == 4 ? build_v4(ld, m) : build_v56(ld, m);
    }
    if (s != WRK_OK) {
        delete m;
        return s;
    }
    *out = m;
    return WRK_OK;
}

int32_t wrk_model_info_get(const wrk_model* m, wrk_model_info* info) {
    WRK_REQUIRE(m && info, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *info = m->info;
    return WRK_OK;
}

int32_t wrk_model_retain(wrk_model* m) {
    WRK_REQUIRE(m, WRK_ERR_INVALID_ARGUMENT, "null argument");
    m->refs.fetch_add(1);
    return WRK_OK;
}

int32_t wrk_model_release(wrk_model* m) {
    if (!m) return WRK_OK;
    if (m->refs.fetch_sub(1) == 1) delete m;
    return WRK_OK;
}

int32_t wrk_model_matrix(wrk_model* m, uint32_t layer, const char* name, wrk_matrix** out) {
    WRK_REQUIRE(m && name && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    const std::string n = name;
    if (n == "head.w") {
        *out = m->head_w;
        return WRK_OK;
    }
    WRK_REQUIRE(layer < m->layers.size(), WRK_ERR_INVALID_ARGUMENT, "layer %u out of range", layer);
    Layer& L = m->layers[layer];
    wrk_matrix* r = nullptr;
    if (n == "att.w_k") r = L.att_w_k;
    else if (n == "att.w_v") r = L.att_w_v;
    else if (n == "att.w_r") r = L.att_w_r;
    else if (n == "att.w_g") r = L.att_w_g;
    else if (n == "att.w_o") r = L.att_w_o;
    else if (n == "ffn.w_k") r = L.ffn_w_k;
    else if (n == "ffn.w_v") r = L.ffn_w_v;
    else if (n == "ffn.w_r") r = L.ffn_w_r;
    WRK_REQUIRE(r, WRK_ERR_INVALID_ARGUMENT, "no matrix %s in layer %u", name, layer);
    *out = r;
    return WRK_OK;
}

}  // extern "C"
