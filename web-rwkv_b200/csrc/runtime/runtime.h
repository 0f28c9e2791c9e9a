// Internal structures of the run() job runtime (model, bundle, scheduling).
#pragma once

#include <algorithm>
#include <map>
#include <regex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../../include/wrk_runtime.h"
#include "../common.h"

namespace wrk {
namespace rt {

struct RnnInfo {
    std::vector<uint32_t> lens;
    std::vector<int32_t> options;  // wrk_rnn_option; WRK_RNN_NONE = None
    uint32_t num_token() const {
        uint32_t n = 0;
        for (auto l : lens) n += l;
        return n;
    }
};

struct RnnRedirect {
    std::vector<uint32_t> headers;
    std::vector<std::pair<uint32_t, uint32_t>> inputs, outputs;
};

struct RnnIter {
    struct Batch {
        bool gen;      // BatchState::Gen
        size_t read;   // BatchState::Read(n)
        int32_t option;
    };
    std::vector<Batch> batches;
    size_t token_chunk_size = 0;
    RnnInfo next();
};

RnnRedirect redirect(const RnnInfo& info);

// RAII handles over the C objects.
struct TensorH {
    wrk_tensor* p = nullptr;
    TensorH() = default;
    explicit TensorH(wrk_tensor* t) : p(t) {}
    TensorH(const TensorH& o) : p(o.p) { if (p) wrk_tensor_retain(p); }
    TensorH(TensorH&& o) noexcept : p(o.p) { o.p = nullptr; }
    TensorH& operator=(TensorH o) { std::swap(p, o.p); return *this; }
    ~TensorH() { if (p) wrk_tensor_release(p); }
    operator wrk_tensor*() const { return p; }
};

struct MatrixH {
    wrk_matrix* p = nullptr;
    MatrixH() = default;
    explicit MatrixH(wrk_matrix* m) : p(m) {}
    MatrixH(const MatrixH& o) : p(o.p) { if (p) p->refs.fetch_add(1); }
    MatrixH(MatrixH&& o) noexcept : p(o.p) { o.p = nullptr; }
    MatrixH& operator=(MatrixH o) { std::swap(p, o.p); return *this; }
    ~MatrixH() { if (p) wrk_matrix_release(p); }
    operator wrk_matrix*() const { return p; }
};

struct LayerNorm { TensorH w, b; };

// Union of the v5 / v6 / v7 layer tensors (src/runtime/v5.rs:68-118, v6.rs:77-118, v7.rs:77-133).
struct Layer {
    LayerNorm att_ln, ffn_ln, gn;
    // v5 / v6
    TensorH time_decay, time_first;              // v5: f32 exp(-exp(.)) [C]; v6: f16 [C] (added per token)
    TensorH time_mix_x, time_mix;                // v6: [C] and [C, 1, 5]
    TensorH time_mix_k, time_mix_v, time_mix_r, time_mix_g;  // v5 att
    MatrixH time_decay_w1, time_decay_w2, time_mix_w1, time_mix_w2;  // v6 adapters
    MatrixH att_w_k, att_w_v, att_w_r, att_w_g, att_w_o;
    TensorH ffn_time_mix_k, ffn_time_mix_r;
    MatrixH ffn_w_k, ffn_w_v, ffn_w_r;
    // v7
    TensorH x_r, x_w, x_k, x_v, x_a, x_g, w0, a0, v0, r_k, k_k, k_a, ffn_x_k;
    MatrixH w1, w2, a1, a2, g1, g2, v1, v2;
};

}  // namespace rt
}  // namespace wrk

struct wrk_rnn_input {
    struct Batch {
        std::vector<uint32_t> tokens;
        int32_t option = WRK_RNN_LAST;
    };
    std::vector<Batch> batches;
    size_t token_chunk_size = 128;
};

struct wrk_rnn_iter {
    wrk::rt::RnnIter it;
};

namespace wrk {
namespace rt {
RnnIter make_iter(const wrk_rnn_input& in);
}
}  // namespace wrk

namespace wrk {
namespace rt {
// One rank's part of a model split across GPUs: time-mix channels [c0, c1) (whole heads), FFN columns [f0, f1)
// and vocabulary rows [v0, v1); world == 1 means the whole model.
struct Shard {
    uint32_t rank = 0, world = 1;
    uint32_t c0 = 0, c1 = 0, f0 = 0, f1 = 0, v0 = 0, v1 = 0;
    bool on() const { return world > 1; }
};
// `world` contiguous ranges over `total`, each a whole number of `align`-sized units, sizes differing by at most
// one unit (larger ranges first).
int32_t shard_range(const char* what, uint32_t total, uint32_t align, uint32_t world, uint32_t rank, uint32_t* begin, uint32_t* end);
}  // namespace rt
}  // namespace wrk

struct wrk_model_builder {
    struct Entry {
        std::vector<uint64_t> shape;  // outermost first
        std::vector<uint16_t> data;   // fp16 bits
        std::vector<uint64_t> full;   // shape before the rank's slice was cut (empty: not sliced)
    };
    // sharded build: set before the first tensor is added; every tensor is cut to the rank's slice as it arrives
    uint32_t shard_rank = 0, shard_world = 1, shard_head_size = 64, shard_block = 1;
    // `Lora` of src/runtime/loader.rs:104-113: named fp16 tensors and an ordered list of (pattern, alpha)
    struct Lora {
        std::map<std::string, Entry> tensors;
        std::vector<std::pair<std::regex, float>> blend;
    };
    wrk_context* ctx = nullptr;
    std::map<std::string, Entry> tensors;
    std::vector<Lora> loras;
    std::unordered_map<uint32_t, int32_t> quant;
    size_t rescale = 0;  // 0 = default of the version
    size_t sep = 0;
    bool rescale_set = false;
};

struct wrk_model {
    std::atomic<int> refs{1};
    wrk_context* ctx = nullptr;
    wrk_model_info info{};
    size_t rescale = 6;
    size_t sep = 1024;
    uint32_t num_vocab_padded = 0;
    wrk::rt::Shard shard;  // info keeps the dimensions of the whole model
    wrk::rt::LayerNorm embed_ln, head_ln;
    uint16_t* embed_host = nullptr;  // pinned [num_vocab_padded][num_emb] fp16 (the reference keeps it on the CPU)
    wrk::rt::MatrixH head_w;
    std::vector<wrk::rt::Layer> layers;
    ~wrk_model();
};
