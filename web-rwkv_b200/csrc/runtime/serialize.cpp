// Quantized-model (de)serialization: the built model (packed weights, block scales, code tables, vectors) written
// to and restored from one file, so that a model is quantized once.
//
// The reference serializes its `Model` struct with serde: every tensor becomes a `TensorBlob {shape, data}` read
// back from the GPU (src/tensor/serialization.rs:11-75), a model is restored through `Seed<Context, _>`
// (src/tensor/serialization.rs:96-159), and examples/serde.rs:218-268 round-trips the result through CBOR.  This
// file writes the same tree in the same encoding: structs as CBOR maps keyed by the reference's field names in
// declaration order (src/runtime/v5.rs:60-125, v6.rs:28-130, v7.rs:55-150), `Shape` as an array of four integers,
// tensor bytes as one byte string, `Matrix` as its externally tagged variants `Fp16`, `Int8 {w, m}` and
// `Fp4 {q, w, m}` (src/tensor/matrix.rs:82-94), unit values (`Context`) as null.  The reader walks the tree by key,
// so the order of fields in a file does not matter to it.
#include <sys/mman.h>
#include <sys/stat.h>

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <memory>
#include <unistd.h>

#include "runtime.h"

using namespace wrk;
using namespace wrk::rt;

namespace {

// ---- CBOR (RFC 8949), the subset serde emits for this tree: unsigned integers, byte and text strings, arrays,
// maps, null ----
enum Major : uint8_t { kUint = 0, kBytes = 2, kText = 3, kArray = 4, kMap = 5, kSimple = 7 };

struct Writer {
    FILE* f = nullptr;
    bool failed = false;
    void raw(const void* p, size_t n) {
        if (n && std::fwrite(p, 1, n, f) != n) failed = true;
    }
    void head(Major major, uint64_t v) {
        uint8_t b[9];
        size_t n;
        const uint8_t m = (uint8_t)(major << 5);
        if (v < 24) {
            b[0] = m | (uint8_t)v;
            n = 1;
        } else if (v <= 0xff) {
            b[0] = m | 24;
            b[1] = (uint8_t)v;
            n = 2;
        } else if (v <= 0xffff) {
            b[0] = m | 25;
            b[1] = (uint8_t)(v >> 8);
            b[2] = (uint8_t)v;
            n = 3;
        } else if (v <= 0xffffffffull) {
            b[0] = m | 26;
            for (int i = 0; i < 4; ++i) b[1 + i] = (uint8_t)(v >> (24 - 8 * i));
            n = 5;
        } else {
            b[0] = m | 27;
            for (int i = 0; i < 8; ++i) b[1 + i] = (uint8_t)(v >> (56 - 8 * i));
            n = 9;
        }
        raw(b, n);
    }
    void text(const char* s) {
        const size_t n = std::strlen(s);
        head(kText, n);
        raw(s, n);
    }
    void null() {
        const uint8_t b = 0xf6;
        raw(&b, 1);
    }
};

struct Node {
    Major major = kSimple;
    uint64_t value = 0;           // kUint: the integer; kSimple: the simple value (22 = null)
    const uint8_t* data = nullptr;  // kBytes / kText
    size_t len = 0;
    std::vector<Node> items;  // kArray: elements; kMap: key, value, key, value, ...
    const Node* find(const char* key) const {
        if (major != kMap) return nullptr;
        const size_t n = std::strlen(key);
        for (size_t i = 0; i + 1 < items.size(); i += 2)
            if (items[i].major == kText && items[i].len == n && std::memcmp(items[i].data, key, n) == 0) return &items[i + 1];
        return nullptr;
    }
};

struct Parser {
    const uint8_t* p;
    const uint8_t* end;
    int depth = 0;
    bool parse(Node* out) {
        if (p >= end || depth > 16) return false;
        const uint8_t b = *p++;
        const uint8_t major = b >> 5, info = b & 31;
        uint64_t v = info;
        if (info >= 24 && info <= 27) {
            const int n = 1 << (info - 24);
            if (end - p < n) return false;
            v = 0;
            for (int i = 0; i < n; ++i) v = (v << 8) | *p++;
        } else if (info > 27) {
            return false;  // indefinite lengths and reserved values are never written
        }
        out->major = (Major)major;
        out->value = v;
        switch (major) {
            case kUint: return true;
            case kBytes:
            case kText:
                if ((uint64_t)(end - p) < v) return false;
                out->data = p;
                out->len = (size_t)v;
                p += v;
                return true;
            case kArray:
            case kMap: {
                const uint64_t n = major == kMap ? 2 * v : v;
                if (n > (uint64_t)(end - p)) return false;
                out->items.resize((size_t)n);
                ++depth;
                for (auto& item : out->items)
                    if (!parse(&item)) return false;
                --depth;
                return true;
            }
            case kSimple: return info == 22;  // null
            default: return false;            // negative integers, tags: not part of this tree
        }
    }
};

// ---- the model tree, written and read by the same description ----
struct Saver {
    Writer w;
    wrk_context* ctx;
    std::vector<uint8_t> bounce;
    int32_t map(const char* key, size_t fields) {
        if (key) w.text(key);
        w.head(kMap, fields);
        return WRK_OK;
    }
    int32_t end() { return WRK_OK; }
    int32_t blob(const uint32_t shape[4], const void* host, size_t bytes) {
        w.head(kMap, 2);
        w.text("shape");
        w.head(kArray, 4);
        for (int i = 0; i < 4; ++i) w.head(kUint, shape[i]);
        w.text("data");
        w.head(kBytes, bytes);
        w.raw(host, bytes);
        return w.failed ? WRK_ERR_INVALID_ARGUMENT : WRK_OK;
    }
    int32_t tensor(const char* key, TensorH& t) {
        WRK_REQUIRE(t.p, WRK_ERR_INVALID_ARGUMENT, "model field %s is empty", key);
        if (key) w.text(key);
        bounce.resize(t.p->bytes());
        WRK_CUDA(cudaMemcpyAsync(bounce.data(), t.p->ptr(), bounce.size(), cudaMemcpyDeviceToHost, ctx->stream));
        WRK_CUDA(cudaStreamSynchronize(ctx->stream));
        return blob(t.p->shape.v, bounce.data(), bounce.size());
    }
    int32_t matrix(const char* key, MatrixH& m) {
        WRK_REQUIRE(m.p, WRK_ERR_INVALID_ARGUMENT, "model field %s is empty", key);
        if (key) w.text(key);
        TensorH tw(m.p->w), tm(m.p->m), tq(m.p->q);
        for (wrk_tensor* t : {m.p->w, m.p->m, m.p->q})
            if (t) wrk_tensor_retain(t);
        w.head(kMap, 1);
        if (m.p->kind == 0) {
            WRK_TRY(tensor("Fp16", tw));
        } else if (m.p->kind == 1) {
            w.text("Int8");
            w.head(kMap, 2);
            WRK_TRY(tensor("w", tw));
            WRK_TRY(tensor("m", tm));
        } else {
            w.text("Fp4");
            w.head(kMap, 3);
            WRK_TRY(tensor("q", tq));
            WRK_TRY(tensor("w", tw));
            WRK_TRY(tensor("m", tm));
        }
        return WRK_OK;
    }
    int32_t host_f16(const char* key, uint16_t*& host, uint32_t x, uint32_t y) {
        w.text(key);
        const uint32_t shape[4] = {x, y, 1, 1};
        return blob(shape, host, (size_t)x * y * 2);
    }
    int32_t uint(const char* key, uint64_t& v) {
        w.text(key);
        w.head(kUint, v);
        return WRK_OK;
    }
    int32_t variant(const char* key, const char* const* names, size_t count, uint32_t& index) {
        w.text(key);
        WRK_REQUIRE(index < count, WRK_ERR_INVALID_ARGUMENT, "%s: no variant %u", key, index);
        w.text(names[index]);
        return WRK_OK;
    }
    int32_t unit(const char* key) {
        w.text(key);
        w.null();
        return WRK_OK;
    }
    int32_t array(const char* key, size_t& count) {
        w.text(key);
        w.head(kArray, count);
        return WRK_OK;
    }
    int32_t custom(wrk_model_info& info);
};

struct Restorer {
    wrk_context* ctx;
    std::vector<const Node*> stack;
    std::vector<size_t> cursor;  // next element of the array on top of the stack
    const Node* child(const char* key) {
        const Node* top = stack.back();
        if (key) return top->find(key);
        if (top->major != kArray || cursor.back() >= top->items.size()) return nullptr;
        return &top->items[cursor.back()++];
    }
    int32_t map(const char* key, size_t) {
        const Node* n = child(key);
        WRK_REQUIRE(n && n->major == kMap, WRK_ERR_INVALID_ARGUMENT, "serialized model: no map %s", key ? key : "(element)");
        stack.push_back(n);
        cursor.push_back(0);
        return WRK_OK;
    }
    int32_t end() {
        stack.pop_back();
        cursor.pop_back();
        return WRK_OK;
    }
    static int32_t blob(const Node* n, const char* key, uint32_t shape[4], const Node** data) {
        const Node* s = n && n->major == kMap ? n->find("shape") : nullptr;
        const Node* d = n && n->major == kMap ? n->find("data") : nullptr;
        WRK_REQUIRE(s && d && s->major == kArray && s->items.size() == 4 && d->major == kBytes, WRK_ERR_INVALID_ARGUMENT,
                    "serialized model: %s is not a tensor", key);
        for (int i = 0; i < 4; ++i) {
            WRK_REQUIRE(s->items[i].major == kUint && s->items[i].value >= 1 && s->items[i].value <= 0xffffffffull,
                        WRK_ERR_SHAPE, "serialized model: shape of %s", key);
            shape[i] = (uint32_t)s->items[i].value;
        }
        *data = d;
        return WRK_OK;
    }
    int32_t tensor_of(const Node* n, const char* key, int dtype, TensorH& t) {
        uint32_t shape[4];
        const Node* d;
        WRK_TRY(blob(n, key, shape, &d));
        const size_t len = (size_t)shape[0] * shape[1] * shape[2] * shape[3];
        WRK_REQUIRE(d->len == len * dtype_size(dtype), WRK_ERR_SHAPE, "serialized model: %s holds %zu bytes for %zu elements of %zu",
                    key, d->len, len, dtype_size(dtype));
        wrk_tensor* out = nullptr;
        WRK_TRY(tensor_alloc(ctx, dtype, shape, false, &out));
        t = TensorH(out);
        WRK_CUDA(cudaMemcpyAsync(out->ptr(), d->data, d->len, cudaMemcpyHostToDevice, ctx->stream));
        return WRK_OK;
    }
    // dtype of a field: what the reference's struct declares for it
    int32_t tensor(const char* key, TensorH& t, int dtype = WRK_F16) { return tensor_of(child(key), key, dtype, t); }
    int32_t matrix(const char* key, MatrixH& m) {
        const Node* n = child(key);
        WRK_REQUIRE(n && n->major == kMap && n->items.size() == 2, WRK_ERR_INVALID_ARGUMENT, "serialized model: no matrix %s", key);
        auto out = std::unique_ptr<wrk_matrix>(new wrk_matrix());
        TensorH w, s, q;
        const Node* body = &n->items[1];
        if (n->find("Fp16")) {
            out->kind = 0;
            WRK_TRY(tensor_of(body, key, WRK_F16, w));
        } else if (n->find("Int8")) {
            out->kind = 1;
            WRK_REQUIRE(body->major == kMap, WRK_ERR_INVALID_ARGUMENT, "serialized model: matrix %s", key);
            WRK_TRY(tensor_of(body->find("w"), key, WRK_U8, w));
            WRK_TRY(tensor_of(body->find("m"), key, WRK_F16, s));
        } else if (n->find("Fp4") || n->find("Nf4")) {  // `Nf4` is the variant's older name (src/tensor/matrix.rs:88)
            out->kind = 2;
            WRK_REQUIRE(body->major == kMap, WRK_ERR_INVALID_ARGUMENT, "serialized model: matrix %s", key);
            WRK_TRY(tensor_of(body->find("q"), key, WRK_F32, q));
            WRK_TRY(tensor_of(body->find("w"), key, WRK_U8, w));
            WRK_TRY(tensor_of(body->find("m"), key, WRK_F16, s));
        } else {
            WRK_REQUIRE(false, WRK_ERR_INVALID_ARGUMENT, "serialized model: matrix %s has an unknown variant", key);
        }
        for (wrk_tensor* t : {w.p, s.p, q.p})
            if (t) wrk_tensor_retain(t);
        out->w = w.p;
        out->m = s.p;
        out->q = q.p;
        m = MatrixH(out.release());
        return WRK_OK;
    }
    int32_t host_f16(const char* key, uint16_t*& host, uint32_t x, uint32_t y) {
        uint32_t shape[4];
        const Node* d;
        WRK_TRY(blob(child(key), key, shape, &d));
        WRK_REQUIRE(shape[0] == x && shape[1] == y && shape[2] == 1 && shape[3] == 1 && d->len == (size_t)x * y * 2, WRK_ERR_SHAPE,
                    "serialized model: %s is [%u, %u], the model needs [%u, %u]", key, shape[0], shape[1], x, y);
        WRK_CUDA(cudaMallocHost(&host, d->len));
        std::memcpy(host, d->data, d->len);
        return WRK_OK;
    }
    int32_t uint(const char* key, uint64_t& v) {
        const Node* n = child(key);
        WRK_REQUIRE(n && n->major == kUint, WRK_ERR_INVALID_ARGUMENT, "serialized model: no integer %s", key);
        v = n->value;
        return WRK_OK;
    }
    int32_t variant(const char* key, const char* const* names, size_t count, uint32_t& index) {
        const Node* n = child(key);
        WRK_REQUIRE(n && n->major == kText, WRK_ERR_INVALID_ARGUMENT, "serialized model: no variant %s", key);
        for (size_t i = 0; i < count; ++i)
            if (std::strlen(names[i]) == n->len && std::memcmp(names[i], n->data, n->len) == 0) {
                index = (uint32_t)i;
                return WRK_OK;
            }
        WRK_REQUIRE(false, WRK_ERR_INVALID_ARGUMENT, "serialized model: unknown variant of %s", key);
    }
    int32_t unit(const char*) { return WRK_OK; }
    int32_t array(const char* key, size_t& count) {
        const Node* n = child(key);
        WRK_REQUIRE(n && n->major == kArray, WRK_ERR_INVALID_ARGUMENT, "serialized model: no array %s", key);
        count = n->items.size();
        stack.push_back(n);
        cursor.push_back(0);
        return WRK_OK;
    }
    int32_t custom(wrk_model_info& info);
};

// Saver::tensor takes no dtype (the tensor knows its own); the walk passes one for the reader
struct SaverAdapter : Saver {
    int32_t tensor(const char* key, TensorH& t, int = WRK_F16) { return Saver::tensor(key, t); }
};

// `ModelCustomInfo` (src/runtime/model.rs:65-72): None | V6 {time_mix, time_decay} | V7 {w, a, g, v}
int32_t Saver::custom(wrk_model_info& info) {
    w.text("custom");
    if (info.version == 6) {
        w.head(kMap, 1);
        w.text("V6");
        w.head(kMap, 2);
        w.text("time_mix");
        w.head(kUint, info.custom[0]);
        w.text("time_decay");
        w.head(kUint, info.custom[1]);
    } else if (info.version == 7) {
        static const char* names[4] = {"w", "a", "g", "v"};
        w.head(kMap, 1);
        w.text("V7");
        w.head(kMap, 4);
        for (int i = 0; i < 4; ++i) {
            w.text(names[i]);
            w.head(kUint, info.custom[i]);
        }
    } else {
        w.text("None");
    }
    return WRK_OK;
}

int32_t Restorer::custom(wrk_model_info& info) {
    const Node* n = child("custom");
    WRK_REQUIRE(n, WRK_ERR_INVALID_ARGUMENT, "serialized model: no custom info");
    std::memset(info.custom, 0, sizeof(info.custom));
    if (n->major == kText) return WRK_OK;  // None
    const Node* v6 = n->find("V6");
    const Node* v7 = n->find("V7");
    auto field = [&](const Node* m, const char* key, uint32_t* out) -> int32_t {
        const Node* f = m->find(key);
        WRK_REQUIRE(f && f->major == kUint, WRK_ERR_INVALID_ARGUMENT, "serialized model: custom info field %s", key);
        *out = (uint32_t)f->value;
        return WRK_OK;
    };
    if (v6) {
        WRK_TRY(field(v6, "time_mix", &info.custom[0]));
        WRK_TRY(field(v6, "time_decay", &info.custom[1]));
    } else if (v7) {
        static const char* names[4] = {"w", "a", "g", "v"};
        for (int i = 0; i < 4; ++i) WRK_TRY(field(v7, names[i], &info.custom[i]));
    } else {
        WRK_REQUIRE(false, WRK_ERR_INVALID_ARGUMENT, "serialized model: unknown custom info");
    }
    return WRK_OK;
}

template <class V>
int32_t walk_layer_norm(V& v, const char* key, LayerNorm& ln) {
    WRK_TRY(v.map(key, 2));
    WRK_TRY(v.tensor("w", ln.w));
    WRK_TRY(v.tensor("b", ln.b));
    return v.end();
}

// `Layer` of v4 (src/runtime/v4.rs:67-103)
template <class V>
int32_t walk_layer_v4(V& v, Layer& L) {
    WRK_TRY(v.map(nullptr, 4));
    WRK_TRY(walk_layer_norm(v, "att_layer_norm", L.att_ln));
    WRK_TRY(walk_layer_norm(v, "ffn_layer_norm", L.ffn_ln));
    WRK_TRY(v.map("att", 9));
    WRK_TRY(v.tensor("time_decay", L.time_decay, WRK_F32));
    WRK_TRY(v.tensor("time_first", L.time_first, WRK_F32));
    WRK_TRY(v.tensor("time_mix_k", L.time_mix_k));
    WRK_TRY(v.tensor("time_mix_v", L.time_mix_v));
    WRK_TRY(v.tensor("time_mix_r", L.time_mix_r));
    WRK_TRY(v.matrix("w_k", L.att_w_k));
    WRK_TRY(v.matrix("w_v", L.att_w_v));
    WRK_TRY(v.matrix("w_r", L.att_w_r));
    WRK_TRY(v.matrix("w_o", L.att_w_o));
    WRK_TRY(v.end());
    WRK_TRY(v.map("ffn", 5));
    WRK_TRY(v.tensor("time_mix_k", L.ffn_time_mix_k));
    WRK_TRY(v.tensor("time_mix_r", L.ffn_time_mix_r));
    WRK_TRY(v.matrix("w_k", L.ffn_w_k));
    WRK_TRY(v.matrix("w_v", L.ffn_w_v));
    WRK_TRY(v.matrix("w_r", L.ffn_w_r));
    WRK_TRY(v.end());
    return v.end();
}

// `Layer` of v5 (src/runtime/v5.rs:68-118) and v6 (src/runtime/v6.rs:77-118)
template <class V>
int32_t walk_layer_v56(V& v, uint32_t version, Layer& L) {
    WRK_TRY(v.map(nullptr, 4));
    WRK_TRY(walk_layer_norm(v, "att_layer_norm", L.att_ln));
    WRK_TRY(walk_layer_norm(v, "ffn_layer_norm", L.ffn_ln));
    WRK_TRY(v.map("att", version == 5 ? 12 : 14));
    if (version == 5) {
        WRK_TRY(v.tensor("time_decay", L.time_decay, WRK_F32));
        WRK_TRY(v.tensor("time_first", L.time_first, WRK_F32));
        WRK_TRY(v.tensor("time_mix_k", L.time_mix_k));
        WRK_TRY(v.tensor("time_mix_v", L.time_mix_v));
        WRK_TRY(v.tensor("time_mix_r", L.time_mix_r));
        WRK_TRY(v.tensor("time_mix_g", L.time_mix_g));
    } else {
        WRK_TRY(v.tensor("time_decay", L.time_decay));
        WRK_TRY(v.tensor("time_first", L.time_first, WRK_F32));
        WRK_TRY(v.tensor("time_mix_x", L.time_mix_x));
        WRK_TRY(v.tensor("time_mix", L.time_mix));
        WRK_TRY(v.matrix("time_decay_w1", L.time_decay_w1));
        WRK_TRY(v.matrix("time_decay_w2", L.time_decay_w2));
        WRK_TRY(v.matrix("time_mix_w1", L.time_mix_w1));
        WRK_TRY(v.matrix("time_mix_w2", L.time_mix_w2));
    }
    WRK_TRY(v.matrix("w_k", L.att_w_k));
    WRK_TRY(v.matrix("w_v", L.att_w_v));
    WRK_TRY(v.matrix("w_r", L.att_w_r));
    WRK_TRY(v.matrix("w_g", L.att_w_g));
    WRK_TRY(v.matrix("w_o", L.att_w_o));
    WRK_TRY(walk_layer_norm(v, "group_norm", L.gn));
    WRK_TRY(v.end());
    WRK_TRY(v.map("ffn", 5));
    WRK_TRY(v.tensor("time_mix_k", L.ffn_time_mix_k));
    WRK_TRY(v.tensor("time_mix_r", L.ffn_time_mix_r));
    WRK_TRY(v.matrix("w_k", L.ffn_w_k));
    WRK_TRY(v.matrix("w_v", L.ffn_w_v));
    WRK_TRY(v.matrix("w_r", L.ffn_w_r));
    WRK_TRY(v.end());
    return v.end();
}

// `Layer` of v7 (src/runtime/v7.rs:77-133)
template <class V>
int32_t walk_layer_v7(V& v, Layer& L) {
    WRK_TRY(v.map(nullptr, 4));
    WRK_TRY(walk_layer_norm(v, "att_ln", L.att_ln));
    WRK_TRY(walk_layer_norm(v, "ffn_ln", L.ffn_ln));
    WRK_TRY(v.map("att", 25));
    WRK_TRY(v.tensor("x_r", L.x_r));
    WRK_TRY(v.tensor("x_w", L.x_w));
    WRK_TRY(v.tensor("x_k", L.x_k));
    WRK_TRY(v.tensor("x_v", L.x_v));
    WRK_TRY(v.tensor("x_a", L.x_a));
    WRK_TRY(v.tensor("x_g", L.x_g));
    WRK_TRY(v.tensor("w0", L.w0));
    WRK_TRY(v.tensor("a0", L.a0));
    WRK_TRY(v.tensor("v0", L.v0));
    WRK_TRY(v.matrix("w1", L.w1));
    WRK_TRY(v.matrix("w2", L.w2));
    WRK_TRY(v.matrix("a1", L.a1));
    WRK_TRY(v.matrix("a2", L.a2));
    WRK_TRY(v.matrix("g1", L.g1));
    WRK_TRY(v.matrix("g2", L.g2));
    WRK_TRY(v.matrix("v1", L.v1));
    WRK_TRY(v.matrix("v2", L.v2));
    WRK_TRY(v.tensor("r_k", L.r_k));
    WRK_TRY(v.tensor("k_k", L.k_k));
    WRK_TRY(v.tensor("k_a", L.k_a));
    WRK_TRY(v.matrix("w_k", L.att_w_k));
    WRK_TRY(v.matrix("w_v", L.att_w_v));
    WRK_TRY(v.matrix("w_r", L.att_w_r));
    WRK_TRY(v.matrix("w_o", L.att_w_o));
    WRK_TRY(walk_layer_norm(v, "gn", L.gn));
    WRK_TRY(v.end());
    WRK_TRY(v.map("ffn", 3));
    WRK_TRY(v.tensor("x_k", L.ffn_x_k));
    WRK_TRY(v.matrix("w_k", L.ffn_w_k));
    WRK_TRY(v.matrix("w_v", L.ffn_w_v));
    WRK_TRY(v.end());
    return v.end();
}

// `Model` (src/runtime/v6.rs:36-43 and the same struct in v5.rs / v7.rs)
template <class V>
int32_t walk_model(V& v, wrk_model* m, bool restoring) {
    static const char* versions[4] = {"V4", "V5", "V6", "V7"};
    wrk_model_info& info = m->info;
    WRK_TRY(v.map(nullptr, 5));
    WRK_TRY(v.unit("context"));
    WRK_TRY(v.map("info", 7));
    uint32_t version = info.version - 4;
    WRK_TRY(v.variant("version", versions, 4, version));
    info.version = version + 4;
    uint64_t fields[5] = {info.num_layer, info.num_emb, info.num_hidden, info.num_vocab, info.num_head};
    static const char* names[5] = {"num_layer", "num_emb", "num_hidden", "num_vocab", "num_head"};
    for (int i = 0; i < 5; ++i) {
        WRK_TRY(v.uint(names[i], fields[i]));
        WRK_REQUIRE(fields[i] >= 1 && fields[i] <= 0xffffffffull, WRK_ERR_INVALID_ARGUMENT, "serialized model: %s", names[i]);
    }
    info.num_layer = (uint32_t)fields[0];
    info.num_emb = (uint32_t)fields[1];
    info.num_hidden = (uint32_t)fields[2];
    info.num_vocab = (uint32_t)fields[3];
    info.num_head = (uint32_t)fields[4];
    WRK_TRY(v.custom(info));
    WRK_TRY(v.end());
    uint64_t rescale = m->rescale, sep = m->sep;
    WRK_TRY(v.uint("rescale", rescale));
    WRK_TRY(v.uint("sep", sep));
    m->rescale = (size_t)rescale;
    m->sep = (size_t)sep;
    WRK_REQUIRE(m->rescale >= 1 && info.num_emb % info.num_head == 0, WRK_ERR_INVALID_ARGUMENT, "serialized model: model info");
    const bool v7 = info.version == 7;
    WRK_TRY(v.map("tensor", 3));
    WRK_TRY(v.map("embed", 2));
    WRK_TRY(walk_layer_norm(v, v7 ? "ln" : "layer_norm", m->embed_ln));
    m->num_vocab_padded = (info.num_vocab + 7) / 8 * 8;  // load_matrix_f16_padded_cpu in every version
    WRK_TRY(v.host_f16("w", m->embed_host, info.num_emb, m->num_vocab_padded));
    WRK_TRY(v.end());
    WRK_TRY(v.map("head", 2));
    WRK_TRY(walk_layer_norm(v, v7 ? "ln" : "layer_norm", m->head_ln));
    WRK_TRY(v.matrix("w", m->head_w));
    WRK_TRY(v.end());
    size_t count = m->layers.size();
    WRK_TRY(v.array("layers", count));
    if (restoring) {
        WRK_REQUIRE(count == info.num_layer, WRK_ERR_INVALID_ARGUMENT, "serialized model: %zu layers, info says %u", count, info.num_layer);
        m->layers.resize(count);
    }
    for (auto& L : m->layers) WRK_TRY(v7 ? walk_layer_v7(v, L) : info.version == 4 ? walk_layer_v4(v, L) : walk_layer_v56(v, info.version, L));
    if (restoring) WRK_TRY(v.end());
    WRK_TRY(v.end());
    return v.end();
}

}  // namespace

extern "C" {

int32_t wrk_model_save(wrk_model* m, const char* path) {
    WRK_REQUIRE(m && path, WRK_ERR_INVALID_ARGUMENT, "null argument");
    SaverAdapter s;
    s.ctx = m->ctx;
    s.w.f = std::fopen(path, "wb");
    WRK_REQUIRE(s.w.f, WRK_ERR_INVALID_ARGUMENT, "cannot open %s for writing: %s", path, std::strerror(errno));
    std::vector<char> buffer(8u << 20);
    std::setvbuf(s.w.f, buffer.data(), _IOFBF, buffer.size());
    int32_t status = walk_model(s, m, false);
    if (std::fclose(s.w.f) != 0 || s.w.failed) {
        if (status == WRK_OK) {
            status = wrk::set_error(WRK_ERR_INVALID_ARGUMENT, "writing %s failed: %s", path, std::strerror(errno));
        }
    }
    if (status != WRK_OK) std::remove(path);
    return status;
}

int32_t wrk_model_load(wrk_context* ctx, const char* path, wrk_model** out) {
    WRK_REQUIRE(ctx && path && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    const int fd = ::open(path, O_RDONLY);
    WRK_REQUIRE(fd >= 0, WRK_ERR_INVALID_ARGUMENT, "cannot open %s: %s", path, std::strerror(errno));
    struct stat st {};
    void* map = MAP_FAILED;
    if (::fstat(fd, &st) == 0 && st.st_size > 0) map = ::mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    WRK_REQUIRE(map != MAP_FAILED, WRK_ERR_INVALID_ARGUMENT, "cannot map %s", path);
    const size_t size = (size_t)st.st_size;
    int32_t status = WRK_OK;
    auto m = new wrk_model();
    m->ctx = ctx;
    {
        Node root;
        Parser parser{static_cast<const uint8_t*>(map), static_cast<const uint8_t*>(map) + size};
        if (!parser.parse(&root) || parser.p != parser.end) {
            status = wrk::set_error(WRK_ERR_INVALID_ARGUMENT, "%s is not a serialized model (malformed at byte %zu of %zu)", path,
                                    (size_t)(parser.p - static_cast<const uint8_t*>(map)), size);
        } else {
            Node holder;  // the walk opens the root as an array element
            holder.major = kArray;
            holder.items.push_back(std::move(root));
            Restorer r;
            r.ctx = ctx;
            r.stack.push_back(&holder);
            r.cursor.push_back(0);
            status = walk_model(r, m, true);
        }
    }
    // the copies read the mapping: they have to land before it goes
    const cudaError_t sync = cudaStreamSynchronize(ctx->stream);
    ::munmap(map, size);
    if (status == WRK_OK && sync != cudaSuccess) {
        status = wrk::set_error(WRK_ERR_CUDA, "cudaStreamSynchronize failed: %s", cudaGetErrorString(sync));
    }
    if (status != WRK_OK) {
        delete m;
        return status;
    }
    *out = m;
    return WRK_OK;
}

}  // extern "C"
