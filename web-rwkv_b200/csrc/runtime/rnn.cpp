// Token scheduling of the run() jobs: RnnInput, RnnIter, RnnInfo::redirect.
// Pure host logic restated from src/runtime/infer/rnn.rs (token_chunk_size / num_batch semantics).
#include "runtime.h"

using namespace wrk;

namespace wrk {
namespace rt {

// RnnIter::next, src/runtime/infer/rnn.rs:283-334.
// The job takes min(sum of remaining, token_chunk_size) tokens, rounded down to a multiple of 32 when
// above 32, and hands them out greedily: repeatedly every non-empty batch receives
// min(shortest remaining batch, budget left), in batch order.
RnnInfo RnnIter::next() {
    const size_t nb = batches.size();
    std::vector<size_t> remains(nb);
    for (size_t i = 0; i < nb; ++i) remains[i] = batches[i].gen ? 1 : batches[i].read;

    size_t num_token = 0;
    for (auto r : remains) num_token += r;
    num_token = std::min(num_token, token_chunk_size);
    if (num_token > WRK_MIN_TOKEN_CHUNK_SIZE) num_token -= num_token % WRK_MIN_TOKEN_CHUNK_SIZE;

    RnnInfo info;
    info.lens.assign(nb, 0);
    info.options.assign(nb, WRK_RNN_NONE);
    while (num_token > 0) {
        size_t mid = 0;
        bool any = false;
        for (auto r : remains)
            if (r > 0 && (!any || r < mid)) {
                mid = r;
                any = true;
            }
        if (!any) break;  // the reference would spin here; unreachable because num_token <= sum(remains)
        for (size_t i = 0; i < nb; ++i) {
            if (remains[i] == 0) continue;
            const size_t take = std::min(mid, num_token);
            num_token -= take;
            info.lens[i] += (uint32_t)take;
            remains[i] -= take;
        }
    }
    for (size_t i = 0; i < nb; ++i) {
        if (info.lens[i] > 0) {
            batches[i].gen = remains[i] == 0;
            batches[i].read = remains[i];
        }
        if (batches[i].option == WRK_RNN_FULL) info.options[i] = WRK_RNN_FULL;
        else info.options[i] = remains[i] == 0 ? WRK_RNN_LAST : WRK_RNN_NONE;
    }
    return info;
}

RnnIter make_iter(const wrk_rnn_input& in) {
    RnnIter it;
    it.token_chunk_size = in.token_chunk_size;
    for (auto& b : in.batches) it.batches.push_back({false, b.tokens.size(), b.option});
    return it;
}

// RnnInfo::redirect, src/runtime/infer/rnn.rs:41-81.
RnnRedirect redirect(const RnnInfo& info) {
    RnnRedirect r;
    const size_t nb = info.lens.size();
    r.inputs.assign(nb, {0, 0});
    r.outputs.assign(nb, {0, 0});
    uint32_t p_in = 0, p_out = 0;
    for (size_t b = 0; b < nb; ++b) {
        const uint32_t len = info.lens[b];
        r.inputs[b] = {p_in, p_in + len};
        switch (info.options[b]) {
            case WRK_RNN_LAST:
                if (len == 0) {
                    r.outputs[b] = {p_out, p_out};
                } else {
                    r.outputs[b] = {p_out, p_out + 1};
                    r.headers.push_back(p_in + len - 1);
                    p_out += 1;
                }
                break;
            case WRK_RNN_FULL:
                r.outputs[b] = {p_out, p_out + len};
                for (uint32_t i = 0; i < len; ++i) r.headers.push_back(p_in + i);
                p_out += len;
                break;
            default: r.outputs[b] = {p_out, p_out}; break;
        }
        p_in += len;
    }
    return r;
}

}  // namespace rt
}  // namespace wrk

extern "C" {

int32_t wrk_rnn_input_create(uint32_t num_batch, uint32_t token_chunk_size, wrk_rnn_input** out) {
    WRK_REQUIRE(out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    auto in = new wrk_rnn_input();
    in->batches.resize(num_batch);
    // RnnInput::new: at least 32, rounded up to a multiple of 32 (rnn.rs:204-208)
    size_t s = std::max<size_t>(token_chunk_size, WRK_MIN_TOKEN_CHUNK_SIZE);
    s = (s + WRK_MIN_TOKEN_CHUNK_SIZE - 1) / WRK_MIN_TOKEN_CHUNK_SIZE * WRK_MIN_TOKEN_CHUNK_SIZE;
    in->token_chunk_size = s;
    *out = in;
    return WRK_OK;
}

int32_t wrk_rnn_input_destroy(wrk_rnn_input* in) {
    delete in;
    return WRK_OK;
}

int32_t wrk_rnn_input_set_option(wrk_rnn_input* in, uint32_t batch, int32_t option) {
    WRK_REQUIRE(in, WRK_ERR_INVALID_ARGUMENT, "null argument");
    if (batch >= in->batches.size())
        return set_error(WRK_ERR_BATCH_OUT_OF_RANGE, "batch %u out of range of max %zu", batch, in->batches.size());
    WRK_REQUIRE(option == WRK_RNN_LAST || option == WRK_RNN_FULL, WRK_ERR_INVALID_ARGUMENT, "unknown option %d", option);
    in->batches[batch].option = option;
    return WRK_OK;
}

int32_t wrk_rnn_input_append(wrk_rnn_input* in, uint32_t batch, const uint32_t* tokens, size_t count) {
    WRK_REQUIRE(in && (tokens || count == 0), WRK_ERR_INVALID_ARGUMENT, "null argument");
    if (batch >= in->batches.size())
        return set_error(WRK_ERR_BATCH_OUT_OF_RANGE, "batch %u out of range of max %zu", batch, in->batches.size());
    auto& t = in->batches[batch].tokens;
    t.insert(t.end(), tokens, tokens + count);
    return WRK_OK;
}

int32_t wrk_rnn_input_token_chunk_size(const wrk_rnn_input* in, uint32_t* size) {
    WRK_REQUIRE(in && size, WRK_ERR_INVALID_ARGUMENT, "null argument");
    *size = (uint32_t)in->token_chunk_size;
    return WRK_OK;
}

int32_t wrk_rnn_input_num_token(const wrk_rnn_input* in, uint64_t* count) {
    WRK_REQUIRE(in && count, WRK_ERR_INVALID_ARGUMENT, "null argument");
    uint64_t n = 0;
    for (auto& b : in->batches) n += b.tokens.size();
    *count = n;
    return WRK_OK;
}

int32_t wrk_rnn_input_remaining(const wrk_rnn_input* in, uint32_t batch, uint64_t* count) {
    WRK_REQUIRE(in && count, WRK_ERR_INVALID_ARGUMENT, "null argument");
    if (batch >= in->batches.size())
        return set_error(WRK_ERR_BATCH_OUT_OF_RANGE, "batch %u out of range of max %zu", batch, in->batches.size());
    *count = in->batches[batch].tokens.size();
    return WRK_OK;
}

// JobInput::step, rnn.rs:233-240: drop the tokens the next job takes.
int32_t wrk_rnn_input_step(wrk_rnn_input* in) {
    WRK_REQUIRE(in, WRK_ERR_INVALID_ARGUMENT, "null argument");
    rt::RnnIter it = rt::make_iter(*in);
    rt::RnnInfo info = it.next();
    for (size_t b = 0; b < in->batches.size(); ++b) {
        auto& t = in->batches[b].tokens;
        t.erase(t.begin(), t.begin() + std::min<size_t>(info.lens[b], t.size()));
    }
    return WRK_OK;
}

int32_t wrk_rnn_iter_create(const wrk_rnn_input* in, wrk_rnn_iter** out) {
    WRK_REQUIRE(in && out, WRK_ERR_INVALID_ARGUMENT, "null argument");
    auto it = new wrk_rnn_iter();
    it->it = rt::make_iter(*in);
    *out = it;
    return WRK_OK;
}

int32_t wrk_rnn_iter_next(wrk_rnn_iter* it, uint32_t* lens, int32_t* options) {
    WRK_REQUIRE(it && lens && options, WRK_ERR_INVALID_ARGUMENT, "null argument");
    rt::RnnInfo info = it->it.next();
    for (size_t b = 0; b < info.lens.size(); ++b) {
        lens[b] = info.lens[b];
        options[b] = info.options[b];
    }
    return WRK_OK;
}

int32_t wrk_rnn_iter_destroy(wrk_rnn_iter* it) {
    delete it;
    return WRK_OK;
}

int32_t wrk_rnn_redirect(const uint32_t* lens, const int32_t* options, uint32_t num_batch, uint32_t* headers,
                         uint32_t* num_headers, uint32_t* inputs, uint32_t* outputs) {
    WRK_REQUIRE(lens && options && num_headers, WRK_ERR_INVALID_ARGUMENT, "null argument");
    rt::RnnInfo info;
    info.lens.assign(lens, lens + num_batch);
    info.options.assign(options, options + num_batch);
    rt::RnnRedirect r = rt::redirect(info);
    *num_headers = (uint32_t)r.headers.size();
    if (headers)
        for (size_t i = 0; i < r.headers.size(); ++i) headers[i] = r.headers[i];
    for (uint32_t b = 0; b < num_batch; ++b) {
        if (inputs) {
            inputs[2 * b] = r.inputs[b].first;
            inputs[2 * b + 1] = r.inputs[b].second;
        }
        if (outputs) {
            outputs[2 * b] = r.outputs[b].first;
            outputs[2 * b + 1] = r.outputs[b].second;
        }
    }
    return WRK_OK;
}

}  // extern "C"
