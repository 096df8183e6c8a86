// The token-level half of the reference's engine (crates/bobcat-cli/src/engine.rs): one sequence
// with the bookkeeping that lets a request reuse what earlier requests left on the device.
//  - generate (engine.rs:510-647): a request's tokens that extend what the sequence has consumed
//    continue from there; tokens that extend the recorded history of the conversation restore the
//    checkpoint taken at the last turn; anything else starts over. Greedy requests run the
//    pipelined generate_stream; sampled requests pick each token on the device (bc_seq_sample)
//    where the reference reads the logits back and samples on the host (engine.rs:615-630).
//  - score (engine.rs:372-446): log-probabilities of label tokens after each of several prompts,
//    the prompts' longest common prefix run once and every prompt continued from its checkpoint.
// Text (templates, tokenizer, tool calls, stop strings) stays with the caller: everything here is
// token ids in, token ids and numbers out.

#include <algorithm>
#include <cmath>
#include <memory>
#include <vector>

#include "seq.h"

using namespace bc;

struct bc_engine {
    bc_seq* seq = nullptr;       // owned
    uint32_t context = 0;
    std::vector<uint32_t> consumed;  // tokens the sequence's state holds (engine.rs `consumed`)
    std::vector<uint32_t> history;   // tokens up to the last turn start, with their checkpoint
    bc_checkpoint* checkpoint = nullptr;
    uint64_t rng = 0;            // state of the draw generator
    uint32_t last_cached = 0;

    void forget() {
        consumed.clear();
        history.clear();
        if (checkpoint) bc_checkpoint_free(checkpoint);
        checkpoint = nullptr;
    }
    ~bc_engine() {
        if (checkpoint) bc_checkpoint_free(checkpoint);
        if (seq) bc_seq_free(seq);
    }
};

namespace {

bool starts_with(const uint32_t* tokens, size_t n, const std::vector<uint32_t>& prefix) {
    return prefix.size() <= n && std::equal(prefix.begin(), prefix.end(), tokens);
}

// A uniform draw in [0, 1) from a splitmix64 stream (the reference draws from fastrand; which
// generator feeds the sampler is the host's choice).
float next_uniform(uint64_t* state) {
    uint64_t z = (*state += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

bool is_greedy(const bc_sampling* s) { return !s || (s->temperature <= 0.f && std::fabs(s->repeat_penalty - 1.0f) <= 1.1920929e-7f); }

struct Collector {
    bc_emit_fn emit;
    void* user;
    uint32_t* out;
    size_t cap, n;
};

int32_t collect(uint32_t token, void* user) {
    Collector* c = static_cast<Collector*>(user);
    if (c->n < c->cap) c->out[c->n] = token;
    c->n += 1;
    return c->emit ? c->emit(token, c->user) : 1;
}

}  // namespace

extern "C" {

bc_status bc_engine_new(bc_model* model, bc_backend* backend, uint32_t n_ctx, int32_t kv_half, uint64_t seed, bc_engine** out) {
    if (!out) return fail(BC_ERR_ARGUMENT, "out must be non-null");
    std::unique_ptr<bc_engine> e(new bc_engine());
    BC_TRY(bc_seq_new(model, backend, n_ctx, kv_half, &e->seq));
    e->context = n_ctx;
    e->rng = seed;
    *out = e.release();
    return BC_OK;
}

void bc_engine_free(bc_engine* engine) { delete engine; }

bc_status bc_engine_generate(bc_engine* e, const uint32_t* tokens, size_t n_tokens, int64_t turn, uint32_t max_tokens,
                             const bc_sampling* sampling, bc_emit_fn emit, void* user, uint32_t* out, size_t out_cap, size_t* n_out,
                             uint32_t* cached_tokens) {
    if (!e || (!tokens && n_tokens) || !n_out) return fail(BC_ERR_ARGUMENT, "engine, tokens and n_out must be non-null");
    *n_out = 0;
    if (n_tokens == 0) return fail(BC_ERR_ARGUMENT, "a request needs at least one token");
    if (n_tokens >= e->context)
        return fail(BC_ERR_CONTEXT_FULL, "the conversation holds %zu tokens, which fills the context of %u", n_tokens, e->context);
    if (turn >= (int64_t)n_tokens) return fail(BC_ERR_ARGUMENT, "the turn starts inside the request's tokens");
    bc_seq* s = e->seq;
    // What the device already holds of this request (engine.rs:561-574).
    size_t cached = 0;
    bc_status st = BC_OK;
    if (!e->consumed.empty() && starts_with(tokens, n_tokens, e->consumed) && e->consumed.size() < n_tokens) {
        cached = e->consumed.size();
    } else if (e->checkpoint && starts_with(tokens, n_tokens, e->history) && e->history.size() < n_tokens) {
        st = bc_seq_restore(s, e->checkpoint);
        cached = e->history.size();
    } else {
        st = bc_seq_reset(s);
        e->history.clear();
        if (e->checkpoint) bc_checkpoint_free(e->checkpoint);
        e->checkpoint = nullptr;
    }
    auto failed = [&](bc_status status) {
        // The device may hold part of the failed reply: the next request starts over (engine.rs:501-507).
        e->forget();
        bc_seq_reset(s);
        return status;
    };
    if (st != BC_OK) return failed(st);
    e->consumed.assign(tokens, tokens + cached);
    // The prompt up to the reply's turn becomes the history the next request may resume from (:575-585).
    size_t start = cached;
    if (turn > (int64_t)cached) {
        if ((st = bc_seq_prefill(s, tokens + cached, (size_t)turn - cached, nullptr, 0, nullptr, 0, nullptr)) != BC_OK) return failed(st);
        e->history.assign(tokens, tokens + turn);
        if (e->checkpoint) bc_checkpoint_free(e->checkpoint);
        e->checkpoint = nullptr;
        if ((st = bc_seq_checkpoint(s, &e->checkpoint)) != BC_OK) return failed(st);
        start = (size_t)turn;
    }
    if ((st = bc_seq_prefill(s, tokens + start, n_tokens - start, nullptr, 0, nullptr, 0, nullptr)) != BC_OK) return failed(st);
    e->consumed.assign(tokens, tokens + n_tokens);
    e->last_cached = (uint32_t)cached;
    if (cached_tokens) *cached_tokens = (uint32_t)cached;

    const uint32_t room = e->context - (uint32_t)n_tokens;
    uint32_t remaining = std::min(max_tokens, room);
    if (is_greedy(sampling)) {
        // Several steps ahead of the host; steps already submitted when the caller stops still
        // run, and their tokens join the consumed history (:595-619).
        Collector c{emit, user, out, out_cap, 0};
        std::vector<uint32_t> gained(remaining ? remaining : 1);
        size_t n_gained = 0;
        if ((st = bc_seq_generate_stream(s, remaining, collect, &c, gained.data(), gained.size(), &n_gained)) != BC_OK) return failed(st);
        e->consumed.insert(e->consumed.end(), gained.begin(), gained.begin() + n_gained);
        *n_out = std::min(c.n, out_cap);
        return BC_OK;
    }
    // Sampled: pick on the device from the logits the last step left there, then step (:620-634).
    size_t produced = 0;
    while (remaining > 0) {
        uint32_t token = 0;
        if ((st = bc_seq_sample(s, sampling, next_uniform(&e->rng), e->consumed.data(), e->consumed.size(), &token)) != BC_OK) return failed(st);
        remaining -= 1;
        if (produced < out_cap) out[produced] = token;
        produced += 1;
        const bool go_on = emit ? emit(token, user) != 0 : true;
        if (!go_on || remaining == 0) break;
        // The step's logits stay on the device, where the next pick reads them.
        if ((st = bc_seq_step_on_device(s, token)) != BC_OK) return failed(st);
        e->consumed.push_back(token);
    }
    *n_out = std::min(produced, out_cap);
    return BC_OK;
}

bc_status bc_engine_score(bc_engine* e, const uint32_t* prompt_tokens, const size_t* prompt_offsets, size_t n_prompts, const uint32_t* label_tokens,
                          const size_t* label_offsets, double* scores) {
    if (!e || !prompt_tokens || !prompt_offsets || !label_offsets || !scores || (!label_tokens && n_prompts && label_offsets[n_prompts]))
        return fail(BC_ERR_ARGUMENT, "engine, prompts, labels and scores must be non-null");
    bc_seq* s = e->seq;
    const uint32_t n_vocab = s->hp.n_vocab;
    for (size_t i = 0; i < n_prompts; ++i) {
        const size_t len = prompt_offsets[i + 1] - prompt_offsets[i];
        if (len == 0) return fail(BC_ERR_ARGUMENT, "a scored sequence needs at least one token");
        if (len >= e->context) return fail(BC_ERR_CONTEXT_FULL, "the prompt has %zu tokens, which does not fit the context of %u tokens", len, e->context);
        for (size_t t = prompt_offsets[i]; t < prompt_offsets[i + 1]; ++t)
            if (prompt_tokens[t] >= n_vocab) return fail(BC_ERR_TOKEN, "token %u lies outside the vocabulary", prompt_tokens[t]);
        for (size_t t = label_offsets[i]; t < label_offsets[i + 1]; ++t)
            if (label_tokens[t] >= n_vocab) return fail(BC_ERR_TOKEN, "label token %u lies outside the vocabulary", label_tokens[t]);
    }
    // Scoring runs sequences of its own, so the next reply starts over (:397-400).
    e->forget();
    BC_TRY(bc_seq_reset(s));
    if (n_prompts == 0) return BC_OK;
    // The longest common prefix, leaving every prompt at least its last token (:401-415).
    size_t shared = SIZE_MAX;
    for (size_t i = 0; i < n_prompts; ++i) shared = std::min(shared, prompt_offsets[i + 1] - prompt_offsets[i] - 1);
    const uint32_t* first = prompt_tokens + prompt_offsets[0];
    for (size_t i = 1; i < n_prompts; ++i) {
        const uint32_t* other = prompt_tokens + prompt_offsets[i];
        size_t same = 0;
        while (same < shared && first[same] == other[same]) ++same;
        shared = same;
    }
    bc_checkpoint* start = nullptr;
    struct Free {
        bc_checkpoint*& c;
        ~Free() { if (c) bc_checkpoint_free(c); }
    } free_start{start};
    if (shared > 0) {
        BC_TRY(bc_seq_prefill(s, first, shared, nullptr, 0, nullptr, 0, nullptr));
        BC_TRY(bc_seq_checkpoint(s, &start));
    }
    std::vector<float> logits(n_vocab);
    for (size_t i = 0; i < n_prompts; ++i) {
        if (start) BC_TRY(bc_seq_restore(s, start));
        else BC_TRY(bc_seq_reset(s));
        const uint32_t* prompt = prompt_tokens + prompt_offsets[i];
        const size_t len = prompt_offsets[i + 1] - prompt_offsets[i];
        BC_TRY(bc_seq_prefill(s, prompt + shared, len - shared, logits.data(), logits.size(), nullptr, 0, nullptr));
        // log-softmax in f64 (:425-433).
        double top = -INFINITY;
        for (float v : logits) top = std::max(top, (double)v);
        double sum = 0.0;
        for (float v : logits) sum += std::exp((double)v - top);
        const double log_sum = top + std::log(sum);
        for (size_t t = label_offsets[i]; t < label_offsets[i + 1]; ++t) scores[t] = (double)logits[label_tokens[t]] - log_sum;
    }
    return bc_seq_reset(s);
}

uint32_t bc_engine_consumed(const bc_engine* engine) { return engine ? (uint32_t)engine->consumed.size() : 0; }

}  // extern "C"
