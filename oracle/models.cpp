// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// CPU restatement of bobcat's scalar forward passes: LFM2 / LFM2-MoE
// (crates/bobcat/src/lfm2.rs:308-560, :678-716) and Qwen3.5 (crates/bobcat/src/qwen35.rs:284-516,
// :754-778), together with the loader's metadata keys, tensor names and shape checks
// (lfm2.rs:737-1004, qwen35.rs:629-752). It exists so the tests, the smoke check and the
// benchmark's CPU-baseline leg have the reference's arithmetic to compare against; the shipped
// CUDA library never links it.
//
// The caller (Python, through ctypes) parses the GGUF file with the `gguf` package and hands this
// code the metadata values and the tensor bytes by name; no file parsing happens here, which keeps
// this checker independent of the product's own GGUF reader.
//
// Parity pin: the reference ships no golden vectors for these passes (its model dumps are
// downloaded artefacts). This restatement is pinned instead against float32 `transformers` runs
// of randomly initialised models of the same architecture — the authority the reference's own
// scalar tests compare with — whose outputs are committed under tests/golden/.

#include <algorithm>
#include <cstdio>
#include <map>
#include <numeric>
#include <string>

#include "scalar.h"

namespace oracle {

struct Tensor {
    uint32_t type = 0;
    const uint8_t* data = nullptr;
    std::vector<uint64_t> shape;  // innermost first, as GGUF stores it
};

struct Matrix {
    const Tensor* t = nullptr;
    uint32_t n_rows = 0, n_cols = 0;
};

struct Vec {
    std::vector<float> v;
};

struct Source {
    std::map<std::string, uint32_t> u32s;
    std::map<std::string, float> f32s;
    std::map<std::string, std::vector<uint32_t>> arrays;
    std::map<std::string, Tensor> tensors;
    std::string architecture;
    std::string error;
    int threads = 1;

    bool fail(const std::string& why) {
        if (error.empty()) error = why;
        return false;
    }
    bool u32(const std::string& key, uint32_t* out) {
        auto it = u32s.find(key);
        if (it == u32s.end()) return fail("missing metadata " + key);
        *out = it->second;
        return true;
    }
    bool f32(const std::string& key, float* out) {
        auto it = f32s.find(key);
        if (it == f32s.end()) return fail("missing metadata " + key);
        *out = it->second;
        return true;
    }
    const Tensor* tensor(const std::string& name) const {
        auto it = tensors.find(name);
        return it == tensors.end() ? nullptr : &it->second;
    }
    // lfm2.rs:834-850
    const Tensor* require(const std::string& name, const std::vector<uint64_t>& want) {
        const Tensor* t = tensor(name);
        if (!t) { fail("missing tensor " + name); return nullptr; }
        if (t->shape != want) { fail("tensor " + name + " has the wrong shape"); return nullptr; }
        return t;
    }
    // lfm2.rs:853-868
    bool matrix(const std::string& name, uint64_t n_cols, uint64_t n_rows, Matrix* out) {
        const Tensor* t = require(name, {n_cols, n_rows});
        if (!t) return false;
        *out = {t, (uint32_t)n_rows, (uint32_t)n_cols};
        return true;
    }
    // lfm2.rs:872-891 — stacked experts become one matrix of n_experts * n_rows rows.
    bool experts(const std::string& name, uint64_t n_cols, uint64_t n_rows, uint64_t n_experts, Matrix* out) {
        const Tensor* t = require(name, {n_cols, n_rows, n_experts});
        if (!t) return false;
        *out = {t, (uint32_t)(n_rows * n_experts), (uint32_t)n_cols};
        return true;
    }
    // lfm2.rs:895-914 — vectors must be F32.
    bool vector(const std::string& name, const std::vector<uint64_t>& want, Vec* out) {
        const Tensor* t = require(name, want);
        if (!t) return false;
        if (t->type != T_F32) return fail("tensor " + name + " must be F32");
        size_t n = 1;
        for (uint64_t d : want) n *= (size_t)d;
        out->v.resize(n);
        std::memcpy(out->v.data(), t->data, n * 4);
        return true;
    }
};

static void add_in_place(float* h, const float* d, size_t n) {
    for (size_t i = 0; i < n; ++i) h[i] += d[i];
}

static float sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

// A float's position in IEEE total order, as Rust's f32::total_cmp ranks it.
static int32_t total_order_key(float f) {
    int32_t b;
    std::memcpy(&b, &f, 4);
    b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
    return b;
}

// ------------------------------------------------------------------------------------------
// LFM2 / LFM2-MoE
// ------------------------------------------------------------------------------------------

struct Lfm2Layer {
    bool attention = false;
    uint32_t cache_index = 0;
    Vec attn_norm, ffn_norm;
    // attention
    Matrix q, k, v, output;
    Vec q_norm, k_norm;
    // conv
    Vec taps;
    Matrix in_proj, out_proj;
    // ffn
    bool moe = false;
    Matrix gate, up, down, router;
    Vec expert_bias;
};

struct Lfm2 {
    uint32_t n_layers = 0, n_attention_layers = 0, n_conv_layers = 0, n_embd = 0, n_ff = 0;
    uint32_t n_experts = 0, n_experts_used = 0, n_ff_expert = 0, n_heads = 0, n_kv_heads = 0;
    uint32_t head_dim = 0, n_vocab = 0, conv_kernel = 0;
    float rope_theta = 0, norm_eps = 0;
    std::vector<Lfm2Layer> layers;
    Matrix token_embd, output;
    Vec output_norm;
};

struct Lfm2State {
    uint32_t n_ctx = 0, n_past = 0;
    std::vector<float> k_cache, v_cache, conv_history, hidden, normed, block_out, bcx, conv_out;
    std::vector<float> q, k, v, attn, scores, gate, up, router, expert_out;
    std::vector<uint32_t> experts;
};

// lfm2.rs:737-808 and :186-233, :919-1004
static bool load_lfm2(Source& s, Lfm2& m) {
    bool moe;
    if (s.architecture == "lfm2") moe = false;
    else if (s.architecture == "lfm2moe") moe = true;
    else return s.fail("architecture " + s.architecture);
    std::string p = s.architecture + ".";
    uint32_t n_dense = 0;
    if (!s.u32(p + "block_count", &m.n_layers) || !s.u32(p + "embedding_length", &m.n_embd) ||
        !s.u32(p + "feed_forward_length", &m.n_ff) || !s.u32(p + "attention.head_count", &m.n_heads) ||
        !s.u32(p + "shortconv.l_cache", &m.conv_kernel) || !s.f32(p + "rope.freq_base", &m.rope_theta) ||
        !s.f32(p + "attention.layer_norm_rms_epsilon", &m.norm_eps))
        return false;
    if (moe) {
        uint32_t gating = 0;
        if (!s.u32(p + "expert_gating_func", &gating)) return false;
        if (gating != 2) return s.fail("expert_gating_func must be 2 (sigmoid)");
        if (!s.u32(p + "expert_count", &m.n_experts) || !s.u32(p + "expert_used_count", &m.n_experts_used) ||
            !s.u32(p + "expert_feed_forward_length", &m.n_ff_expert))
            return false;
        auto it = s.u32s.find(p + "leading_dense_block_count");
        n_dense = it == s.u32s.end() ? 0 : it->second;
    } else {
        n_dense = m.n_layers;
    }
    if (m.n_layers == 0 || m.n_embd == 0 || m.n_ff == 0 || m.n_heads == 0 || m.n_embd % m.n_heads != 0 ||
        m.conv_kernel < 2 ||
        (moe && (m.n_experts_used == 0 || m.n_experts_used > m.n_experts || m.n_ff_expert == 0)))
        return s.fail("hyperparameters");
    m.head_dim = m.n_embd / m.n_heads;
    if (m.head_dim % 2 != 0) return s.fail("odd head_dim");

    const uint64_t n_embd = m.n_embd;
    const std::string kv_key = p + "attention.head_count_kv";
    m.layers.resize(m.n_layers);
    for (uint32_t il = 0; il < m.n_layers; ++il) {
        Lfm2Layer& L = m.layers[il];
        auto name = [&](const char* suffix) { return "blk." + std::to_string(il) + "." + suffix + ".weight"; };
        // lfm2.rs:819-831 — one count per layer (0 marks a conv layer) or one scalar for all.
        uint32_t n_kv = 0;
        auto arr = s.arrays.find(kv_key);
        if (arr != s.arrays.end() && arr->second.size() == m.n_layers) n_kv = arr->second[il];
        else if (!s.u32(kv_key, &n_kv)) return false;

        if (!s.vector(name("attn_norm"), {n_embd}, &L.attn_norm) || !s.vector(name("ffn_norm"), {n_embd}, &L.ffn_norm))
            return false;
        if (il < n_dense) {
            if (!s.matrix(name("ffn_gate"), n_embd, m.n_ff, &L.gate) || !s.matrix(name("ffn_up"), n_embd, m.n_ff, &L.up) ||
                !s.matrix(name("ffn_down"), m.n_ff, n_embd, &L.down))
                return false;
        } else {
            L.moe = true;
            if (!s.matrix(name("ffn_gate_inp"), n_embd, m.n_experts, &L.router) ||
                !s.vector("blk." + std::to_string(il) + ".exp_probs_b.bias", {m.n_experts}, &L.expert_bias) ||
                !s.experts(name("ffn_gate_exps"), n_embd, m.n_ff_expert, m.n_experts, &L.gate) ||
                !s.experts(name("ffn_up_exps"), n_embd, m.n_ff_expert, m.n_experts, &L.up) ||
                !s.experts(name("ffn_down_exps"), m.n_ff_expert, n_embd, m.n_experts, &L.down))
                return false;
        }
        if (n_kv == 0) {
            if (!s.vector(name("shortconv.conv"), {m.conv_kernel, n_embd}, &L.taps) ||
                !s.matrix(name("shortconv.in_proj"), n_embd, 3 * n_embd, &L.in_proj) ||
                !s.matrix(name("shortconv.out_proj"), n_embd, n_embd, &L.out_proj))
                return false;
            L.cache_index = m.n_conv_layers++;
        } else {
            if (m.n_kv_heads == 0) m.n_kv_heads = n_kv;
            if (n_kv != m.n_kv_heads || m.n_heads % n_kv != 0) return s.fail("kv heads");
            uint64_t hd = m.head_dim, q_dim = (uint64_t)m.n_heads * hd, kv_dim = (uint64_t)n_kv * hd;
            L.attention = true;
            if (!s.matrix(name("attn_q"), n_embd, q_dim, &L.q) || !s.matrix(name("attn_k"), n_embd, kv_dim, &L.k) ||
                !s.matrix(name("attn_v"), n_embd, kv_dim, &L.v) || !s.matrix(name("attn_output"), q_dim, n_embd, &L.output) ||
                !s.vector(name("attn_q_norm"), {hd}, &L.q_norm) || !s.vector(name("attn_k_norm"), {hd}, &L.k_norm))
                return false;
            L.cache_index = m.n_attention_layers++;
        }
    }
    const Tensor* embd = s.tensor("token_embd.weight");
    if (!embd || embd->shape.size() != 2) return s.fail("missing tensor token_embd.weight");
    m.n_vocab = (uint32_t)embd->shape[1];
    if (!s.matrix("token_embd.weight", n_embd, m.n_vocab, &m.token_embd) ||
        !s.vector("token_embd_norm.weight", {n_embd}, &m.output_norm))
        return false;
    // lfm2.rs:217-223 — the output matrix is the token embedding unless the file has its own.
    if (s.tensor("output.weight")) {
        if (!s.matrix("output.weight", n_embd, m.n_vocab, &m.output)) return false;
    } else {
        m.output = m.token_embd;
    }
    return true;
}

// lfm2.rs:593-627
static void lfm2_state_init(const Lfm2& m, uint32_t n_ctx, Lfm2State& st) {
    size_t n_embd = m.n_embd, kv_dim = (size_t)m.n_kv_heads * m.head_dim, q_dim = (size_t)m.n_heads * m.head_dim;
    size_t cache = (size_t)m.n_attention_layers * n_ctx * kv_dim;
    size_t n_ff = std::max(m.n_ff, m.n_ff_expert);
    st.n_ctx = n_ctx;
    st.n_past = 0;
    st.k_cache.assign(cache, 0.f);
    st.v_cache.assign(cache, 0.f);
    st.conv_history.assign((size_t)m.n_conv_layers * (m.conv_kernel - 1) * n_embd, 0.f);
    st.hidden.assign(n_embd, 0.f);
    st.normed.assign(n_embd, 0.f);
    st.block_out.assign(n_embd, 0.f);
    st.bcx.assign(3 * n_embd, 0.f);
    st.conv_out.assign(n_embd, 0.f);
    st.q.assign(q_dim, 0.f);
    st.k.assign(kv_dim, 0.f);
    st.v.assign(kv_dim, 0.f);
    st.attn.assign(q_dim, 0.f);
    st.scores.assign(n_ctx, 0.f);
    st.gate.assign(n_ff, 0.f);
    st.up.assign(n_ff, 0.f);
    st.router.assign(m.n_experts, 0.f);
    st.experts.assign(m.n_experts, 0);
    st.expert_out.assign(n_embd, 0.f);
}

static void mv(const Matrix& w, const float* x, float* y, int threads, size_t first_row = 0, size_t n_rows = 0) {
    size_t rows = n_rows ? n_rows : w.n_rows;
    const uint8_t* base = w.t->data + first_row * row_bytes(w.t->type, w.n_cols);
    matvec(w.t->type, base, x, w.n_cols, y, rows, threads);
}

// lfm2.rs:691-709 — sigmoid scores; stable sort of ids by (score + bias) descending under total
// order; weights = score / (f32 sum of picked scores + 1e-6).
static void lfm2_route(float* scores, const float* bias, size_t n_experts, size_t n_used, uint32_t* experts) {
    for (size_t i = 0; i < n_experts; ++i) scores[i] = 1.0f / (1.0f + expf(-scores[i]));
    std::iota(experts, experts + n_experts, 0u);
    std::stable_sort(experts, experts + n_experts, [&](uint32_t a, uint32_t b) {
        return total_order_key(scores[b] + bias[b]) < total_order_key(scores[a] + bias[a]);
    });
    float sum = 0.f;
    for (size_t i = 0; i < n_used; ++i) sum += scores[experts[i]];
    float norm = sum + 1e-6f;
    for (size_t i = 0; i < n_used; ++i) scores[experts[i]] /= norm;
}

// lfm2.rs:444-478
static void lfm2_conv_block(const Lfm2& m, const Lfm2Layer& L, Lfm2State& st, int threads) {
    size_t n_embd = m.n_embd, kernel = m.conv_kernel;
    float* history = st.conv_history.data() + (size_t)L.cache_index * (kernel - 1) * n_embd;
    mv(L.in_proj, st.normed.data(), st.bcx.data(), threads);
    const float* b = st.bcx.data();
    const float* c = b + n_embd;
    const float* x = c + n_embd;
    for (size_t ch = 0; ch < n_embd; ++ch) {
        const float* taps = L.taps.v.data() + ch * kernel;
        float bx = b[ch] * x[ch];
        double sum = (double)taps[kernel - 1] * (double)bx;
        for (size_t k = 0; k + 1 < kernel; ++k) sum += (double)taps[k] * (double)history[k * n_embd + ch];
        for (size_t k = 0; k + 2 < kernel; ++k) history[k * n_embd + ch] = history[(k + 1) * n_embd + ch];
        history[(kernel - 2) * n_embd + ch] = bx;
        st.conv_out[ch] = c[ch] * (float)sum;
    }
    mv(L.out_proj, st.conv_out.data(), st.block_out.data(), threads);
}

// lfm2.rs:482-560
static void lfm2_attention_block(const Lfm2& m, const Lfm2Layer& L, Lfm2State& st, uint32_t pos, int threads) {
    size_t hd = m.head_dim, kv_dim = (size_t)m.n_kv_heads * hd, group = m.n_heads / m.n_kv_heads;
    float scale = 1.0f / sqrtf((float)m.head_dim);
    size_t layer_len = (size_t)st.n_ctx * kv_dim;
    float* k_cache = st.k_cache.data() + (size_t)L.cache_index * layer_len;
    float* v_cache = st.v_cache.data() + (size_t)L.cache_index * layer_len;
    mv(L.q, st.normed.data(), st.q.data(), threads);
    mv(L.k, st.normed.data(), st.k.data(), threads);
    mv(L.v, st.normed.data(), st.v.data(), threads);
    for (size_t h = 0; h < m.n_heads; ++h) {
        float* head = st.q.data() + h * hd;
        rms_norm(head, L.q_norm.v.data(), hd, m.norm_eps, head);
        rope_neox(head, hd, pos, m.rope_theta);
    }
    for (size_t h = 0; h < m.n_kv_heads; ++h) {
        float* head = st.k.data() + h * hd;
        rms_norm(head, L.k_norm.v.data(), hd, m.norm_eps, head);
        rope_neox(head, hd, pos, m.rope_theta);
    }
    std::memcpy(k_cache + (size_t)pos * kv_dim, st.k.data(), kv_dim * 4);
    std::memcpy(v_cache + (size_t)pos * kv_dim, st.v.data(), kv_dim * 4);

    size_t n_keys = (size_t)pos + 1;
    float* scores = st.scores.data();
    for (size_t h = 0; h < m.n_heads; ++h) {
        const float* qh = st.q.data() + h * hd;
        float* out = st.attn.data() + h * hd;
        size_t kv_offset = h / group * hd;
        for (size_t t = 0; t < n_keys; ++t) scores[t] = scale * dot(qh, k_cache + t * kv_dim + kv_offset, hd);
        softmax(scores, n_keys);
        for (size_t d = 0; d < hd; ++d) {
            double sum = 0.0;
            for (size_t t = 0; t < n_keys; ++t) sum += (double)scores[t] * (double)v_cache[t * kv_dim + kv_offset + d];
            out[d] = (float)sum;
        }
    }
    mv(L.output, st.attn.data(), st.block_out.data(), threads);
}

static void swiglu(float* gate, const float* up, size_t n) {
    for (size_t i = 0; i < n; ++i) gate[i] = silu(gate[i]) * up[i];
}

// lfm2.rs:404-440
static void lfm2_ffn(const Lfm2& m, const Lfm2Layer& L, Lfm2State& st, int threads) {
    if (!L.moe) {
        mv(L.gate, st.normed.data(), st.gate.data(), threads);
        mv(L.up, st.normed.data(), st.up.data(), threads);
        swiglu(st.gate.data(), st.up.data(), m.n_ff);
        mv(L.down, st.gate.data(), st.block_out.data(), threads);
        return;
    }
    size_t n_embd = m.n_embd, n_ff = m.n_ff_expert, n_used = m.n_experts_used;
    mv(L.router, st.normed.data(), st.router.data(), threads);
    lfm2_route(st.router.data(), L.expert_bias.v.data(), m.n_experts, n_used, st.experts.data());
    std::fill(st.block_out.begin(), st.block_out.end(), 0.f);
    for (size_t i = 0; i < n_used; ++i) {
        size_t e = st.experts[i];
        mv(L.gate, st.normed.data(), st.gate.data(), threads, e * n_ff, n_ff);
        mv(L.up, st.normed.data(), st.up.data(), threads, e * n_ff, n_ff);
        swiglu(st.gate.data(), st.up.data(), n_ff);
        mv(L.down, st.gate.data(), st.expert_out.data(), threads, e * n_embd, n_embd);
        float weight = st.router[e];
        for (size_t j = 0; j < n_embd; ++j) st.block_out[j] += weight * st.expert_out[j];
    }
}

struct TraceOut {
    float* embedding;
    float* layers;
    float* final_norm;
    int32_t* experts;  // optional: n_layers * n_used picked expert ids, -1 for dense layers
};

// lfm2.rs:308-394. Returns 0, or 1 ContextFull, 2 Token.
static int lfm2_step(const Lfm2& m, Lfm2State& st, uint32_t token, float* logits, const TraceOut* trace, int threads) {
    size_t n_embd = m.n_embd;
    uint32_t pos = st.n_past;
    if (pos >= st.n_ctx) return 1;
    if (token >= m.n_vocab) return 2;
    get_row(m.token_embd.t->type, m.token_embd.t->data, token, n_embd, st.hidden.data());
    if (trace && trace->embedding) std::memcpy(trace->embedding, st.hidden.data(), n_embd * 4);
    for (size_t il = 0; il < m.layers.size(); ++il) {
        const Lfm2Layer& L = m.layers[il];
        rms_norm(st.hidden.data(), L.attn_norm.v.data(), n_embd, m.norm_eps, st.normed.data());
        if (L.attention) lfm2_attention_block(m, L, st, pos, threads);
        else lfm2_conv_block(m, L, st, threads);
        add_in_place(st.hidden.data(), st.block_out.data(), n_embd);
        rms_norm(st.hidden.data(), L.ffn_norm.v.data(), n_embd, m.norm_eps, st.normed.data());
        lfm2_ffn(m, L, st, threads);
        add_in_place(st.hidden.data(), st.block_out.data(), n_embd);
        if (trace && trace->layers) std::memcpy(trace->layers + il * n_embd, st.hidden.data(), n_embd * 4);
        if (trace && trace->experts && m.n_experts_used) {
            for (uint32_t i = 0; i < m.n_experts_used; ++i)
                trace->experts[il * m.n_experts_used + i] = L.moe ? (int32_t)st.experts[i] : -1;
        }
    }
    rms_norm(st.hidden.data(), m.output_norm.v.data(), n_embd, m.norm_eps, st.normed.data());
    if (trace && trace->final_norm) std::memcpy(trace->final_norm, st.normed.data(), n_embd * 4);
    if (logits) mv(m.output, st.normed.data(), logits, threads);
    st.n_past += 1;
    return 0;
}

// ------------------------------------------------------------------------------------------
// Qwen3.5
// ------------------------------------------------------------------------------------------

struct QwenLayer {
    bool attention = false;
    uint32_t cache_index = 0;
    Vec attn_norm, ffn_norm;
    Matrix gate, up, down;
    // attention
    Matrix q, k, v, output;
    Vec q_norm, k_norm;
    // delta net
    Matrix qkv, z, beta, alpha, out;
    Vec conv, dt_bias, a, norm;
};

struct Qwen {
    uint32_t n_layers = 0, n_attention_layers = 0, n_delta_layers = 0, n_embd = 0, n_ff = 0, n_vocab = 0;
    uint32_t n_heads = 0, n_kv_heads = 0, head_dim = 0, n_rot = 0, conv_kernel = 0;
    uint32_t n_k_heads = 0, n_v_heads = 0, k_head_dim = 0, v_head_dim = 0;
    float rope_theta = 0, norm_eps = 0;
    std::vector<QwenLayer> layers;
    Matrix token_embd, output;
    Vec output_norm;
    uint32_t key_dim() const { return n_k_heads * k_head_dim; }
    uint32_t value_dim() const { return n_v_heads * v_head_dim; }
    uint32_t conv_dim() const { return 2 * key_dim() + value_dim(); }
};

struct QwenState {
    uint32_t n_ctx = 0, n_past = 0;
    std::vector<std::vector<float>> cache_k, cache_v, rec_conv, rec_state;
    std::vector<float> h, x, mixer_out, ffn_gate, ffn_up, q_gate, q, attn_gate, k, v, attn, scores;
    std::vector<float> qkv, conv_out, z, beta, alpha, delta, delta_out;
};

// qwen35.rs:629-752
static bool load_qwen(Source& s, Qwen& m) {
    if (s.architecture != "qwen35") return s.fail("architecture " + s.architecture);
    const std::string p = "qwen35.";
    uint32_t block_count = 0, n_nextn = 0, inner = 0, value_length = 0;
    if (!s.u32(p + "block_count", &block_count)) return false;
    auto nn = s.u32s.find(p + "nextn_predict_layers");
    if (nn != s.u32s.end()) n_nextn = nn->second;
    if (n_nextn > block_count) return s.fail("hyperparameters");
    m.n_layers = block_count - n_nextn;
    if (!s.u32(p + "attention.key_length", &m.head_dim) || !s.u32(p + "ssm.time_step_rank", &m.n_v_heads) ||
        !s.u32(p + "ssm.inner_size", &inner) || !s.u32(p + "embedding_length", &m.n_embd) ||
        !s.u32(p + "feed_forward_length", &m.n_ff) || !s.u32(p + "attention.head_count", &m.n_heads) ||
        !s.u32(p + "attention.head_count_kv", &m.n_kv_heads) || !s.u32(p + "rope.dimension_count", &m.n_rot) ||
        !s.f32(p + "rope.freq_base", &m.rope_theta) || !s.f32(p + "attention.layer_norm_rms_epsilon", &m.norm_eps) ||
        !s.u32(p + "ssm.conv_kernel", &m.conv_kernel) || !s.u32(p + "ssm.group_count", &m.n_k_heads) ||
        !s.u32(p + "ssm.state_size", &m.k_head_dim) || !s.u32(p + "attention.value_length", &value_length))
        return false;
    m.v_head_dim = m.n_v_heads ? inner / m.n_v_heads : 0;
    if (m.n_layers == 0 || m.n_embd == 0 || m.n_heads == 0 || m.n_kv_heads == 0 || m.n_heads % m.n_kv_heads != 0 ||
        m.head_dim == 0 || value_length != m.head_dim || m.n_rot == 0 || m.n_rot % 2 != 0 || m.n_rot > m.head_dim ||
        m.conv_kernel < 2 || m.n_k_heads == 0 || m.n_v_heads == 0 || m.n_v_heads % m.n_k_heads != 0 ||
        m.k_head_dim == 0 || m.v_head_dim == 0 || (uint64_t)m.n_v_heads * m.v_head_dim != inner)
        return s.fail("hyperparameters");

    const Tensor* embd = s.tensor("token_embd.weight");
    if (!embd || embd->shape.size() != 2) return s.fail("missing tensor token_embd.weight");
    m.n_vocab = (uint32_t)embd->shape[1];
    uint64_t n_embd = m.n_embd, n_ff = m.n_ff;
    m.layers.resize(m.n_layers);
    for (uint32_t il = 0; il < m.n_layers; ++il) {
        QwenLayer& L = m.layers[il];
        auto name = [&](const char* suffix) { return "blk." + std::to_string(il) + "." + suffix; };
        if (s.tensor(name("ssm_a"))) {
            uint64_t value_dim = m.value_dim(), conv_dim = m.conv_dim(), n_v = m.n_v_heads;
            if (!s.matrix(name("attn_qkv.weight"), n_embd, conv_dim, &L.qkv) ||
                !s.matrix(name("attn_gate.weight"), n_embd, value_dim, &L.z) ||
                !s.matrix(name("ssm_beta.weight"), n_embd, n_v, &L.beta) ||
                !s.matrix(name("ssm_alpha.weight"), n_embd, n_v, &L.alpha) ||
                !s.vector(name("ssm_conv1d.weight"), {m.conv_kernel, conv_dim}, &L.conv) ||
                !s.vector(name("ssm_dt.bias"), {n_v}, &L.dt_bias) || !s.vector(name("ssm_a"), {n_v}, &L.a) ||
                !s.vector(name("ssm_norm.weight"), {m.v_head_dim}, &L.norm) ||
                !s.matrix(name("ssm_out.weight"), value_dim, n_embd, &L.out))
                return false;
            L.cache_index = m.n_delta_layers++;
        } else {
            uint64_t hd = m.head_dim, q_dim = (uint64_t)m.n_heads * hd, kv_dim = (uint64_t)m.n_kv_heads * hd;
            L.attention = true;
            if (!s.matrix(name("attn_q.weight"), n_embd, 2 * q_dim, &L.q) ||
                !s.matrix(name("attn_k.weight"), n_embd, kv_dim, &L.k) ||
                !s.matrix(name("attn_v.weight"), n_embd, kv_dim, &L.v) ||
                !s.matrix(name("attn_output.weight"), q_dim, n_embd, &L.output) ||
                !s.vector(name("attn_q_norm.weight"), {hd}, &L.q_norm) ||
                !s.vector(name("attn_k_norm.weight"), {hd}, &L.k_norm))
                return false;
            L.cache_index = m.n_attention_layers++;
        }
        if (!s.vector(name("attn_norm.weight"), {n_embd}, &L.attn_norm) ||
            !s.vector(name("post_attention_norm.weight"), {n_embd}, &L.ffn_norm) ||
            !s.matrix(name("ffn_gate.weight"), n_embd, n_ff, &L.gate) ||
            !s.matrix(name("ffn_up.weight"), n_embd, n_ff, &L.up) ||
            !s.matrix(name("ffn_down.weight"), n_ff, n_embd, &L.down))
            return false;
    }
    if (!s.matrix("token_embd.weight", n_embd, m.n_vocab, &m.token_embd) ||
        !s.vector("output_norm.weight", {n_embd}, &m.output_norm))
        return false;
    if (s.tensor("output.weight")) {
        if (!s.matrix("output.weight", n_embd, m.n_vocab, &m.output)) return false;
    } else {
        m.output = m.token_embd;
    }
    return true;
}

// qwen35.rs:573-619
static void qwen_state_init(const Qwen& m, uint32_t n_ctx, QwenState& st) {
    size_t hd = m.head_dim, kv_dim = (size_t)m.n_kv_heads * hd, q_dim = (size_t)m.n_heads * hd;
    size_t conv_dim = m.conv_dim(), value_dim = m.value_dim();
    st.n_ctx = n_ctx;
    st.n_past = 0;
    st.cache_k.assign(m.n_attention_layers, std::vector<float>((size_t)n_ctx * kv_dim, 0.f));
    st.cache_v = st.cache_k;
    st.rec_conv.assign(m.n_delta_layers, std::vector<float>(conv_dim * (m.conv_kernel - 1), 0.f));
    st.rec_state.assign(m.n_delta_layers, std::vector<float>((size_t)m.n_v_heads * m.k_head_dim * m.v_head_dim, 0.f));
    st.h.assign(m.n_embd, 0.f);
    st.x.assign(m.n_embd, 0.f);
    st.mixer_out.assign(m.n_embd, 0.f);
    st.ffn_gate.assign(m.n_ff, 0.f);
    st.ffn_up.assign(m.n_ff, 0.f);
    st.q_gate.assign(2 * q_dim, 0.f);
    st.q.assign(q_dim, 0.f);
    st.attn_gate.assign(q_dim, 0.f);
    st.k.assign(kv_dim, 0.f);
    st.v.assign(kv_dim, 0.f);
    st.attn.assign(q_dim, 0.f);
    st.scores.assign(n_ctx, 0.f);
    st.qkv.assign(conv_dim, 0.f);
    st.conv_out.assign(conv_dim, 0.f);
    st.z.assign(value_dim, 0.f);
    st.beta.assign(m.n_v_heads, 0.f);
    st.alpha.assign(m.n_v_heads, 0.f);
    st.delta.assign(m.v_head_dim, 0.f);
    st.delta_out.assign(value_dim, 0.f);
}

// qwen35.rs:762-768 — the sum of squares stays in f32.
static void l2_normalize(float* x, size_t n, float scale) {
    float sum = 0.f;
    for (size_t i = 0; i < n; ++i) sum += x[i] * x[i];
    float factor = scale / sqrtf(sum + 1e-6f);
    for (size_t i = 0; i < n; ++i) x[i] *= factor;
}

// qwen35.rs:776-778
static float softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// qwen35.rs:369-426
static void qwen_attention(const Qwen& m, const QwenLayer& L, QwenState& st, uint32_t pos, int threads) {
    size_t hd = m.head_dim, n_rot = m.n_rot, n_heads = m.n_heads, n_kv = m.n_kv_heads;
    size_t kv_dim = n_kv * hd, group = n_heads / n_kv;
    mv(L.q, st.x.data(), st.q_gate.data(), threads);
    mv(L.k, st.x.data(), st.k.data(), threads);
    mv(L.v, st.x.data(), st.v.data(), threads);
    for (size_t head = 0; head < n_heads; ++head) {
        const float* block = st.q_gate.data() + 2 * head * hd;
        float* q = st.q.data() + head * hd;
        std::memcpy(q, block, hd * 4);
        rms_norm(q, L.q_norm.v.data(), hd, m.norm_eps, q);
        rope_neox(q, n_rot, pos, m.rope_theta);
        std::memcpy(st.attn_gate.data() + head * hd, block + hd, hd * 4);
    }
    for (size_t head = 0; head < n_kv; ++head) {
        float* k = st.k.data() + head * hd;
        rms_norm(k, L.k_norm.v.data(), hd, m.norm_eps, k);
        rope_neox(k, n_rot, pos, m.rope_theta);
    }
    float* ck = st.cache_k[L.cache_index].data();
    float* cv = st.cache_v[L.cache_index].data();
    std::memcpy(ck + (size_t)pos * kv_dim, st.k.data(), kv_dim * 4);
    std::memcpy(cv + (size_t)pos * kv_dim, st.v.data(), kv_dim * 4);

    size_t n_keys = (size_t)pos + 1;
    float scale = 1.0f / sqrtf((float)m.head_dim);
    float* scores = st.scores.data();
    for (size_t head = 0; head < n_heads; ++head) {
        size_t kv_head = head / group;
        const float* q = st.q.data() + head * hd;
        for (size_t t = 0; t < n_keys; ++t) scores[t] = dot(q, ck + t * kv_dim + kv_head * hd, hd) * scale;
        softmax(scores, n_keys);
        float* out = st.attn.data() + head * hd;
        std::fill(out, out + hd, 0.f);
        // The weighted sum of values stays in f32, in position order.
        for (size_t t = 0; t < n_keys; ++t) {
            const float* v = cv + t * kv_dim + kv_head * hd;
            float w = scores[t];
            for (size_t d = 0; d < hd; ++d) out[d] += w * v[d];
        }
    }
    for (size_t i = 0; i < n_heads * hd; ++i) st.attn[i] *= sigmoid(st.attn_gate[i]);
    mv(L.output, st.attn.data(), st.mixer_out.data(), threads);
}

// qwen35.rs:430-516
static void qwen_delta_net(const Qwen& m, const QwenLayer& L, QwenState& st, int threads) {
    size_t kernel = m.conv_kernel, history = kernel - 1, n_k = m.n_k_heads, n_v = m.n_v_heads;
    size_t kd = m.k_head_dim, vd = m.v_head_dim, key_dim = m.key_dim(), conv_dim = m.conv_dim();
    float* rconv = st.rec_conv[L.cache_index].data();
    float* rstate = st.rec_state[L.cache_index].data();
    mv(L.qkv, st.x.data(), st.qkv.data(), threads);
    mv(L.z, st.x.data(), st.z.data(), threads);
    mv(L.beta, st.x.data(), st.beta.data(), threads);
    mv(L.alpha, st.x.data(), st.alpha.data(), threads);

    // Causal convolution with SiLU; the history holds raw inputs, oldest first; f32 sum starting
    // from the newest tap's term.
    for (size_t c = 0; c < conv_dim; ++c) {
        const float* taps = L.conv.v.data() + c * kernel;
        float* past = rconv + c * history;
        float input = st.qkv[c];
        float sum = taps[history] * input;
        for (size_t i = 0; i < history; ++i) sum += taps[i] * past[i];
        st.conv_out[c] = silu(sum);
        for (size_t i = 0; i + 1 < history; ++i) past[i] = past[i + 1];
        past[history - 1] = input;
    }
    float* q = st.conv_out.data();
    float* k = q + key_dim;
    float* v = k + key_dim;
    float q_scale = 1.0f / sqrtf((float)m.k_head_dim);
    for (size_t head = 0; head < n_k; ++head) {
        l2_normalize(q + head * kd, kd, q_scale);
        l2_normalize(k + head * kd, kd, 1.0f);
    }
    for (size_t head = 0; head < n_v; ++head) {
        // Value head j reads key head j % n_k_heads.
        size_t key_head = head % n_k;
        const float* qh = q + key_head * kd;
        const float* kh = k + key_head * kd;
        const float* vh = v + head * vd;
        float beta = sigmoid(st.beta[head]);
        float decay = expf(L.a.v[head] * softplus(st.alpha[head] + L.dt_bias.v[head]));
        float* S = rstate + head * kd * vd;  // kd rows of vd elements
        for (size_t i = 0; i < kd * vd; ++i) S[i] *= decay;
        float* r = st.delta.data();
        std::fill(r, r + vd, 0.f);
        for (size_t i = 0; i < kd; ++i)
            for (size_t j = 0; j < vd; ++j) r[j] += S[i * vd + j] * kh[i];
        for (size_t j = 0; j < vd; ++j) r[j] = (vh[j] - r[j]) * beta;
        float* out = st.delta_out.data() + head * vd;
        std::fill(out, out + vd, 0.f);
        for (size_t i = 0; i < kd; ++i)
            for (size_t j = 0; j < vd; ++j) {
                S[i * vd + j] += kh[i] * r[j];
                out[j] += S[i * vd + j] * qh[i];
            }
        rms_norm(out, L.norm.v.data(), vd, m.norm_eps, out);
        const float* gate = st.z.data() + head * vd;
        for (size_t j = 0; j < vd; ++j) out[j] *= silu(gate[j]);
    }
    mv(L.out, st.delta_out.data(), st.mixer_out.data(), threads);
}

// qwen35.rs:284-365
static int qwen_step(const Qwen& m, QwenState& st, uint32_t token, float* logits, const TraceOut* trace, int threads) {
    size_t n_embd = m.n_embd;
    uint32_t pos = st.n_past;
    if (pos >= st.n_ctx) return 1;
    if (token >= m.n_vocab) return 2;
    get_row(m.token_embd.t->type, m.token_embd.t->data, token, n_embd, st.h.data());
    if (trace && trace->embedding) std::memcpy(trace->embedding, st.h.data(), n_embd * 4);
    for (size_t il = 0; il < m.layers.size(); ++il) {
        const QwenLayer& L = m.layers[il];
        rms_norm(st.h.data(), L.attn_norm.v.data(), n_embd, m.norm_eps, st.x.data());
        if (L.attention) qwen_attention(m, L, st, pos, threads);
        else qwen_delta_net(m, L, st, threads);
        add_in_place(st.h.data(), st.mixer_out.data(), n_embd);
        rms_norm(st.h.data(), L.ffn_norm.v.data(), n_embd, m.norm_eps, st.x.data());
        mv(L.gate, st.x.data(), st.ffn_gate.data(), threads);
        mv(L.up, st.x.data(), st.ffn_up.data(), threads);
        swiglu(st.ffn_gate.data(), st.ffn_up.data(), m.n_ff);
        mv(L.down, st.ffn_gate.data(), st.mixer_out.data(), threads);
        add_in_place(st.h.data(), st.mixer_out.data(), n_embd);
        if (trace && trace->layers) std::memcpy(trace->layers + il * n_embd, st.h.data(), n_embd * 4);
    }
    rms_norm(st.h.data(), m.output_norm.v.data(), n_embd, m.norm_eps, st.x.data());
    if (trace && trace->final_norm) std::memcpy(trace->final_norm, st.x.data(), n_embd * 4);
    if (logits) mv(m.output, st.x.data(), logits, threads);
    st.n_past += 1;
    return 0;
}

struct Model {
    Source src;
    bool is_qwen = false;
    Lfm2 lfm2;
    Qwen qwen;
};

struct State {
    const Model* model;
    Lfm2State lfm2;
    QwenState qwen;
};

}  // namespace oracle

// ------------------------------------------------------------------------------------------
// C entry points for ctypes
// ------------------------------------------------------------------------------------------
using namespace oracle;

extern "C" {

void* orc_model_new(const char* architecture) {
    Model* m = new Model();
    m->src.architecture = architecture;
    return m;
}
void orc_model_free(void* m) { delete (Model*)m; }
void orc_model_set_u32(void* m, const char* key, uint32_t v) { ((Model*)m)->src.u32s[key] = v; }
void orc_model_set_f32(void* m, const char* key, float v) { ((Model*)m)->src.f32s[key] = v; }
void orc_model_set_array(void* m, const char* key, const uint32_t* v, uint64_t n) {
    ((Model*)m)->src.arrays[key] = std::vector<uint32_t>(v, v + n);
}
// `data` must stay valid for the model's life. `shape` is innermost-first, as the file stores it.
void orc_model_add_tensor(void* m, const char* name, uint32_t type, const void* data, const uint64_t* shape, uint32_t n_dims) {
    Tensor t;
    t.type = type;
    t.data = (const uint8_t*)data;
    t.shape.assign(shape, shape + n_dims);
    ((Model*)m)->src.tensors[name] = t;
}
void orc_model_set_threads(void* m, int threads) { ((Model*)m)->src.threads = threads < 1 ? 1 : threads; }
// Returns 0 on success; otherwise orc_model_error names the first failed check.
int orc_model_finish(void* mp) {
    Model* m = (Model*)mp;
    m->is_qwen = m->src.architecture == "qwen35";
    bool ok = m->is_qwen ? load_qwen(m->src, m->qwen) : load_lfm2(m->src, m->lfm2);
    return ok ? 0 : 1;
}
const char* orc_model_error(void* m) { return ((Model*)m)->src.error.c_str(); }

// Hyperparameters in a fixed order: n_layers, n_embd, n_vocab, n_attention_layers, n_other_layers,
// n_heads, n_kv_heads, head_dim, n_ff, n_experts, n_experts_used.
void orc_model_shape(void* mp, uint32_t* out) {
    Model* m = (Model*)mp;
    if (m->is_qwen) {
        const Qwen& q = m->qwen;
        uint32_t v[11] = {q.n_layers, q.n_embd, q.n_vocab, q.n_attention_layers, q.n_delta_layers, q.n_heads, q.n_kv_heads, q.head_dim, q.n_ff, 0, 0};
        std::memcpy(out, v, sizeof v);
    } else {
        const Lfm2& l = m->lfm2;
        uint32_t v[11] = {l.n_layers, l.n_embd, l.n_vocab, l.n_attention_layers, l.n_conv_layers, l.n_heads, l.n_kv_heads, l.head_dim, l.n_ff, l.n_experts, l.n_experts_used};
        std::memcpy(out, v, sizeof v);
    }
}

void* orc_state_new(void* mp, uint32_t n_ctx) {
    Model* m = (Model*)mp;
    if (n_ctx == 0) return nullptr;
    State* st = new State();
    st->model = m;
    if (m->is_qwen) qwen_state_init(m->qwen, n_ctx, st->qwen);
    else lfm2_state_init(m->lfm2, n_ctx, st->lfm2);
    return st;
}
void orc_state_free(void* st) { delete (State*)st; }
uint32_t orc_state_n_past(void* sp) {
    State* st = (State*)sp;
    return st->model->is_qwen ? st->qwen.n_past : st->lfm2.n_past;
}

// One token through the model. Null outputs are skipped. `experts` (LFM2-MoE only) receives the
// picked expert ids of every layer. Returns 0, 1 = context full, 2 = token outside the vocabulary.
int orc_step(void* sp, uint32_t token, float* logits, float* trace_embedding, float* trace_layers,
             float* trace_final, int32_t* experts) {
    State* st = (State*)sp;
    const Model* m = st->model;
    TraceOut trace{trace_embedding, trace_layers, trace_final, experts};
    if (m->is_qwen) return qwen_step(m->qwen, st->qwen, token, logits, &trace, m->src.threads);
    return lfm2_step(m->lfm2, st->lfm2, token, logits, &trace, m->src.threads);
}

// Read the state the GPU path must reproduce. Each returns the float count and fills `out` when
// it is non-null.
uint64_t orc_state_conv(void* sp, uint32_t index, float* out) {
    State* st = (State*)sp;
    const std::vector<float>* v;
    if (st->model->is_qwen) v = &st->qwen.rec_conv[index];
    else v = &st->lfm2.conv_history;
    if (out) std::memcpy(out, v->data(), v->size() * 4);
    return v->size();
}
uint64_t orc_state_delta(void* sp, uint32_t index, float* out) {
    State* st = (State*)sp;
    if (!st->model->is_qwen) return 0;
    const std::vector<float>& v = st->qwen.rec_state[index];
    if (out) std::memcpy(out, v.data(), v.size() * 4);
    return v.size();
}
// K (which = 0) or V (which = 1) cache of attention layer `index`: n_ctx rows of kv_dim floats.
uint64_t orc_state_kv(void* sp, uint32_t index, int which, float* out) {
    State* st = (State*)sp;
    const float* p;
    size_t n;
    if (st->model->is_qwen) {
        const std::vector<float>& v = which ? st->qwen.cache_v[index] : st->qwen.cache_k[index];
        p = v.data();
        n = v.size();
    } else {
        const Lfm2& m = st->model->lfm2;
        n = (size_t)st->lfm2.n_ctx * m.n_kv_heads * m.head_dim;
        p = (which ? st->lfm2.v_cache.data() : st->lfm2.k_cache.data()) + index * n;
    }
    if (out) std::memcpy(out, p, n * 4);
    return n;
}

// Scalar ops, for the per-kernel parity tests.
void orc_dequantize(uint32_t type, const void* bytes, uint64_t n, float* out) { dequantize(type, (const uint8_t*)bytes, n, out); }
void orc_matvec(uint32_t type, const void* w, const float* x, uint64_t n_cols, float* y, uint64_t n_rows, int threads) {
    matvec(type, (const uint8_t*)w, x, n_cols, y, n_rows, threads);
}
void orc_rms_norm(const float* x, const float* w, uint64_t n, float eps, float* out) { rms_norm(x, w, n, eps, out); }
void orc_rope_neox(float* vec, uint64_t len, uint32_t pos, float theta) { rope_neox(vec, len, pos, theta); }
void orc_softmax(float* x, uint64_t n) { softmax(x, n); }
float orc_silu(float x) { return silu(x); }
float orc_dot(const float* a, const float* b, uint64_t n) { return dot(a, b, n); }
void orc_lfm2_route(float* scores, const float* bias, uint64_t n_experts, uint64_t n_used, uint32_t* experts) {
    lfm2_route(scores, bias, n_experts, n_used, experts);
}
float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

}  // extern "C"
