#include "seq.h"

#include <algorithm>
#include <initializer_list>
#include <cstring>

using namespace bc;

namespace bc {
bc_status model_check_supported(const bc_model& m);
}

namespace {

using Clock = std::chrono::steady_clock;
double since(Clock::time_point start) { return std::chrono::duration<double>(Clock::now() - start).count(); }

// Records forward passes of one sequence onto its backend's stream.
struct Recorder {
    bc_seq& s;
    const bc_hparams& hp;
    cudaStream_t stream;
    bc_status status = BC_OK;
    // When set, single-token passes read their position from s.step_pos on the device, so the
    // launches can be captured once and replayed at every position.
    bool replayed = false;
    // Traced passes of a mixture-of-experts model: where the next router launch's routes are copied to.
    uint32_t* route_trace = nullptr;

    explicit Recorder(bc_seq& seq) : s(seq), hp(seq.model->hp), stream(seq.backend->stream) {}

    k::Pos at(uint32_t pos) const { return replayed ? k::Pos{s.step_pos, 0} : k::Pos{nullptr, pos}; }

    // Launch helper: counts the kernel, keeps the first failure.
    template <typename F>
    void run(const char* name, uint32_t rows, uint32_t cols, uint64_t bytes, int kernels, F&& f) {
        if (status != BC_OK) return;
        // Timing diagnostics: a launch kind left out of the pass (its outputs keep stale values).
        if (!s.skip_name.empty() && s.skip_name == name && (s.skip_rows == 0 || s.skip_rows == rows) && (s.skip_cols == 0 || s.skip_cols == cols)) return;
        s.launches += (uint64_t)kernels;
        status = s.backend->run(name, rows, cols, bytes, kernels, f);
    }

    k::Norm norm(const float* weight) const { return k::Norm{weight, hp.norm_eps}; }

    void matvec(const k::Mat& w, const float* x, float* y, k::Norm nm, bool accumulate) {
        k::MatvecSegment seg{w, y};
        run("matvec", w.n_rows, w.n_cols, w.bytes(), 1, [&] { return k::matvec(stream, &seg, 1, x, nm, accumulate); });
    }

    void matmul(const k::Mat& w, const float* x, float* y, uint32_t n, int store) {
        void* pack = nullptr;
        if (status == BC_OK && k::matmul_umma_supported(w, n)) status = s.backend->pack_scratch(k::matmul_scratch_bytes(w, n), &pack);
        run("matmul", w.n_rows, w.n_cols, w.bytes(), pack ? k::matmul_umma_launches(w, n) : 1, [&] { return k::matmul(stream, w, x, y, n, w.n_rows, store, pack); });
    }

    // RMSNorm of the batch, then products that all read the normalised rows. When every product
    // runs on the tensor-core kernel the normalised rows are packed to fp16 once, straight from the
    // residual stream, and the f32 copy is never written; otherwise s.normed takes them first.
    struct Product {
        const k::Mat* w;
        float* y;
        int store;
    };
    // ffn = silu(gate x^) * (up x^) over the batch, x^ the normalised rows.
    void normed_swiglu(const float* x, const float* norm_weight, uint32_t n, const k::Mat& gate, const k::Mat& up, float* y) {
        if (!k::matmul_umma_swiglu_supported(gate, up, n)) {
            // The up projection's store combines with the gate projection already in the buffer.
            normed_matmuls(x, norm_weight, n, {{&gate, y, BC_STORE_OVERWRITE}, {&up, y, BC_STORE_SWIGLU}});
            return;
        }
        const uint32_t cols = hp.n_embd;
        void* scratch = nullptr;
        if (status == BC_OK) status = s.backend->pack_scratch(k::matmul_pack_bytes(n, cols), &scratch);
        run("pack_norm", n, cols, 0, 1, [&] { return k::matmul_pack_norm(stream, x, norm(norm_weight), n, cols, scratch); });
        run("matmul_swiglu", gate.n_rows, gate.n_cols, 2 * gate.bytes(), 1,
            [&] { return k::matmul_umma_swiglu(stream, gate, up, scratch, y, n, gate.n_rows); });
    }

    void normed_matmuls(const float* x, const float* norm_weight, uint32_t n, std::initializer_list<Product> products) {
        const uint32_t cols = hp.n_embd;
        bool fused = true;
        size_t bytes = 0;
        for (const Product& q : products) {
            fused = fused && k::matmul_umma_supported(*q.w, n);
            bytes = std::max(bytes, (size_t)k::matmul_scratch_bytes(*q.w, n));
        }
        if (!fused) {
            run("rms_norm", n, cols, 0, 1, [&] { return k::rms_norm(stream, x, norm_weight, s.normed, cols, n, hp.norm_eps); });
            for (const Product& q : products) matmul(*q.w, s.normed, q.y, n, q.store);
            return;
        }
        void* scratch = nullptr;
        if (status == BC_OK) status = s.backend->pack_scratch(bytes, &scratch);
        run("pack_norm", n, cols, 0, 1, [&] { return k::matmul_pack_norm(stream, x, norm(norm_weight), n, cols, scratch); });
        for (const Product& q : products) {
            const k::Mat& w = *q.w;
            run("matmul", w.n_rows, w.n_cols, w.bytes(), k::matmul_umma_launches(w, n) - 1,
                [&] { return k::matmul_umma(stream, w, scratch, q.y, n, w.n_rows, q.store); });
        }
    }

    size_t kv_element_bytes() const { return s.kv_half ? 2 : 4; }
    size_t kv_dim() const { return (size_t)hp.n_kv_heads * hp.head_dim; }
    // lfm2_metal.rs:1064-1067: layer-major, then position, then KV head, then element.
    size_t layer_base(uint32_t cache_index) const { return (size_t)cache_index * s.n_ctx * kv_dim(); }
    void* cache_at(void* cache, size_t element) const { return static_cast<char*>(cache) + element * kv_element_bytes(); }

    // ---- LFM2 (lfm2_metal.rs:993-1156)

    void lfm2_conv(const DeviceLayer& D, uint32_t cache_index) {
        float* history = s.conv_state + (size_t)cache_index * (hp.conv_kernel - 1) * hp.n_embd;
        run("matvec_conv", 3 * hp.n_embd, D.in_proj.n_cols, D.in_proj.bytes(), 1, [&] {
            return k::matvec_conv(stream, D.in_proj, s.hidden, norm(D.attn_norm), D.taps, history, s.conv_out, hp.n_embd, hp.conv_kernel);
        });
        matvec(D.out_proj, s.conv_out, s.hidden, k::Norm{}, true);
    }

    // Norm and rotation of q and k, cache stores, attention over positions [0, pos + n).
    void rotate_and_attend(const DeviceLayer& D, uint32_t cache_index, uint32_t pos, uint32_t n, uint32_t q_stride, uint32_t q_head_stride) {
        size_t slot = layer_base(cache_index) + (size_t)pos * kv_dim();
        run("norm_rope", hp.n_heads * n, hp.head_dim, 0, 1, [&] {
            return k::norm_rope(stream, s.q, s.q, false, D.q_norm, hp.n_heads, hp.head_dim, q_head_stride, hp.n_rot, pos, n, q_stride, q_stride,
                                hp.rope_theta, hp.norm_eps);
        });
        run("norm_rope", hp.n_kv_heads * n, hp.head_dim, 0, 1, [&] {
            return k::norm_rope(stream, s.k, cache_at(s.k_cache, slot), s.kv_half, D.k_norm, hp.n_kv_heads, hp.head_dim, hp.head_dim, hp.n_rot,
                                pos, n, (uint32_t)kv_dim(), (uint32_t)kv_dim(), hp.rope_theta, hp.norm_eps);
        });
        if (s.kv_half)
            run("convert_half", 1, n * (uint32_t)kv_dim(), 0, 1,
                [&] { return k::convert_half(stream, s.v, static_cast<__half*>(cache_at(s.v_cache, slot)), (uint64_t)n * kv_dim()); });
        k::AttentionShape shape{hp.n_heads, hp.n_kv_heads, hp.head_dim, pos, n, s.n_ctx, q_stride, q_head_stride};
        int kernels = k::attention_launches(s.kv_half, shape);
        uint64_t kv_bytes = (uint64_t)(pos + n) * kv_dim() * kv_element_bytes() * 2;
        run("attention", n, pos + n, kv_bytes, kernels, [&] {
            return k::attention(stream, s.q, cache_at(s.k_cache, layer_base(cache_index)), cache_at(s.v_cache, layer_base(cache_index)), s.kv_half,
                                s.scores, s.attn, shape);
        });
    }

    float* value_target(uint32_t cache_index, uint32_t pos) {
        if (s.kv_half) return s.v;
        return static_cast<float*>(cache_at(s.v_cache, layer_base(cache_index) + (size_t)pos * kv_dim()));
    }

    // One token: norm and rotation of q and k, the K and V rows of position `pos` into the caches
    // (one launch), then attention over positions [0, pos].
    void decode_attend(const DeviceLayer& D, uint32_t cache_index, uint32_t pos, uint32_t q_stride, uint32_t q_head_stride) {
        k::RopeStore rs{s.q, s.k, s.v, cache_at(s.k_cache, layer_base(cache_index)), cache_at(s.v_cache, layer_base(cache_index)),
                        D.q_norm, D.k_norm, hp.n_heads, hp.n_kv_heads, hp.head_dim, q_head_stride, hp.n_rot, hp.rope_theta, hp.norm_eps, s.kv_half, s.rope_table};
        k::Pos p = at(pos);
        k::AttentionShape shape{hp.n_heads, hp.n_kv_heads, hp.head_dim, p.value, 1, s.n_ctx, q_stride, q_head_stride, p.ptr};
        uint64_t kv_bytes = (uint64_t)(pos + 1) * kv_dim() * kv_element_bytes() * 2;
        if (k::attention_step_supported(rs, shape)) {
            run("attention_step", 1, pos + 1, kv_bytes, 2, [&] { return k::attention_step(stream, rs, s.scores, s.attn, shape); });
            return;
        }
        run("rope_store", hp.n_heads + 2 * hp.n_kv_heads, hp.head_dim, 0, 1, [&] { return k::rope_store(stream, rs, p); });
        run("attention", 1, pos + 1, kv_bytes, k::attention_launches(s.kv_half, shape), [&] {
            return k::attention(stream, s.q, cache_at(s.k_cache, layer_base(cache_index)), cache_at(s.v_cache, layer_base(cache_index)), s.kv_half,
                                s.scores, s.attn, shape);
        });
    }

    void lfm2_attention(const DeviceLayer& D, uint32_t cache_index, uint32_t pos) {
        // The three projections share the normalised input, so one launch computes them.
        k::MatvecSegment segs[3] = {{D.q, s.q}, {D.k, s.k}, {D.v, s.v}};
        uint64_t bytes = D.q.bytes() + D.k.bytes() + D.v.bytes();
        run("matvec_qkv", D.q.n_rows + D.k.n_rows + D.v.n_rows, D.q.n_cols, bytes, 1,
            [&] { return k::matvec(stream, segs, 3, s.hidden, norm(D.attn_norm), false); });
        uint32_t q_dim = hp.n_heads * hp.head_dim;
        decode_attend(D, cache_index, pos, q_dim, hp.head_dim);
        matvec(D.output, s.attn, s.hidden, k::Norm{}, true);
    }

    void lfm2_dense_ffn(const DeviceLayer& D) {
        run("matvec_swiglu", D.gate.n_rows, D.gate.n_cols, D.gate.bytes() * 2, 1,
            [&] { return k::matvec_swiglu(stream, D.gate, D.up, s.hidden, norm(D.ffn_norm), s.ffn); });
        matvec(D.down, s.ffn, s.hidden, k::Norm{}, true);
    }

    // The mixture of experts on the n tokens of the batch, added to the residual stream
    // (lfm2_metal.rs:1251-1370). With `fused_norm` the router launch normalises the residual stream
    // into the normed buffer first; otherwise the normed buffer already holds the tokens. One token
    // runs matrix-vector products on its experts; a batch groups its tokens by expert so each
    // expert's weights stream once.
    void lfm2_moe(const DeviceLayer& D, uint32_t n, bool fused_norm) {
        const uint32_t n_used = hp.n_experts_used, n_ff = hp.n_ff_expert, n_embd = hp.n_embd;
        const float* input = fused_norm ? s.hidden : s.normed;
        k::Norm nm = fused_norm ? norm(D.ffn_norm) : k::Norm{};
        run("moe_route", hp.n_experts, n_embd, D.router.bytes(), 1, [&] {
            return k::moe_route(stream, input, nm, s.normed, static_cast<const float*>(D.router.data), D.expert_bias, s.route, n_embd, hp.n_experts,
                                n_used, n);
        });
        if (route_trace) run("copy", 1, n * 2 * n_used, 0, 0, [&] {
            return k::copy_floats(stream, reinterpret_cast<const float*>(s.route), reinterpret_cast<float*>(route_trace), (uint64_t)n * 2 * n_used);
        });
        // Bytes the experts stream: the picked experts of each token (decode) or every expert once (batch).
        uint64_t expert_bytes = D.gate.bytes() / hp.n_experts;
        if (n == 1) {
            run("matvec_experts_swiglu", n_ff, n_embd, 2 * expert_bytes * n_used, 1,
                [&] { return k::matvec_experts_swiglu(stream, D.gate, D.up, n_ff, s.normed, s.route, n_used, s.ffn, n); });
            run("matvec_experts_down", n_embd, n_ff, expert_bytes * n_used, k::matvec_experts_down_launches(D.down, n_embd, n_used, n, true),
                [&] { return k::matvec_experts_down(stream, D.down, n_embd, s.ffn, s.route, n_used, s.hidden, n, s.expert_out); });
            return;
        }
        run("moe_group", n, hp.n_experts, 0, 1, [&] { return k::moe_group(stream, s.route, s.expert_offsets, s.expert_entries, hp.n_experts, n_used, n); });
        // Q4_0 experts run on the tensor-core kernel in its grouped mode, from a gathered fp16 packing.
        void* up_scratch = nullptr;
        void* down_scratch = nullptr;
        const bool tensor_up = k::matmul_experts_umma_supported(D.gate, &D.up, n), tensor_down = k::matmul_experts_umma_supported(D.down, nullptr, n);
        if (status == BC_OK && (tensor_up || tensor_down)) {
            size_t bytes = (size_t)std::max(tensor_up ? k::matmul_experts_scratch_bytes(hp.n_experts, n, n_embd) : 0,
                                            tensor_down ? k::matmul_experts_scratch_bytes(hp.n_experts, n, n_ff) : 0);
            void* scratch = nullptr;
            status = s.backend->pack_scratch(bytes, &scratch);
            if (tensor_up) up_scratch = scratch;
            if (tensor_down) down_scratch = scratch;
        }
        run("matmul_experts", n_ff, n_embd, 2 * D.gate.bytes(), up_scratch ? 2 : 1, [&] {
            return k::matmul_experts(stream, D.gate, &D.up, n_ff, hp.n_experts, s.normed, true, s.expert_offsets, s.expert_entries, n_used, s.ffn, n,
                                     up_scratch);
        });
        run("matmul_experts", n_embd, n_ff, D.down.bytes(), down_scratch ? 2 : 1, [&] {
            return k::matmul_experts(stream, D.down, nullptr, n_embd, hp.n_experts, s.ffn, false, s.expert_offsets, s.expert_entries, n_used,
                                     s.expert_out, n, down_scratch);
        });
        run("moe_combine", n, n_embd, 0, 1, [&] { return k::moe_combine(stream, s.expert_out, s.route, s.hidden, n_embd, n_used, n); });
    }

    void copy(const float* src, float* dst, uint64_t n) {
        run("copy", 1, (uint32_t)n, 0, 0, [&] { return k::copy_floats(stream, src, dst, n); });
    }

    // lfm2_metal.rs:1162-1242
    void lfm2_step(uint32_t pos, bool want_logits, bool traced) {
        const DeviceModel& W = *s.weights;
        run("embed", 1, hp.n_embd, 0, 1, [&] { return k::embed(stream, W.token_embd, s.tokens, at(pos), s.hidden, 1); });
        if (traced) copy(s.hidden, s.trace_embedding, hp.n_embd);
        for (size_t il = 0; il < W.layers.size(); ++il) {
            const LayerSpec& S = s.model->layers[il];
            const DeviceLayer& D = W.layers[il];
            if (S.mixer == Mixer::Attention) lfm2_attention(D, S.cache_index, pos);
            else lfm2_conv(D, S.cache_index);
            if (S.moe) {
                route_trace = traced ? s.trace_routes + il * (size_t)s.trace_rows * 2 * hp.n_experts_used : nullptr;
                lfm2_moe(D, 1, true);
            } else lfm2_dense_ffn(D);
            if (traced) copy(s.hidden, s.trace_layers + il * hp.n_embd, hp.n_embd);
        }
        if (traced)
            run("rms_norm", 1, hp.n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, W.output_norm, s.trace_final, hp.n_embd, 1, hp.norm_eps); });
        if (want_logits) matvec(W.output, s.hidden, s.logits, norm(W.output_norm), false);
    }

    // lfm2_metal.rs:1455-1548
    void lfm2_batch(uint32_t pos, uint32_t n, bool want_logits, bool traced, size_t trace_stride) {
        const DeviceModel& W = *s.weights;
        const uint32_t n_embd = hp.n_embd;
        run("embed", n, n_embd, 0, 1, [&] { return k::embed(stream, W.token_embd, s.tokens, k::Pos{nullptr, pos}, s.hidden, n); });
        if (traced) copy(s.hidden, s.trace_embedding, (uint64_t)n * n_embd);
        for (size_t il = 0; il < W.layers.size(); ++il) {
            const LayerSpec& S = s.model->layers[il];
            const DeviceLayer& D = W.layers[il];
            if (S.mixer == Mixer::Attention) {
                normed_matmuls(s.hidden, D.attn_norm, n,
                               {{&D.q, s.q, BC_STORE_OVERWRITE}, {&D.k, s.k, BC_STORE_OVERWRITE}, {&D.v, value_target(S.cache_index, pos), BC_STORE_OVERWRITE}});
                uint32_t q_dim = hp.n_heads * hp.head_dim;
                rotate_and_attend(D, S.cache_index, pos, n, q_dim, hp.head_dim);
                matmul(D.output, s.attn, s.hidden, n, BC_STORE_ACCUMULATE);
            } else {
                float* history = s.conv_state + (size_t)S.cache_index * (hp.conv_kernel - 1) * n_embd;
                normed_matmuls(s.hidden, D.attn_norm, n, {{&D.in_proj, s.bcx, BC_STORE_OVERWRITE}});
                run("short_conv", n, n_embd, 0, 2,
                    [&] { return k::short_conv(stream, s.bcx, D.taps, history, s.conv_out, n_embd, hp.conv_kernel, n); });
                matmul(D.out_proj, s.conv_out, s.hidden, n, BC_STORE_ACCUMULATE);
            }
            if (S.moe) {
                run("rms_norm", n, n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, D.ffn_norm, s.normed, n_embd, n, hp.norm_eps); });
                route_trace = traced ? s.trace_routes + il * (size_t)s.trace_rows * 2 * hp.n_experts_used : nullptr;
                lfm2_moe(D, n, false);
            } else {
                normed_swiglu(s.hidden, D.ffn_norm, n, D.gate, D.up, s.ffn);
                matmul(D.down, s.ffn, s.hidden, n, BC_STORE_ACCUMULATE);
            }
            if (traced) copy(s.hidden, s.trace_layers + il * trace_stride, (uint64_t)n * n_embd);
        }
        if (traced)
            run("rms_norm", n, n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, W.output_norm, s.trace_final, n_embd, n, hp.norm_eps); });
        if (want_logits) matvec(W.output, s.hidden + (size_t)(n - 1) * n_embd, s.logits, norm(W.output_norm), false);
    }

    // ---- Qwen3.5 (qwen35_metal.rs:867-1134)

    uint32_t conv_dim() const { return 2 * hp.n_k_heads * hp.k_head_dim + hp.n_v_heads * hp.v_head_dim; }
    uint32_t value_dim() const { return hp.n_v_heads * hp.v_head_dim; }

    // The DeltaNet mixer from the conv onward, over n tokens whose projections sit in gdn_qkv,
    // gdn_z, gdn_beta and gdn_alpha (qwen35_metal.rs:965-1033). The recurrence normalises q and k itself.
    void qwen_delta_tail(const DeviceLayer& D, uint32_t cache_index, uint32_t n) {
        const uint32_t K = hp.conv_kernel;
        float* history = s.conv_state + (size_t)cache_index * conv_dim() * (K - 1);
        float* state = s.delta_state + (size_t)cache_index * hp.n_v_heads * hp.k_head_dim * hp.v_head_dim;
        if (n == 1 && k::gdn_step_supported(hp.n_k_heads, hp.n_v_heads, hp.k_head_dim, hp.v_head_dim, K)) {
            // A decode step: the whole tail in one launch.
            uint64_t step_bytes = (uint64_t)hp.n_v_heads * hp.k_head_dim * hp.v_head_dim * 4 * 2;
            run("gdn_step", 1, value_dim(), step_bytes, 1, [&] {
                return k::gdn_step(stream, s.gdn_qkv, D.conv1d, history, s.gdn_beta, s.gdn_alpha, D.a, D.dt_bias, state, s.gdn_z, D.ssm_norm, s.gdn_out,
                                   hp.n_k_heads, hp.n_v_heads, hp.k_head_dim, hp.v_head_dim, K, hp.norm_eps);
            });
            return;
        }
        run("gdn_conv", n, conv_dim(), 0, k::gdn_conv_launches(n), [&] { return k::gdn_conv(stream, s.gdn_qkv, D.conv1d, history, s.gdn_conv_out, conv_dim(), K, n); });
        run("gdn_gates", n, hp.n_v_heads, 0, 1, [&] { return k::gdn_gates(stream, s.gdn_beta, s.gdn_alpha, D.a, D.dt_bias, hp.n_v_heads, n); });
        uint64_t state_bytes = (uint64_t)hp.n_v_heads * hp.k_head_dim * hp.v_head_dim * 4 * 2;
        run("gdn_recurrence", n, value_dim(), state_bytes, 1, [&] {
            return k::gdn_recurrence(stream, s.gdn_conv_out, s.gdn_beta, s.gdn_alpha, state, s.gdn_out, hp.n_k_heads, hp.n_v_heads, hp.k_head_dim,
                                     hp.v_head_dim, n, true);
        });
        run("gdn_gated_norm", n * hp.n_v_heads, hp.v_head_dim, 0, 1,
            [&] { return k::gdn_gated_norm(stream, s.gdn_out, s.gdn_z, D.ssm_norm, hp.v_head_dim, n * hp.n_v_heads, hp.norm_eps); });
    }

    // qwen35_metal.rs:1038-1134
    void qwen_step(uint32_t pos, bool want_logits, bool traced) {
        const DeviceModel& W = *s.weights;
        const uint32_t q_dim = hp.n_heads * hp.head_dim;
        run("embed", 1, hp.n_embd, 0, 1, [&] { return k::embed(stream, W.token_embd, s.tokens, at(pos), s.hidden, 1); });
        if (traced) copy(s.hidden, s.trace_embedding, hp.n_embd);
        for (size_t il = 0; il < W.layers.size(); ++il) {
            const LayerSpec& S = s.model->layers[il];
            const DeviceLayer& D = W.layers[il];
            if (S.mixer == Mixer::Attention) {
                // Each query head's rows hold its queries, then the gate of its output.
                k::MatvecSegment segs[3] = {{D.q, s.q}, {D.k, s.k}, {D.v, s.v}};
                run("matvec_qkv", D.q.n_rows + D.k.n_rows + D.v.n_rows, D.q.n_cols, D.q.bytes() + D.k.bytes() + D.v.bytes(), 1,
                    [&] { return k::matvec(stream, segs, 3, s.hidden, norm(D.attn_norm), false); });
                decode_attend(D, S.cache_index, pos, 2 * q_dim, 2 * hp.head_dim);
                run("attention_gate", 1, q_dim, 0, 1, [&] { return k::attention_gate(stream, s.attn, s.q, hp.n_heads, hp.head_dim, 1); });
                matvec(D.output, s.attn, s.hidden, k::Norm{}, true);
            } else {
                k::MatvecSegment segs[4] = {{D.qkv, s.gdn_qkv}, {D.z, s.gdn_z}, {D.beta, s.gdn_beta}, {D.alpha, s.gdn_alpha}};
                uint64_t bytes = D.qkv.bytes() + D.z.bytes() + D.beta.bytes() + D.alpha.bytes();
                run("matvec_delta", D.qkv.n_rows + D.z.n_rows + 2 * D.beta.n_rows, D.qkv.n_cols, bytes, 1,
                    [&] { return k::matvec(stream, segs, 4, s.hidden, norm(D.attn_norm), false); });
                qwen_delta_tail(D, S.cache_index, 1);
                matvec(D.ssm_out, s.gdn_out, s.hidden, k::Norm{}, true);
            }
            lfm2_dense_ffn(D);
            if (traced) copy(s.hidden, s.trace_layers + il * hp.n_embd, hp.n_embd);
        }
        if (traced)
            run("rms_norm", 1, hp.n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, W.output_norm, s.trace_final, hp.n_embd, 1, hp.norm_eps); });
        if (want_logits) matvec(W.output, s.hidden, s.logits, norm(W.output_norm), false);
    }

    // qwen35_metal.rs:1142-1240
    void qwen_batch(uint32_t pos, uint32_t n, bool want_logits, bool traced, size_t trace_stride) {
        const DeviceModel& W = *s.weights;
        const uint32_t n_embd = hp.n_embd, q_dim = hp.n_heads * hp.head_dim;
        run("embed", n, n_embd, 0, 1, [&] { return k::embed(stream, W.token_embd, s.tokens, k::Pos{nullptr, pos}, s.hidden, n); });
        if (traced) copy(s.hidden, s.trace_embedding, (uint64_t)n * n_embd);
        for (size_t il = 0; il < W.layers.size(); ++il) {
            const LayerSpec& S = s.model->layers[il];
            const DeviceLayer& D = W.layers[il];
            if (S.mixer == Mixer::Attention) {
                normed_matmuls(s.hidden, D.attn_norm, n,
                               {{&D.q, s.q, BC_STORE_OVERWRITE}, {&D.k, s.k, BC_STORE_OVERWRITE}, {&D.v, value_target(S.cache_index, pos), BC_STORE_OVERWRITE}});
                size_t slot = layer_base(S.cache_index) + (size_t)pos * kv_dim();
                // The rotated queries go to their own compact rows; the gates stay in the projection.
                run("norm_rope", hp.n_heads * n, hp.head_dim, 0, 1, [&] {
                    return k::norm_rope(stream, s.q, s.q_rot, false, D.q_norm, hp.n_heads, hp.head_dim, 2 * hp.head_dim, hp.n_rot, pos, n, 2 * q_dim,
                                        q_dim, hp.rope_theta, hp.norm_eps);
                });
                run("norm_rope", hp.n_kv_heads * n, hp.head_dim, 0, 1, [&] {
                    return k::norm_rope(stream, s.k, cache_at(s.k_cache, slot), s.kv_half, D.k_norm, hp.n_kv_heads, hp.head_dim, hp.head_dim,
                                        hp.n_rot, pos, n, (uint32_t)kv_dim(), (uint32_t)kv_dim(), hp.rope_theta, hp.norm_eps);
                });
                if (s.kv_half)
                    run("convert_half", 1, n * (uint32_t)kv_dim(), 0, 1,
                        [&] { return k::convert_half(stream, s.v, static_cast<__half*>(cache_at(s.v_cache, slot)), (uint64_t)n * kv_dim()); });
                k::AttentionShape shape{hp.n_heads, hp.n_kv_heads, hp.head_dim, pos, n, s.n_ctx, q_dim, hp.head_dim};
                run("attention", n, pos + n, (uint64_t)(pos + n) * kv_dim() * kv_element_bytes() * 2, k::attention_launches(s.kv_half, shape), [&] {
                    return k::attention(stream, s.q_rot, cache_at(s.k_cache, layer_base(S.cache_index)), cache_at(s.v_cache, layer_base(S.cache_index)),
                                        s.kv_half, s.scores, s.attn, shape);
                });
                run("attention_gate", n, q_dim, 0, 1, [&] { return k::attention_gate(stream, s.attn, s.q, hp.n_heads, hp.head_dim, n); });
                matmul(D.output, s.attn, s.hidden, n, BC_STORE_ACCUMULATE);
            } else {
                normed_matmuls(s.hidden, D.attn_norm, n,
                               {{&D.qkv, s.gdn_qkv, BC_STORE_OVERWRITE}, {&D.z, s.gdn_z, BC_STORE_OVERWRITE}, {&D.beta, s.gdn_beta, BC_STORE_OVERWRITE},
                                {&D.alpha, s.gdn_alpha, BC_STORE_OVERWRITE}});
                qwen_delta_tail(D, S.cache_index, n);
                matmul(D.ssm_out, s.gdn_out, s.hidden, n, BC_STORE_ACCUMULATE);
            }
            normed_swiglu(s.hidden, D.ffn_norm, n, D.gate, D.up, s.ffn);
            matmul(D.down, s.ffn, s.hidden, n, BC_STORE_ACCUMULATE);
            if (traced) copy(s.hidden, s.trace_layers + il * trace_stride, (uint64_t)n * n_embd);
        }
        if (traced)
            run("rms_norm", n, n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, W.output_norm, s.trace_final, n_embd, n, hp.norm_eps); });
        if (want_logits) matvec(W.output, s.hidden + (size_t)(n - 1) * n_embd, s.logits, norm(W.output_norm), false);
    }

    void step(uint32_t pos, bool want_logits, bool traced) {
        if (hp.architecture == BC_ARCH_QWEN35) qwen_step(pos, want_logits, traced);
        else lfm2_step(pos, want_logits, traced);
    }

    void batch(uint32_t pos, uint32_t n, bool want_logits, bool traced, size_t trace_stride) {
        if (hp.architecture == BC_ARCH_QWEN35) qwen_batch(pos, n, want_logits, traced, trace_stride);
        else lfm2_batch(pos, n, want_logits, traced, trace_stride);
    }

    void argmax(const float* x, uint32_t* out, uint32_t* readback) {
        run("argmax", 1, hp.n_vocab, 0, 1, [&] { return k::argmax(stream, x, hp.n_vocab, out, readback); });
    }
};

bc_status ensure_trace_rows(bc_seq* s, uint32_t rows) {
    if (rows <= s->trace_rows) return BC_OK;
    const bc_hparams& hp = s->model->hp;
    BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    cudaFree(s->trace_embedding);
    cudaFree(s->trace_layers);
    cudaFree(s->trace_final);
    cudaFree(s->trace_routes);
    s->trace_embedding = s->trace_layers = s->trace_final = nullptr;
    s->trace_routes = nullptr;
    s->trace_rows = 0;
    size_t floats = (size_t)rows * hp.n_embd;
    size_t route_words = std::max<size_t>(1, (size_t)rows * hp.n_layers * 2 * hp.n_experts_used);
    if (cudaMalloc(&s->trace_embedding, floats * 4) != cudaSuccess || cudaMalloc(&s->trace_layers, floats * 4 * hp.n_layers) != cudaSuccess ||
        cudaMalloc(&s->trace_final, floats * 4) != cudaSuccess || cudaMalloc(&s->trace_routes, route_words * 4) != cudaSuccess ||
        cudaMemset(s->trace_routes, 0, route_words * 4) != cudaSuccess)
        return fail(BC_ERR_ALLOCATION, "cannot allocate trace buffers for %u tokens", rows);
    s->trace_rows = rows;
    return BC_OK;
}

bc_status check_trace(const bc_seq* s, const bc_trace* trace, uint32_t n_tokens, const char* why) {
    if (!trace) return BC_OK;
    if (!trace->embedding || !trace->layers || !trace->final_norm || trace->n_tokens != n_tokens) return fail(BC_ERR_ARGUMENT, "%s", why);
    (void)s;
    return BC_OK;
}

bc_status read_floats(bc_seq* s, const float* device, float* host, size_t n) {
    BC_CUDA(cudaMemcpyAsync(host, device, n * 4, cudaMemcpyDeviceToHost, s->backend->stream));
    return BC_OK;
}

// Bracket recorded work with events so last_gpu_seconds reports device time.
bc_status timing_begin(bc_seq* s) {
    BC_CUDA(cudaEventRecord(s->timing_start, s->backend->stream));
    return BC_OK;
}

bc_status timing_end(bc_seq* s, double* seconds) {
    BC_CUDA(cudaEventRecord(s->timing_end, s->backend->stream));
    cudaError_t e = cudaEventSynchronize(s->timing_end);
    if (e != cudaSuccess) return cuda_fail(e, "recorded work");
    float ms = 0.f;
    cudaEventElapsedTime(&ms, s->timing_start, s->timing_end);
    *seconds = ms * 1e-3;
    return kernel_wait_status();
}

// Replay needs a stream that can be captured (not the legacy default stream) and no per-launch
// event timing.
bool replay_enabled(const bc_seq* s) {
    return s->use_graphs && !s->backend->profiling && s->backend->stream != nullptr && s->backend->stream != cudaStreamLegacy;
}

// Capture one generated step into a graph. The generate variant picks tokens[pos] from the logits,
// then runs the forward pass at pos; the stream variant runs the forward pass at pos, then picks
// tokens[pos + 1] and mirrors it into the host-mapped ring at slot pos % kGenerateInFlight. Both
// start by adding one to s->step_pos, so the host seeds it with the first position minus one.
bc_status capture_step(bc_seq* s, bool stream_variant) {
    cudaStream_t stream = s->backend->stream;
    const uint32_t n_vocab = s->model->hp.n_vocab;
    uint64_t before = s->launches;
    BC_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    Recorder r(*s);
    r.replayed = true;
    if (stream_variant) {
        r.run("advance", 1, 1, 0, 1, [&] { return k::advance(stream, s->step_pos); });
        r.step(0, true, false);
        r.run("argmax", 1, n_vocab, 0, 1,
              [&] { return k::argmax_step(stream, s->logits, n_vocab, s->step_pos, false, s->tokens, 1, s->readback, kGenerateInFlight); });
    } else {
        r.run("argmax", 1, n_vocab, 0, 1,
              [&] { return k::argmax_step(stream, s->logits, n_vocab, s->step_pos, true, s->tokens, 0, nullptr, 1); });
        r.step(0, true, false);
    }
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(stream, &graph);
    uint64_t kernels = s->launches - before;
    s->launches = before;  // capturing launches nothing
    if (r.status != BC_OK) {
        if (graph) cudaGraphDestroy(graph);
        return r.status;
    }
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture");
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
    if (stream_variant) {
        s->stream_graph = exec;
        s->stream_graph_kernels = kernels;
    } else {
        s->generate_graph = exec;
        s->generate_graph_kernels = kernels;
    }
    return BC_OK;
}

// Make sure the wanted graph exists and seed the device position for a run that starts at `first`.
bc_status prepare_replay(bc_seq* s, bool stream_variant, uint32_t first) {
    if (stream_variant ? !s->stream_graph : !s->generate_graph) BC_TRY(capture_step(s, stream_variant));
    s->host_pos = first - 1;  // first >= 1: generation needs a prompt
    BC_CUDA(cudaMemcpyAsync(s->step_pos, &s->host_pos, 4, cudaMemcpyHostToDevice, s->backend->stream));
    return BC_OK;
}

bc_status generate_inner(bc_seq* s, uint32_t* out, size_t count, bool select_next) {
    if (!s || (!out && count)) return fail(BC_ERR_ARGUMENT, "seq and out must be non-null");
    if (count > UINT32_MAX) return fail(BC_ERR_ARGUMENT, "too many tokens");
    uint32_t n = (uint32_t)count;
    uint32_t remaining = s->n_ctx - s->n_past;
    if (s->n_past == 0) return fail(BC_ERR_ARGUMENT, "generation needs a prompt first");
    if (n > remaining) return fail(BC_ERR_CONTEXT_FULL, "context full: %u tokens requested, %u remaining", n, remaining);
    if (s->backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(s->backend->activate());
    if (n == 0) return BC_OK;

    auto encode_start = Clock::now();
    const bool replay = replay_enabled(s);
    if (replay) BC_TRY(prepare_replay(s, /*stream_variant=*/false, s->n_past));
    BC_TRY(timing_begin(s));
    Recorder r(*s);
    for (uint32_t i = 0; i < n && r.status == BC_OK; ++i) {
        uint32_t pos = s->n_past + i;
        // Bound the steps in flight, so the CPU runs only a few steps ahead of the device.
        int slot = (int)(i % kGenerateInFlight);
        if (i >= (uint32_t)kGenerateInFlight) {
            cudaError_t e = cudaEventSynchronize(s->slot_done[slot]);
            if (e != cudaSuccess) return cuda_fail(e, "generation step");
        }
        if (replay) {
            BC_CUDA(cudaGraphLaunch(s->generate_graph, s->backend->stream));
            s->launches += s->generate_graph_kernels;
        } else {
            r.argmax(s->logits, s->tokens + pos, nullptr);
            r.step(pos, true, false);
        }
        if (select_next && i + 1 == n) r.argmax(s->logits, s->greedy_token, nullptr);
        if (r.status == BC_OK) BC_CUDA(cudaEventRecord(s->slot_done[slot], s->backend->stream));
    }
    double encode = since(encode_start);
    double gpu = 0;
    bc_status finish = timing_end(s, &gpu);
    if (r.status != BC_OK) return r.status;
    BC_TRY(finish);

    BC_CUDA(cudaMemcpyAsync(out, s->tokens + s->n_past, (size_t)n * 4, cudaMemcpyDeviceToHost, s->backend->stream));
    BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    if (select_next) {
        std::rotate(out, out + 1, out + n);
        BC_CUDA(cudaMemcpyAsync(out + n - 1, s->greedy_token, 4, cudaMemcpyDeviceToHost, s->backend->stream));
        BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    }
    s->n_past += n;
    s->last_encode_seconds = encode;
    s->last_gpu_seconds = gpu;
    return BC_OK;
}

}  // namespace

bc_seq::~bc_seq() {
    if (backend) {
        cudaSetDevice(backend->device);
        cudaStreamSynchronize(backend->stream);
    }
    cudaFree(arena);
    cudaFree(trace_embedding);
    cudaFree(trace_layers);
    cudaFree(trace_final);
    cudaFree(trace_routes);
    if (readback) cudaFreeHost(readback);
    if (generate_graph) cudaGraphExecDestroy(generate_graph);
    if (stream_graph) cudaGraphExecDestroy(stream_graph);
    for (cudaEvent_t e : slot_done)
        if (e) cudaEventDestroy(e);
    if (timing_start) cudaEventDestroy(timing_start);
    if (timing_end) cudaEventDestroy(timing_end);
}

extern "C" {

bc_status bc_seq_new(bc_model* model, bc_backend* backend, uint32_t n_ctx, int32_t kv_half, bc_seq** out) {
    if (!model || !backend || !out) return fail(BC_ERR_ARGUMENT, "model, backend and out must be non-null");
    if (n_ctx == 0) return fail(BC_ERR_ARGUMENT, "the context must hold a token");
    BC_TRY(model_check_supported(*model));
    BC_TRY(backend->activate());
    std::unique_ptr<bc_seq> s(new bc_seq());
    s->model = model;
    s->backend = backend;
    s->n_ctx = n_ctx;
    s->kv_half = kv_half != 0;
    s->batch = std::min(n_ctx, kPrefillBatch);
    BC_TRY(model->device_model(backend, &s->weights));

    const bc_hparams& hp = model->hp;
    const size_t n_embd = hp.n_embd, rows = s->batch;
    const size_t kv_dim = (size_t)hp.n_kv_heads * hp.head_dim, q_dim = (size_t)hp.n_heads * hp.head_dim;
    const size_t q_width = hp.architecture == BC_ARCH_QWEN35 ? 2 * q_dim : q_dim;  // Qwen's q holds [q | gate]
    const size_t cache_bytes = (size_t)hp.n_attention_layers * n_ctx * kv_dim * (s->kv_half ? 2 : 4);
    const size_t key_dim = (size_t)hp.n_k_heads * hp.k_head_dim, value_dim = (size_t)hp.n_v_heads * hp.v_head_dim;
    const size_t conv_dim = 2 * key_dim + value_dim;
    const bool qwen = hp.architecture == BC_ARCH_QWEN35;
    // LFM2: [conv layer][K - 1][n_embd] of B*X products. Qwen3.5: [delta layer][channel][K - 1] raw inputs.
    s->conv_floats = qwen ? (size_t)hp.n_delta_layers * conv_dim * (hp.conv_kernel - 1) : (size_t)hp.n_conv_layers * (hp.conv_kernel - 1) * n_embd;
    s->delta_floats = (size_t)hp.n_delta_layers * hp.n_v_heads * hp.k_head_dim * hp.v_head_dim;
    const size_t ffn_width = std::max<size_t>(hp.n_ff, (size_t)hp.n_experts_used * hp.n_ff_expert);
    const size_t scratch_floats = hp.n_attention_layers ? k::attention_scratch_floats(hp.n_heads, hp.head_dim, n_ctx, s->batch) : 0;

    // Plan the arena: (pointer slot, bytes) pairs, each aligned to 256 bytes.
    struct Item { void** slot; size_t bytes; };
    std::vector<Item> items = {
        {&s->k_cache, cache_bytes},
        {&s->v_cache, cache_bytes},
        {(void**)&s->k, rows * kv_dim * 4},
        {(void**)&s->v, rows * kv_dim * 4},
        {(void**)&s->conv_state, s->conv_floats * 4},
        {(void**)&s->hidden, rows * n_embd * 4},
        {(void**)&s->normed, rows * n_embd * 4},
        {(void**)&s->bcx, rows * 3 * n_embd * 4},
        {(void**)&s->conv_out, rows * n_embd * 4},
        {(void**)&s->q, rows * q_width * 4},
        {(void**)&s->attn, rows * q_dim * 4},
        {(void**)&s->scores, scratch_floats * 4},
        {(void**)&s->ffn, rows * ffn_width * 4},
        {(void**)&s->logits, (size_t)hp.n_vocab * 4},
        {(void**)&s->tokens, ((size_t)n_ctx + 1) * 4},
        {(void**)&s->greedy_token, 4},
        {(void**)&s->route, rows * 2 * hp.n_experts_used * 4},
        {(void**)&s->expert_offsets, ((size_t)hp.n_experts + 1) * 4},
        {(void**)&s->expert_entries, rows * hp.n_experts_used * 4},
        {(void**)&s->expert_out, rows * hp.n_experts_used * n_embd * 4},
        {(void**)&s->delta_state, s->delta_floats * 4},
        {(void**)&s->gdn_qkv, rows * conv_dim * 4},
        {(void**)&s->gdn_conv_out, rows * conv_dim * 4},
        {(void**)&s->gdn_z, rows * value_dim * 4},
        {(void**)&s->gdn_beta, rows * hp.n_v_heads * 4},
        {(void**)&s->gdn_alpha, rows * hp.n_v_heads * 4},
        {(void**)&s->gdn_out, rows * value_dim * 4},
        {(void**)&s->q_rot, qwen ? rows * q_dim * 4 : 0},
        {(void**)&s->step_pos, 4},
        {(void**)&s->rope_table, hp.n_attention_layers && !qwen ? (size_t)n_ctx * (hp.n_rot / 2) * sizeof(float2) : 0},
    };
    const char* no_graph = getenv("BOBCAT_NO_GRAPH");
    s->use_graphs = !(no_graph && no_graph[0] == '1');
    // Kernels whose input vector outgrows the default shared-memory limit get their limit raised
    // now, so no launch inside a capture has to.
    uint32_t widest = std::max({hp.n_embd, hp.n_ff, hp.n_ff_expert, (uint32_t)q_dim, hp.n_v_heads * hp.v_head_dim});
    BC_CUDA(k::matvec_prepare(widest));
    size_t total = 0;
    for (Item& it : items) total += round_up(std::max<size_t>(it.bytes, 4), 256);
    cudaError_t e = cudaMalloc(&s->arena, total);
    if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate %zu bytes of sequence state: %s", total, cudaGetErrorString(e));
    s->arena_bytes = total;
    BC_CUDA(cudaMemsetAsync(s->arena, 0, total, backend->stream));
    char* p = static_cast<char*>(s->arena);
    for (Item& it : items) {
        *it.slot = p;
        p += round_up(std::max<size_t>(it.bytes, 4), 256);
    }
    if (hp.n_attention_layers && !qwen) BC_CUDA(k::rope_table(backend->stream, s->rope_table, n_ctx, hp.n_rot, hp.rope_theta));
    BC_TRY(ensure_trace_rows(s.get(), 1));
    e = cudaHostAlloc((void**)&s->readback, sizeof(uint32_t) * kGenerateInFlight, cudaHostAllocMapped);
    if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate the token readback: %s", cudaGetErrorString(e));
    for (int i = 0; i < kGenerateInFlight; ++i) BC_CUDA(cudaEventCreateWithFlags(&s->slot_done[i], cudaEventDisableTiming));
    BC_CUDA(cudaEventCreate(&s->timing_start));
    BC_CUDA(cudaEventCreate(&s->timing_end));
    BC_CUDA(cudaStreamSynchronize(backend->stream));
    *out = s.release();
    return BC_OK;
}

void bc_seq_free(bc_seq* seq) { delete seq; }
uint32_t bc_seq_n_past(const bc_seq* seq) { return seq ? seq->n_past : 0; }
uint64_t bc_seq_launches(const bc_seq* seq) { return seq ? seq->launches : 0; }

bc_status bc_seq_step(bc_seq* s, uint32_t token, float* logits, size_t logits_len, bc_trace* trace) {
    if (!s) return fail(BC_ERR_ARGUMENT, "seq must be non-null");
    const bc_hparams& hp = s->model->hp;
    uint32_t pos = s->n_past;
    if (pos >= s->n_ctx) return fail(BC_ERR_CONTEXT_FULL, "context full: 1 token requested, 0 remaining");
    if (token >= hp.n_vocab) return fail(BC_ERR_TOKEN, "token %u outside the vocabulary of %u", token, hp.n_vocab);
    if (logits && logits_len != hp.n_vocab) return fail(BC_ERR_ARGUMENT, "logits must hold n_vocab floats");
    BC_TRY(check_trace(s, trace, 1, "the trace must hold one token"));
    if (s->backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;

    BC_CUDA(cudaMemcpyAsync(s->tokens + pos, &token, 4, cudaMemcpyHostToDevice, stream));
    auto encode_start = Clock::now();
    BC_TRY(timing_begin(s));
    Recorder r(*s);
    r.step(pos, logits != nullptr, trace != nullptr);
    double encode = since(encode_start);
    double gpu = 0;
    bc_status finish = timing_end(s, &gpu);
    if (r.status != BC_OK) return r.status;
    BC_TRY(finish);
    if (logits) BC_TRY(read_floats(s, s->logits, logits, hp.n_vocab));
    if (trace) {
        BC_TRY(read_floats(s, s->trace_embedding, trace->embedding, hp.n_embd));
        BC_TRY(read_floats(s, s->trace_layers, trace->layers, (size_t)hp.n_layers * hp.n_embd));
        BC_TRY(read_floats(s, s->trace_final, trace->final_norm, hp.n_embd));
    }
    BC_CUDA(cudaStreamSynchronize(stream));
    s->n_past += 1;
    s->last_encode_seconds = encode;
    s->last_gpu_seconds = gpu;
    return BC_OK;
}

bc_status bc_seq_prefill(bc_seq* s, const uint32_t* tokens, size_t n_tokens, float* logits, size_t logits_len, float* final_norm,
                         size_t final_norm_len, bc_trace* trace) {
    if (!s || (!tokens && n_tokens)) return fail(BC_ERR_ARGUMENT, "seq and tokens must be non-null");
    const bc_hparams& hp = s->model->hp;
    if (n_tokens > UINT32_MAX) return fail(BC_ERR_ARGUMENT, "too many tokens");
    uint32_t n = (uint32_t)n_tokens, remaining = s->n_ctx - s->n_past;
    if (n == 0) return fail(BC_ERR_ARGUMENT, "the prompt must hold a token");
    if (n > remaining) return fail(BC_ERR_CONTEXT_FULL, "context full: %u tokens requested, %u remaining", n, remaining);
    for (uint32_t i = 0; i < n; ++i)
        if (tokens[i] >= hp.n_vocab) return fail(BC_ERR_TOKEN, "token %u outside the vocabulary of %u", tokens[i], hp.n_vocab);
    if (logits && logits_len != hp.n_vocab) return fail(BC_ERR_ARGUMENT, "logits must hold n_vocab floats");
    if (final_norm && final_norm_len != hp.n_embd) return fail(BC_ERR_ARGUMENT, "final_norm must hold n_embd floats");
    BC_TRY(check_trace(s, trace, n, "the trace must hold every prompt token"));
    if (s->backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;
    const size_t n_embd = hp.n_embd;

    BC_CUDA(cudaMemcpyAsync(s->tokens + s->n_past, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, stream));
    // Qwen's final_norm output comes from the trace buffer of the last batch.
    bool traced = trace != nullptr;
    if (traced || final_norm) BC_TRY(ensure_trace_rows(s, s->batch));

    double encode = 0, gpu = 0;
    BC_TRY(timing_begin(s));
    uint32_t done = 0;
    while (done < n) {
        uint32_t count = std::min(n - done, s->batch);
        uint32_t pos = s->n_past + done;
        bool last = done + count == n;
        auto encode_start = Clock::now();
        Recorder r(*s);
        size_t layer_stride = (size_t)s->trace_rows * n_embd;
        r.batch(pos, count, last, traced || (final_norm && last), layer_stride);
        encode += since(encode_start);
        if (r.status != BC_OK) {
            cudaStreamSynchronize(stream);
            return r.status;
        }
        if (traced) {
            // A traced batch is copied out before the next batch overwrites the trace buffers.
            size_t start = (size_t)done * n_embd, row_floats = (size_t)count * n_embd;
            BC_TRY(read_floats(s, s->trace_embedding, trace->embedding + start, row_floats));
            BC_TRY(read_floats(s, s->trace_final, trace->final_norm + start, row_floats));
            for (uint32_t il = 0; il < hp.n_layers; ++il)
                BC_TRY(read_floats(s, s->trace_layers + il * layer_stride, trace->layers + ((size_t)il * n + done) * n_embd, row_floats));
            BC_CUDA(cudaStreamSynchronize(stream));
        }
        if (final_norm && last) BC_TRY(read_floats(s, s->trace_final + (size_t)(count - 1) * n_embd, final_norm, n_embd));
        done += count;
    }
    BC_TRY(timing_end(s, &gpu));
    if (logits) BC_TRY(read_floats(s, s->logits, logits, hp.n_vocab));
    BC_CUDA(cudaStreamSynchronize(stream));
    s->n_past += n;
    s->last_encode_seconds = encode;
    s->last_gpu_seconds = gpu;
    return BC_OK;
}

bc_status bc_seq_greedy_token(bc_seq* s, uint32_t* token) {
    if (!s || !token) return fail(BC_ERR_ARGUMENT, "seq and token must be non-null");
    if (s->n_past == 0) return fail(BC_ERR_ARGUMENT, "generation needs a prompt first");
    if (s->backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(s->backend->activate());
    auto start = Clock::now();
    BC_TRY(timing_begin(s));
    Recorder r(*s);
    r.argmax(s->logits, s->greedy_token, nullptr);
    double encode = since(start), gpu = 0;
    bc_status finish = timing_end(s, &gpu);
    if (r.status != BC_OK) return r.status;
    BC_TRY(finish);
    BC_CUDA(cudaMemcpyAsync(token, s->greedy_token, 4, cudaMemcpyDeviceToHost, s->backend->stream));
    BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    s->last_encode_seconds = encode;
    s->last_gpu_seconds = gpu;
    return BC_OK;
}

bc_status bc_seq_generate(bc_seq* s, uint32_t* out, size_t n) { return generate_inner(s, out, n, false); }
bc_status bc_seq_generate_next(bc_seq* s, uint32_t* out, size_t n) { return generate_inner(s, out, n, true); }

bc_status bc_seq_generate_stream(bc_seq* s, uint32_t max_tokens, bc_emit_fn emit, void* user, uint32_t* gained, size_t gained_cap,
                                 size_t* n_gained) {
    if (!s || !emit || !n_gained) return fail(BC_ERR_ARGUMENT, "seq, emit and n_gained must be non-null");
    *n_gained = 0;
    if (max_tokens == 0) return BC_OK;
    uint32_t first = 0;
    BC_TRY(bc_seq_greedy_token(s, &first));
    if (!emit(first, user)) return BC_OK;
    // Each step runs one token and selects the next, so the first token needs no step.
    uint32_t steps = std::min(max_tokens - 1, s->n_ctx - s->n_past);
    if (gained_cap < steps && !(gained == nullptr && steps == 0))
        if (gained_cap < steps) return fail(BC_ERR_ARGUMENT, "gained must hold %u tokens", steps);
    uint32_t start = s->n_past;
    cudaStream_t stream = s->backend->stream;
    bool emitting = true;
    uint32_t committed = 0;
    bool pending[kGenerateInFlight] = {};
    double encode = 0;
    bc_status result = BC_OK;
    BC_TRY(timing_begin(s));

    auto finish_slot = [&](int slot) -> bc_status {
        cudaError_t e = cudaEventSynchronize(s->slot_done[slot]);
        pending[slot] = false;
        if (e != cudaSuccess) return cuda_fail(e, "generation step");
        if (emitting) emitting = emit(s->readback[slot], user) != 0;
        return BC_OK;
    };
    const bool replay = replay_enabled(s);
    if (replay && steps > 0) {
        Recorder first_pick(*s);
        first_pick.argmax(s->logits, s->tokens + start, nullptr);
        if (first_pick.status != BC_OK) return first_pick.status;
        BC_TRY(prepare_replay(s, /*stream_variant=*/true, start));
    }

    for (uint32_t step = 0; step < steps; ++step) {
        // The slot's previous step selected the token that goes out next. A step at position p
        // uses slot p % kGenerateInFlight, which is also where the replayed argmax writes.
        uint32_t pos = start + step;
        int slot = (int)(pos % kGenerateInFlight);
        if (pending[slot] && (result = finish_slot(slot)) != BC_OK) break;
        if (!emitting) break;
        auto encode_start = Clock::now();
        Recorder r(*s);
        if (replay) {
            cudaError_t ge = cudaGraphLaunch(s->stream_graph, stream);
            if (ge != cudaSuccess) r.status = cuda_fail(ge, "cudaGraphLaunch");
            else s->launches += s->stream_graph_kernels;
        } else {
            if (step == 0) r.argmax(s->logits, s->tokens + pos, nullptr);
            r.step(pos, true, false);
            // tokens has n_ctx + 1 slots, so the pick at the last position has a place to go.
            r.argmax(s->logits, s->tokens + pos + 1, s->readback + slot);
        }
        if (r.status != BC_OK) {
            result = r.status;
            break;
        }
        cudaError_t e = cudaEventRecord(s->slot_done[slot], stream);
        if (e != cudaSuccess) {
            result = cuda_fail(e, "cudaEventRecord");
            break;
        }
        pending[slot] = true;
        ++committed;
        encode += since(encode_start);
    }
    // Finish the steps still in flight in submission order, which is the order of their tokens.
    for (int offset = 0; offset < kGenerateInFlight; ++offset) {
        int slot = (int)((start + committed + offset) % kGenerateInFlight);
        if (!pending[slot]) continue;
        bc_status st = finish_slot(slot);
        if (st != BC_OK && result == BC_OK) result = st;
    }
    double gpu = 0;
    bc_status finish = timing_end(s, &gpu);
    s->n_past += committed;
    s->last_encode_seconds = encode;
    s->last_gpu_seconds = gpu;
    if (result != BC_OK) return result;
    BC_TRY(finish);
    if (committed) {
        BC_CUDA(cudaMemcpyAsync(gained, s->tokens + start, (size_t)committed * 4, cudaMemcpyDeviceToHost, stream));
        BC_CUDA(cudaStreamSynchronize(stream));
    }
    *n_gained = committed;
    return BC_OK;
}

bc_status bc_seq_reset(bc_seq* s) {
    if (!s) return fail(BC_ERR_ARGUMENT, "seq must be non-null");
    BC_TRY(s->backend->activate());
    // A new sequence starts from zero convolution history (and zero DeltaNet state). The KV cache
    // needs no clearing, because attention reads only the positions a sequence has written.
    if (s->conv_floats) BC_CUDA(cudaMemsetAsync(s->conv_state, 0, s->conv_floats * 4, s->backend->stream));
    if (s->delta_floats) BC_CUDA(cudaMemsetAsync(s->delta_state, 0, s->delta_floats * 4, s->backend->stream));
    BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    s->n_past = 0;
    s->resets += 1;
    return BC_OK;
}

bc_status bc_seq_checkpoint(bc_seq* s, bc_checkpoint** out) {
    if (!s || !out) return fail(BC_ERR_ARGUMENT, "seq and out must be non-null");
    BC_TRY(s->backend->activate());
    std::unique_ptr<bc_checkpoint> c(new bc_checkpoint());
    c->owner = s;
    c->resets = s->resets;
    c->n_past = s->n_past;
    c->conv_state.resize(s->conv_floats);
    c->logits.resize(s->model->hp.n_vocab);
    cudaStream_t stream = s->backend->stream;
    if (s->conv_floats) BC_CUDA(cudaMemcpyAsync(c->conv_state.data(), s->conv_state, s->conv_floats * 4, cudaMemcpyDeviceToHost, stream));
    c->delta_state.resize(s->delta_floats);
    if (s->delta_floats) BC_CUDA(cudaMemcpyAsync(c->delta_state.data(), s->delta_state, s->delta_floats * 4, cudaMemcpyDeviceToHost, stream));
    BC_CUDA(cudaMemcpyAsync(c->logits.data(), s->logits, c->logits.size() * 4, cudaMemcpyDeviceToHost, stream));
    BC_CUDA(cudaStreamSynchronize(stream));
    *out = c.release();
    return BC_OK;
}

bc_status bc_seq_restore(bc_seq* s, const bc_checkpoint* c) {
    if (!s || !c) return fail(BC_ERR_ARGUMENT, "seq and checkpoint must be non-null");
    // A checkpoint holds the recurrent state only; the KV rows of its prefix live in the cache of
    // the sequence that took it, so no other sequence can continue from it.
    if (c->owner != s) return fail(BC_ERR_ARGUMENT, "the checkpoint belongs to another sequence");
    if (c->resets != s->resets) return fail(BC_ERR_ARGUMENT, "the checkpoint predates a reset");
    if (c->conv_state.size() != s->conv_floats || c->delta_state.size() != s->delta_floats || c->logits.size() != s->model->hp.n_vocab || c->n_past > s->n_ctx)
        return fail(BC_ERR_ARGUMENT, "the checkpoint comes from a different model or context");
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;
    if (s->conv_floats) BC_CUDA(cudaMemcpyAsync(s->conv_state, c->conv_state.data(), s->conv_floats * 4, cudaMemcpyHostToDevice, stream));
    if (s->delta_floats) BC_CUDA(cudaMemcpyAsync(s->delta_state, c->delta_state.data(), s->delta_floats * 4, cudaMemcpyHostToDevice, stream));
    BC_CUDA(cudaMemcpyAsync(s->logits, c->logits.data(), c->logits.size() * 4, cudaMemcpyHostToDevice, stream));
    BC_CUDA(cudaStreamSynchronize(stream));
    s->n_past = c->n_past;
    return BC_OK;
}

void bc_checkpoint_free(bc_checkpoint* c) { delete c; }

bc_status bc_seq_timings(const bc_seq* s, double* encode_seconds, double* gpu_seconds) {
    if (!s) return fail(BC_ERR_ARGUMENT, "seq must be non-null");
    if (encode_seconds) *encode_seconds = s->last_encode_seconds;
    if (gpu_seconds) *gpu_seconds = s->last_gpu_seconds;
    return BC_OK;
}

bc_status bc_seq_set_skip(bc_seq* s, const char* name, uint32_t n_rows, uint32_t n_cols) {
    if (!s) return fail(BC_ERR_ARGUMENT, "seq must be non-null");
    BC_TRY(s->backend->activate());
    BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    s->skip_name = name ? name : "";
    s->skip_rows = n_rows;
    s->skip_cols = n_cols;
    // The captured steps hold the old launch list.
    if (s->generate_graph) cudaGraphExecDestroy(s->generate_graph);
    if (s->stream_graph) cudaGraphExecDestroy(s->stream_graph);
    s->generate_graph = s->stream_graph = nullptr;
    return BC_OK;
}

bc_status bc_seq_read_state(bc_seq* s, int32_t which, uint32_t layer, float* out, size_t cap, size_t* n) {
    if (!s || !n) return fail(BC_ERR_ARGUMENT, "seq and n must be non-null");
    const bc_hparams& hp = s->model->hp;
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;
    if (which == 0) {
        *n = s->conv_floats;
        if (!out) return BC_OK;
        if (cap < *n) return fail(BC_ERR_ARGUMENT, "out must hold %zu floats", *n);
        if (*n) BC_CUDA(cudaMemcpyAsync(out, s->conv_state, *n * 4, cudaMemcpyDeviceToHost, stream));
        BC_CUDA(cudaStreamSynchronize(stream));
        return BC_OK;
    }
    if (which == 1 || which == 2) {
        if (layer >= hp.n_attention_layers) return fail(BC_ERR_ARGUMENT, "no attention layer %u", layer);
        size_t count = (size_t)s->n_ctx * hp.n_kv_heads * hp.head_dim;
        *n = count;
        if (!out) return BC_OK;
        if (cap < count) return fail(BC_ERR_ARGUMENT, "out must hold %zu floats", count);
        const char* cache = static_cast<const char*>(which == 1 ? s->k_cache : s->v_cache);
        if (s->kv_half) {
            std::vector<uint16_t> halfs(count);
            BC_CUDA(cudaMemcpyAsync(halfs.data(), cache + (size_t)layer * count * 2, count * 2, cudaMemcpyDeviceToHost, stream));
            BC_CUDA(cudaStreamSynchronize(stream));
            for (size_t i = 0; i < count; ++i) {
                out[i] = __half2float(__half(__half_raw{halfs[i]}));
            }
        } else {
            BC_CUDA(cudaMemcpyAsync(out, cache + (size_t)layer * count * 4, count * 4, cudaMemcpyDeviceToHost, stream));
            BC_CUDA(cudaStreamSynchronize(stream));
        }
        return BC_OK;
    }
    if (which == 3) {
        if (layer >= hp.n_delta_layers) return fail(BC_ERR_ARGUMENT, "no DeltaNet layer %u", layer);
        size_t count = (size_t)hp.n_v_heads * hp.k_head_dim * hp.v_head_dim;
        *n = count;
        if (!out) return BC_OK;
        if (cap < count) return fail(BC_ERR_ARGUMENT, "out must hold %zu floats", count);
        BC_CUDA(cudaMemcpyAsync(out, s->delta_state + (size_t)layer * count, count * 4, cudaMemcpyDeviceToHost, stream));
        BC_CUDA(cudaStreamSynchronize(stream));
        return BC_OK;
    }
    if (which == 4) {
        // The routes the last traced pass recorded, [layer][trace row][2 * n_used] 32-bit words (ids,
        // then weights as float bits), copied out bit for bit.
        size_t count = (size_t)s->trace_rows * hp.n_layers * 2 * hp.n_experts_used;
        *n = count;
        if (!out) return BC_OK;
        if (cap < count) return fail(BC_ERR_ARGUMENT, "out must hold %zu words", count);
        if (count) BC_CUDA(cudaMemcpyAsync(out, s->trace_routes, count * 4, cudaMemcpyDeviceToHost, stream));
        BC_CUDA(cudaStreamSynchronize(stream));
        return BC_OK;
    }
    return fail(BC_ERR_ARGUMENT, "unknown state %d", which);
}

}  // extern "C"
