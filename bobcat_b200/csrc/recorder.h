// The recorder of forward passes: the launch sequences of one token, a batch of one sequence's
// tokens, and one token of each of several sequences. Shared by the sequence API (seq.cpp) and the
// multi-sequence API (batch.cpp).
#pragma once

#include <algorithm>
#include <initializer_list>

#include "comm.h"
#include "seq.h"

namespace bc {

// Expert parallelism of a multi-sequence pass: this rank multiplies experts
// [first_expert, first_expert + n_local_experts) for the rows of every rank.
struct ExpertParallel {
    bc_comm* comm = nullptr;
    uint32_t first_expert = 0, n_local_experts = 0;
};

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
    // Batches with fewer rows than this multiply on the f32 tile kernels. A prefill's short tail
    // keeps f32 operands that way; a pass over several sequences lowers it to 1, because its few
    // rows (a rank's share of the sequences) still read every weight and the tensor-core kernel
    // reads them faster.
    uint32_t min_tensor_rows = 16;

    explicit Recorder(bc_seq& seq) : s(seq), hp(seq.hp), stream(seq.backend->stream) {}

    k::Pos at(uint32_t pos) const { return replayed ? k::Pos{s.step_pos, 0} : k::Pos{nullptr, pos}; }

    // A split-K product into the residual stream whose partial products are not added up yet
    // (in the backend's partial scratch). The normalisation that reads the stream next takes the
    // sum itself; any other launch that comes first triggers the separate sum.
    k::Deferred open_sum{};
    float* open_sum_y = nullptr;

    void close_sum() {
        if (!open_sum.partial) return;
        const k::Deferred d = open_sum;
        open_sum = k::Deferred{};
        float* y = open_sum_y;
        run("reduce", d.n_tokens, d.n_rows, 0, 1, [&] { return k::matmul_reduce(stream, d, y); });
    }

    // Launch helper: counts the kernel, keeps the first failure.
    template <typename F>
    void run(const char* name, uint32_t rows, uint32_t cols, uint64_t bytes, int kernels, F&& f) {
        if (status != BC_OK) return;
        if (open_sum.partial) close_sum();
        // Timing diagnostics: a launch kind left out of the pass (its outputs keep stale values).
        if (!s.skip_name.empty() && s.skip_name == name && (s.skip_rows == 0 || s.skip_rows == rows) && (s.skip_cols == 0 || s.skip_cols == cols)) return;
        s.launches += (uint64_t)kernels;
        status = s.backend->run(name, rows, cols, bytes, kernels, f);
    }

    // A recorded step that reports a status of its own (collectives).
    template <typename F>
    void run_status(F&& f) {
        if (status != BC_OK) return;
        if (open_sum.partial) close_sum();
        status = f();
    }

    k::Norm norm(const float* weight) const { return k::Norm{weight, hp.norm_eps}; }

    // Batched products run on the tensor cores with half-precision operands (as the reference's
    // Q4_0 prefill does, matmul.metal:519-521) unless the sequence asks for f32 operands, which
    // the f32 tile kernels provide at a lower rate.
    bool tensor_products() const { return !s.exact_products; }

    void matvec(const k::Mat& w, const float* x, float* y, k::Norm nm, bool accumulate) {
        k::MatvecSegment seg{w, y};
        run("matvec", w.n_rows, w.n_cols, w.bytes(), 1, [&] { return k::matvec(stream, &seg, 1, x, nm, accumulate); });
    }

    // y += W x where, on a tensor-parallel rank, W holds the rank's columns of an output projection
    // and x the matching slice of its input: the partial products are summed over ranks first
    // (qwen35.rs:369-516 computes the whole product on one device), then added to y on every rank.
    void matvec_reduced(const k::Mat& w, const float* x, float* y) {
        if (!s.tp) {
            matvec(w, x, y, k::Norm{}, true);
            return;
        }
        matvec(w, x, s.partial, k::Norm{}, false);
        // One kernel over NVLink peer memory when the ranks could map each other's buffers
        // (kernels_comm.cu), else ncclAllReduce and an add.
        s.launches += 1;
        run_status([&] { return comm_all_reduce_add(s.tp, s.partial, y, w.n_rows); });
    }
    void matmul_reduced(const k::Mat& w, const float* x, float* y, uint32_t n) {
        if (!s.tp) {
            matmul(w, x, y, n, BC_STORE_ACCUMULATE);
            return;
        }
        matmul(w, x, s.partial, n, BC_STORE_OVERWRITE);
        s.launches += 1;
        run_status([&] { return comm_all_reduce_add(s.tp, s.partial, y, (size_t)n * w.n_rows); });
    }
    // The logits: on a tensor-parallel rank the output matrix holds the rank's vocabulary rows;
    // every rank ends with all of them.
    void logits_product(const float* x) {
        const DeviceModel& W = *s.weights;
        if (!s.tp) {
            matvec(W.output, x, s.logits, norm(W.output_norm), false);
            return;
        }
        matvec(W.output, x, s.logits + W.first_vocab_row, norm(W.output_norm), false);
        run_status([&] { return comm_all_gather(s.tp, s.logits + W.first_vocab_row, s.logits, W.n_vocab_rows); });
    }

    void matmul(const k::Mat& w, const float* x, float* y, uint32_t n, int store) {
        if (status == BC_OK && tensor_products() && k::matmul_umma_supported(w, n, min_tensor_rows)) {
            void* pack = nullptr;
            status = s.backend->pack_scratch(k::matmul_pack_bytes(n, w.n_cols), &pack);
            run("pack", n, w.n_cols, 0, 1, [&] { return k::matmul_pack(stream, x, n, w.n_cols, pack); });
            product_of_packed(w, pack, y, n, store);
            return;
        }
        run("matmul", w.n_rows, w.n_cols, w.bytes(), 1, [&] { return k::matmul(stream, w, x, y, n, w.n_rows, store, nullptr); });
    }

    // The tensor-core product of packed inputs. Split-K shapes put their partial products into the
    // backend's partial scratch; when the product adds to y, the sum stays open for the next
    // normalisation of y (open_sum), else it is taken at once.
    void product_of_packed(const k::Mat& w, const void* packed, float* y, uint32_t n, int store) {
        close_sum();  // the partial scratch is about to be reused (or regrown)
        void* partial = nullptr;
        const uint64_t partial_bytes = k::matmul_partial_bytes(w, n);
        if (status == BC_OK && partial_bytes) status = s.backend->partial_scratch(partial_bytes, &partial);
        k::Deferred left{};
        // The normalisation that would take the sum runs one CTA per 4 tokens: with few rows the
        // separate, wide sum is quicker.
        const bool may_defer = store == BC_STORE_ACCUMULATE && n >= 128;
        run("matmul", w.n_rows, w.n_cols, w.bytes(), 1, [&] {
            return k::matmul_umma(stream, w, packed, y, n, w.n_rows, store, static_cast<float*>(partial), may_defer ? &left : nullptr);
        });
        if (status != BC_OK) return;
        if (left.partial) {
            open_sum = left;
            open_sum_y = y;
        } else if (partial_bytes) {
            s.launches += 1;  // the sum ran inside matmul_umma
        }
    }

    // The fused normalisation and packing of x, taking an open sum into x along the way.
    void pack_normed(float* x, const float* norm_weight, uint32_t n, uint32_t cols, void* packed) {
        k::Deferred add{};
        if (open_sum.partial && open_sum_y == x && open_sum.n_tokens == n && open_sum.n_rows == cols) {
            add = open_sum;
            open_sum = k::Deferred{};
        }
        run("pack_norm", n, cols, 0, 1, [&] { return k::matmul_pack_norm(stream, x, norm(norm_weight), n, cols, packed, &add); });
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
        if (!tensor_products() || !k::matmul_umma_swiglu_supported(gate, up, n, min_tensor_rows)) {
            // The up projection's store combines with the gate projection already in the buffer.
            normed_matmuls(x, norm_weight, n, {{&gate, y, BC_STORE_OVERWRITE}, {&up, y, BC_STORE_SWIGLU}});
            return;
        }
        const uint32_t cols = hp.n_embd;
        void* scratch = nullptr;
        if (status == BC_OK) status = s.backend->pack_scratch(k::matmul_pack_bytes(n, cols), &scratch);
        pack_normed(const_cast<float*>(x), norm_weight, n, cols, scratch);
        run("matmul_swiglu", gate.n_rows, gate.n_cols, 2 * gate.bytes(), 1,
            [&] { return k::matmul_umma_swiglu(stream, gate, up, scratch, y, n, gate.n_rows); });
    }

    // hidden += down (silu(gate x^) * (up x^)) over the batch, x^ the normalised rows of hidden
    // (lfm2.rs:405-411, qwen35.rs:505-516). On the tensor-core path the gate / up launch writes its
    // result as the packed fp16 input of the down product, so the f32 intermediate and its
    // packing launch do not exist.
    void normed_ffn(float* hidden, const float* norm_weight, uint32_t n, const k::Mat& gate, const k::Mat& up, const k::Mat& down) {
        const bool direct = tensor_products() && k::matmul_umma_swiglu_supported(gate, up, n, min_tensor_rows) && k::matmul_umma_supported(down, n, min_tensor_rows) &&
                            down.n_cols == gate.n_rows && gate.n_rows % 64 == 0;
        if (!direct) {
            normed_swiglu(hidden, norm_weight, n, gate, up, s.ffn);
            matmul_reduced(down, s.ffn, hidden, n);
            return;
        }
        const uint32_t cols = hp.n_embd;
        const size_t down_bytes = (k::matmul_pack_bytes(n, down.n_cols) + 255) & ~(size_t)255;
        void* scratch = nullptr;
        if (status == BC_OK) status = s.backend->pack_scratch(down_bytes + k::matmul_pack_bytes(n, cols), &scratch);
        void* in_pack = static_cast<char*>(scratch) + down_bytes;
        pack_normed(hidden, norm_weight, n, cols, in_pack);
        run("matmul_swiglu", gate.n_rows, gate.n_cols, 2 * gate.bytes(), 1,
            [&] { return k::matmul_umma_swiglu(stream, gate, up, in_pack, nullptr, n, gate.n_rows, scratch); });
        product_of_packed(down, scratch, s.tp ? s.partial : hidden, n, s.tp ? BC_STORE_OVERWRITE : BC_STORE_ACCUMULATE);
        if (s.tp) {
            s.launches += 1;
            run_status([&] { return comm_all_reduce_add(s.tp, s.partial, hidden, (size_t)n * down.n_rows); });
        }
    }

    void normed_matmuls(const float* x, const float* norm_weight, uint32_t n, std::initializer_list<Product> products) {
        const uint32_t cols = hp.n_embd;
        bool fused = true;
        size_t bytes = 0;
        for (const Product& q : products) {
            fused = fused && tensor_products() && k::matmul_umma_supported(*q.w, n, min_tensor_rows);
            bytes = std::max(bytes, (size_t)k::matmul_scratch_bytes(*q.w, n));
        }
        if (!fused) {
            run("rms_norm", n, cols, 0, 1, [&] { return k::rms_norm(stream, x, norm_weight, s.normed, cols, n, hp.norm_eps); });
            for (const Product& q : products) matmul(*q.w, s.normed, q.y, n, q.store);
            return;
        }
        void* scratch = nullptr;
        if (status == BC_OK) status = s.backend->pack_scratch(bytes, &scratch);
        pack_normed(const_cast<float*>(x), norm_weight, n, cols, scratch);
        // Products that only overwrite their outputs (q, k, v; a DeltaNet layer's four projections) share one launch.
        bool together = products.size() > 1 && products.size() <= 4;
        for (const Product& q : products) together = together && q.store == BC_STORE_OVERWRITE;
        if (together) {
            const k::Mat* ws[4];
            float* ys[4];
            uint32_t rows = 0;
            uint64_t bytes_read = 0;
            int count = 0;
            for (const Product& q : products) {
                ws[count] = q.w;
                ys[count++] = q.y;
                rows += q.w->n_rows;
                bytes_read += q.w->bytes();
            }
            run("matmul", rows, cols, bytes_read, 1, [&] { return k::matmul_umma_several(stream, ws, ys, count, scratch, n); });
            return;
        }
        for (const Product& q : products) product_of_packed(*q.w, scratch, q.y, n, q.store);
    }

    size_t kv_element_bytes() const { return s.kv_half ? 2 : 4; }
    size_t kv_dim() const { return (size_t)hp.n_kv_heads * hp.head_dim; }
    // lfm2_metal.rs:1064-1067: layer-major, then position, then KV head, then element.
    size_t layer_base(uint32_t cache_index) const { return (size_t)cache_index * s.kv_stride * kv_dim(); }
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

    void qwen_dense_ffn(const DeviceLayer& D) {
        run("matvec_swiglu", D.gate.n_rows, D.gate.n_cols, D.gate.bytes() * 2, 1,
            [&] { return k::matvec_swiglu(stream, D.gate, D.up, s.hidden, norm(D.ffn_norm), s.ffn); });
        matvec_reduced(D.down, s.ffn, s.hidden);
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
        const bool tensor_up = tensor_products() && k::matmul_experts_umma_supported(D.gate, &D.up, n);
        const bool tensor_down = tensor_products() && k::matmul_experts_umma_supported(D.down, nullptr, n);
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

    // The mixture of experts of a multi-sequence pass with the experts sharded over ranks
    // (lfm2.rs:413-440 split by expert). s.hidden holds this rank's n_local rows. Dispatch: the
    // normalised rows of all ranks are gathered on every rank, which then routes all of them
    // identically (the router is replicated; f64 sums, so the ids agree bit for bit). Each rank
    // multiplies the entries of its own experts; the other entries' output rows stay zero.
    // Combine: the output rows are summed over ranks (one nonzero contributor each, so the sum is
    // exact) and scattered to the rank that owns the row's sequence, which adds its slots in route
    // order. All buffers are this GPU's own; NCCL moves the data.
    void lfm2_moe_expert_parallel(const DeviceLayer& D, uint32_t n_local, const ExpertParallel& ep) {
        const uint32_t n_used = hp.n_experts_used, n_ff = hp.n_ff_expert, n_embd = hp.n_embd;
        const uint32_t world = (uint32_t)ep.comm->world, rank = (uint32_t)ep.comm->rank, n = n_local * world;
        float* mine = s.normed + (size_t)rank * n_local * n_embd;
        run("rms_norm", n_local, n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, D.ffn_norm, mine, n_embd, n_local, hp.norm_eps); });
        run_status([&] { return comm_all_gather(ep.comm, mine, s.normed, (size_t)n_local * n_embd); });
        run("moe_route", hp.n_experts, n_embd, D.router.bytes(), 1, [&] {
            return k::moe_route(stream, s.normed, k::Norm{}, s.normed, static_cast<const float*>(D.router.data), D.expert_bias, s.route, n_embd, hp.n_experts,
                                n_used, n);
        });
        run("moe_group", n, ep.n_local_experts, 0, 1,
            [&] { return k::moe_group(stream, s.route, s.expert_offsets, s.expert_entries, ep.n_local_experts, n_used, n, ep.first_expert); });
        run_status([&]() -> bc_status {
            BC_CUDA(cudaMemsetAsync(s.expert_out, 0, (size_t)n * n_used * n_embd * 4, stream));
            return BC_OK;
        });
        const k::Mat gate = D.gate.rows(ep.first_expert * n_ff, ep.n_local_experts * n_ff), up = D.up.rows(ep.first_expert * n_ff, ep.n_local_experts * n_ff);
        const k::Mat down = D.down.rows(ep.first_expert * n_embd, ep.n_local_experts * n_embd);
        void* up_scratch = nullptr;
        void* down_scratch = nullptr;
        const bool tensor_up = tensor_products() && k::matmul_experts_umma_supported(gate, &up, n);
        const bool tensor_down = tensor_products() && k::matmul_experts_umma_supported(down, nullptr, n);
        if (status == BC_OK && (tensor_up || tensor_down)) {
            size_t bytes = (size_t)std::max(tensor_up ? k::matmul_experts_scratch_bytes(ep.n_local_experts, n, n_embd) : 0,
                                            tensor_down ? k::matmul_experts_scratch_bytes(ep.n_local_experts, n, n_ff) : 0);
            void* scratch = nullptr;
            status = s.backend->pack_scratch(bytes, &scratch);
            if (tensor_up) up_scratch = scratch;
            if (tensor_down) down_scratch = scratch;
        }
        run("matmul_experts", n_ff, n_embd, 2 * gate.bytes(), up_scratch ? 2 : 1, [&] {
            return k::matmul_experts(stream, gate, &up, n_ff, ep.n_local_experts, s.normed, true, s.expert_offsets, s.expert_entries, n_used, s.ffn, n, up_scratch);
        });
        run("matmul_experts", n_embd, n_ff, down.bytes(), down_scratch ? 2 : 1, [&] {
            return k::matmul_experts(stream, down, nullptr, n_embd, ep.n_local_experts, s.ffn, false, s.expert_offsets, s.expert_entries, n_used,
                                     s.expert_out, n, down_scratch);
        });
        float* my_rows = s.expert_out + (size_t)rank * n_local * n_used * n_embd;
        run_status([&] { return comm_reduce_scatter_sum(ep.comm, s.expert_out, my_rows, (size_t)n_local * n_used * n_embd); });
        const uint32_t* my_routes = s.route + (size_t)rank * n_local * 2 * n_used;
        run("moe_combine", n_local, n_embd, 0, 1, [&] { return k::moe_combine(stream, my_rows, my_routes, s.hidden, n_embd, n_used, n_local); });
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
                if (tensor_products() && k::matmul_umma_supported(D.out_proj, n, min_tensor_rows) && n_embd % 64 == 0) {
                    // The convolution writes the packed input of the output projection itself.
                    void* pack = nullptr;
                    if (status == BC_OK) status = s.backend->pack_scratch(k::matmul_pack_bytes(n, n_embd), &pack);
                    run("short_conv", n, n_embd, 0, 2,
                        [&] { return k::short_conv(stream, s.bcx, D.taps, history, nullptr, n_embd, hp.conv_kernel, n, pack); });
                    product_of_packed(D.out_proj, pack, s.hidden, n, BC_STORE_ACCUMULATE);
                } else {
                    run("short_conv", n, n_embd, 0, 2,
                        [&] { return k::short_conv(stream, s.bcx, D.taps, history, s.conv_out, n_embd, hp.conv_kernel, n); });
                    matmul(D.out_proj, s.conv_out, s.hidden, n, BC_STORE_ACCUMULATE);
                }
            }
            if (S.moe) {
                run("rms_norm", n, n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, D.ffn_norm, s.normed, n_embd, n, hp.norm_eps); });
                route_trace = traced ? s.trace_routes + il * (size_t)s.trace_rows * 2 * hp.n_experts_used : nullptr;
                lfm2_moe(D, n, false);
            } else {
                normed_ffn(s.hidden, D.ffn_norm, n, D.gate, D.up, D.down);
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
        run("gdn_qk_norm", n * 2 * hp.n_k_heads, hp.k_head_dim, 0, 1,
            [&] { return k::gdn_qk_norm(stream, s.gdn_conv_out, hp.n_k_heads, hp.n_v_heads, hp.k_head_dim, hp.v_head_dim, n); });
        run("gdn_recurrence", n, value_dim(), state_bytes, 1, [&] {
            return k::gdn_recurrence(stream, s.gdn_conv_out, s.gdn_beta, s.gdn_alpha, state, s.gdn_out, hp.n_k_heads, hp.n_v_heads, hp.k_head_dim,
                                     hp.v_head_dim, n, false);
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
                matvec_reduced(D.output, s.attn, s.hidden);
            } else {
                k::MatvecSegment segs[4] = {{D.qkv, s.gdn_qkv}, {D.z, s.gdn_z}, {D.beta, s.gdn_beta}, {D.alpha, s.gdn_alpha}};
                uint64_t bytes = D.qkv.bytes() + D.z.bytes() + D.beta.bytes() + D.alpha.bytes();
                        run("matvec_delta", D.qkv.n_rows + D.z.n_rows + 2 * D.beta.n_rows, D.qkv.n_cols, bytes, 1,
                    [&] { return k::matvec(stream, segs, 4, s.hidden, norm(D.attn_norm), false); });
                        qwen_delta_tail(D, S.cache_index, 1);
                matvec_reduced(D.ssm_out, s.gdn_out, s.hidden);
            }
            qwen_dense_ffn(D);
            if (traced) copy(s.hidden, s.trace_layers + il * hp.n_embd, hp.n_embd);
        }
        if (traced)
            run("rms_norm", 1, hp.n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, W.output_norm, s.trace_final, hp.n_embd, 1, hp.norm_eps); });
        if (want_logits) logits_product(s.hidden);
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
                matmul_reduced(D.output, s.attn, s.hidden, n);
            } else {
                normed_matmuls(s.hidden, D.attn_norm, n,
                               {{&D.qkv, s.gdn_qkv, BC_STORE_OVERWRITE}, {&D.z, s.gdn_z, BC_STORE_OVERWRITE}, {&D.beta, s.gdn_beta, BC_STORE_OVERWRITE},
                                {&D.alpha, s.gdn_alpha, BC_STORE_OVERWRITE}});
                qwen_delta_tail(D, S.cache_index, n);
                matmul_reduced(D.ssm_out, s.gdn_out, s.hidden, n);
            }
            normed_ffn(s.hidden, D.ffn_norm, n, D.gate, D.up, D.down);
            if (traced) copy(s.hidden, s.trace_layers + il * trace_stride, (uint64_t)n * n_embd);
        }
        if (traced)
            run("rms_norm", n, n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, W.output_norm, s.trace_final, n_embd, n, hp.norm_eps); });
        if (want_logits) logits_product(s.hidden + (size_t)(n - 1) * n_embd);
    }

    // ---- one token of each of n sequences (the multi-sequence decode step). Row b of every
    // activation buffer belongs to sequence b; `seqs` reaches each sequence's caches, history and
    // position. Weight products are the batched ones, so every weight is read once for all rows;
    // each row computes what lfm2_step computes for its sequence (lfm2_metal.rs:1162-1242).
    // `tokens` holds the n token ids; logits go to `all_logits` ([n][n_vocab]).
    void lfm2_seqs_step(const uint32_t* tokens, uint32_t n, k::SeqTable seqs, float* all_logits, const ExpertParallel* ep = nullptr) {
        const DeviceModel& W = *s.weights;
        const uint32_t n_embd = hp.n_embd, q_dim = hp.n_heads * hp.head_dim;
        run("embed", n, n_embd, 0, 1, [&] { return k::embed(stream, W.token_embd, tokens, k::Pos{nullptr, 0}, s.hidden, n); });
        for (size_t il = 0; il < W.layers.size(); ++il) {
            const LayerSpec& S = s.model->layers[il];
            const DeviceLayer& D = W.layers[il];
            if (S.mixer == Mixer::Attention) {
                normed_matmuls(s.hidden, D.attn_norm, n, {{&D.q, s.q, BC_STORE_OVERWRITE}, {&D.k, s.k, BC_STORE_OVERWRITE}, {&D.v, s.v, BC_STORE_OVERWRITE}});
                seqs.layer_offset = layer_base(S.cache_index);
                k::RopeStore rs{s.q, s.k, s.v, nullptr, nullptr, D.q_norm, D.k_norm, hp.n_heads, hp.n_kv_heads, hp.head_dim, hp.head_dim, hp.n_rot,
                                hp.rope_theta, hp.norm_eps, s.kv_half, nullptr};
                run("rope_store_seqs", (hp.n_heads + 2 * hp.n_kv_heads) * n, hp.head_dim, 0, 1, [&] { return k::rope_store_seqs(stream, rs, seqs, q_dim, n); });
                run("attention_seqs", n, hp.n_heads, 0, 1, [&] {
                    return k::attention_seqs(stream, s.q, s.attn, seqs, s.kv_half, hp.n_heads, hp.n_kv_heads, hp.head_dim, q_dim, hp.head_dim, n);
                });
                matmul(D.output, s.attn, s.hidden, n, BC_STORE_ACCUMULATE);
            } else {
                normed_matmuls(s.hidden, D.attn_norm, n, {{&D.in_proj, s.bcx, BC_STORE_OVERWRITE}});
                seqs.conv_offset = (uint64_t)S.cache_index * (hp.conv_kernel - 1) * n_embd;
                run("short_conv_seqs", n, n_embd, 0, 1, [&] { return k::short_conv_seqs(stream, s.bcx, D.taps, seqs, s.conv_out, n_embd, hp.conv_kernel, n); });
                matmul(D.out_proj, s.conv_out, s.hidden, n, BC_STORE_ACCUMULATE);
            }
            if (S.moe && ep && ep->comm->world > 1) {
                lfm2_moe_expert_parallel(D, n, *ep);
            } else if (S.moe) {
                run("rms_norm", n, n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, D.ffn_norm, s.normed, n_embd, n, hp.norm_eps); });
                route_trace = nullptr;
                lfm2_moe(D, n, false);
            } else {
                normed_ffn(s.hidden, D.ffn_norm, n, D.gate, D.up, D.down);
            }
        }
        // Every row needs its logits, so the output matrix is one batched product too.
        run("rms_norm", n, n_embd, 0, 1, [&] { return k::rms_norm(stream, s.hidden, W.output_norm, s.normed, n_embd, n, hp.norm_eps); });
        matmul(W.output, s.normed, all_logits, n, BC_STORE_OVERWRITE);
    }

    void step(uint32_t pos, bool want_logits, bool traced) {
        if (hp.architecture == BC_ARCH_QWEN35) qwen_step(pos, want_logits, traced);
        else lfm2_step(pos, want_logits, traced);
    }

    void batch(uint32_t pos, uint32_t n, bool want_logits, bool traced, size_t trace_stride) {
        if (hp.architecture == BC_ARCH_QWEN35) qwen_batch(pos, n, want_logits, traced, trace_stride);
        else lfm2_batch(pos, n, want_logits, traced, trace_stride);
        close_sum();  // the last layer's product, when no logits were asked for
    }

    void argmax(const float* x, uint32_t* out, uint32_t* readback) {
        run("argmax", 1, hp.n_vocab, 0, 1, [&] { return k::argmax(stream, x, hp.n_vocab, out, readback); });
    }
};

}  // namespace bc
