// Bounds-checked op wrappers of the mixture-of-experts launches
// (crates/bobcat-metal/src/backend.rs:1428-1737).

#include "backend.h"

using namespace bc;

namespace {

bc_status recording(bc_backend* b) {
    if (!b) return fail(BC_ERR_ARGUMENT, "backend must be non-null");
    if (!b->recording) return fail(BC_ERR_NOT_RECORDING, "no recording is open");
    return b->activate();
}

template <typename T>
T* at(bc_buffer* buffer, size_t offset) {
    return reinterpret_cast<T*>(static_cast<char*>(buffer->ptr) + offset);
}

// check_expert_limits, backend.rs:2730-2736
bc_status expert_limits(uint32_t n_experts, uint32_t n_used) {
    if (n_experts > 128 || n_used > 8 || n_used == 0 || n_used > n_experts)
        return fail(BC_ERR_EXPERT_LIMITS, "at most 8 of 128 experts per token and at least one, got %u of %u", n_used, n_experts);
    return BC_OK;
}

// The stacked expert matrices a (buffer, offset) view names: n_experts * n_rows rows from offset 0.
bc_status experts_view(bc_backend* b, bc_buffer* buffer, size_t offset, int32_t format, uint32_t n_rows, uint32_t n_cols, uint32_t n_experts,
                       const char* op, k::Mat* out) {
    if (!buffer) return fail(BC_ERR_ARGUMENT, "the %s launch got a null buffer", op);
    if (buffer->backend != b) return fail(BC_ERR_FOREIGN_BUFFER, "the buffer belongs to another backend");
    if (!buffer->is_matrix) return fail(BC_ERR_ARGUMENT, "the %s launch needs weights from bc_matrix_upload", op);
    if (format != BC_Q4_0 && format != BC_F16 && format != BC_F32) return fail(BC_ERR_NO_EXPERTS, "format %d cannot hold experts", format);
    const k::Mat& m = buffer->matrix;
    if (m.format != format || m.n_cols != n_cols || offset != 0) return fail(BC_ERR_ARGUMENT, "the %s launch names a different format, width or offset than the upload", op);
    if ((uint64_t)n_rows * n_experts > m.n_rows)
        return fail(BC_ERR_OUT_OF_BOUNDS, "the %s launch needs %llu rows of a %u-row matrix", op, (unsigned long long)n_rows * n_experts, m.n_rows);
    *out = m;
    return BC_OK;
}

}  // namespace

extern "C" {

size_t bc_route_bytes(uint32_t n_used, uint32_t n_tokens) { return (size_t)2 * n_used * n_tokens * 4; }

bc_status bc_op_moe_route(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* norm, size_t norm_off, float eps, bc_buffer* normed,
                          size_t normed_off, bc_buffer* router, size_t router_off, bc_buffer* bias, size_t bias_off, bc_buffer* route,
                          size_t route_off, uint32_t n_cols, uint32_t n_experts, uint32_t n_used, uint32_t n_tokens) {
    BC_TRY(recording(b));
    BC_TRY(expert_limits(n_experts, n_used));
    size_t token_bytes = (size_t)n_tokens * n_cols * 4;
    BC_TRY(check_range(b, x, x_off, token_bytes, "moe_route"));
    BC_TRY(check_range(b, router, router_off, (size_t)n_experts * n_cols * 4, "moe_route"));
    BC_TRY(check_range(b, bias, bias_off, (size_t)n_experts * 4, "moe_route"));
    BC_TRY(check_range(b, route, route_off, bc_route_bytes(n_used, n_tokens), "moe_route"));
    k::Norm nm;
    float* normed_ptr = nullptr;
    if (norm) {
        BC_TRY(check_range(b, norm, norm_off, (size_t)n_cols * 4, "moe_route"));
        BC_TRY(check_range(b, normed, normed_off, token_bytes, "moe_route"));
        nm = k::Norm{at<const float>(norm, norm_off), eps};
        normed_ptr = at<float>(normed, normed_off);
    }
    return b->run("moe_route", n_experts, n_cols, (uint64_t)n_experts * n_cols * 4, 1, [&] {
        return k::moe_route(b->stream, at<const float>(x, x_off), nm, normed_ptr, at<const float>(router, router_off), at<const float>(bias, bias_off),
                            at<uint32_t>(route, route_off), n_cols, n_experts, n_used, n_tokens);
    });
}

bc_status bc_op_moe_group(bc_backend* b, bc_buffer* route, size_t route_off, bc_buffer* offsets, size_t off_off, bc_buffer* entries,
                          size_t ent_off, uint32_t n_experts, uint32_t n_used, uint32_t n_tokens) {
    BC_TRY(recording(b));
    BC_TRY(expert_limits(n_experts, n_used));
    BC_TRY(check_range(b, route, route_off, bc_route_bytes(n_used, n_tokens), "moe_group"));
    BC_TRY(check_range(b, offsets, off_off, ((size_t)n_experts + 1) * 4, "moe_group"));
    BC_TRY(check_range(b, entries, ent_off, (size_t)n_tokens * n_used * 4, "moe_group"));
    return b->run("moe_group", n_tokens, n_experts, 0, 1, [&] {
        return k::moe_group(b->stream, at<const uint32_t>(route, route_off), at<uint32_t>(offsets, off_off), at<uint32_t>(entries, ent_off), n_experts,
                            n_used, n_tokens);
    });
}

bc_status bc_op_matvec_experts_swiglu(bc_backend* b, int32_t format, bc_buffer* gate, size_t gate_off, bc_buffer* up, size_t up_off,
                                      uint32_t n_rows, uint32_t n_cols, uint32_t n_experts, bc_buffer* x, size_t x_off, bc_buffer* route,
                                      size_t route_off, uint32_t n_used, bc_buffer* y, size_t y_off, uint32_t n_tokens) {
    BC_TRY(recording(b));
    BC_TRY(expert_limits(n_experts, n_used));
    k::Mat g, u;
    BC_TRY(experts_view(b, gate, gate_off, format, n_rows, n_cols, n_experts, "matvec_experts_swiglu", &g));
    BC_TRY(experts_view(b, up, up_off, format, n_rows, n_cols, n_experts, "matvec_experts_swiglu", &u));
    BC_TRY(check_range(b, x, x_off, (size_t)n_tokens * n_cols * 4, "matvec_experts_swiglu"));
    BC_TRY(check_range(b, route, route_off, bc_route_bytes(n_used, n_tokens), "matvec_experts_swiglu"));
    BC_TRY(check_range(b, y, y_off, (size_t)n_tokens * n_used * n_rows * 4, "matvec_experts_swiglu"));
    uint64_t bytes = 2ull * n_used * n_tokens * n_rows * type_row_bytes((uint32_t)format, n_cols);
    return b->run("matvec_experts_swiglu", n_rows, n_cols, bytes, 1, [&] {
        return k::matvec_experts_swiglu(b->stream, g, u, n_rows, at<const float>(x, x_off), at<const uint32_t>(route, route_off), n_used,
                                        at<float>(y, y_off), n_tokens);
    });
}

bc_status bc_op_matvec_experts_down(bc_backend* b, int32_t format, bc_buffer* down, size_t down_off, uint32_t n_rows, uint32_t n_cols,
                                    uint32_t n_experts, bc_buffer* x, size_t x_off, bc_buffer* route, size_t route_off, uint32_t n_used,
                                    bc_buffer* y, size_t y_off, uint32_t n_tokens) {
    BC_TRY(recording(b));
    BC_TRY(expert_limits(n_experts, n_used));
    k::Mat d;
    BC_TRY(experts_view(b, down, down_off, format, n_rows, n_cols, n_experts, "matvec_experts_down", &d));
    BC_TRY(check_range(b, x, x_off, (size_t)n_tokens * n_used * n_cols * 4, "matvec_experts_down"));
    BC_TRY(check_range(b, route, route_off, bc_route_bytes(n_used, n_tokens), "matvec_experts_down"));
    BC_TRY(check_range(b, y, y_off, (size_t)n_tokens * n_rows * 4, "matvec_experts_down"));
    uint64_t bytes = (uint64_t)n_used * n_tokens * n_rows * type_row_bytes((uint32_t)format, n_cols);
    // A single token on the tile kernel leaves its slots' outputs in the backend's scratch first.
    void* slots = nullptr;
    const int launches = k::matvec_experts_down_launches(d, n_rows, n_used, n_tokens, true);
    if (launches == 2) BC_TRY(b->pack_scratch((size_t)n_used * n_rows * 4, &slots));
    return b->run("matvec_experts_down", n_rows, n_cols, bytes, launches, [&] {
        return k::matvec_experts_down(b->stream, d, n_rows, at<const float>(x, x_off), at<const uint32_t>(route, route_off), n_used, at<float>(y, y_off),
                                      n_tokens, static_cast<float*>(slots));
    });
}

bc_status bc_op_matmul_experts(bc_backend* b, int32_t format, bc_buffer* weights, size_t w_off, bc_buffer* up, size_t up_off, uint32_t n_rows,
                               uint32_t n_cols, uint32_t n_experts, bc_buffer* x, size_t x_off, int32_t gather, bc_buffer* offsets,
                               size_t off_off, bc_buffer* entries, size_t ent_off, uint32_t n_used, bc_buffer* y, size_t y_off,
                               uint32_t n_tokens) {
    BC_TRY(recording(b));
    BC_TRY(expert_limits(n_experts, n_used));
    k::Mat w, u;
    BC_TRY(experts_view(b, weights, w_off, format, n_rows, n_cols, n_experts, "matmul_experts", &w));
    if (up) BC_TRY(experts_view(b, up, up_off, format, n_rows, n_cols, n_experts, "matmul_experts", &u));
    size_t in_rows = gather ? n_tokens : (size_t)n_tokens * n_used;
    BC_TRY(check_range(b, x, x_off, in_rows * n_cols * 4, "matmul_experts"));
    BC_TRY(check_range(b, offsets, off_off, ((size_t)n_experts + 1) * 4, "matmul_experts"));
    BC_TRY(check_range(b, entries, ent_off, (size_t)n_tokens * n_used * 4, "matmul_experts"));
    BC_TRY(check_range(b, y, y_off, (size_t)n_tokens * n_used * n_rows * 4, "matmul_experts"));
    void* scratch = nullptr;
    if (k::matmul_experts_umma_supported(w, up ? &u : nullptr, n_tokens))
        BC_TRY(b->pack_scratch(k::matmul_experts_scratch_bytes(n_experts, n_tokens, n_cols), &scratch));
    return b->run("matmul_experts", n_rows, n_cols, w.bytes() * (up ? 2 : 1), scratch ? 2 : 1, [&] {
        return k::matmul_experts(b->stream, w, up ? &u : nullptr, n_rows, n_experts, at<const float>(x, x_off), gather != 0,
                                 at<const uint32_t>(offsets, off_off), at<const uint32_t>(entries, ent_off), n_used, at<float>(y, y_off), n_tokens,
                                 scratch);
    });
}

bc_status bc_op_moe_combine(bc_backend* b, bc_buffer* expert_out, size_t eo_off, bc_buffer* route, size_t route_off, bc_buffer* y, size_t y_off,
                            uint32_t n_embd, uint32_t n_used, uint32_t n_tokens) {
    BC_TRY(recording(b));
    BC_TRY(check_range(b, expert_out, eo_off, (size_t)n_tokens * n_used * n_embd * 4, "moe_combine"));
    BC_TRY(check_range(b, route, route_off, bc_route_bytes(n_used, n_tokens), "moe_combine"));
    BC_TRY(check_range(b, y, y_off, (size_t)n_tokens * n_embd * 4, "moe_combine"));
    return b->run("moe_combine", n_tokens, n_embd, 0, 1, [&] {
        return k::moe_combine(b->stream, at<const float>(expert_out, eo_off), at<const uint32_t>(route, route_off), at<float>(y, y_off), n_embd, n_used,
                              n_tokens);
    });
}

}  // extern "C"
