// Bounds-checked op wrappers of the Qwen3.5 launches (crates/bobcat-metal/src/backend.rs:1739-2032).

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

}  // namespace

extern "C" {

bc_status bc_op_gdn_conv(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* taps, size_t taps_off, bc_buffer* history, size_t hist_off,
                         bc_buffer* out, size_t out_off, uint32_t conv_dim, uint32_t kernel, uint32_t n_tokens) {
    BC_TRY(recording(b));
    if (kernel < 2 || kernel > 8) return fail(BC_ERR_DELTANET_LIMITS, "a DeltaNet convolution of 2 to 8 taps, got %u", kernel);
    BC_TRY(check_range(b, x, x_off, (size_t)n_tokens * conv_dim * 4, "gdn_conv"));
    BC_TRY(check_range(b, taps, taps_off, (size_t)conv_dim * kernel * 4, "gdn_conv"));
    BC_TRY(check_range(b, history, hist_off, (size_t)conv_dim * (kernel - 1) * 4, "gdn_conv"));
    BC_TRY(check_range(b, out, out_off, (size_t)n_tokens * conv_dim * 4, "gdn_conv"));
    return b->run("gdn_conv", n_tokens, conv_dim, 0, k::gdn_conv_launches(n_tokens), [&] {
        return k::gdn_conv(b->stream, at<const float>(x, x_off), at<const float>(taps, taps_off), at<float>(history, hist_off), at<float>(out, out_off),
                           conv_dim, kernel, n_tokens);
    });
}

bc_status bc_op_gdn_gates(bc_backend* b, bc_buffer* beta, size_t beta_off, bc_buffer* alpha, size_t alpha_off, bc_buffer* a, size_t a_off,
                          bc_buffer* dt_bias, size_t dt_off, uint32_t n_v_heads, uint32_t n_tokens) {
    BC_TRY(recording(b));
    BC_TRY(check_range(b, beta, beta_off, (size_t)n_tokens * n_v_heads * 4, "gdn_gates"));
    BC_TRY(check_range(b, alpha, alpha_off, (size_t)n_tokens * n_v_heads * 4, "gdn_gates"));
    BC_TRY(check_range(b, a, a_off, (size_t)n_v_heads * 4, "gdn_gates"));
    BC_TRY(check_range(b, dt_bias, dt_off, (size_t)n_v_heads * 4, "gdn_gates"));
    return b->run("gdn_gates", n_tokens, n_v_heads, 0, 1, [&] {
        return k::gdn_gates(b->stream, at<float>(beta, beta_off), at<float>(alpha, alpha_off), at<const float>(a, a_off), at<const float>(dt_bias, dt_off),
                            n_v_heads, n_tokens);
    });
}

bc_status bc_op_gdn_recurrence(bc_backend* b, bc_buffer* qkv, size_t qkv_off, bc_buffer* beta, size_t beta_off, bc_buffer* decay,
                               size_t decay_off, bc_buffer* state, size_t state_off, bc_buffer* out, size_t out_off, uint32_t n_k_heads,
                               uint32_t n_v_heads, uint32_t k_dim, uint32_t v_dim, uint32_t n_tokens, int32_t normalize) {
    BC_TRY(recording(b));
    if (n_k_heads == 0 || n_v_heads == 0 || n_v_heads % n_k_heads != 0 || k_dim == 0 || k_dim % 32 != 0 || k_dim > 128 || v_dim == 0 ||
        v_dim % 32 != 0 || v_dim > 256)
        return fail(BC_ERR_DELTANET_LIMITS,
                    "DeltaNet needs key heads of a multiple of 32 up to 128, value heads of a multiple of 32 up to 256 and a whole number of "
                    "value heads per key head, got %u x %u and %u x %u",
                    n_k_heads, k_dim, n_v_heads, v_dim);
    size_t conv_dim = 2 * (size_t)n_k_heads * k_dim + (size_t)n_v_heads * v_dim;
    BC_TRY(check_range(b, qkv, qkv_off, (size_t)n_tokens * conv_dim * 4, "gdn_recurrence"));
    BC_TRY(check_range(b, beta, beta_off, (size_t)n_tokens * n_v_heads * 4, "gdn_recurrence"));
    BC_TRY(check_range(b, decay, decay_off, (size_t)n_tokens * n_v_heads * 4, "gdn_recurrence"));
    BC_TRY(check_range(b, state, state_off, (size_t)n_v_heads * k_dim * v_dim * 4, "gdn_recurrence"));
    BC_TRY(check_range(b, out, out_off, (size_t)n_tokens * n_v_heads * v_dim * 4, "gdn_recurrence"));
    return b->run("gdn_recurrence", n_tokens, n_v_heads * v_dim, (uint64_t)n_v_heads * k_dim * v_dim * 8, 1, [&] {
        return k::gdn_recurrence(b->stream, at<const float>(qkv, qkv_off), at<const float>(beta, beta_off), at<const float>(decay, decay_off),
                                 at<float>(state, state_off), at<float>(out, out_off), n_k_heads, n_v_heads, k_dim, v_dim, n_tokens, normalize != 0);
    });
}

bc_status bc_op_gdn_gated_norm(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* z, size_t z_off, bc_buffer* weight, size_t w_off,
                               uint32_t v_dim, uint32_t n_rows, float eps) {
    BC_TRY(recording(b));
    BC_TRY(check_range(b, x, x_off, (size_t)n_rows * v_dim * 4, "gdn_gated_norm"));
    BC_TRY(check_range(b, z, z_off, (size_t)n_rows * v_dim * 4, "gdn_gated_norm"));
    BC_TRY(check_range(b, weight, w_off, (size_t)v_dim * 4, "gdn_gated_norm"));
    return b->run("gdn_gated_norm", n_rows, v_dim, 0, 1, [&] {
        return k::gdn_gated_norm(b->stream, at<float>(x, x_off), at<const float>(z, z_off), at<const float>(weight, w_off), v_dim, n_rows, eps);
    });
}

bc_status bc_op_attention_gate(bc_backend* b, bc_buffer* out, size_t out_off, bc_buffer* q_gate, size_t qg_off, uint32_t n_heads,
                               uint32_t head_dim, uint32_t n_tokens) {
    BC_TRY(recording(b));
    if (head_dim == 0 || n_heads == 0) return fail(BC_ERR_GATE_SHAPE, "attention gates need heads of at least one float, got %u x %u", n_heads, head_dim);
    BC_TRY(check_range(b, out, out_off, (size_t)n_tokens * n_heads * head_dim * 4, "attention_gate"));
    BC_TRY(check_range(b, q_gate, qg_off, (size_t)n_tokens * n_heads * head_dim * 8, "attention_gate"));
    return b->run("attention_gate", n_tokens, n_heads * head_dim, 0, 1, [&] {
        return k::attention_gate(b->stream, at<float>(out, out_off), at<const float>(q_gate, qg_off), n_heads, head_dim, n_tokens);
    });
}

}  // extern "C"
