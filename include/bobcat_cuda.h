/* bobcat-cuda: the C ABI of the B200 (sm_100a) decode / prefill path for bobcat.
 *
 * Every entry point is plain C: opaque handles, pointers and sizes. Nothing here allocates with or
 * depends on any Python or tensor library. Each group names the reference interface it stands in
 * for (paths are relative to the bobcat repository root).
 *
 * Conventions
 *  - Every call returns a bc_status. On failure bc_last_error() holds a message for the calling
 *    thread. The library never prints, aborts or throws across this boundary
 *    (the reference's rule: AGENTS.md "library code never prints, panics or exits").
 *  - Arguments are validated before any device work; sequence positions advance only on success
 *    (crates/bobcat/src/lfm2_metal.rs:314-332, :363).
 *  - Handles are not thread-safe; distinct handles are independent
 *    (crates/bobcat/tests/metal_commands.rs:12-59).
 *  - Views of activation vectors (x, y, norm weights, q, out) must start on a 16-byte boundary; the
 *    kernels read them with 128-bit loads. Ops with a scalar variant fall back to it; the others
 *    reject the offset with BC_ERR_ARGUMENT before launching anything.
 *  - There is no CPU fallback. Opening a backend without a CUDA device fails with BC_ERR_NO_DEVICE.
 */
#ifndef BOBCAT_CUDA_H
#define BOBCAT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: crates/bobcat/src/error.rs:10-97 and crates/bobcat-metal/src/backend.rs:163-298 */
typedef int32_t bc_status;
enum {
    BC_OK = 0,
    BC_ERR_IO = 1,               /* Error::Io */
    BC_ERR_GGUF = 2,             /* Error::Gguf (any bobcat_gguf::Error) */
    BC_ERR_METADATA = 3,         /* Error::Metadata */
    BC_ERR_ARCHITECTURE = 4,     /* Error::Architecture */
    BC_ERR_HYPERPARAMETERS = 5,  /* Error::Hyperparameters */
    BC_ERR_ODD_HEAD_DIM = 6,     /* Error::OddHeadDim */
    BC_ERR_MISSING_TENSOR = 7,   /* Error::MissingTensor */
    BC_ERR_TENSOR_SHAPE = 8,     /* Error::TensorShape */
    BC_ERR_TENSOR_TYPE = 9,      /* Error::TensorType */
    BC_ERR_KV_HEADS = 10,        /* Error::KvHeads */
    BC_ERR_TOKEN = 11,           /* Error::Token */
    BC_ERR_CONTEXT_FULL = 12,    /* Error::ContextFull */
    BC_ERR_ARGUMENT = 13,        /* Error::Argument */
    BC_ERR_UNSUPPORTED = 14,     /* Error::MetalUnsupported */
    BC_ERR_NO_DEVICE = 20,       /* bobcat_metal::Error::NoDevice */
    BC_ERR_ALLOCATION = 21,      /* ::Allocation */
    BC_ERR_NOT_RECORDING = 22,   /* ::NotRecording */
    BC_ERR_ALREADY_RECORDING = 23, /* ::AlreadyRecording */
    BC_ERR_OUT_OF_BOUNDS = 24,   /* ::OutOfBounds and ::Access */
    BC_ERR_FOREIGN_BUFFER = 25,  /* ::ForeignBuffer */
    BC_ERR_BUSY = 26,            /* ::Busy */
    BC_ERR_ATTENTION_LIMITS = 27, /* ::AttentionLimits */
    BC_ERR_GATE_SHAPE = 28,      /* ::GateShape */
    BC_ERR_NO_FUSED_CONV = 29,   /* ::NoFusedConv */
    BC_ERR_NO_EXPANSION = 30,    /* ::NoExpansion */
    BC_ERR_NO_EXPERTS = 31,      /* ::NoExperts */
    BC_ERR_DELTANET_LIMITS = 32, /* ::DeltaNetLimits */
    BC_ERR_EXPERT_LIMITS = 33,   /* ::ExpertLimits */
    BC_ERR_EXECUTION = 34        /* ::Execution (a CUDA error while running recorded work) */
};

/* The message of the calling thread's latest failure ("" when none). */
const char* bc_last_error(void);
/* The library's version string. */
const char* bc_version(void);

/* ---- weight formats: bobcat_metal::Format (crates/bobcat-metal/src/backend.rs:408-449).
 * The numeric values are the ggml type ids (crates/bobcat-gguf/src/lib.rs:126-152). */
enum { BC_F32 = 0, BC_F16 = 1, BC_Q4_0 = 2, BC_Q8_0 = 8, BC_Q6_K = 14 };

/* ---- how a batched multiply combines with its output: bobcat_metal::Store (backend.rs:361-370) */
enum { BC_STORE_OVERWRITE = 0, BC_STORE_ACCUMULATE = 1, BC_STORE_SWIGLU = 2 };

/* ============================================================================================
 * Backend: one CUDA device + one stream + the buffers allocated on it.
 * Stands in for `bobcat_metal::Metal` (crates/bobcat-metal/src/backend.rs:1027-1340).
 * ============================================================================================ */
typedef struct bc_backend bc_backend;
typedef struct bc_buffer bc_buffer;

/* Metal::open (backend.rs:1083). `stream` may be an existing cudaStream_t the caller owns (work is
 * then ordered with the caller's other work on it) or NULL for a stream the backend creates. */
bc_status bc_backend_open(int32_t device, void* stream, bc_backend** out);
void bc_backend_close(bc_backend* backend);
/* The cudaStream_t every launch of this backend goes to. */
void* bc_backend_stream(bc_backend* backend);

/* Metal::new_buffer (backend.rs:1124): `len` zeroed bytes of device memory. */
bc_status bc_buffer_new(bc_backend* backend, size_t len, bc_buffer** out);
void bc_buffer_free(bc_buffer* buffer);
size_t bc_buffer_len(const bc_buffer* buffer);
/* The device address, for callers that share the buffer with their own CUDA code. */
void* bc_buffer_device_ptr(bc_buffer* buffer);
/* Metal::write / Metal::read (backend.rs:1180-1205): host <-> device copies, complete on return.
 * Fail with BC_ERR_BUSY while a recording is open, BC_ERR_OUT_OF_BOUNDS past the end. */
bc_status bc_buffer_write(bc_buffer* buffer, size_t offset, const void* data, size_t len);
bc_status bc_buffer_read(bc_buffer* buffer, size_t offset, void* out, size_t len);

/* Convert a matrix of `format` from its GGUF byte layout (`data`, n_rows * row_bytes) into the
 * device layout the kernels read, in a new buffer. F32, F16, Q8_0 and Q6_K are copied unchanged.
 * Q4_0 is split into 16-byte quant groups followed by the fp16 scales; values are unchanged bit
 * for bit. (Q8_0 and Q6_K - the embedding type of the published Q4_0 files,
 * crates/bobcat/tests/lfm2_reference.rs:39 - run on the general kernels: every op takes them, at a
 * lower rate than Q4_0.)
 * No reference counterpart by name: the reference reads the mapped file in place
 * (crates/bobcat/src/lfm2_metal.rs:137-146); a discrete GPU uploads once instead. */
bc_status bc_matrix_upload(bc_backend* backend, int32_t format, const void* data, uint32_t n_rows,
                           uint32_t n_cols, bc_buffer** out);

/* Metal::begin / barrier / commit / wait / end / discard (backend.rs:1244-1279). Launches are
 * legal only between begin and commit/end. `barrier` orders later launches after earlier ones;
 * on a CUDA stream that order already holds, so it records nothing. A ticket is complete once
 * bc_wait returns; `seconds` (nullable) receives the GPU time of the recorded work. */
typedef uint64_t bc_ticket;
bc_status bc_begin(bc_backend* backend);
bc_status bc_barrier(bc_backend* backend);
bc_status bc_commit(bc_backend* backend, bc_ticket* ticket);
bc_status bc_wait(bc_backend* backend, bc_ticket ticket, double* seconds);
bc_status bc_end(bc_backend* backend, double* seconds);
void bc_discard(bc_backend* backend);

/* Metal::set_profiling / profile (backend.rs:1285-1340): per (kernel, n_rows, n_cols) totals. */
typedef struct bc_profile_entry {
    const char* name;
    uint32_t n_rows, n_cols;
    uint64_t calls;
    double seconds;
    uint64_t bytes; /* weight bytes the launches read, for GB/s */
} bc_profile_entry;
bc_status bc_set_profiling(bc_backend* backend, int32_t enabled);
/* Copies up to `capacity` entries; `count` receives the number available. */
bc_status bc_profile(bc_backend* backend, bc_profile_entry* out, size_t capacity, size_t* count);

/* ---- ops. A (buffer, byte offset) pair is the reference's `View` (backend.rs:337-341). Every
 * op checks its ranges before launching (check_range, backend.rs:2772-2790). */

/* Metal::matvec (backend.rs:1344-1380): y[r] (+)= sum_c W[r,c] * x^[c], with x^ = RMSNorm(x) *
 * norm_weight when `norm` is non-null. `weights` must come from bc_matrix_upload. */
bc_status bc_op_matvec(bc_backend* b, int32_t format, bc_buffer* weights, size_t w_off, uint32_t n_rows,
                       uint32_t n_cols, bc_buffer* x, size_t x_off, bc_buffer* y, size_t y_off,
                       bc_buffer* norm, size_t norm_off, float eps, int32_t accumulate);
/* Metal::matvec_swiglu (backend.rs:1385-1417): y = silu(gate x^) * (up x^). */
bc_status bc_op_matvec_swiglu(bc_backend* b, int32_t format, bc_buffer* gate, size_t gate_off, bc_buffer* up,
                              size_t up_off, uint32_t n_rows, uint32_t n_cols, bc_buffer* x, size_t x_off,
                              bc_buffer* norm, size_t norm_off, float eps, bc_buffer* y, size_t y_off);
/* Metal::matvec_conv (backend.rs:2329-2382): LFM2 decode conv block up to the output projection:
 * RMSNorm, in_proj rows (ch, n_embd+ch, 2 n_embd+ch) -> B, C, X, bx = B*X, taps over bx and the
 * history, history shift, out = C * conv. */
bc_status bc_op_matvec_conv(bc_backend* b, int32_t format, bc_buffer* in_proj, size_t w_off, uint32_t n_cols,
                            bc_buffer* x, size_t x_off, bc_buffer* norm, size_t norm_off, float eps,
                            bc_buffer* taps, size_t taps_off, bc_buffer* history, size_t hist_off,
                            bc_buffer* out, size_t out_off, uint32_t n_embd, uint32_t kernel);
/* Metal::short_conv / short_conv_batch (backend.rs:2384-2468): the same conv over `n_tokens` rows
 * of a [n_tokens][3 n_embd] B|C|X projection. */
bc_status bc_op_short_conv(bc_backend* b, bc_buffer* bcx, size_t bcx_off, bc_buffer* taps, size_t taps_off,
                           bc_buffer* history, size_t hist_off, bc_buffer* out, size_t out_off,
                           uint32_t n_embd, uint32_t kernel, uint32_t n_tokens);
/* Metal::matmul (backend.rs:2470-2517): Y[t,r] = sum_c W[r,c] X[t,c] for n_tokens rows, combined
 * with Y as `store` says. Q4_0 weights are multiplied on the tensor cores in half precision with
 * f32 accumulation, inputs rounded to half, as the reference's Q4_0 path does
 * (crates/bobcat-metal/src/matmul.metal:519-521). */
bc_status bc_op_matmul(bc_backend* b, int32_t format, bc_buffer* weights, size_t w_off, uint32_t n_rows,
                       uint32_t n_cols, bc_buffer* x, size_t x_off, bc_buffer* y, size_t y_off,
                       uint32_t n_tokens, int32_t store);
/* Metal::expand (backend.rs:2519-2550), widened: dequantise a whole uploaded matrix to contiguous
 * rows of f32 (out_half = 0) or half (out_half = 1). The f32 result is bit-identical to
 * scalar::dequantize (crates/bobcat/src/scalar.rs:59-105). */
bc_status bc_op_expand(bc_backend* b, int32_t format, bc_buffer* weights, size_t w_off, bc_buffer* out,
                       size_t out_off, uint32_t n_rows, uint32_t n_cols, int32_t out_half);
/* Metal::embed (backend.rs:2570-2610): rows of the embedding matrix picked by `n_tokens` ids. */
bc_status bc_op_embed(bc_backend* b, int32_t format, bc_buffer* weights, size_t w_off, uint32_t n_vocab,
                      bc_buffer* tokens, size_t tok_off, bc_buffer* out, size_t out_off, uint32_t n_embd,
                      uint32_t n_tokens);
/* Metal::rms_norm (backend.rs:2034-2068). */
bc_status bc_op_rms_norm(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* weight, size_t w_off,
                         bc_buffer* out, size_t out_off, uint32_t n_cols, uint32_t n_rows, float eps);
/* Metal::norm_rope (backend.rs:2070-2123): per-head RMSNorm, NeoX rotation of the first n_rot
 * elements at positions first_pos.., store as f32 or half. Strides are in elements per token. */
bc_status bc_op_norm_rope(bc_backend* b, bc_buffer* src, size_t src_off, bc_buffer* dst, size_t dst_off,
                          int32_t dst_half, bc_buffer* weight, size_t w_off, uint32_t n_heads, uint32_t head_dim,
                          uint32_t head_stride, uint32_t n_rot, uint32_t first_pos, uint32_t n_tokens,
                          uint32_t src_stride, uint32_t dst_stride, float theta, float eps);
/* Metal::convert_half / copy (backend.rs:2126-2148, :2552-2568). */
bc_status bc_op_convert_half(bc_backend* b, bc_buffer* src, size_t src_off, bc_buffer* dst, size_t dst_off, uint32_t n);
bc_status bc_op_copy(bc_backend* b, bc_buffer* src, size_t src_off, bc_buffer* dst, size_t dst_off, uint32_t n);
/* Metal::attention (backend.rs:2150-2320): causal grouped-query attention of n_queries tokens at
 * positions first_pos.. over cache rows [0, first_pos + i]. The caches are [n_ctx][n_kv_heads *
 * head_dim] f32 or half. `scratch` needs bc_attention_scratch_floats floats. */
bc_status bc_op_attention(bc_backend* b, bc_buffer* q, size_t q_off, bc_buffer* k_cache, size_t k_off,
                          bc_buffer* v_cache, size_t v_off, int32_t kv_half, bc_buffer* scratch, size_t s_off,
                          bc_buffer* out, size_t out_off, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                          uint32_t first_pos, uint32_t n_queries, uint32_t n_ctx);
/* attention_scratch_floats (backend.rs:2739-2748). */
size_t bc_attention_scratch_floats(uint32_t n_heads, uint32_t head_dim, uint32_t n_ctx, uint32_t n_queries);
/* Attention for callers that may not allocate device memory. No counterpart in the reference.
 *
 * Who needs it: an embedding engine that plans one device pool up front and gives a plugin only
 * the tensors of the call, or a serving loop that cannot take the device-wide synchronisation of
 * cudaMalloc in the middle of a decode. bc_op_attention wants a scratch buffer for its chunk
 * partials; this variant keeps them in an 8 MiB array built into the library (2 Mi floats, held by
 * every GPU that loads the library until the process exits) and calls no cudaMalloc, cudaFree or
 * other allocating routine. Same kernels, same results as bc_op_attention.
 *
 * All pointers are device pointers on the current device; `stream` is a cudaStream_t (NULL for the
 * default stream). q and out are [n_queries][n_heads * head_dim] f32; the caches are
 * [n_ctx][n_kv_heads * head_dim] f32 or half. Shapes whose partials do not fit
 * (bc_attention_scratch_floats(...) > 2 Mi) fail with BC_ERR_ARGUMENT and launch nothing.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 * that call with the device current and before starting any stream capture. Every call shares the
 * one array, which keeps the previous call's contents: the kernels write every partial before they
 * read it, so nothing needs clearing, but two calls that overlap on the GPU (different streams, or
 * different threads) race on it. Serialise them. */
bc_status bc_attention_static(void* stream, const float* q, const void* k_cache, const void* v_cache, int32_t kv_half,
                              float* out, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t first_pos,
                              uint32_t n_queries, uint32_t n_ctx);
/* Sampler::sample (crates/bobcat-cli/src/sampler.rs:45-112) on the device, in llama.cpp's order:
 * the repetition penalty (each distinct token among the last 64 of `recent` once: positive logits
 * divided, the others multiplied), top-k, top-p and min-p on the softmax at temperature one, the
 * temperature on the survivors, then the draw. temperature <= 0 picks the most likely token (ties
 * to the lowest index). Mirrors bobcat::Sampling (crates/bobcat/src/lfm2.rs:273-282). */
typedef struct bc_sampling {
    float temperature;
    uint32_t top_k; /* 0: no limit */
    float top_p, min_p, repeat_penalty;
} bc_sampling;
/* The pick from `n` logits at `logits` (changed in place by the penalty, as the reference changes
 * its slice) goes to the 32-bit word at `out`. `recent` holds n_recent token ids (may be null with
 * n_recent 0). `uniform` in [0, 1) is the random draw: the reference takes it from its host-side
 * generator, whose stream a caller keeps on the host. Logits equal to a cut value are all kept
 * where the reference's unstable sort keeps an arbitrary subset. */
bc_status bc_op_sample(bc_backend* b, bc_buffer* logits, size_t logits_off, uint32_t n, bc_buffer* recent, size_t recent_off,
                       uint32_t n_recent, const bc_sampling* settings, float uniform, bc_buffer* out, size_t out_off);
/* Metal::argmax (backend.rs:2612-2617): index of the largest of n floats, ties to the lowest. */
bc_status bc_op_argmax(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* out, size_t out_off, uint32_t n);
/* Readback / Metal::new_readback / argmax_readback / read_readback (backend.rs:324-333,
 * :2619-2676): token slots the CPU reads while later recordings still run. argmax_readback stores
 * the index at `out` and in `slot`; bc_read_readback returns the slot's token once the recording
 * that last wrote it has finished, BC_ERR_BUSY before that, BC_ERR_OUT_OF_BOUNDS for a slot no
 * recording has written. */
typedef struct bc_readback bc_readback;
bc_status bc_readback_new(bc_backend* backend, size_t slots, bc_readback** out);
void bc_readback_free(bc_readback* readback);
bc_status bc_op_argmax_readback(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* out, size_t out_off, bc_readback* readback,
                                size_t slot, uint32_t n);
bc_status bc_read_readback(bc_backend* b, const bc_readback* readback, size_t slot, uint32_t* token);
/* ---- mixture of experts. A token's route is 2 * n_used 32-bit words: the picked expert ids, then
 * their weights as float bits (crates/bobcat-metal/src/moe.metal:4-6); bc_route_bytes sizes it
 * (route_bytes, backend.rs:2724). At most 128 experts, 8 used (backend.rs:97-100). */
size_t bc_route_bytes(uint32_t n_used, uint32_t n_tokens);
/* Metal::moe_route (backend.rs:1428-1479): sigmoid router scores of an F32 router matrix, the
 * n_used largest of score + bias with ties to the lower expert, weights score / (sum + 1e-6).
 * With `norm` non-null each token is RMS-normalised first and stored at `normed`. The picked ids
 * equal the reference's `route` (crates/bobcat/src/lfm2.rs:691-709) on the same input. */
bc_status bc_op_moe_route(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* norm, size_t norm_off, float eps,
                          bc_buffer* normed, size_t normed_off, bc_buffer* router, size_t router_off, bc_buffer* bias,
                          size_t bias_off, bc_buffer* route, size_t route_off, uint32_t n_cols, uint32_t n_experts,
                          uint32_t n_used, uint32_t n_tokens);
/* Metal::moe_group (backend.rs:1599-1637): offsets[n_experts + 1], entries[n_tokens * n_used]. */
bc_status bc_op_moe_group(bc_backend* b, bc_buffer* route, size_t route_off, bc_buffer* offsets, size_t off_off,
                          bc_buffer* entries, size_t ent_off, uint32_t n_experts, uint32_t n_used, uint32_t n_tokens);
/* Metal::matvec_experts_swiglu (backend.rs:1481-1536): `gate` and `up` hold n_experts stacked
 * matrices of n_rows rows; y[token][slot][row] = silu(gate_e x) * (up_e x). */
bc_status bc_op_matvec_experts_swiglu(bc_backend* b, int32_t format, bc_buffer* gate, size_t gate_off, bc_buffer* up,
                                      size_t up_off, uint32_t n_rows, uint32_t n_cols, uint32_t n_experts, bc_buffer* x,
                                      size_t x_off, bc_buffer* route, size_t route_off, uint32_t n_used, bc_buffer* y,
                                      size_t y_off, uint32_t n_tokens);
/* Metal::matvec_experts_down (backend.rs:1538-1597): y[token][row] += sum over slots of
 * weight * (down_e row . x[token][slot]). */
bc_status bc_op_matvec_experts_down(bc_backend* b, int32_t format, bc_buffer* down, size_t down_off, uint32_t n_rows,
                                    uint32_t n_cols, uint32_t n_experts, bc_buffer* x, size_t x_off, bc_buffer* route,
                                    size_t route_off, uint32_t n_used, bc_buffer* y, size_t y_off, uint32_t n_tokens);
/* Metal::matmul_experts (backend.rs:1639-1703): grouped multiply over the entries of moe_group.
 * `up` non-null pairs gate and up with a SwiGLU store. `gather` reads a token's shared input row;
 * otherwise each entry reads its own row. Output rows are the entries'. */
bc_status bc_op_matmul_experts(bc_backend* b, int32_t format, bc_buffer* weights, size_t w_off, bc_buffer* up, size_t up_off,
                               uint32_t n_rows, uint32_t n_cols, uint32_t n_experts, bc_buffer* x, size_t x_off,
                               int32_t gather, bc_buffer* offsets, size_t off_off, bc_buffer* entries, size_t ent_off,
                               uint32_t n_used, bc_buffer* y, size_t y_off, uint32_t n_tokens);
/* Metal::moe_combine (backend.rs:1705-1737): y[t] += sum_s weight[t, s] * expert_out[t * n_used + s]. */
bc_status bc_op_moe_combine(bc_backend* b, bc_buffer* expert_out, size_t eo_off, bc_buffer* route, size_t route_off,
                            bc_buffer* y, size_t y_off, uint32_t n_embd, uint32_t n_used, uint32_t n_tokens);
/* ---- Qwen3.5 Gated DeltaNet and gated attention. Shapes follow DeltaShape (backend.rs:2704-2722):
 * n_k_heads key heads of k_dim, n_v_heads value heads of v_dim (a multiple of n_k_heads), conv_dim =
 * 2 * n_k_heads * k_dim + n_v_heads * v_dim. Limits: conv kernel 2..8, k_dim a multiple of 32 up to
 * 128, v_dim a multiple of 32 up to 256 (backend.rs:109-112, :1899-1911). */
/* Metal::gdn_conv (backend.rs:1739-1817): causal convolution + SiLU over the q|k|v channels of
 * n_tokens rows; `history` holds the last kernel - 1 raw inputs of each channel, [conv_dim][kernel - 1]. */
bc_status bc_op_gdn_conv(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* taps, size_t taps_off, bc_buffer* history,
                         size_t hist_off, bc_buffer* out, size_t out_off, uint32_t conv_dim, uint32_t kernel, uint32_t n_tokens);
/* Metal::gdn_gates (backend.rs:1851-1886), in place: beta = sigmoid(beta);
 * alpha = exp(a * softplus(alpha + dt_bias)) over [n_tokens][n_v_heads]. */
bc_status bc_op_gdn_gates(bc_backend* b, bc_buffer* beta, size_t beta_off, bc_buffer* alpha, size_t alpha_off, bc_buffer* a,
                          size_t a_off, bc_buffer* dt_bias, size_t dt_off, uint32_t n_v_heads, uint32_t n_tokens);
/* Metal::gdn_recurrence (backend.rs:1888-1979): the gated delta rule over n_tokens rows of the
 * convolved q|k|v, carrying `state` [n_v_heads][k_dim][v_dim]. Value head h reads key head
 * h % n_k_heads. `normalize` L2-normalises q (times 1/sqrt(k_dim)) and k first. */
bc_status bc_op_gdn_recurrence(bc_backend* b, bc_buffer* qkv, size_t qkv_off, bc_buffer* beta, size_t beta_off, bc_buffer* decay,
                               size_t decay_off, bc_buffer* state, size_t state_off, bc_buffer* out, size_t out_off,
                               uint32_t n_k_heads, uint32_t n_v_heads, uint32_t k_dim, uint32_t v_dim, uint32_t n_tokens,
                               int32_t normalize);
/* Metal::gdn_gated_norm (backend.rs:1819-1849): x = RMSNorm(x) * weight * silu(z) per row of v_dim. */
bc_status bc_op_gdn_gated_norm(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* z, size_t z_off, bc_buffer* weight,
                               size_t w_off, uint32_t v_dim, uint32_t n_rows, float eps);
/* Metal::attention_gate (backend.rs:2001-2032): out[t][h][d] *= sigmoid(q_gate[t][h][head_dim + d])
 * with q_gate the interleaved [q | gate] projection of [n_tokens][n_heads][2 * head_dim]. */
bc_status bc_op_attention_gate(bc_backend* b, bc_buffer* out, size_t out_off, bc_buffer* q_gate, size_t qg_off, uint32_t n_heads,
                               uint32_t head_dim, uint32_t n_tokens);
/* Metal::silu_mul (backend.rs:1983-1999): x = silu(gate) * x, elementwise. */
bc_status bc_op_silu_mul(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* gate, size_t g_off, uint32_t n);

/* ============================================================================================
 * Model: a parsed GGUF file + its hyperparameters (host side).
 * Stands in for lfm2::Model::load (crates/bobcat/src/lfm2.rs:186-233) and
 * qwen35::Model::load (crates/bobcat/src/qwen35.rs:179-229); the architecture is read from
 * `general.architecture` and may be "lfm2", "lfm2moe" or "qwen35".
 * ============================================================================================ */
typedef struct bc_model bc_model;

enum { BC_ARCH_LFM2 = 0, BC_ARCH_LFM2MOE = 1, BC_ARCH_QWEN35 = 2 };

/* lfm2::Hyperparameters (lfm2.rs:18-49) and qwen35::Hyperparameters (qwen35.rs:33-68) in one
 * record; fields a family lacks are zero. */
typedef struct bc_hparams {
    int32_t architecture;
    uint32_t n_layers, n_attention_layers, n_conv_layers, n_delta_layers;
    uint32_t n_embd, n_ff, n_vocab;
    uint32_t n_heads, n_kv_heads, head_dim, n_rot;
    uint32_t conv_kernel;
    uint32_t n_experts, n_experts_used, n_ff_expert;
    uint32_t n_k_heads, n_v_heads, k_head_dim, v_head_dim;
    float rope_theta, norm_eps;
} bc_hparams;

bc_status bc_model_load(const char* path, bc_model** out);
void bc_model_free(bc_model* model);
bc_status bc_model_hparams(const bc_model* model, bc_hparams* out);
/* Writes 1 for each attention layer and 0 for each other layer (Model::attention_layers,
 * lfm2.rs:241-245). `out` holds n_layers bytes. */
bc_status bc_model_attention_layers(const bc_model* model, uint8_t* out, size_t len);

/* ============================================================================================
 * Sequence: the device state of one decode.
 * Stands in for `Lfm2Metal` (crates/bobcat/src/lfm2_metal.rs:103-762) and `Qwen35Metal`
 * (crates/bobcat/src/qwen35_metal.rs:112-676).
 * ============================================================================================ */
typedef struct bc_seq bc_seq;
typedef struct bc_checkpoint bc_checkpoint;

/* Buffers that receive activations: lfm2::Trace (lfm2.rs:630-675). Each pointer is nullable as a
 * group (all three or none); `n_tokens` is the token count the caller sized them for. */
typedef struct bc_trace {
    float* embedding;  /* [n_tokens][n_embd] */
    float* layers;     /* [n_layers][n_tokens][n_embd] */
    float* final_norm; /* [n_tokens][n_embd] */
    uint32_t n_tokens;
} bc_trace;

/* Lfm2Metal::new / Qwen35Metal::new (lfm2_metal.rs:125, qwen35_metal.rs:112). Uploads the model's
 * weights to the backend's device on first use and shares them between sequences. */
bc_status bc_seq_new(bc_model* model, bc_backend* backend, uint32_t n_ctx, int32_t kv_half, bc_seq** out);
void bc_seq_free(bc_seq* seq);
/* Qwen35Metal::n_past (qwen35_metal.rs:231). */
uint32_t bc_seq_n_past(const bc_seq* seq);
/* step (lfm2_metal.rs:308): `logits` (n_vocab floats) and `trace` (one token) are nullable. */
bc_status bc_seq_step(bc_seq* seq, uint32_t token, float* logits, size_t logits_len, bc_trace* trace);
/* prefill (lfm2_metal.rs:662; qwen35_metal.rs:557): `final_norm` (n_embd floats of the last token,
 * Qwen's extra output) is nullable. */
bc_status bc_seq_prefill(bc_seq* seq, const uint32_t* tokens, size_t n_tokens, float* logits, size_t logits_len,
                         float* final_norm, size_t final_norm_len, bc_trace* trace);
/* greedy_token (lfm2_metal.rs:372). */
bc_status bc_seq_greedy_token(bc_seq* seq, uint32_t* token);
/* generate / generate_next (lfm2_metal.rs:401, :411). */
bc_status bc_seq_generate(bc_seq* seq, uint32_t* out, size_t n);
bc_status bc_seq_generate_next(bc_seq* seq, uint32_t* out, size_t n);
/* generate_stream (lfm2_metal.rs:425): `emit` runs on the calling thread and returns nonzero to
 * continue. `gained` (capacity `gained_cap`) receives the tokens the sequence gained. */
typedef int32_t (*bc_emit_fn)(uint32_t token, void* user);
bc_status bc_seq_generate_stream(bc_seq* seq, uint32_t max_tokens, bc_emit_fn emit, void* user, uint32_t* gained,
                                 size_t gained_cap, size_t* n_gained);
/* The engine's sampled decode step without the logits leaving the device
 * (crates/bobcat-cli/src/engine.rs:615-630 reads them back and samples on the host): pick the next
 * token from the sequence's current logits with bc_op_sample's rules and return it. The caller
 * feeds it to bc_seq_step (with or without logits) to advance. */
bc_status bc_seq_sample(bc_seq* seq, const bc_sampling* settings, float uniform, const uint32_t* recent, size_t n_recent, uint32_t* token);
/* step (lfm2_metal.rs:308) whose logits are computed but stay on the device, for a following
 * bc_seq_sample or bc_seq_greedy_token. */
bc_status bc_seq_step_on_device(bc_seq* seq, uint32_t token);
/* reset / checkpoint / restore (lfm2_metal.rs:238-288; qwen35_metal.rs:238-297). */
bc_status bc_seq_reset(bc_seq* seq);
bc_status bc_seq_checkpoint(bc_seq* seq, bc_checkpoint** out);
bc_status bc_seq_restore(bc_seq* seq, const bc_checkpoint* checkpoint);
void bc_checkpoint_free(bc_checkpoint* checkpoint);
/* ---- paged KV cache and cached prefixes.
 * The reference keeps each sequence's KV cache as one buffer indexed layer * n_ctx * kv_dim + pos *
 * kv_dim + kv_head * head_dim + d (crates/bobcat/src/lfm2_metal.rs:1064-1067) and reuses a prompt
 * prefix only inside the sequence that computed it (checkpoint / restore, lfm2_metal.rs:250-288;
 * the engine's prefix cache, crates/bobcat-cli/src/engine.rs:561-584). Here a sequence made with
 * bc_seq_new_paged keeps that index - its kernels see one contiguous range per cache - but the
 * memory behind the range comes in physical pages (one page = page_positions positions of one layer
 * of K or V), and sequences that continue the same cached prefix map the same pages. */
/* Lfm2Metal::new with paged caches. Fails with BC_ERR_UNSUPPORTED when a KV row does not divide
 * the device's page size. */
bc_status bc_seq_new_paged(bc_model* model, bc_backend* backend, uint32_t n_ctx, int32_t kv_half, bc_seq** out);
/* The arithmetic of the page table: the flat index above (with `stride`, the positions between two
 * layers: n_ctx rounded up to whole pages) and the page (numbered layer * stride / page_positions +
 * pos / page_positions) and element offset inside the page that hold it. flat_index ==
 * page * page_positions * kv_dim + offset for every element, which is what keeps the kernels'
 * indexing the reference's. */
bc_status bc_kv_page_locate(uint32_t kv_dim, uint32_t head_dim, uint32_t page_positions, uint32_t stride, uint32_t layer, uint32_t pos,
                            uint32_t kv_head, uint32_t d, uint64_t* flat_index, uint32_t* page, uint64_t* offset);
/* Page size in positions, pages mapped (K and V) and how many of them are shared with a prefix or
 * another sequence; zeros for a sequence with contiguous caches. */
bc_status bc_seq_kv_pages(const bc_seq* seq, uint32_t* page_positions, uint32_t* pages, uint32_t* shared_pages);
/* A cached prefix: the state of `seq` at its current position - recurrent state (convolution
 * history, DeltaNet state), logits, and the KV rows [0, n_past) - kept on the device. Full pages of
 * a paged sequence are held by reference, everything else is copied device to device. The prefix
 * outlives the sequence. */
typedef struct bc_prefix bc_prefix;
bc_status bc_seq_prefix_save(bc_seq* seq, bc_prefix** out);
/* Start `seq` (same model, device and cache type; n_ctx at least the prefix's length) from the
 * prefix: afterwards it stands at the prefix's position exactly as the sequence that computed it
 * did, and prefill / step / generate continue from there. A paged sequence maps the prefix's full
 * pages (no copy) and keeps pages of its own from the first partly-filled page on; a prefix of a
 * paged sequence loads only into paged sequences. bc_seq_reset gives the sequence private pages
 * again. */
bc_status bc_seq_prefix_load(bc_seq* seq, const bc_prefix* prefix);
void bc_prefix_free(bc_prefix* prefix);
uint32_t bc_prefix_n_past(const bc_prefix* prefix);
/* last_encode_seconds / last_gpu_seconds (lfm2_metal.rs:223-230). */
bc_status bc_seq_timings(const bc_seq* seq, double* encode_seconds, double* gpu_seconds);

/* ============================================================================================
 * Engine: one sequence plus the bookkeeping of the reference's engine that lets a request reuse
 * what earlier requests left on the device (crates/bobcat-cli/src/engine.rs). Token ids in, token
 * ids and numbers out: templates, tokenizer, stop strings and tool calls stay with the caller.
 * ============================================================================================ */
typedef struct bc_engine bc_engine;
/* Engine::new's device half: a sequence of n_ctx positions; `seed` starts the stream of draws for
 * sampled requests. */
bc_status bc_engine_new(bc_model* model, bc_backend* backend, uint32_t n_ctx, int32_t kv_half, uint64_t seed, bc_engine** out);
void bc_engine_free(bc_engine* engine);
/* Engine::generate_inner (engine.rs:510-647) on the rendered prompt `tokens`. Tokens that extend
 * what the sequence has consumed continue from there; tokens that extend the history recorded at
 * the previous request's turn restore its checkpoint; anything else starts over. `turn` is the
 * index of the prompt's last turn-opening token (the reply's turn; the prompt up to it becomes the
 * next history), or -1. At most max_tokens tokens (and no more than the context holds) are
 * generated: greedily through the pipelined stream when `sampling` is null or greedy, else picked
 * on the device by bc_seq_sample's rules with draws from the engine's stream. `emit` (nullable)
 * sees every token and returns zero to stop. out (capacity out_cap) receives the tokens, n_out
 * their count, cached_tokens (nullable) how many prompt tokens were already on the device. */
bc_status bc_engine_generate(bc_engine* engine, const uint32_t* tokens, size_t n_tokens, int64_t turn, uint32_t max_tokens,
                             const bc_sampling* sampling, bc_emit_fn emit, void* user, uint32_t* out, size_t out_cap, size_t* n_out,
                             uint32_t* cached_tokens);
/* Engine::score (engine.rs:372-446): scores[t] = log-probability of label_tokens[t] after prompt i,
 * for t in [label_offsets[i], label_offsets[i + 1]); prompt i is prompt_tokens[prompt_offsets[i] ..
 * prompt_offsets[i + 1]). The prompts' longest common prefix runs once; every prompt continues
 * from its checkpoint. The log-softmax is taken in f64 over the whole vocabulary. */
bc_status bc_engine_score(bc_engine* engine, const uint32_t* prompt_tokens, const size_t* prompt_offsets, size_t n_prompts,
                          const uint32_t* label_tokens, const size_t* label_offsets, double* scores);
/* Tokens the engine's sequence currently holds. */
uint32_t bc_engine_consumed(const bc_engine* engine);

/* ============================================================================================
 * Batch: n_seqs independent sequences of one model decoding together, one token each per pass,
 * so that a pass reads every weight once for all of them (LFM2 and LFM2-MoE models).
 * The reference has one sequence per runner and serves one request at a time
 * (crates/bobcat/src/lfm2_metal.rs:103-105, crates/bobcat-cli/src/serve.rs:4-7); a batch is n_seqs
 * such runners plus a pass whose row b computes what Lfm2Metal::step (lfm2_metal.rs:308) computes
 * for sequence b. Each sequence keeps its own KV cache, convolution history, position and logits.
 * ============================================================================================ */
typedef struct bc_batch bc_batch;

/* n_seqs sequences of `n_ctx` positions each (Lfm2Metal::new, lfm2_metal.rs:125, n_seqs times).
 * n_ctx must be at least n_seqs. */
bc_status bc_batch_new(bc_model* model, bc_backend* backend, uint32_t n_seqs, uint32_t n_ctx, int32_t kv_half, bc_batch** out);
void bc_batch_free(bc_batch* batch);
uint32_t bc_batch_n_seqs(const bc_batch* batch);
/* Sequence `index` of the batch, for the single-sequence calls (bc_seq_prefill to give it its
 * prompt, bc_seq_reset, bc_seq_n_past, bc_seq_step). The batch owns it: do not free it. */
bc_status bc_batch_seq(bc_batch* batch, uint32_t index, bc_seq** out);
/* Lfm2Metal::generate (lfm2_metal.rs:401) for every sequence at once: each sequence, which must
 * hold a prompt, gains `n` greedy tokens; out[b * n + i] is token i of sequence b. The sequences
 * may stand at different positions. Tokens equal those of n_seqs separate bc_seq_generate calls up
 * to the rounding of the batched products (half-precision operands, as in prefill). */
bc_status bc_batch_generate(bc_batch* batch, uint32_t* out, size_t n);
/* Which arithmetic the batched pass multiplies with. 0 (the default): half-precision operands on
 * the tensor cores, f32 accumulation - the arithmetic of the reference's batched Q4_0 products
 * (crates/bobcat-metal/src/matmul.metal:519-521), accurate to the 5e-3 class of its batched path.
 * Nonzero: f32 operands on the f32 tile kernels, accurate to the 1e-5 class of the single-token
 * products, at a lower rate. The difference matters where a small change of the activations picks
 * a different expert: with f32 operands every sequence decodes as it does alone. */
bc_status bc_batch_set_exact(bc_batch* batch, int32_t exact);
/* GPU seconds of the last bc_batch_generate and the kernels the batch has launched in total. */
bc_status bc_batch_timings(const bc_batch* batch, double* gpu_seconds, uint64_t* launches);

/* ============================================================================================
 * Communicator: one rank per GPU over NCCL, for the sharded configurations. No reference
 * counterpart (the reference is single-GPU, crates/bobcat-metal/src/lib.rs:5-8). NCCL is bound at
 * run time; a world of one needs no NCCL at all.
 * ============================================================================================ */
typedef struct bc_comm bc_comm;
#define BC_COMM_ID_BYTES 128
/* ncclGetUniqueId: rank 0 makes the id and hands it to the other ranks by any host-side means. */
bc_status bc_comm_unique_id(uint8_t* out, size_t len);
/* ncclCommInitRank on the backend's device; collectives run on the backend's stream. */
bc_status bc_comm_init(bc_backend* backend, const uint8_t* id, size_t id_len, int32_t rank, int32_t world, bc_comm** out);
void bc_comm_free(bc_comm* comm);
int32_t bc_comm_rank(const bc_comm* comm);
int32_t bc_comm_world(const bc_comm* comm);
/* Collectives this communicator has recorded so far, and how many of them were sums over ranks
 * taken by this library's own kernel over NVLink peer memory (each rank stores its partial vector
 * into buffers the ranks mapped from one another at bc_comm_init, then adds the ranks' vectors in
 * rank order) rather than by NCCL. BOBCAT_NO_PEER_REDUCE=1 leaves every collective to NCCL. */
uint64_t bc_comm_collectives(const bc_comm* comm);
uint64_t bc_comm_peer_reduces(const bc_comm* comm);

/* Expert-parallel multi-sequence decode of a mixture-of-experts model (moe_block,
 * crates/bobcat/src/lfm2.rs:413-440, sharded): this rank holds `n_seqs` of the world's sequences
 * and runs the experts [rank * n_experts / world, (rank + 1) * n_experts / world) for every
 * sequence of every rank. Per mixture-of-experts layer the ranks exchange tokens twice: the
 * normalised rows of all ranks' sequences are gathered on every rank (the dispatch: every rank then
 * routes all rows identically, lfm2.rs:691-709), each rank multiplies the rows that picked its
 * experts, and the expert outputs return to the rank that owns the sequence (the combine), where
 * they are added in the reference's slot order (lfm2.rs:426-439). An output row has exactly one
 * nonzero contributor, so the combine's sum over ranks is exact. Attention, convolution and dense
 * feed-forward layers run on the rank's own sequences. n_experts must be a multiple of the world
 * size; every rank must call bc_batch_generate together with the same token count. */
bc_status bc_batch_new_expert_parallel(bc_model* model, bc_backend* backend, bc_comm* comm, uint32_t n_seqs, uint32_t n_ctx,
                                       int32_t kv_half, bc_batch** out);

/* Tensor-parallel sequence of a Qwen3.5 model (Qwen35Metal::new, crates/bobcat/src/qwen35_metal.rs:112,
 * sharded): every rank of the communicator creates one and calls the same sequence methods with
 * the same arguments. A rank holds the weights of its share of the attention heads (whole KV heads
 * with the query heads that read them; ranks beyond the KV-head count share a KV head and split
 * its query heads), of the DeltaNet heads (key heads, and the value heads j with j % n_k_heads
 * among them, crates/bobcat-metal/src/gdn.metal:244), of the feed-forward rows and of the
 * vocabulary rows of the output matrix, with the KV cache, convolution history and DeltaNet state
 * of those heads. Each mixer and each feed-forward block ends in a sum over ranks of its output
 * projection (ncclAllReduce); the logits are gathered from every rank's vocabulary rows. The
 * residual stream, the logits and the picked tokens are the same on every rank. Sums over ranks
 * associate differently from the one-device sum, so results agree with bc_seq_new's to rounding
 * (the 1e-5 class of the single-token products), not bit for bit. */
bc_status bc_seq_new_tensor_parallel(bc_model* model, bc_backend* backend, bc_comm* comm, uint32_t n_ctx, int32_t kv_half,
                                     bc_seq** out);

#ifdef __cplusplus
}
#endif
#endif /* BOBCAT_CUDA_H */
