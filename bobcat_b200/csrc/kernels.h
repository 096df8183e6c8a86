// Launch functions of every CUDA kernel in the library. All pointers are device pointers; all
// launches go to `stream` and return the launch status without synchronising.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <utility>

#include <cstdint>

namespace bc {
namespace k {

// A matrix in the device layout.
//  F32 / F16: `data` holds n_rows contiguous rows.
//  Q4_0: `data` holds n_rows * (n_cols / 32) 16-byte quant groups, row-major, with the byte and
//  nibble order of the GGUF block (low nibbles are elements 0..15, high nibbles 16..31); `scales`
//  holds the matching fp16 scales. The split keeps every quant group 16-byte aligned so one lane
//  reads a block with one 128-bit load and a warp reads 512 contiguous bytes.
struct Mat {
    int32_t format = 0;
    const void* data = nullptr;
    const __half* scales = nullptr;
    // Q4_0 only, optional: the same values in the 16-row tile layout the tensor-core decode kernel
    // streams (see kernels_matvec_mma.cu). Null when the matrix has no such copy.
    const void* tiles = nullptr;
    uint32_t n_rows = 0, n_cols = 0;
    // Rows [first, first + rows) of this matrix.
    Mat rows(uint32_t first, uint32_t count) const;
    uint64_t bytes() const;  // bytes a full pass over the matrix reads
};

struct Norm {
    const float* weight = nullptr;  // null: no normalisation
    float eps = 0.f;
};

// Up to four matrices that share an input vector, multiplied in one launch.
struct MatvecSegment {
    Mat w;
    float* y = nullptr;
};

// Launch `kernel` with the programmatic-dependent-launch attribute (unless BOBCAT_NO_PDL=1), so it
// may start while the launch before it still runs. Only for kernels that call pdl_wait() before
// touching memory other launches write. `args` is the usual array of pointers to the arguments.
cudaError_t launch_kernel(const void* kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, void** args);
// Whether launches carry the programmatic-dependency attribute (BOBCAT_NO_PDL=1 turns it off).
bool pdl_enabled();
// launch_kernel for a kernel given by name, with its arguments as written in a <<<>>> launch. The
// kernel must call pdl_wait() before it touches what an earlier launch wrote or still reads.
template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}
// Raise `kernel`'s dynamic shared-memory limit to `smem` bytes on the current device if needed.
cudaError_t ensure_dynamic_smem(const void* kernel, size_t smem);
// Number of SMs of the current device.
int sm_count();

// Repack GGUF Q4_0 bytes (18-byte blocks) already on the device into the split layout.
cudaError_t repack_q4_0(cudaStream_t stream, const uint8_t* raw, uint64_t n_blocks, void* quants, __half* scales);

// The tile layout of a Q4_0 matrix: its size, whether this width has one, and the conversion from
// the split layout (both already on the device).
uint64_t tiles_bytes(uint32_t n_rows, uint32_t n_cols);
bool tiles_supported(uint32_t n_cols);
cudaError_t repack_tiles(cudaStream_t stream, const void* quants, const __half* scales, uint32_t n_rows, uint32_t n_cols, void* tiles);
// The tensor-core decode kernels; every matrix must carry `tiles`. matvec / matvec_swiglu /
// matvec_conv below pick them when they can.
cudaError_t matvec_mma(cudaStream_t stream, const MatvecSegment* segments, int n_segments, const float* x, Norm norm, bool accumulate);
// One token's experts on the same kernel: the stacked matrices' tiles, the slot's expert read from
// route on the device. swiglu: y[slot][n_rows] from x; down: expert_out[slot][n_rows] from
// x[slot][n_cols], to be added to the residual stream by moe_combine.
bool matvec_experts_mma_supported(const Mat& w, uint32_t n_rows, uint32_t n_used);
cudaError_t matvec_experts_swiglu_mma(cudaStream_t stream, const Mat& gate, const Mat& up, uint32_t n_rows, const float* x, const uint32_t* route,
                                      uint32_t n_used, float* y);
cudaError_t matvec_experts_down_mma(cudaStream_t stream, const Mat& down, uint32_t n_rows, const float* x, const uint32_t* route, uint32_t n_used,
                                    float* expert_out);
cudaError_t matvec_swiglu_mma(cudaStream_t stream, const Mat& gate, const Mat& up, const float* x, Norm norm, float* y);
cudaError_t matvec_conv_mma(cudaStream_t stream, const Mat& in_proj, const float* x, Norm norm, const float* taps, float* history,
                            float* out, uint32_t n_embd, uint32_t kernel);
cudaError_t matvec_mma_prepare(uint32_t widest_cols);
// Nonzero once a bounded wait inside a kernel gave up (1: a ring slot never freed, 2: a chunk never
// arrived). Reading clears it.
int matvec_error_flag();
// Raise the shared-memory limit of every matvec kernel for input vectors of up to `widest_cols`.
cudaError_t matvec_prepare(uint32_t widest_cols);
cudaError_t matvec(cudaStream_t stream, const MatvecSegment* segments, int n_segments, const float* x, Norm norm,
                   bool accumulate);
cudaError_t matvec_swiglu(cudaStream_t stream, const Mat& gate, const Mat& up, const float* x, Norm norm, float* y);
cudaError_t matvec_conv(cudaStream_t stream, const Mat& in_proj, const float* x, Norm norm, const float* taps,
                        float* history, float* out, uint32_t n_embd, uint32_t kernel);
// With `packed` (matmul_pack_bytes(n_tokens, n_embd) bytes; n_embd a multiple of 64) the results go
// out as the packed fp16 input of the product that consumes them, and `out` is not written.
cudaError_t short_conv(cudaStream_t stream, const float* bcx, const float* taps, float* history, float* out,
                       uint32_t n_embd, uint32_t kernel, uint32_t n_tokens, void* packed = nullptr);
cudaError_t expand(cudaStream_t stream, const Mat& w, void* out, bool out_half);
// A position that is either immediate or read from device memory at run time (`*ptr + value`), so
// one captured launch sequence can be replayed at every position of a decode.
struct Pos {
    const uint32_t* ptr = nullptr;
    uint32_t value = 0;
};
// `tokens + pos` names the first token id.
cudaError_t embed(cudaStream_t stream, const Mat& w, const uint32_t* tokens, Pos pos, float* out, uint32_t n_tokens);
// Decode-time fusion of the three per-token stores of an attention layer: per-head RMSNorm and
// rotation of q in place; the same for k, stored into the cache row of `pos`; v copied (or rounded
// to half) into its cache row. Caches point at the layer's first row.
struct RopeStore {
    float* q;
    const float* k;
    const float* v;
    void* k_cache;
    void* v_cache;
    const float* q_norm;
    const float* k_norm;
    uint32_t n_heads, n_kv_heads, head_dim, q_head_stride, n_rot;
    float theta, eps;
    bool kv_half;
    // Optional [position][n_rot / 2] table of (cos, sin) from rope_table, read by attention_step
    // in place of computing them.
    const float2* table = nullptr;
};
// (cos, sin) of every rotation pair at positions [0, n_positions), the values rope_store computes.
cudaError_t rope_table(cudaStream_t stream, float2* table, uint32_t n_positions, uint32_t n_rot, float theta);
cudaError_t rope_store(cudaStream_t stream, const RopeStore& p, Pos pos);
// One thread: *counter += 1.
cudaError_t advance(cudaStream_t stream, uint32_t* counter);
// argmax for a replayed decode: pos = *counter (after adding 1 to it when `advance`), then
// tokens[pos + offset] = argmax(x) and, when `ring` is non-null, ring[pos % ring_slots] too.
cudaError_t argmax_step(cudaStream_t stream, const float* x, uint32_t n, uint32_t* counter, bool advance, uint32_t* tokens,
                        uint32_t offset, uint32_t* ring, uint32_t ring_slots);
cudaError_t rms_norm(cudaStream_t stream, const float* x, const float* weight, float* out, uint32_t n_cols,
                     uint32_t n_rows, float eps);
cudaError_t norm_rope(cudaStream_t stream, const float* src, void* dst, bool dst_half, const float* weight,
                      uint32_t n_heads, uint32_t head_dim, uint32_t head_stride, uint32_t n_rot, uint32_t first_pos,
                      uint32_t n_tokens, uint32_t src_stride, uint32_t dst_stride, float theta, float eps);
cudaError_t convert_half(cudaStream_t stream, const float* src, __half* dst, uint64_t n);
cudaError_t copy_floats(cudaStream_t stream, const float* src, float* dst, uint64_t n);
cudaError_t silu_mul(cudaStream_t stream, float* x, const float* gate, uint64_t n);
// y[i] += x[i]
cudaError_t add_floats(cudaStream_t stream, float* y, const float* x, uint64_t n);

// Causal grouped-query attention of n_queries tokens at positions first_pos.. over the cache.
// q and out are [n_queries][n_heads * head_dim]; caches are [n_ctx][n_kv_heads * head_dim].
// q_stride is the element stride between tokens of q (Qwen interleaves q and gate per head, so
// q_head_stride is the element stride between heads).
struct AttentionShape {
    uint32_t n_heads, n_kv_heads, head_dim, first_pos, n_queries, n_ctx;
    uint32_t q_stride, q_head_stride;
    const uint32_t* pos_ptr = nullptr;  // when set, first_pos is *pos_ptr + first_pos and the grid covers n_ctx
};
uint64_t attention_scratch_floats(uint32_t n_heads, uint32_t head_dim, uint32_t n_ctx, uint32_t n_queries);
cudaError_t attention(cudaStream_t stream, const float* q, const void* k_cache, const void* v_cache, bool kv_half,
                      float* scratch, float* out, const AttentionShape& shape);
// Kernels `attention` launches for this shape.
int attention_launches(bool kv_half, const AttentionShape& shape);
// One decoded token of an attention layer in two launches: the chunk pass normalises and rotates
// the raw q itself, and the CTA whose chunk ends at the new position prepares that position's key
// and value rows, stores them in the caches and uses them; then the combine pass. Covers
// half-precision caches, heads of 64, 128 or 256 elements rotated whole, 16-byte aligned rows.
bool attention_step_supported(const RopeStore& r, const AttentionShape& shape);
cudaError_t attention_step(cudaStream_t stream, const RopeStore& r, float* scratch, float* out, const AttentionShape& shape);
// The tensor-core prefill kernel (kernels_attention_flash.cu): heads of 64 elements, f16 cache, at
// least 32 queries, positions known at launch. `attention` picks it when it applies.
bool attention_flash_supported(bool kv_half, const AttentionShape& shape);
cudaError_t attention_flash(cudaStream_t stream, const float* q, const void* k_cache, const void* v_cache, float* out,
                            const AttentionShape& shape);

// argmax over n floats, ties to the lowest index. `out` is a device word; `readback` (nullable) is
// a host-mapped word that receives the same value.
cudaError_t argmax(cudaStream_t stream, const float* x, uint32_t n, uint32_t* out, uint32_t* readback);

// ---- tensor-parallel decode (kernels_comm.cu): y += sum over ranks of `partial`, through buffers
// every rank has mapped from every other rank (plain peer stores over NVLink; see the kernel).
constexpr int kMaxPeers = 8;
constexpr uint32_t kPeerSlotFloats = 16384;
struct PeerBuffers {
    void* base[kMaxPeers];   // every rank's buffer as this GPU addresses it (base[rank] is its own)
    uint32_t world, rank;
    uint32_t slot_floats;    // floats per slot; slots are [parity 2][world] from the start of a buffer
    uint64_t flags_offset;   // byte offset of the flags, uint32 [parity 2][world]
    uint64_t epoch_offset;   // byte offset of the rank's epoch counter
};
inline uint64_t peer_buffer_bytes(uint32_t world) { return (uint64_t)2 * world * kPeerSlotFloats * 4 + 2 * world * 4 + 64; }
cudaError_t peer_all_reduce_add(cudaStream_t stream, const PeerBuffers& peers, const float* partial, float* y, uint32_t count);
// Nonzero once a rank's flag did not arrive within the wait's limit (1 + that rank). Reading clears it.
int peer_error_flag();

// ---- sampling (kernels_sample.cu): Sampler::sample of crates/bobcat-cli/src/sampler.rs:45-112.
struct Sampling {
    float temperature = 0.f;   // <= 0: the most likely token
    uint32_t top_k = 0;        // 0: no limit
    float top_p = 1.f, min_p = 0.f, repeat_penalty = 1.f;
};
// Picks a token from `logits` (n floats, changed in place by the repetition penalty over the last
// 64 of `recent`): penalty, top-k, top-p, min-p, temperature, then the draw `uniform` in [0, 1).
cudaError_t sample(cudaStream_t stream, float* logits, uint32_t n, const uint32_t* recent, uint32_t n_recent, const Sampling& settings,
                   float uniform, uint32_t* out, uint32_t* readback);

// ---- multi-sequence decode (kernels_batch.cu): one new token of each of n_seqs sequences per pass.
// What is per sequence is reached through device arrays indexed by the sequence's row.
struct SeqTable {
    const uint32_t* pos = nullptr;      // [n_seqs] position of each sequence's new token
    void* const* k_cache = nullptr;     // [n_seqs] each sequence's K cache (first layer's first row)
    void* const* v_cache = nullptr;     // [n_seqs] likewise for V
    float* const* conv_state = nullptr; // [n_seqs] each sequence's convolution history (first layer's)
    uint64_t layer_offset = 0;          // elements from a cache base to the layer's first row
    uint64_t conv_offset = 0;           // floats from a history base to the layer's history
};
// rope_store for row b of q / k / v at position pos[b] into sequence b's caches; q_stride is the
// element stride between rows of q.
cudaError_t rope_store_seqs(cudaStream_t stream, const RopeStore& p, const SeqTable& seqs, uint32_t q_stride, uint32_t n_seqs);
// Attention of row b of q over positions [0, pos[b]] of sequence b's caches; out is [n_seqs][n_heads * head_dim].
bool attention_seqs_supported(uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim);
cudaError_t attention_seqs(cudaStream_t stream, const float* q, float* out, const SeqTable& seqs, bool kv_half, uint32_t n_heads,
                           uint32_t n_kv_heads, uint32_t head_dim, uint32_t q_stride, uint32_t q_head_stride, uint32_t n_seqs);
// The LFM2 gated short convolution of one token per sequence, each with its own history.
cudaError_t short_conv_seqs(cudaStream_t stream, const float* bcx, const float* taps, const SeqTable& seqs, float* out, uint32_t n_embd,
                            uint32_t kernel, uint32_t n_seqs);
// picked[r] = argmax of row r of x (n floats each), ties to the lowest index; when `record` is
// non-null record[r * record_stride + record_at] takes it too.
cudaError_t argmax_rows(cudaStream_t stream, const float* x, uint32_t n, uint32_t n_rows, uint32_t* picked, uint32_t* record,
                        uint32_t record_stride, uint32_t record_at);
// pos[b] += 1 for every sequence.
cudaError_t advance_seqs(cudaStream_t stream, uint32_t* pos, uint32_t n_seqs);

// ---- Qwen3.5 (kernels_gdn.cu)
// DeltaNet causal convolution with SiLU over [n_tokens][conv_dim]; history [conv_dim][kernel - 1].
cudaError_t gdn_conv(cudaStream_t stream, const float* x, const float* taps, float* history, float* out, uint32_t conv_dim,
                     uint32_t kernel, uint32_t n_tokens);
int gdn_conv_launches(uint32_t n_tokens);
// In place: beta = sigmoid(beta); alpha = exp(a * softplus(alpha + dt_bias)).
cudaError_t gdn_gates(cudaStream_t stream, float* beta, float* alpha, const float* a, const float* dt_bias, uint32_t n_v_heads,
                      uint32_t n_tokens);
// The gated delta rule over n_tokens; state [n_v_heads][k_dim][v_dim]; `normalize` L2-normalises q and k.
cudaError_t gdn_recurrence(cudaStream_t stream, const float* qkv, const float* beta, const float* decay, float* state, float* out,
                           uint32_t n_k_heads, uint32_t n_v_heads, uint32_t k_dim, uint32_t v_dim, uint32_t n_tokens, bool normalize);
// The q and k heads of qkv ([n_tokens][2 * n_k_heads * k_dim + n_v_heads * v_dim]) L2-normalised in
// place, q also times 1 / sqrt(k_dim): what gdn_recurrence does per token with `normalize`, done
// for the whole batch at once, so the recurrence can run without it.
cudaError_t gdn_qk_norm(cudaStream_t stream, float* qkv, uint32_t n_k_heads, uint32_t n_v_heads, uint32_t k_dim, uint32_t v_dim, uint32_t n_tokens);
// One token through the whole mixer after its projections (conv with history shift, gates, L2
// norms, delta rule, gated norm) in one launch; gdn_step_supported says whether the shape fits.
bool gdn_step_supported(uint32_t n_k_heads, uint32_t n_v_heads, uint32_t k_dim, uint32_t v_dim, uint32_t kernel);
cudaError_t gdn_step(cudaStream_t stream, const float* qkv, const float* taps, float* history, const float* beta, const float* alpha,
                     const float* a, const float* dt_bias, float* state, const float* z, const float* norm_weight, float* out,
                     uint32_t n_k_heads, uint32_t n_v_heads, uint32_t k_dim, uint32_t v_dim, uint32_t kernel, float eps);
// x = RMSNorm(x) * weight * silu(z) per row of v_dim.
cudaError_t gdn_gated_norm(cudaStream_t stream, float* x, const float* z, const float* weight, uint32_t v_dim, uint32_t n_rows,
                           float eps);
// out *= sigmoid(gate), the gate read from the interleaved [q | gate] projection.
cudaError_t attention_gate(cudaStream_t stream, float* out, const float* q_gate, uint32_t n_heads, uint32_t head_dim, uint32_t n_tokens);

// ---- mixture of experts (kernels_moe.cu). A token's route is 2 * n_used words: expert ids, then
// weights as float bits.
// Router: optional RMSNorm (normalised tokens also go to `normed`), F32 router logits in f64,
// sigmoid, top n_used of score + bias with ties to the lower id, weights = score / (sum + 1e-6).
cudaError_t moe_route(cudaStream_t stream, const float* x, Norm norm, float* normed, const float* router, const float* bias,
                      uint32_t* route, uint32_t n_cols, uint32_t n_experts, uint32_t n_used, uint32_t n_tokens);
// Counting sort of the (token, slot) entries by expert: offsets[n_experts + 1], entries[n_tokens * n_used].
// With first_expert > 0 (or fewer experts than the router has) only the entries of experts
// [first_expert, first_expert + n_experts) are kept, numbered from zero: offsets[n_experts] is then
// the number of kept entries, which the grouped products read from the device.
cudaError_t moe_group(cudaStream_t stream, const uint32_t* route, uint32_t* offsets, uint32_t* entries, uint32_t n_experts,
                      uint32_t n_used, uint32_t n_tokens, uint32_t first_expert = 0);
// Decode: y[token][slot][row] = silu(gate_e x) * (up_e x) for the slot's expert e; n_rows per expert.
cudaError_t matvec_experts_swiglu(cudaStream_t stream, const Mat& gate, const Mat& up, uint32_t n_rows, const float* x,
                                  const uint32_t* route, uint32_t n_used, float* y, uint32_t n_tokens);
// Decode: y[token][row] += sum over slots of weight * (down_e row . x[token][slot]).
// With `expert_out` ([n_used][n_rows] floats of scratch) a single token may run on the tile kernel,
// its slots' outputs added to y by moe_combine: two launches, see matvec_experts_down_launches.
cudaError_t matvec_experts_down(cudaStream_t stream, const Mat& down, uint32_t n_rows, const float* x, const uint32_t* route,
                                uint32_t n_used, float* y, uint32_t n_tokens, float* expert_out = nullptr);
int matvec_experts_down_launches(const Mat& down, uint32_t n_rows, uint32_t n_used, uint32_t n_tokens, bool has_scratch);
// Prefill: for each expert, its entries times its rows; with `up` the store is silu(gate) * up.
// Input rows are the tokens' (gather) or the entries' own; output rows are the entries'.
// With `scratch` (matmul_experts_scratch_bytes) and Q4_0 experts the tcgen05 kernel runs in its
// grouped mode (two launches: gather-pack, then the product); otherwise the SIMT tile kernel.
cudaError_t matmul_experts(cudaStream_t stream, const Mat& w, const Mat* up, uint32_t n_rows, uint32_t n_experts, const float* x,
                           bool gather, const uint32_t* offsets, const uint32_t* entries, uint32_t n_used, float* y, uint32_t n_tokens,
                           void* scratch);
bool matmul_experts_umma_supported(const Mat& w, const Mat* up, uint32_t n_tokens);
uint64_t matmul_experts_scratch_bytes(uint32_t n_experts, uint32_t n_tokens, uint32_t n_cols);
cudaError_t matmul_experts_umma(cudaStream_t stream, const Mat& w, const Mat* up, uint32_t n_rows, uint32_t n_experts, const float* x, bool gather,
                                const uint32_t* offsets, const uint32_t* entries, uint32_t n_used, float* y, uint32_t n_tokens, void* scratch);
cudaError_t moe_combine(cudaStream_t stream, const float* expert_out, const uint32_t* route, float* y, uint32_t n_embd,
                        uint32_t n_used, uint32_t n_tokens);

// Y[t][r] (store) sum_c W[r][c] X[t][c]. X is [n_tokens][n_cols] f32, Y is [n_tokens][y_stride].
// With `pack` (matmul_scratch_bytes(w, n_tokens) bytes of scratch) and a matrix the tensor-core
// kernel supports, the inputs are packed to fp16 there and the tcgen05 kernel runs
// (matmul_umma_launches launches); otherwise the f32 SIMT tile kernel runs. y_stride must be
// w.n_rows on the tensor-core path's split-K shapes, which is what every caller passes.
cudaError_t matmul(cudaStream_t stream, const Mat& w, const float* x, float* y, uint32_t n_tokens, uint32_t y_stride,
                   int32_t store, void* pack);
// The tensor-core prefill kernel (kernels_matmul_umma.cu) and its input packing.
// Batches below `min_tokens` rows are left to the f32 tile kernel unless the caller lowers the bound
// (rows are padded to 16 either way).
bool matmul_umma_supported(const Mat& w, uint32_t n_tokens, uint32_t min_tokens = 16);
uint64_t matmul_pack_bytes(uint32_t n_tokens, uint32_t n_cols);
// Packed inputs plus, for shapes that split K, the partial products.
uint64_t matmul_scratch_bytes(const Mat& w, uint32_t n_tokens);
int matmul_umma_launches(const Mat& w, uint32_t n_tokens);
cudaError_t matmul_pack(cudaStream_t stream, const float* x, uint32_t n_tokens, uint32_t n_cols, void* packed);
// RMSNorm fused into the packing: packed = fp16(weight * (x * scale)), so a normalised batch that only feeds
// tensor-core products never exists in f32.
// The partial products of a split-K launch whose sum into y has not been taken yet: `split`
// arrays of [n_tokens][n_rows] floats, to be added to y in index order.
struct Deferred {
    const float* partial = nullptr;
    uint32_t split = 0, n_tokens = 0, n_rows = 0;
};
// Bytes of partial products matmul_umma writes for this shape (zero when it does not split K).
uint64_t matmul_partial_bytes(const Mat& w, uint32_t n_tokens);
// With `add` (for this x: n_tokens rows of n_cols), x += the deferred partial products first, so
// the sum a split-K product into the residual stream left open costs no launch of its own.
cudaError_t matmul_pack_norm(cudaStream_t stream, float* x, Norm norm, uint32_t n_tokens, uint32_t n_cols, void* packed,
                             const Deferred* add = nullptr);
// `partial`: where a split-K launch puts its partial products (matmul_partial_bytes; by default
// behind the packed inputs, as matmul_scratch_bytes sizes the scratch). With `defer`, an
// accumulating split-K product into rows of n_rows floats leaves the sum of the partial products
// open and describes it there (defer->partial stays null when the launch did not split).
cudaError_t matmul_umma(cudaStream_t stream, const Mat& w, const void* packed, float* y, uint32_t n_tokens, uint32_t y_stride,
                        int32_t store, float* partial = nullptr, Deferred* defer = nullptr);
// Up to four products that read the same packed inputs, in one launch (q, k and v of an attention
// layer; the projections of a DeltaNet layer): ys[i] = ws[i] x for every token, rows of ws[i]->n_rows floats, overwritten.
cudaError_t matmul_umma_several(cudaStream_t stream, const Mat* const* ws, float* const* ys, int n, const void* packed, uint32_t n_tokens);
// y += the deferred partial products, in index order.
cudaError_t matmul_reduce(cudaStream_t stream, const Deferred& d, float* y);
// Gate and up of a SwiGLU in one launch: both weight tiles meet the same token tile, two
// accumulators in tensor memory, y = silu(gate x) * (up x).
bool matmul_umma_swiglu_supported(const Mat& gate, const Mat& up, uint32_t n_tokens, uint32_t min_tokens = 16);
// With `packed_out` the result is written as the packed fp16 input of the product that consumes it
// (what matmul_pack would make of it, for gate.n_rows columns; gate.n_rows a multiple of 64) and y
// is not touched.
cudaError_t matmul_umma_swiglu(cudaStream_t stream, const Mat& gate, const Mat& up, const void* packed, float* y, uint32_t n_tokens,
                               uint32_t y_stride, void* packed_out = nullptr);
// The same products for at most 32 tokens (kernels_matmul_few.cu): the matrices' decode tiles against
// the packed inputs on warp-level MMAs, one launch, no split of K left open. matmul_umma,
// matmul_umma_several, matmul_umma_swiglu and matmul_experts_umma hand over to these whenever the
// shape allows (BOBCAT_NO_FEW_MATMUL=1 keeps them on the tcgen05 kernel).
bool matmul_few_supported(const Mat& w, uint32_t n_tokens);
// Nonzero once a warp of that kernel gave up waiting for its weights.
int matmul_few_error_flag();
cudaError_t matmul_few(cudaStream_t stream, const Mat* const* ws, float* const* ys, const uint32_t* strides, int n, const void* packed,
                       uint32_t n_tokens, int32_t store);
cudaError_t matmul_few_swiglu(cudaStream_t stream, const Mat& gate, const Mat& up, const void* packed, float* y, uint32_t n_tokens, uint32_t y_stride,
                              void* packed_out);
// A matrix too wide for matmul_few (more packed tokens than a CTA keeps): the number of slices of
// K it is cut into (0: not this kernel's), and the product as that many arrays of
// [n_tokens][w.n_rows] partial sums, to be added in index order.
uint32_t matmul_few_slices(const Mat& w, uint32_t n_tokens);
cudaError_t matmul_few_sliced(cudaStream_t stream, const Mat& w, const void* packed, float* partial, uint32_t n_tokens);
bool matmul_few_experts_supported(const Mat& w, const Mat* up, uint32_t n_rows, uint32_t n_experts, uint32_t n_tokens);
cudaError_t matmul_few_experts(cudaStream_t stream, const Mat& w, const Mat* up, uint32_t n_rows, uint32_t n_experts, const void* packed,
                               const uint32_t* offsets, const uint32_t* entries, float* y, uint32_t n_tokens, uint32_t n_entries);
// Nonzero once a bounded wait inside the tensor-core prefill kernel gave up (1: producers on a free
// stage, 2: epilogue on the accumulator, 3: token copy on a free stage, 4: MMA thread on a full stage).
int matmul_error_flag();

}  // namespace k
}  // namespace bc
