// The device state of one decode and the recording of its forward passes. Stands in for
// `Lfm2Metal` (crates/bobcat/src/lfm2_metal.rs) and `Qwen35Metal` (crates/bobcat/src/qwen35_metal.rs).
#pragma once

#include <chrono>
#include <memory>
#include <string>
#include <vector>

#include "kv_pages.h"
#include "model.h"

// Generation keeps up to this many steps submitted ahead of the device
// (GENERATE_IN_FLIGHT, crates/bobcat/src/lfm2_metal.rs:29-31).
constexpr int kGenerateInFlight = 3;
// Prefill runs the prompt this many tokens at a time (PREFILL_BATCH, lfm2_metal.rs:33-34).
constexpr uint32_t kPrefillBatch = 512;

// A cached prefix: everything a sequence needs to continue from position n_past - the recurrent
// state, the logits, and the KV rows [0, n_past) of every attention layer. Of a paged sequence the
// full pages are held by reference (shared with every sequence that loads the prefix) and only the
// rows of the last, partial page are copied; of a contiguous sequence all rows are copied.
struct bc_prefix {
    const bc_model* model = nullptr;
    int device = 0;
    bool kv_half = false;
    bc_hparams hp{};
    uint32_t n_past = 0;
    size_t conv_floats = 0, delta_floats = 0;
    float* state = nullptr;  // device: conv history, DeltaNet state, logits
    bool paged = false;
    bc::PageGeometry geometry;
    uint32_t full_pages = 0;  // per layer
    std::vector<std::shared_ptr<bc::PhysicalPage>> k_pages, v_pages;  // [layer][full page]
    void* tail = nullptr;     // device: [K, V][layer][tail_rows][kv_dim] rows from position full_pages * page_positions on
    uint32_t tail_rows = 0;
    ~bc_prefix();
};

struct bc_checkpoint {
    const bc_seq* owner = nullptr;
    uint64_t resets = 0;
    uint32_t n_past = 0;
    std::vector<float> conv_state;   // LFM2 conv history, or Qwen conv history of every DeltaNet layer
    std::vector<float> delta_state;  // Qwen DeltaNet state matrices
    std::vector<float> logits;
};

struct bc_comm;

struct bc_seq {
    bc_model* model = nullptr;
    bc_backend* backend = nullptr;
    // The shapes this sequence's kernels run with: the model's hyperparameters, or, on a
    // tensor-parallel rank, those with the rank's share of heads and feed-forward rows.
    bc_hparams hp{};
    // Tensor parallelism: the communicator whose ranks share this sequence (null otherwise), and
    // rows of n_embd floats for an output projection's partial result before the sum over ranks.
    bc_comm* tp = nullptr;
    float* partial = nullptr;
    std::shared_ptr<bc::DeviceModel> weights;
    uint32_t n_ctx = 0, n_past = 0, batch = 0;
    uint64_t resets = 0;
    bool kv_half = false;
    double last_encode_seconds = 0, last_gpu_seconds = 0;
    uint64_t launches = 0;

    // One device allocation carved into the buffers below.
    void* arena = nullptr;
    size_t arena_bytes = 0;
    void *k_cache = nullptr, *v_cache = nullptr;
    // Positions between two layers of a cache: n_ctx, or n_ctx rounded up to whole pages when the
    // caches are paged (then k_cache / v_cache are the bases of the paged ranges below).
    uint32_t kv_stride = 0;
    std::unique_ptr<bc::PagedCache> k_pages, v_pages;
    uint32_t shared_positions = 0;  // positions [0, shared_positions) lie in pages shared with a prefix
    float *k = nullptr, *v = nullptr, *conv_state = nullptr, *hidden = nullptr, *normed = nullptr, *bcx = nullptr;
    float *conv_out = nullptr, *q = nullptr, *attn = nullptr, *scores = nullptr, *ffn = nullptr, *logits = nullptr;
    float *trace_embedding = nullptr, *trace_layers = nullptr, *trace_final = nullptr;
    uint32_t* trace_routes = nullptr;  // [layer][trace_rows][2 * n_used]: routes of the last traced pass
    uint32_t* tokens = nullptr;        // n_ctx + 1 ids; the extra slot takes the pick at the last position
    uint32_t* greedy_token = nullptr;
    // Mixture of experts: each token's route, the routes grouped by expert, and one row of n_embd
    // floats per routed expert of each token (lfm2_metal.rs:59-65).
    uint32_t *route = nullptr, *expert_offsets = nullptr, *expert_entries = nullptr;
    float* expert_out = nullptr;
    // Qwen3.5 (qwen35_metal.rs:161-196): the DeltaNet state matrices [delta layer][value head][k_dim]
    // [v_dim] (the conv history lives in conv_state as [delta layer][channel][K - 1]), the scratch
    // rows of a DeltaNet layer, and the rotated queries of a batch.
    float *delta_state = nullptr, *gdn_qkv = nullptr, *gdn_conv_out = nullptr, *gdn_z = nullptr, *gdn_beta = nullptr;
    float *gdn_alpha = nullptr, *gdn_out = nullptr, *q_rot = nullptr;
    size_t delta_floats = 0;
    size_t conv_floats = 0;
    uint32_t trace_rows = 0;
    // Host-mapped words the device writes picked tokens into, one per step in flight.
    uint32_t* readback = nullptr;
    cudaEvent_t slot_done[kGenerateInFlight] = {};
    cudaEvent_t timing_start = nullptr, timing_end = nullptr;

    // Replayed decode: the launches of one generated step are captured once into a CUDA graph whose
    // kernels read the position from `step_pos` on the device, then replayed once per token
    // (the reference's plan for stable commands, docs/design.md:94-98).
    float2* rope_table = nullptr;             // (cos, sin) per position and rotation pair, for the decode attention step
    uint32_t* step_pos = nullptr;             // device word: position of the step being run
    cudaGraphExec_t generate_graph = nullptr; // argmax -> tokens[pos], forward pass at pos
    cudaGraphExec_t stream_graph = nullptr;   // forward pass at pos, argmax -> tokens[pos + 1] and the readback ring
    uint64_t generate_graph_kernels = 0, stream_graph_kernels = 0;  // kernels per replay, for the launch count
    uint32_t host_pos = 0;                    // staging for the seed of step_pos
    // Timing diagnostics (bc_seq_set_skip): launches of this name (and shape, when nonzero) are left out.
    std::string skip_name;
    uint32_t skip_rows = 0, skip_cols = 0;
    // Batched products with f32 operands on the f32 tile kernels instead of half-precision operands
    // on the tensor cores (the multi-sequence decode's precise mode).
    bool exact_products = false;
    bool use_graphs = true;                   // BOBCAT_NO_GRAPH=1 turns replay off (launch every kernel eagerly)

    void release();
    ~bc_seq();
};
