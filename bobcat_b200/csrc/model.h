// The host-side model (parsed GGUF + hyperparameters + tensor table, restating the loader checks
// of crates/bobcat/src/lfm2.rs:737-1004 and crates/bobcat/src/qwen35.rs:629-752) and its weights
// on one device.
#pragma once

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "backend.h"

namespace bc {

struct HostMatrix {
    const GgufTensor* t = nullptr;
    uint32_t n_rows = 0, n_cols = 0;
};

struct HostVector {
    const GgufTensor* t = nullptr;
    size_t n = 0;
};

enum class Mixer { Conv, Attention, Delta };

struct LayerSpec {
    Mixer mixer = Mixer::Conv;
    uint32_t cache_index = 0;
    HostVector attn_norm, ffn_norm;
    // attention (LFM2 and Qwen3.5; Qwen's q holds [q | gate] per head)
    HostMatrix q, k, v, output;
    HostVector q_norm, k_norm;
    // LFM2 gated short convolution
    HostVector taps;
    HostMatrix in_proj, out_proj;
    // Qwen3.5 gated delta net
    HostMatrix qkv, z, beta, alpha, ssm_out;
    HostVector conv1d, dt_bias, a, ssm_norm;
    // feed-forward
    bool moe = false;
    HostMatrix gate, up, down, router;
    HostVector expert_bias;
};

// Device copies of one layer's tensors.
struct DeviceLayer {
    k::Mat q, k, v, output, in_proj, out_proj, qkv, z, beta, alpha, ssm_out, gate, up, down, router;
    const float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr, *taps = nullptr;
    const float *conv1d = nullptr, *dt_bias = nullptr, *a = nullptr, *ssm_norm = nullptr, *expert_bias = nullptr;
};

struct DeviceModel {
    int device = 0;
    void* arena = nullptr;
    size_t arena_bytes = 0;
    std::vector<DeviceLayer> layers;
    k::Mat token_embd, output;
    const float* output_norm = nullptr;
    // Tensor-parallel shards are allocated one by one (freed with the model).
    std::vector<void*> extra;
    // Tensor parallelism: the rows of the output matrix this rank multiplies (all of them otherwise).
    uint32_t first_vocab_row = 0, n_vocab_rows = 0;
    ~DeviceModel();
};

// The head and row counts a tensor-parallel rank works with: the model's hyperparameters with the
// per-rank share of attention heads, DeltaNet heads and feed-forward rows.
bc_hparams tensor_parallel_hparams(const bc_hparams& hp, int rank, int world);

}  // namespace bc

struct bc_model {
    bc::Gguf gguf;
    bc_hparams hp{};
    std::vector<bc::LayerSpec> layers;
    bc::HostMatrix token_embd, output;
    bc::HostVector output_norm;
    bool tied_output = true;
    std::mutex mutex;
    std::map<int, std::shared_ptr<bc::DeviceModel>> on_device;  // by CUDA device

    std::map<std::pair<int, std::pair<int, int>>, std::shared_ptr<bc::DeviceModel>> on_device_tp;  // by (device, (rank, world))

    // Upload the weights to the backend's device on first use; later sequences share them.
    bc_status device_model(bc_backend* backend, std::shared_ptr<bc::DeviceModel>* out);
    // The shard of rank `rank` of `world` tensor-parallel ranks (Qwen3.5 models).
    bc_status device_model_tp(bc_backend* backend, int rank, int world, std::shared_ptr<bc::DeviceModel>* out);
};
