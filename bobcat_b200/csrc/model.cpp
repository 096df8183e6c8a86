#include "model.h"

#include <cstring>

using namespace bc;

namespace {

// ---- loader helpers: lfm2.rs:724-914

struct Loader {
    const Gguf& g;
    explicit Loader(const Gguf& gguf) : g(gguf) {}

    bc_status u32(const std::string& key, uint32_t* out) const {
        if (!g.u32(key, out)) return fail(BC_ERR_METADATA, "missing or invalid metadata %s", key.c_str());
        return BC_OK;
    }
    bc_status f32(const std::string& key, float* out) const {
        if (!g.f32(key, out)) return fail(BC_ERR_METADATA, "missing or invalid metadata %s", key.c_str());
        return BC_OK;
    }
    bc_status tensor(const std::string& name, const std::vector<uint64_t>& want, const GgufTensor** out) const {
        const GgufTensor* t = g.tensor(name);
        if (!t) return fail(BC_ERR_MISSING_TENSOR, "missing tensor %s", name.c_str());
        if (t->shape != want) {
            std::string got, need;
            for (uint64_t d : t->shape) got += std::to_string(d) + " ";
            for (uint64_t d : want) need += std::to_string(d) + " ";
            return fail(BC_ERR_TENSOR_SHAPE, "tensor %s has shape [%s], want [%s]", name.c_str(), got.c_str(), need.c_str());
        }
        *out = t;
        return BC_OK;
    }
    bc_status matrix(const std::string& name, uint64_t n_cols, uint64_t n_rows, HostMatrix* out) const {
        const GgufTensor* t;
        BC_TRY(tensor(name, {n_cols, n_rows}, &t));
        if (n_rows > UINT32_MAX || n_cols > UINT32_MAX) return fail(BC_ERR_HYPERPARAMETERS, "invalid hyperparameters");
        *out = HostMatrix{t, (uint32_t)n_rows, (uint32_t)n_cols};
        return BC_OK;
    }
    bc_status experts(const std::string& name, uint64_t n_cols, uint64_t n_rows, uint64_t n_experts, HostMatrix* out) const {
        const GgufTensor* t;
        BC_TRY(tensor(name, {n_cols, n_rows, n_experts}, &t));
        if (n_rows * n_experts > UINT32_MAX || n_cols > UINT32_MAX) return fail(BC_ERR_HYPERPARAMETERS, "invalid hyperparameters");
        *out = HostMatrix{t, (uint32_t)(n_rows * n_experts), (uint32_t)n_cols};
        return BC_OK;
    }
    bc_status vector(const std::string& name, const std::vector<uint64_t>& want, HostVector* out) const {
        const GgufTensor* t;
        BC_TRY(tensor(name, want, &t));
        if (t->type != T_F32) return fail(BC_ERR_TENSOR_TYPE, "tensor %s has type %u, want F32", name.c_str(), t->type);
        size_t n = 1;
        for (uint64_t d : want) n *= (size_t)d;
        *out = HostVector{t, n};
        return BC_OK;
    }
};

// lfm2.rs:737-808, :186-233, :919-1004
bc_status load_lfm2(bc_model& m, bool moe) {
    Loader L(m.gguf);
    bc_hparams& hp = m.hp;
    hp.architecture = moe ? BC_ARCH_LFM2MOE : BC_ARCH_LFM2;
    const std::string p = moe ? "lfm2moe." : "lfm2.";
    BC_TRY(L.u32(p + "block_count", &hp.n_layers));
    BC_TRY(L.u32(p + "embedding_length", &hp.n_embd));
    BC_TRY(L.u32(p + "feed_forward_length", &hp.n_ff));
    BC_TRY(L.u32(p + "attention.head_count", &hp.n_heads));
    BC_TRY(L.u32(p + "shortconv.l_cache", &hp.conv_kernel));
    BC_TRY(L.f32(p + "rope.freq_base", &hp.rope_theta));
    BC_TRY(L.f32(p + "attention.layer_norm_rms_epsilon", &hp.norm_eps));
    uint32_t n_dense = hp.n_layers;
    if (moe) {
        uint32_t gating = 0;
        BC_TRY(L.u32(p + "expert_gating_func", &gating));
        if (gating != 2) return fail(BC_ERR_METADATA, "missing or invalid metadata %sexpert_gating_func", p.c_str());
        BC_TRY(L.u32(p + "expert_count", &hp.n_experts));
        BC_TRY(L.u32(p + "expert_used_count", &hp.n_experts_used));
        BC_TRY(L.u32(p + "expert_feed_forward_length", &hp.n_ff_expert));
        n_dense = 0;
        m.gguf.u32(p + "leading_dense_block_count", &n_dense);
    }
    if (hp.n_layers == 0 || hp.n_embd == 0 || hp.n_ff == 0 || hp.n_heads == 0 || hp.n_embd % hp.n_heads != 0 || hp.conv_kernel < 2 ||
        (moe && (hp.n_experts_used == 0 || hp.n_experts_used > hp.n_experts || hp.n_ff_expert == 0)))
        return fail(BC_ERR_HYPERPARAMETERS, "invalid hyperparameters");
    hp.head_dim = hp.n_embd / hp.n_heads;
    hp.n_rot = hp.head_dim;
    if (hp.head_dim % 2 != 0) return fail(BC_ERR_ODD_HEAD_DIM, "head_dim %u is odd", hp.head_dim);

    const uint64_t n_embd = hp.n_embd;
    const std::string kv_key = p + "attention.head_count_kv";
    m.layers.resize(hp.n_layers);
    for (uint32_t il = 0; il < hp.n_layers; ++il) {
        LayerSpec& S = m.layers[il];
        auto name = [&](const char* suffix) { return "blk." + std::to_string(il) + "." + suffix + ".weight"; };
        uint32_t n_kv = 0;
        uint64_t len = 0;
        if (!(m.gguf.array_len(kv_key, &len) && len == hp.n_layers && m.gguf.array_u32(kv_key, il, &n_kv))) BC_TRY(L.u32(kv_key, &n_kv));

        BC_TRY(L.vector(name("attn_norm"), {n_embd}, &S.attn_norm));
        BC_TRY(L.vector(name("ffn_norm"), {n_embd}, &S.ffn_norm));
        if (il < n_dense) {
            BC_TRY(L.matrix(name("ffn_gate"), n_embd, hp.n_ff, &S.gate));
            BC_TRY(L.matrix(name("ffn_up"), n_embd, hp.n_ff, &S.up));
            BC_TRY(L.matrix(name("ffn_down"), hp.n_ff, n_embd, &S.down));
        } else {
            S.moe = true;
            BC_TRY(L.matrix(name("ffn_gate_inp"), n_embd, hp.n_experts, &S.router));
            BC_TRY(L.vector("blk." + std::to_string(il) + ".exp_probs_b.bias", {hp.n_experts}, &S.expert_bias));
            BC_TRY(L.experts(name("ffn_gate_exps"), n_embd, hp.n_ff_expert, hp.n_experts, &S.gate));
            BC_TRY(L.experts(name("ffn_up_exps"), n_embd, hp.n_ff_expert, hp.n_experts, &S.up));
            BC_TRY(L.experts(name("ffn_down_exps"), hp.n_ff_expert, n_embd, hp.n_experts, &S.down));
        }
        if (n_kv == 0) {
            S.mixer = Mixer::Conv;
            BC_TRY(L.vector(name("shortconv.conv"), {hp.conv_kernel, n_embd}, &S.taps));
            BC_TRY(L.matrix(name("shortconv.in_proj"), n_embd, 3 * n_embd, &S.in_proj));
            BC_TRY(L.matrix(name("shortconv.out_proj"), n_embd, n_embd, &S.out_proj));
            S.cache_index = hp.n_conv_layers++;
        } else {
            if (hp.n_kv_heads == 0) hp.n_kv_heads = n_kv;
            if (n_kv != hp.n_kv_heads || hp.n_heads % n_kv != 0) return fail(BC_ERR_KV_HEADS, "layer %u has %u KV heads", il, n_kv);
            uint64_t hd = hp.head_dim, q_dim = (uint64_t)hp.n_heads * hd, kv_dim = (uint64_t)n_kv * hd;
            S.mixer = Mixer::Attention;
            BC_TRY(L.matrix(name("attn_q"), n_embd, q_dim, &S.q));
            BC_TRY(L.matrix(name("attn_k"), n_embd, kv_dim, &S.k));
            BC_TRY(L.matrix(name("attn_v"), n_embd, kv_dim, &S.v));
            BC_TRY(L.matrix(name("attn_output"), q_dim, n_embd, &S.output));
            BC_TRY(L.vector(name("attn_q_norm"), {hd}, &S.q_norm));
            BC_TRY(L.vector(name("attn_k_norm"), {hd}, &S.k_norm));
            S.cache_index = hp.n_attention_layers++;
        }
    }
    const GgufTensor* embd = m.gguf.tensor("token_embd.weight");
    if (!embd || embd->shape.size() != 2) return fail(BC_ERR_MISSING_TENSOR, "missing tensor token_embd.weight");
    if (embd->shape[1] > UINT32_MAX) return fail(BC_ERR_HYPERPARAMETERS, "invalid hyperparameters");
    hp.n_vocab = (uint32_t)embd->shape[1];
    BC_TRY(L.matrix("token_embd.weight", n_embd, hp.n_vocab, &m.token_embd));
    BC_TRY(L.vector("token_embd_norm.weight", {n_embd}, &m.output_norm));
    if (m.gguf.tensor("output.weight")) {
        BC_TRY(L.matrix("output.weight", n_embd, hp.n_vocab, &m.output));
        m.tied_output = false;
    } else {
        m.output = m.token_embd;
        m.tied_output = true;
    }
    return BC_OK;
}

// qwen35.rs:629-752, :193-229
bc_status load_qwen35(bc_model& m) {
    Loader L(m.gguf);
    bc_hparams& hp = m.hp;
    hp.architecture = BC_ARCH_QWEN35;
    const std::string p = "qwen35.";
    uint32_t block_count = 0, n_nextn = 0, inner = 0, value_length = 0;
    BC_TRY(L.u32(p + "block_count", &block_count));
    m.gguf.u32(p + "nextn_predict_layers", &n_nextn);
    if (n_nextn > block_count) return fail(BC_ERR_HYPERPARAMETERS, "invalid hyperparameters");
    hp.n_layers = block_count - n_nextn;
    BC_TRY(L.u32(p + "attention.key_length", &hp.head_dim));
    BC_TRY(L.u32(p + "ssm.time_step_rank", &hp.n_v_heads));
    BC_TRY(L.u32(p + "ssm.inner_size", &inner));
    BC_TRY(L.u32(p + "embedding_length", &hp.n_embd));
    BC_TRY(L.u32(p + "feed_forward_length", &hp.n_ff));
    BC_TRY(L.u32(p + "attention.head_count", &hp.n_heads));
    BC_TRY(L.u32(p + "attention.head_count_kv", &hp.n_kv_heads));
    BC_TRY(L.u32(p + "rope.dimension_count", &hp.n_rot));
    BC_TRY(L.f32(p + "rope.freq_base", &hp.rope_theta));
    BC_TRY(L.f32(p + "attention.layer_norm_rms_epsilon", &hp.norm_eps));
    BC_TRY(L.u32(p + "ssm.conv_kernel", &hp.conv_kernel));
    BC_TRY(L.u32(p + "ssm.group_count", &hp.n_k_heads));
    BC_TRY(L.u32(p + "ssm.state_size", &hp.k_head_dim));
    hp.v_head_dim = hp.n_v_heads ? inner / hp.n_v_heads : 0;
    BC_TRY(L.u32(p + "attention.value_length", &value_length));
    if (hp.n_layers == 0 || hp.n_embd == 0 || hp.n_heads == 0 || hp.n_kv_heads == 0 || hp.n_heads % hp.n_kv_heads != 0 || hp.head_dim == 0 ||
        value_length != hp.head_dim || hp.n_rot == 0 || hp.n_rot % 2 != 0 || hp.n_rot > hp.head_dim || hp.conv_kernel < 2 ||
        hp.n_k_heads == 0 || hp.n_v_heads == 0 || hp.n_v_heads % hp.n_k_heads != 0 || hp.k_head_dim == 0 || hp.v_head_dim == 0 ||
        (uint64_t)hp.n_v_heads * hp.v_head_dim != inner)
        return fail(BC_ERR_HYPERPARAMETERS, "invalid hyperparameters");
    uint64_t key_dim = (uint64_t)hp.n_k_heads * hp.k_head_dim;
    uint64_t conv_dim = 2 * key_dim + inner;
    if (key_dim > UINT32_MAX || conv_dim > UINT32_MAX || (uint64_t)hp.k_head_dim * hp.v_head_dim > UINT32_MAX)
        return fail(BC_ERR_HYPERPARAMETERS, "invalid hyperparameters");

    const GgufTensor* embd = m.gguf.tensor("token_embd.weight");
    if (!embd || embd->shape.size() != 2) return fail(BC_ERR_MISSING_TENSOR, "missing tensor token_embd.weight");
    if (embd->shape[1] > UINT32_MAX) return fail(BC_ERR_HYPERPARAMETERS, "invalid hyperparameters");
    hp.n_vocab = (uint32_t)embd->shape[1];
    const uint64_t n_embd = hp.n_embd, n_ff = hp.n_ff;
    m.layers.resize(hp.n_layers);
    for (uint32_t il = 0; il < hp.n_layers; ++il) {
        LayerSpec& S = m.layers[il];
        auto name = [&](const char* suffix) { return "blk." + std::to_string(il) + "." + suffix; };
        if (m.gguf.tensor(name("ssm_a"))) {
            uint64_t value_dim = inner, n_v = hp.n_v_heads;
            S.mixer = Mixer::Delta;
            BC_TRY(L.matrix(name("attn_qkv.weight"), n_embd, conv_dim, &S.qkv));
            BC_TRY(L.matrix(name("attn_gate.weight"), n_embd, value_dim, &S.z));
            BC_TRY(L.matrix(name("ssm_beta.weight"), n_embd, n_v, &S.beta));
            BC_TRY(L.matrix(name("ssm_alpha.weight"), n_embd, n_v, &S.alpha));
            BC_TRY(L.vector(name("ssm_conv1d.weight"), {hp.conv_kernel, conv_dim}, &S.conv1d));
            BC_TRY(L.vector(name("ssm_dt.bias"), {n_v}, &S.dt_bias));
            BC_TRY(L.vector(name("ssm_a"), {n_v}, &S.a));
            BC_TRY(L.vector(name("ssm_norm.weight"), {hp.v_head_dim}, &S.ssm_norm));
            BC_TRY(L.matrix(name("ssm_out.weight"), value_dim, n_embd, &S.ssm_out));
            S.cache_index = hp.n_delta_layers++;
        } else {
            uint64_t hd = hp.head_dim, q_dim = (uint64_t)hp.n_heads * hd, kv_dim = (uint64_t)hp.n_kv_heads * hd;
            S.mixer = Mixer::Attention;
            BC_TRY(L.matrix(name("attn_q.weight"), n_embd, 2 * q_dim, &S.q));
            BC_TRY(L.matrix(name("attn_k.weight"), n_embd, kv_dim, &S.k));
            BC_TRY(L.matrix(name("attn_v.weight"), n_embd, kv_dim, &S.v));
            BC_TRY(L.matrix(name("attn_output.weight"), q_dim, n_embd, &S.output));
            BC_TRY(L.vector(name("attn_q_norm.weight"), {hd}, &S.q_norm));
            BC_TRY(L.vector(name("attn_k_norm.weight"), {hd}, &S.k_norm));
            S.cache_index = hp.n_attention_layers++;
        }
        BC_TRY(L.vector(name("attn_norm.weight"), {n_embd}, &S.attn_norm));
        BC_TRY(L.vector(name("post_attention_norm.weight"), {n_embd}, &S.ffn_norm));
        BC_TRY(L.matrix(name("ffn_gate.weight"), n_embd, n_ff, &S.gate));
        BC_TRY(L.matrix(name("ffn_up.weight"), n_embd, n_ff, &S.up));
        BC_TRY(L.matrix(name("ffn_down.weight"), n_ff, n_embd, &S.down));
    }
    BC_TRY(L.matrix("token_embd.weight", n_embd, hp.n_vocab, &m.token_embd));
    BC_TRY(L.vector("output_norm.weight", {n_embd}, &m.output_norm));
    if (m.gguf.tensor("output.weight")) {
        BC_TRY(L.matrix("output.weight", n_embd, hp.n_vocab, &m.output));
        m.tied_output = false;
    } else {
        m.output = m.token_embd;
        m.tied_output = true;
    }
    return BC_OK;
}

bool kernel_format(uint32_t type) { return type == T_F32 || type == T_F16 || type == T_Q4_0 || type == T_Q8_0 || type == T_Q6K; }

// What the kernels can run (check_supported, crates/bobcat/src/lfm2_metal.rs:797-866, and the
// DeltaNet limits of crates/bobcat-metal/src/backend.rs:1899-1911).
bc_status check_supported(const bc_model& m) {
    const bc_hparams& hp = m.hp;
    std::vector<const HostMatrix*> all = {&m.token_embd, &m.output};
    for (const LayerSpec& S : m.layers) {
        for (const HostMatrix* hm : {&S.q, &S.k, &S.v, &S.output, &S.in_proj, &S.out_proj, &S.qkv, &S.z, &S.beta, &S.alpha, &S.ssm_out,
                                     &S.gate, &S.up, &S.down, &S.router})
            if (hm->t) all.push_back(hm);
        if (S.gate.t && S.up.t && S.gate.t->type != S.up.t->type)
            return fail(BC_ERR_UNSUPPORTED, "gate and up matrices of one type, got %u and %u", S.gate.t->type, S.up.t->type);
        if (S.moe && S.router.t->type != T_F32) return fail(BC_ERR_UNSUPPORTED, "an F32 router, got type %u", S.router.t->type);
    }
    for (const HostMatrix* hm : all) {
        if (!kernel_format(hm->t->type)) return fail(BC_ERR_UNSUPPORTED, "matrices in Q4_0, Q8_0, Q6_K, F16 or F32, got type %u for %s", hm->t->type, hm->t->name.c_str());
        if (hm->n_cols % 32 != 0) return fail(BC_ERR_UNSUPPORTED, "matrix rows of a multiple of 32 columns, got %u for %s", hm->n_cols, hm->t->name.c_str());
        if (hm->t->type == T_Q6K && hm->n_cols % 256 != 0) return fail(BC_ERR_UNSUPPORTED, "Q6_K rows of whole super-blocks of 256, got %u for %s", hm->n_cols, hm->t->name.c_str());
    }
    uint32_t group = hp.n_heads / (hp.n_kv_heads ? hp.n_kv_heads : 1);
    if (hp.n_attention_layers && (hp.head_dim % 32 != 0 || hp.head_dim > 256 || group > 8))
        return fail(BC_ERR_UNSUPPORTED, "a head size that is a multiple of 32 up to 256 and at most 8 query heads per KV head, got %u and %u",
                    hp.head_dim, group);
    if (hp.conv_kernel > 9) return fail(BC_ERR_UNSUPPORTED, "a convolution of at most 9 taps, got %u", hp.conv_kernel);
    if (hp.n_experts > 128 || hp.n_experts_used > 8)
        return fail(BC_ERR_UNSUPPORTED, "at most 8 of 128 experts per token, got %u of %u", hp.n_experts_used, hp.n_experts);
    if (hp.n_delta_layers && (hp.k_head_dim > 128 || hp.k_head_dim % 32 != 0 || hp.v_head_dim % 32 != 0 || hp.v_head_dim > 256))
        return fail(BC_ERR_UNSUPPORTED, "DeltaNet key heads of a multiple of 32 up to 128 and value heads of a multiple of 32 up to 256, got %u and %u",
                    hp.k_head_dim, hp.v_head_dim);
    return BC_OK;
}

uint64_t aligned(uint64_t n) { return round_up(n, 256); }

uint64_t device_bytes(const HostMatrix& hm) {
    if (!hm.t) return 0;
    uint64_t n = (uint64_t)hm.n_rows * hm.n_cols;
    if (hm.t->type == T_Q4_0) {
        uint64_t tiles = k::tiles_supported(hm.n_cols) ? aligned(k::tiles_bytes(hm.n_rows, hm.n_cols)) : 0;
        return aligned(n / 32 * 16) + aligned(n / 32 * 2) + tiles;
    }
    return aligned(hm.t->n_bytes);
}

}  // namespace

bc::DeviceModel::~DeviceModel() {
    if (arena || !extra.empty()) cudaSetDevice(device);
    if (arena) cudaFree(arena);
    for (void* p : extra) cudaFree(p);
}

bc_status bc_model::device_model(bc_backend* backend, std::shared_ptr<DeviceModel>* out) {
    std::lock_guard<std::mutex> lock(mutex);
    auto found = on_device.find(backend->device);
    if (found != on_device.end()) {
        *out = found->second;
        return BC_OK;
    }
    BC_TRY(backend->activate());
    auto dm = std::make_shared<DeviceModel>();
    dm->device = backend->device;

    // Every tensor the kernels read, each once (a tied output matrix shares the embedding).
    std::map<const GgufTensor*, uint64_t> offsets;
    uint64_t total = 0, largest_raw = 0;
    auto plan_matrix = [&](const HostMatrix& hm) {
        if (!hm.t || offsets.count(hm.t)) return;
        offsets[hm.t] = total;
        total += device_bytes(hm);
        if (hm.t->type == T_Q4_0 && hm.t->n_bytes > largest_raw) largest_raw = hm.t->n_bytes;
    };
    auto plan_vector = [&](const HostVector& hv) {
        if (!hv.t || offsets.count(hv.t)) return;
        offsets[hv.t] = total;
        total += aligned(hv.t->n_bytes);
    };
    plan_matrix(token_embd);
    plan_matrix(output);
    plan_vector(output_norm);
    for (const LayerSpec& S : layers) {
        for (const HostMatrix* hm : {&S.q, &S.k, &S.v, &S.output, &S.in_proj, &S.out_proj, &S.qkv, &S.z, &S.beta, &S.alpha, &S.ssm_out, &S.gate,
                                     &S.up, &S.down, &S.router})
            plan_matrix(*hm);
        for (const HostVector* hv : {&S.attn_norm, &S.ffn_norm, &S.q_norm, &S.k_norm, &S.taps, &S.conv1d, &S.dt_bias, &S.a, &S.ssm_norm, &S.expert_bias})
            plan_vector(*hv);
    }
    cudaError_t e = cudaMalloc(&dm->arena, total ? total : 256);
    if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate %llu bytes of device weights: %s", (unsigned long long)total, cudaGetErrorString(e));
    dm->arena_bytes = total;
    void* staging = nullptr;
    if (largest_raw) {
        e = cudaMalloc(&staging, largest_raw);
        if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate %llu staging bytes: %s", (unsigned long long)largest_raw, cudaGetErrorString(e));
    }
    struct Free {
        void* p;
        ~Free() { if (p) cudaFree(p); }
    } free_staging{staging};
    char* base = static_cast<char*>(dm->arena);
    std::map<const GgufTensor*, bool> uploaded;

    auto upload_matrix = [&](const HostMatrix& hm, k::Mat* mat) -> bc_status {
        if (!hm.t) return BC_OK;
        char* dst = base + offsets[hm.t];
        mat->format = (int32_t)hm.t->type;
        mat->n_rows = hm.n_rows;
        mat->n_cols = hm.n_cols;
        mat->data = dst;
        uint64_t n_blocks = (uint64_t)hm.n_rows * hm.n_cols / 32;
        if (hm.t->type == T_Q4_0) {
            mat->scales = reinterpret_cast<const __half*>(dst + aligned(n_blocks * 16));
            if (k::tiles_supported(hm.n_cols)) mat->tiles = dst + aligned(n_blocks * 16) + aligned(n_blocks * 2);
        }
        if (uploaded[hm.t]) return BC_OK;
        uploaded[hm.t] = true;
        if (hm.t->type == T_Q4_0) {
            // The stream orders each tensor's copy into the staging buffer after the repack of the
            // tensor before it.
            BC_CUDA(cudaMemcpyAsync(staging, gguf.data(*hm.t), hm.t->n_bytes, cudaMemcpyHostToDevice, backend->stream));
            BC_CUDA(k::repack_q4_0(backend->stream, static_cast<const uint8_t*>(staging), n_blocks, dst, const_cast<__half*>(mat->scales)));
            if (k::tiles_supported(hm.n_cols)) {
                // A second copy in the layout the tensor-core decode kernel streams.
                char* tiles = dst + aligned(n_blocks * 16) + aligned(n_blocks * 2);
                BC_CUDA(k::repack_tiles(backend->stream, dst, mat->scales, hm.n_rows, hm.n_cols, tiles));
            }
        } else {
            BC_CUDA(cudaMemcpyAsync(dst, gguf.data(*hm.t), hm.t->n_bytes, cudaMemcpyHostToDevice, backend->stream));
        }
        return BC_OK;
    };
    auto upload_vector = [&](const HostVector& hv, const float** ptr) -> bc_status {
        if (!hv.t) return BC_OK;
        char* dst = base + offsets[hv.t];
        *ptr = reinterpret_cast<const float*>(dst);
        if (uploaded[hv.t]) return BC_OK;
        uploaded[hv.t] = true;
        BC_CUDA(cudaMemcpyAsync(dst, gguf.data(*hv.t), hv.t->n_bytes, cudaMemcpyHostToDevice, backend->stream));
        return BC_OK;
    };

    BC_TRY(upload_matrix(token_embd, &dm->token_embd));
    BC_TRY(upload_matrix(output, &dm->output));
    BC_TRY(upload_vector(output_norm, &dm->output_norm));
    dm->layers.resize(layers.size());
    for (size_t il = 0; il < layers.size(); ++il) {
        const LayerSpec& S = layers[il];
        DeviceLayer& D = dm->layers[il];
        BC_TRY(upload_matrix(S.q, &D.q));
        BC_TRY(upload_matrix(S.k, &D.k));
        BC_TRY(upload_matrix(S.v, &D.v));
        BC_TRY(upload_matrix(S.output, &D.output));
        BC_TRY(upload_matrix(S.in_proj, &D.in_proj));
        BC_TRY(upload_matrix(S.out_proj, &D.out_proj));
        BC_TRY(upload_matrix(S.qkv, &D.qkv));
        BC_TRY(upload_matrix(S.z, &D.z));
        BC_TRY(upload_matrix(S.beta, &D.beta));
        BC_TRY(upload_matrix(S.alpha, &D.alpha));
        BC_TRY(upload_matrix(S.ssm_out, &D.ssm_out));
        BC_TRY(upload_matrix(S.gate, &D.gate));
        BC_TRY(upload_matrix(S.up, &D.up));
        BC_TRY(upload_matrix(S.down, &D.down));
        BC_TRY(upload_matrix(S.router, &D.router));
        BC_TRY(upload_vector(S.attn_norm, &D.attn_norm));
        BC_TRY(upload_vector(S.ffn_norm, &D.ffn_norm));
        BC_TRY(upload_vector(S.q_norm, &D.q_norm));
        BC_TRY(upload_vector(S.k_norm, &D.k_norm));
        BC_TRY(upload_vector(S.taps, &D.taps));
        BC_TRY(upload_vector(S.conv1d, &D.conv1d));
        BC_TRY(upload_vector(S.dt_bias, &D.dt_bias));
        BC_TRY(upload_vector(S.a, &D.a));
        BC_TRY(upload_vector(S.ssm_norm, &D.ssm_norm));
        BC_TRY(upload_vector(S.expert_bias, &D.expert_bias));
    }
    BC_CUDA(cudaStreamSynchronize(backend->stream));
    on_device[backend->device] = dm;
    *out = dm;
    return BC_OK;
}

extern "C" {

bc_status bc_model_load(const char* path, bc_model** out) {
    if (!path || !out) return fail(BC_ERR_ARGUMENT, "path and out must be non-null");
    std::unique_ptr<bc_model> m(new bc_model());
    BC_TRY(m->gguf.open(path));
    std::string architecture;
    if (!m->gguf.string("general.architecture", &architecture)) return fail(BC_ERR_METADATA, "missing or invalid metadata general.architecture");
    if (architecture == "lfm2") BC_TRY(load_lfm2(*m, false));
    else if (architecture == "lfm2moe") BC_TRY(load_lfm2(*m, true));
    else if (architecture == "qwen35") BC_TRY(load_qwen35(*m));
    else return fail(BC_ERR_ARCHITECTURE, "unsupported architecture %s", architecture.c_str());
    *out = m.release();
    return BC_OK;
}

void bc_model_free(bc_model* model) { delete model; }

bc_status bc_model_hparams(const bc_model* model, bc_hparams* out) {
    if (!model || !out) return fail(BC_ERR_ARGUMENT, "model and out must be non-null");
    *out = model->hp;
    return BC_OK;
}

bc_status bc_model_attention_layers(const bc_model* model, uint8_t* out, size_t len) {
    if (!model || !out) return fail(BC_ERR_ARGUMENT, "model and out must be non-null");
    if (len != model->layers.size()) return fail(BC_ERR_ARGUMENT, "out must hold n_layers bytes");
    for (size_t i = 0; i < len; ++i) out[i] = model->layers[i].mixer == Mixer::Attention;
    return BC_OK;
}

uint64_t bc_model_decode_bytes(const bc_model* model) {
    if (!model) return 0;
    const bc_hparams& hp = model->hp;
    uint64_t total = model->output.t->n_bytes;
    for (const LayerSpec& S : model->layers) {
        for (const HostMatrix* hm : {&S.q, &S.k, &S.v, &S.output, &S.in_proj, &S.out_proj, &S.qkv, &S.z, &S.beta, &S.alpha, &S.ssm_out, &S.router})
            if (hm->t) total += hm->t->n_bytes;
        for (const HostMatrix* hm : {&S.gate, &S.up, &S.down}) {
            if (!hm->t) continue;
            // A mixture-of-experts layer reads only the experts the router picks.
            total += S.moe ? hm->t->n_bytes / hp.n_experts * hp.n_experts_used : hm->t->n_bytes;
        }
    }
    return total;
}

}  // extern "C"

// Exposed to the sequence code.
namespace bc {
bc_status model_check_supported(const bc_model& m) { return check_supported(m); }
}  // namespace bc
