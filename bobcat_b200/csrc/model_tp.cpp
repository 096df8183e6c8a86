// Tensor-parallel weight shards of a Qwen3.5 model: what rank r of G uploads.
//
// The reference is single-GPU; the arithmetic each shard must reproduce is qwen35.rs:369-516
// (attention and DeltaNet blocks) and :284-365 (the step around them). The split:
//  - gated attention by KV head: a rank takes whole KV heads and the query heads that read them
//    (query head h reads KV head h / group); with more ranks than KV heads, ranks share a KV head
//    and split its group of query heads. q rows (per head [queries | gate], qwen35.rs:383-390),
//    k and v rows, and the matching columns of the output projection are rank-local.
//  - DeltaNet by key head: a rank takes key heads in a contiguous range and every value head that
//    reads one of them (value head j reads key head j % n_k_heads, crates/bobcat-metal/src/
//    gdn.metal:244), ordered so that the same rule holds on local indices. The q | k | v rows of the
//    qkv projection, their convolution taps, the z, beta and alpha rows, dt_bias and a, and the
//    columns of the output projection are rank-local; the state and the conv history are too.
//  - feed-forward: gate and up rows in a contiguous range, the same range of down's columns.
//  - the output matrix by vocabulary rows (the embedding table itself is whole on every rank).
// Each mixer and each feed-forward block then ends in a sum over ranks of its output projection.
// Shards are assembled on the host from the GGUF bytes (rows, or ranges of blocks of each row) and
// go through the same repacking as whole matrices, so their values are the file's bit for bit.

#include <cstring>

#include "model.h"

using namespace bc;

namespace {

uint64_t aligned(uint64_t n) { return round_up(n, 256); }

struct Range {
    uint32_t first, count;
};

struct Uploader {
    bc_backend* backend;
    const Gguf& gguf;
    DeviceModel& dm;
    void* staging = nullptr;
    size_t staging_cap = 0;

    ~Uploader() {
        if (staging) cudaFree(staging);
    }

    bc_status device_alloc(size_t bytes, char** out) {
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, bytes ? bytes : 256);
        if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate %zu bytes of device weights: %s", bytes, cudaGetErrorString(e));
        dm.extra.push_back(p);
        *out = static_cast<char*>(p);
        return BC_OK;
    }

    // `host` holds n_rows rows in the GGUF byte layout of `type`.
    bc_status matrix_bytes(uint32_t type, const std::vector<uint8_t>& host, uint32_t n_rows, uint32_t n_cols, k::Mat* mat) {
        mat->format = (int32_t)type;
        mat->n_rows = n_rows;
        mat->n_cols = n_cols;
        const uint64_t n_blocks = (uint64_t)n_rows * n_cols / 32;
        cudaStream_t stream = backend->stream;
        if (type == T_Q4_0) {
            const bool tiled = k::tiles_supported(n_cols);
            char* dst = nullptr;
            BC_TRY(device_alloc(aligned(n_blocks * 16) + aligned(n_blocks * 2) + (tiled ? aligned(k::tiles_bytes(n_rows, n_cols)) : 0), &dst));
            mat->data = dst;
            mat->scales = reinterpret_cast<const __half*>(dst + aligned(n_blocks * 16));
            if (host.size() > staging_cap) {
                BC_CUDA(cudaStreamSynchronize(stream));
                if (staging) cudaFree(staging);
                staging = nullptr;
                staging_cap = 0;
                cudaError_t e = cudaMalloc(&staging, host.size() + host.size() / 4);
                if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate %zu staging bytes", host.size());
                staging_cap = host.size() + host.size() / 4;
            }
            // The host vector is gone after this call: finish the copy before returning.
            BC_CUDA(cudaMemcpyAsync(staging, host.data(), host.size(), cudaMemcpyHostToDevice, stream));
            BC_CUDA(k::repack_q4_0(stream, static_cast<const uint8_t*>(staging), n_blocks, dst, const_cast<__half*>(mat->scales)));
            if (tiled) {
                char* tiles = dst + aligned(n_blocks * 16) + aligned(n_blocks * 2);
                mat->tiles = tiles;
                BC_CUDA(k::repack_tiles(stream, dst, mat->scales, n_rows, n_cols, tiles));
            }
            BC_CUDA(cudaStreamSynchronize(stream));
            return BC_OK;
        }
        if (type != T_F32 && type != T_F16) return fail(BC_ERR_UNSUPPORTED, "tensor-parallel shards of tensor type %u", type);
        char* dst = nullptr;
        BC_TRY(device_alloc(host.size(), &dst));
        mat->data = dst;
        BC_CUDA(cudaMemcpyAsync(dst, host.data(), host.size(), cudaMemcpyHostToDevice, stream));
        BC_CUDA(cudaStreamSynchronize(stream));
        return BC_OK;
    }

    // The rows `ranges` of a matrix, in that order.
    bc_status rows(const HostMatrix& hm, const std::vector<Range>& ranges, k::Mat* mat) {
        const uint64_t row_bytes = type_row_bytes(hm.t->type, hm.n_cols);
        const uint8_t* src = gguf.data(*hm.t);
        std::vector<uint8_t> host;
        uint32_t n_rows = 0;
        for (const Range& r : ranges) {
            if ((uint64_t)r.first + r.count > hm.n_rows) return fail(BC_ERR_TENSOR_SHAPE, "a shard reaches past row %u of %s", hm.n_rows, hm.t->name.c_str());
            host.insert(host.end(), src + (uint64_t)r.first * row_bytes, src + (uint64_t)(r.first + r.count) * row_bytes);
            n_rows += r.count;
        }
        return matrix_bytes(hm.t->type, host, n_rows, hm.n_cols, mat);
    }

    // The columns `ranges` (multiples of 32) of every row, in that order.
    bc_status cols(const HostMatrix& hm, const std::vector<Range>& ranges, k::Mat* mat) {
        uint64_t elements = 1, block_bytes = 4;
        type_block(hm.t->type, &elements, &block_bytes);
        const uint64_t row_bytes = type_row_bytes(hm.t->type, hm.n_cols);
        const uint8_t* src = gguf.data(*hm.t);
        uint32_t n_cols = 0;
        for (const Range& r : ranges) {
            if (r.first % 32 || r.count % 32 || (uint64_t)r.first + r.count > hm.n_cols)
                return fail(BC_ERR_TENSOR_SHAPE, "a column shard of %s must be whole blocks of 32 inside the row", hm.t->name.c_str());
            n_cols += r.count;
        }
        std::vector<uint8_t> host;
        host.reserve((size_t)hm.n_rows * n_cols / elements * block_bytes);
        for (uint32_t row = 0; row < hm.n_rows; ++row) {
            const uint8_t* line = src + (uint64_t)row * row_bytes;
            for (const Range& r : ranges) host.insert(host.end(), line + r.first / elements * block_bytes, line + (r.first + r.count) / elements * block_bytes);
        }
        return matrix_bytes(hm.t->type, host, hm.n_rows, n_cols, mat);
    }

    // Groups of `width` floats of an F32 vector, picked by `ranges` of group indices.
    bc_status vector(const HostVector& hv, const std::vector<Range>& ranges, size_t width, const float** out) {
        const float* src = reinterpret_cast<const float*>(gguf.data(*hv.t));
        std::vector<float> host;
        for (const Range& r : ranges) {
            if (((size_t)r.first + r.count) * width > hv.n) return fail(BC_ERR_TENSOR_SHAPE, "a shard reaches past the end of %s", hv.t->name.c_str());
            host.insert(host.end(), src + (size_t)r.first * width, src + ((size_t)r.first + r.count) * width);
        }
        char* dst = nullptr;
        BC_TRY(device_alloc(host.size() * 4, &dst));
        BC_CUDA(cudaMemcpyAsync(dst, host.data(), host.size() * 4, cudaMemcpyHostToDevice, backend->stream));
        BC_CUDA(cudaStreamSynchronize(backend->stream));
        *out = reinterpret_cast<const float*>(dst);
        return BC_OK;
    }

    bc_status whole_vector(const HostVector& hv, const float** out) {
        if (!hv.t) return BC_OK;
        return vector(hv, {Range{0, (uint32_t)hv.n}}, 1, out);
    }
};

// Contiguous share of n items in multiples of `unit`; the first ranks take one unit more.
Range share(int rank, int world, uint32_t n, uint32_t unit) {
    uint32_t units = n / unit, base = units / world, extra = units % world;
    uint32_t first = rank * base + std::min<uint32_t>(rank, extra), count = base + ((uint32_t)rank < extra ? 1 : 0);
    return Range{first * unit, count * unit};
}

struct HeadSplit {
    std::vector<uint32_t> kv, q;      // attention: KV heads and query heads of the rank
    std::vector<uint32_t> keys, values;  // DeltaNet: key heads and value heads of the rank
};

bc_status split_heads(const bc_hparams& hp, int rank, int world, HeadSplit* out) {
    const uint32_t group = hp.n_heads / hp.n_kv_heads;
    if ((uint32_t)world <= hp.n_kv_heads) {
        if (hp.n_kv_heads % world) return fail(BC_ERR_KV_HEADS, "%u KV heads do not split over %d ranks", hp.n_kv_heads, world);
        uint32_t per = hp.n_kv_heads / world;
        for (uint32_t kv = rank * per; kv < (rank + 1) * per; ++kv) {
            out->kv.push_back(kv);
            for (uint32_t g = 0; g < group; ++g) out->q.push_back(kv * group + g);
        }
    } else {
        if (world % hp.n_kv_heads) return fail(BC_ERR_KV_HEADS, "%d ranks do not share %u KV heads evenly", world, hp.n_kv_heads);
        uint32_t sharers = world / hp.n_kv_heads;
        if (group % sharers) return fail(BC_ERR_KV_HEADS, "a group of %u query heads does not split over %u ranks", group, sharers);
        uint32_t kv = rank * hp.n_kv_heads / world, per = group / sharers;
        out->kv.push_back(kv);
        for (uint32_t g = 0; g < per; ++g) out->q.push_back(kv * group + (rank % sharers) * per + g);
    }
    if (hp.n_k_heads % world) return fail(BC_ERR_DELTANET_LIMITS, "%u key heads do not split over %d ranks", hp.n_k_heads, world);
    uint32_t per = hp.n_k_heads / world;
    for (uint32_t k = rank * per; k < (rank + 1) * per; ++k) out->keys.push_back(k);
    for (uint32_t rep = 0; rep < hp.n_v_heads / hp.n_k_heads; ++rep)
        for (uint32_t k : out->keys) out->values.push_back(k + rep * hp.n_k_heads);
    return BC_OK;
}

std::vector<Range> head_ranges(const std::vector<uint32_t>& heads, uint32_t width, uint32_t base = 0) {
    std::vector<Range> ranges;
    for (uint32_t h : heads) ranges.push_back(Range{base + h * width, width});
    return ranges;
}

}  // namespace

bc_hparams bc::tensor_parallel_hparams(const bc_hparams& hp, int rank, int world) {
    bc_hparams local = hp;
    HeadSplit heads;
    if (split_heads(hp, rank, world, &heads) != BC_OK) return local;
    local.n_heads = (uint32_t)heads.q.size();
    local.n_kv_heads = (uint32_t)heads.kv.size();
    local.n_k_heads = (uint32_t)heads.keys.size();
    local.n_v_heads = (uint32_t)heads.values.size();
    local.n_ff = share(rank, world, hp.n_ff, 32).count;
    return local;
}

bc_status bc_model::device_model_tp(bc_backend* backend, int rank, int world, std::shared_ptr<DeviceModel>* out) {
    if (hp.architecture != BC_ARCH_QWEN35) return fail(BC_ERR_UNSUPPORTED, "tensor parallelism of architectures other than qwen35");
    if (world < 1 || rank < 0 || rank >= world) return fail(BC_ERR_ARGUMENT, "rank %d outside a world of %d", rank, world);
    if (hp.n_vocab % (16 * world)) return fail(BC_ERR_ARGUMENT, "a vocabulary of %u rows does not split into %d shares of whole 16-row tiles", hp.n_vocab, world);
    if (hp.n_ff % (32 * world)) return fail(BC_ERR_ARGUMENT, "%u feed-forward rows do not split into %d shares of whole blocks", hp.n_ff, world);
    HeadSplit heads;
    BC_TRY(split_heads(hp, rank, world, &heads));
    std::lock_guard<std::mutex> lock(mutex);
    auto key = std::make_pair(backend->device, std::make_pair(rank, world));
    auto found = on_device_tp.find(key);
    if (found != on_device_tp.end()) {
        *out = found->second;
        return BC_OK;
    }
    BC_TRY(backend->activate());
    auto dm = std::make_shared<DeviceModel>();
    dm->device = backend->device;
    Uploader up{backend, gguf, *dm};

    const uint32_t hd = hp.head_dim, kd = hp.k_head_dim, vd = hp.v_head_dim;
    const uint32_t key_dim = hp.n_k_heads * kd;
    BC_TRY(up.rows(token_embd, {Range{0, token_embd.n_rows}}, &dm->token_embd));
    const Range vocab = share(rank, world, hp.n_vocab, 16);
    dm->first_vocab_row = vocab.first;
    dm->n_vocab_rows = vocab.count;
    if (tied_output) dm->output = dm->token_embd.rows(vocab.first, vocab.count);
    else BC_TRY(up.rows(output, {vocab}, &dm->output));
    BC_TRY(up.whole_vector(output_norm, &dm->output_norm));
    const Range ff = share(rank, world, hp.n_ff, 32);

    dm->layers.resize(layers.size());
    for (size_t il = 0; il < layers.size(); ++il) {
        const LayerSpec& S = layers[il];
        DeviceLayer& D = dm->layers[il];
        BC_TRY(up.whole_vector(S.attn_norm, &D.attn_norm));
        BC_TRY(up.whole_vector(S.ffn_norm, &D.ffn_norm));
        if (S.mixer == Mixer::Attention) {
            BC_TRY(up.rows(S.q, head_ranges(heads.q, 2 * hd), &D.q));
            BC_TRY(up.rows(S.k, head_ranges(heads.kv, hd), &D.k));
            BC_TRY(up.rows(S.v, head_ranges(heads.kv, hd), &D.v));
            BC_TRY(up.cols(S.output, head_ranges(heads.q, hd), &D.output));
            BC_TRY(up.whole_vector(S.q_norm, &D.q_norm));
            BC_TRY(up.whole_vector(S.k_norm, &D.k_norm));
        } else {
            // Channels of the q | k | v projection (and of its convolution): q heads, k heads, v heads.
            std::vector<Range> channels = head_ranges(heads.keys, kd);
            for (const Range& r : head_ranges(heads.keys, kd, key_dim)) channels.push_back(r);
            for (const Range& r : head_ranges(heads.values, vd, 2 * key_dim)) channels.push_back(r);
            BC_TRY(up.rows(S.qkv, channels, &D.qkv));
            BC_TRY(up.vector(S.conv1d, channels, hp.conv_kernel, &D.conv1d));
            BC_TRY(up.rows(S.z, head_ranges(heads.values, vd), &D.z));
            BC_TRY(up.rows(S.beta, head_ranges(heads.values, 1), &D.beta));
            BC_TRY(up.rows(S.alpha, head_ranges(heads.values, 1), &D.alpha));
            BC_TRY(up.vector(S.dt_bias, head_ranges(heads.values, 1), 1, &D.dt_bias));
            BC_TRY(up.vector(S.a, head_ranges(heads.values, 1), 1, &D.a));
            BC_TRY(up.whole_vector(S.ssm_norm, &D.ssm_norm));
            BC_TRY(up.cols(S.ssm_out, head_ranges(heads.values, vd), &D.ssm_out));
        }
        BC_TRY(up.rows(S.gate, {ff}, &D.gate));
        BC_TRY(up.rows(S.up, {ff}, &D.up));
        BC_TRY(up.cols(S.down, {ff}, &D.down));
    }
    on_device_tp[key] = dm;
    *out = dm;
    return BC_OK;
}
