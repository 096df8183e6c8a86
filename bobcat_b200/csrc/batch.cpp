// Multi-sequence decode: n_seqs independent sequences of one model that advance together, one
// token each per pass, so that a pass reads every weight once for all of them.
//
// The reference runs one sequence per runner and one request at a time
// (crates/bobcat/src/lfm2_metal.rs:103-105, crates/bobcat-cli/src/serve.rs:4-7). A batch here is
// n_seqs such runners - each sequence keeps its own KV cache, convolution history, position and
// logits, is prefilled on the single-sequence path, and may be at any position - plus a decode
// pass over all of them whose row b computes what Lfm2Metal::step (lfm2_metal.rs:308) computes for
// sequence b.

#include <memory>
#include <vector>

#include <algorithm>

#include "recorder.h"
#include "seq.h"

using namespace bc;

struct bc_batch {
    bc_model* model = nullptr;
    bc_backend* backend = nullptr;
    std::vector<bc_seq*> seqs;  // owned; seqs[0]'s activation rows also serve the batched pass
    uint32_t n_ctx = 0;
    ExpertParallel ep;  // comm is null unless the experts are sharded over ranks
    // One device allocation: positions, picked tokens, per-sequence pointer tables, logits rows,
    // generated tokens of the current call.
    void* arena = nullptr;
    uint32_t *pos = nullptr, *picked = nullptr, *generated = nullptr;
    void **k_ptrs = nullptr, **v_ptrs = nullptr;
    float** conv_ptrs = nullptr;
    float* logits = nullptr;  // [n_seqs][n_vocab]
    uint32_t generated_cap = 0;
    cudaEvent_t start = nullptr, stop = nullptr;
    double last_gpu_seconds = 0;
    uint64_t launches = 0;

    ~bc_batch() {
        if (backend) {
            cudaSetDevice(backend->device);
            cudaStreamSynchronize(backend->stream);
        }
        for (bc_seq* s : seqs) bc_seq_free(s);
        cudaFree(arena);
        cudaFree(generated);
        if (start) cudaEventDestroy(start);
        if (stop) cudaEventDestroy(stop);
    }
};

extern "C" {

bc_status bc_batch_new(bc_model* model, bc_backend* backend, uint32_t n_seqs, uint32_t n_ctx, int32_t kv_half, bc_batch** out) {
    if (!model || !backend || !out) return fail(BC_ERR_ARGUMENT, "model, backend and out must be non-null");
    if (n_seqs == 0 || n_seqs > 512) return fail(BC_ERR_ARGUMENT, "a batch holds 1 to 512 sequences, got %u", n_seqs);
    const bc_hparams& hp = model->hp;
    if (hp.architecture == BC_ARCH_QWEN35) return fail(BC_ERR_UNSUPPORTED, "multi-sequence decode of Qwen3.5 models");
    if (hp.n_attention_layers && !k::attention_seqs_supported(hp.n_heads, hp.n_kv_heads, hp.head_dim))
        return fail(BC_ERR_ATTENTION_LIMITS, "multi-sequence attention needs heads of 32, 64, 128 or 256 elements and at most 8 query heads per KV head");
    if (n_ctx < n_seqs) return fail(BC_ERR_ARGUMENT, "the context (%u) must be at least the number of sequences (%u): the batched pass uses one sequence's prefill rows", n_ctx, n_seqs);
    BC_TRY(backend->activate());
    std::unique_ptr<bc_batch> b(new bc_batch());
    b->model = model;
    b->backend = backend;
    b->n_ctx = n_ctx;
    for (uint32_t i = 0; i < n_seqs; ++i) {
        bc_seq* s = nullptr;
        BC_TRY(bc_seq_new(model, backend, n_ctx, kv_half, &s));
        b->seqs.push_back(s);
    }
    const size_t words = (size_t)n_seqs;
    size_t bytes = round_up(words * 4, 256) * 2 + round_up(words * sizeof(void*), 256) * 3 + round_up(words * hp.n_vocab * 4, 256);
    cudaError_t e = cudaMalloc(&b->arena, bytes);
    if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate %zu bytes of batch state: %s", bytes, cudaGetErrorString(e));
    BC_CUDA(cudaMemsetAsync(b->arena, 0, bytes, backend->stream));
    char* p = static_cast<char*>(b->arena);
    auto take = [&](size_t n) { char* at = p; p += round_up(n, 256); return at; };
    b->pos = reinterpret_cast<uint32_t*>(take(words * 4));
    b->picked = reinterpret_cast<uint32_t*>(take(words * 4));
    b->k_ptrs = reinterpret_cast<void**>(take(words * sizeof(void*)));
    b->v_ptrs = reinterpret_cast<void**>(take(words * sizeof(void*)));
    b->conv_ptrs = reinterpret_cast<float**>(take(words * sizeof(void*)));
    b->logits = reinterpret_cast<float*>(take(words * hp.n_vocab * 4));
    std::vector<void*> kp(n_seqs), vp(n_seqs), cp(n_seqs);
    for (uint32_t i = 0; i < n_seqs; ++i) {
        kp[i] = b->seqs[i]->k_cache;
        vp[i] = b->seqs[i]->v_cache;
        cp[i] = b->seqs[i]->conv_state;
    }
    BC_CUDA(cudaMemcpyAsync(b->k_ptrs, kp.data(), words * sizeof(void*), cudaMemcpyHostToDevice, backend->stream));
    BC_CUDA(cudaMemcpyAsync(b->v_ptrs, vp.data(), words * sizeof(void*), cudaMemcpyHostToDevice, backend->stream));
    BC_CUDA(cudaMemcpyAsync(b->conv_ptrs, cp.data(), words * sizeof(void*), cudaMemcpyHostToDevice, backend->stream));
    BC_CUDA(cudaStreamSynchronize(backend->stream));
    BC_CUDA(cudaEventCreate(&b->start));
    BC_CUDA(cudaEventCreate(&b->stop));
    *out = b.release();
    return BC_OK;
}

bc_status bc_batch_new_expert_parallel(bc_model* model, bc_backend* backend, bc_comm* comm, uint32_t n_seqs, uint32_t n_ctx, int32_t kv_half,
                                       bc_batch** out) {
    if (!model || !comm || !out) return fail(BC_ERR_ARGUMENT, "model, comm and out must be non-null");
    if (comm->backend != backend) return fail(BC_ERR_FOREIGN_BUFFER, "the communicator belongs to another backend");
    const bc_hparams& hp = model->hp;
    const uint32_t world = (uint32_t)comm->world;
    if (hp.n_experts == 0) return fail(BC_ERR_NO_EXPERTS, "expert parallelism needs a mixture-of-experts model");
    if (hp.n_experts % world != 0) return fail(BC_ERR_EXPERT_LIMITS, "%u experts do not split over %u ranks", hp.n_experts, world);
    // The gathered rows of all ranks pass through one sequence's prefill-sized buffers.
    if ((uint64_t)n_seqs * world > std::min<uint64_t>(n_ctx, kPrefillBatch))
        return fail(BC_ERR_ARGUMENT, "%u sequences on each of %u ranks need a context of at least %u positions (at most %u rows in all)", n_seqs,
                    world, n_seqs * world, kPrefillBatch);
    bc_batch* batch = nullptr;
    BC_TRY(bc_batch_new(model, backend, n_seqs, n_ctx, kv_half, &batch));
    batch->ep.comm = comm;
    batch->ep.n_local_experts = hp.n_experts / world;
    batch->ep.first_expert = (uint32_t)comm->rank * batch->ep.n_local_experts;
    *out = batch;
    return BC_OK;
}

bc_status bc_batch_set_exact(bc_batch* batch, int32_t exact) {
    if (!batch) return fail(BC_ERR_ARGUMENT, "batch must be non-null");
    // The batched pass records through sequence 0's buffers.
    batch->seqs[0]->exact_products = exact != 0;
    return BC_OK;
}

void bc_batch_free(bc_batch* batch) { delete batch; }

uint32_t bc_batch_n_seqs(const bc_batch* batch) { return batch ? (uint32_t)batch->seqs.size() : 0; }

bc_status bc_batch_seq(bc_batch* batch, uint32_t index, bc_seq** out) {
    if (!batch || !out) return fail(BC_ERR_ARGUMENT, "batch and out must be non-null");
    if (index >= batch->seqs.size()) return fail(BC_ERR_ARGUMENT, "no sequence %u in a batch of %zu", index, batch->seqs.size());
    *out = batch->seqs[index];
    return BC_OK;
}

bc_status bc_batch_generate(bc_batch* batch, uint32_t* out, size_t n_tokens) {
    if (!batch || (!out && n_tokens)) return fail(BC_ERR_ARGUMENT, "batch and out must be non-null");
    if (n_tokens > UINT32_MAX) return fail(BC_ERR_ARGUMENT, "too many tokens");
    const uint32_t n = (uint32_t)n_tokens, n_seqs = (uint32_t)batch->seqs.size();
    bc_backend* backend = batch->backend;
    const bc_hparams& hp = batch->model->hp;
    // Validate every sequence before any device work; positions advance only on success.
    for (uint32_t i = 0; i < n_seqs; ++i) {
        const bc_seq* s = batch->seqs[i];
        if (s->n_past == 0) return fail(BC_ERR_ARGUMENT, "sequence %u needs a prompt before it can generate", i);
        if (n > s->n_ctx - s->n_past)
            return fail(BC_ERR_CONTEXT_FULL, "context full: %u tokens requested, %u remaining in sequence %u", n, s->n_ctx - s->n_past, i);
    }
    if (backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(backend->activate());
    if (n == 0) return BC_OK;
    cudaStream_t stream = backend->stream;
    if (batch->generated_cap < n) {
        BC_CUDA(cudaStreamSynchronize(stream));
        cudaFree(batch->generated);
        batch->generated = nullptr;
        batch->generated_cap = 0;
        cudaError_t e = cudaMalloc(&batch->generated, (size_t)n_seqs * n * 4);
        if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate the generated tokens: %s", cudaGetErrorString(e));
        batch->generated_cap = n;
    }
    // Each sequence's logits (left by its prefill or by an earlier pass) become its row, and its
    // position the one its next token takes.
    std::vector<uint32_t> positions(n_seqs);
    for (uint32_t i = 0; i < n_seqs; ++i) {
        positions[i] = batch->seqs[i]->n_past;
        BC_CUDA(cudaMemcpyAsync(batch->logits + (size_t)i * hp.n_vocab, batch->seqs[i]->logits, (size_t)hp.n_vocab * 4, cudaMemcpyDeviceToDevice, stream));
    }
    BC_CUDA(cudaMemcpyAsync(batch->pos, positions.data(), (size_t)n_seqs * 4, cudaMemcpyHostToDevice, stream));
    BC_CUDA(cudaEventRecord(batch->start, stream));

    bc_seq& rows = *batch->seqs[0];
    uint64_t before = rows.launches;
    Recorder r(rows);
    // With the sequences spread over ranks, a rank's share runs on the kernels the whole batch
    // would run on in one process: the tensor-core products when all ranks together hold 16 rows
    // or more, however few of them are this rank's (they still read every weight).
    if (batch->ep.comm && batch->ep.comm->world > 1) r.min_tensor_rows = std::max(1u, (16u + (uint32_t)batch->ep.comm->world - 1) / (uint32_t)batch->ep.comm->world);
    k::SeqTable table;
    table.pos = batch->pos;
    table.k_cache = batch->k_ptrs;
    table.v_cache = batch->v_ptrs;
    table.conv_state = batch->conv_ptrs;
    for (uint32_t i = 0; i < n && r.status == BC_OK; ++i) {
        // Pick each sequence's token from its logits, run it at the sequence's position, move on.
        r.run("argmax_rows", n_seqs, hp.n_vocab, 0, 1,
              [&] { return k::argmax_rows(stream, batch->logits, hp.n_vocab, n_seqs, batch->picked, batch->generated, n, i); });
        r.lfm2_seqs_step(batch->picked, n_seqs, table, batch->logits, batch->ep.comm ? &batch->ep : nullptr);
        r.run("advance_seqs", 1, n_seqs, 0, 1, [&] { return k::advance_seqs(stream, batch->pos, n_seqs); });
    }
    batch->launches += rows.launches - before;
    if (r.status != BC_OK) {
        cudaStreamSynchronize(stream);
        return r.status;
    }
    BC_CUDA(cudaEventRecord(batch->stop, stream));
    // The sequences stay usable on their own: each takes its latest logits back.
    for (uint32_t i = 0; i < n_seqs; ++i)
        BC_CUDA(cudaMemcpyAsync(batch->seqs[i]->logits, batch->logits + (size_t)i * hp.n_vocab, (size_t)hp.n_vocab * 4, cudaMemcpyDeviceToDevice, stream));
    BC_CUDA(cudaMemcpyAsync(out, batch->generated, (size_t)n_seqs * n * 4, cudaMemcpyDeviceToHost, stream));
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return cuda_fail(e, "the multi-sequence decode");
    BC_TRY(kernel_wait_status());
    float ms = 0.f;
    cudaEventElapsedTime(&ms, batch->start, batch->stop);
    batch->last_gpu_seconds = ms * 1e-3;
    for (bc_seq* s : batch->seqs) s->n_past += n;
    return BC_OK;
}

bc_status bc_batch_timings(const bc_batch* batch, double* gpu_seconds, uint64_t* launches) {
    if (!batch) return fail(BC_ERR_ARGUMENT, "batch must be non-null");
    if (gpu_seconds) *gpu_seconds = batch->last_gpu_seconds;
    if (launches) *launches = batch->launches;
    return BC_OK;
}

}  // extern "C"
