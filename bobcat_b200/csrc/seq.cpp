#include "seq.h"
#include "recorder.h"

#include <algorithm>
#include <initializer_list>
#include <cstring>

using namespace bc;

namespace bc {
bc_status model_check_supported(const bc_model& m);
}

namespace {

using Clock = std::chrono::steady_clock;
double since(Clock::time_point start) { return std::chrono::duration<double>(Clock::now() - start).count(); }

bc_status ensure_trace_rows(bc_seq* s, uint32_t rows) {
    if (rows <= s->trace_rows) return BC_OK;
    const bc_hparams& hp = s->hp;
    BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    cudaFree(s->trace_embedding);
    cudaFree(s->trace_layers);
    cudaFree(s->trace_final);
    cudaFree(s->trace_routes);
    s->trace_embedding = s->trace_layers = s->trace_final = nullptr;
    s->trace_routes = nullptr;
    s->trace_rows = 0;
    size_t floats = (size_t)rows * hp.n_embd;
    size_t route_words = std::max<size_t>(1, (size_t)rows * hp.n_layers * 2 * hp.n_experts_used);
    if (cudaMalloc(&s->trace_embedding, floats * 4) != cudaSuccess || cudaMalloc(&s->trace_layers, floats * 4 * hp.n_layers) != cudaSuccess ||
        cudaMalloc(&s->trace_final, floats * 4) != cudaSuccess || cudaMalloc(&s->trace_routes, route_words * 4) != cudaSuccess ||
        cudaMemset(s->trace_routes, 0, route_words * 4) != cudaSuccess)
        return fail(BC_ERR_ALLOCATION, "cannot allocate trace buffers for %u tokens", rows);
    s->trace_rows = rows;
    return BC_OK;
}

bc_status check_trace(const bc_seq* s, const bc_trace* trace, uint32_t n_tokens, const char* why) {
    if (!trace) return BC_OK;
    if (!trace->embedding || !trace->layers || !trace->final_norm || trace->n_tokens != n_tokens) return fail(BC_ERR_ARGUMENT, "%s", why);
    (void)s;
    return BC_OK;
}

bc_status read_floats(bc_seq* s, const float* device, float* host, size_t n) {
    BC_CUDA(cudaMemcpyAsync(host, device, n * 4, cudaMemcpyDeviceToHost, s->backend->stream));
    return BC_OK;
}

// Bracket recorded work with events so last_gpu_seconds reports device time.
bc_status timing_begin(bc_seq* s) {
    BC_CUDA(cudaEventRecord(s->timing_start, s->backend->stream));
    return BC_OK;
}

bc_status timing_end(bc_seq* s, double* seconds) {
    BC_CUDA(cudaEventRecord(s->timing_end, s->backend->stream));
    cudaError_t e = cudaEventSynchronize(s->timing_end);
    if (e != cudaSuccess) return cuda_fail(e, "recorded work");
    float ms = 0.f;
    cudaEventElapsedTime(&ms, s->timing_start, s->timing_end);
    *seconds = ms * 1e-3;
    return kernel_wait_status();
}

// Replay needs a stream that can be captured (not the legacy default stream) and no per-launch
// event timing.
bool replay_enabled(const bc_seq* s) {
    return s->use_graphs && !s->backend->profiling && s->backend->stream != nullptr && s->backend->stream != cudaStreamLegacy;
}

// Capture one generated step into a graph. The generate variant picks tokens[pos] from the logits,
// then runs the forward pass at pos; the stream variant runs the forward pass at pos, then picks
// tokens[pos + 1] and mirrors it into the host-mapped ring at slot pos % kGenerateInFlight. Both
// start by adding one to s->step_pos, so the host seeds it with the first position minus one.
bc_status capture_step(bc_seq* s, bool stream_variant) {
    cudaStream_t stream = s->backend->stream;
    const uint32_t n_vocab = s->hp.n_vocab;
    uint64_t before = s->launches;
    BC_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    Recorder r(*s);
    r.replayed = true;
    if (stream_variant) {
        r.run("advance", 1, 1, 0, 1, [&] { return k::advance(stream, s->step_pos); });
        r.step(0, true, false);
        r.run("argmax", 1, n_vocab, 0, 1,
              [&] { return k::argmax_step(stream, s->logits, n_vocab, s->step_pos, false, s->tokens, 1, s->readback, kGenerateInFlight); });
    } else {
        r.run("argmax", 1, n_vocab, 0, 1,
              [&] { return k::argmax_step(stream, s->logits, n_vocab, s->step_pos, true, s->tokens, 0, nullptr, 1); });
        r.step(0, true, false);
    }
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(stream, &graph);
    uint64_t kernels = s->launches - before;
    s->launches = before;  // capturing launches nothing
    if (r.status != BC_OK) {
        if (graph) cudaGraphDestroy(graph);
        return r.status;
    }
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture");
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
    if (stream_variant) {
        s->stream_graph = exec;
        s->stream_graph_kernels = kernels;
    } else {
        s->generate_graph = exec;
        s->generate_graph_kernels = kernels;
    }
    return BC_OK;
}

// Make sure the wanted graph exists and seed the device position for a run that starts at `first`.
bc_status prepare_replay(bc_seq* s, bool stream_variant, uint32_t first) {
    if (stream_variant ? !s->stream_graph : !s->generate_graph) BC_TRY(capture_step(s, stream_variant));
    s->host_pos = first - 1;  // first >= 1: generation needs a prompt
    BC_CUDA(cudaMemcpyAsync(s->step_pos, &s->host_pos, 4, cudaMemcpyHostToDevice, s->backend->stream));
    return BC_OK;
}

bc_status generate_inner(bc_seq* s, uint32_t* out, size_t count, bool select_next) {
    if (!s || !s->backend || (!out && count)) return fail(BC_ERR_ARGUMENT, "seq and out must be non-null and the backend open");
    if (count > UINT32_MAX) return fail(BC_ERR_ARGUMENT, "too many tokens");
    uint32_t n = (uint32_t)count;
    uint32_t remaining = s->n_ctx - s->n_past;
    if (s->n_past == 0) return fail(BC_ERR_ARGUMENT, "generation needs a prompt first");
    if (n > remaining) return fail(BC_ERR_CONTEXT_FULL, "context full: %u tokens requested, %u remaining", n, remaining);
    if (s->backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(s->backend->activate());
    if (n == 0) return BC_OK;

    auto encode_start = Clock::now();
    const bool replay = replay_enabled(s);
    if (replay) BC_TRY(prepare_replay(s, /*stream_variant=*/false, s->n_past));
    BC_TRY(timing_begin(s));
    Recorder r(*s);
    for (uint32_t i = 0; i < n && r.status == BC_OK; ++i) {
        uint32_t pos = s->n_past + i;
        // Bound the steps in flight, so the CPU runs only a few steps ahead of the device.
        int slot = (int)(i % kGenerateInFlight);
        if (i >= (uint32_t)kGenerateInFlight) {
            cudaError_t e = cudaEventSynchronize(s->slot_done[slot]);
            if (e != cudaSuccess) return cuda_fail(e, "generation step");
        }
        if (replay) {
            BC_CUDA(cudaGraphLaunch(s->generate_graph, s->backend->stream));
            s->launches += s->generate_graph_kernels;
        } else {
            r.argmax(s->logits, s->tokens + pos, nullptr);
            r.step(pos, true, false);
        }
        if (select_next && i + 1 == n) r.argmax(s->logits, s->greedy_token, nullptr);
        if (r.status == BC_OK) BC_CUDA(cudaEventRecord(s->slot_done[slot], s->backend->stream));
    }
    double encode = since(encode_start);
    double gpu = 0;
    bc_status finish = timing_end(s, &gpu);
    if (r.status != BC_OK) return r.status;
    BC_TRY(finish);

    BC_CUDA(cudaMemcpyAsync(out, s->tokens + s->n_past, (size_t)n * 4, cudaMemcpyDeviceToHost, s->backend->stream));
    BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    if (select_next) {
        std::rotate(out, out + 1, out + n);
        BC_CUDA(cudaMemcpyAsync(out + n - 1, s->greedy_token, 4, cudaMemcpyDeviceToHost, s->backend->stream));
        BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    }
    s->n_past += n;
    s->last_encode_seconds = encode;
    s->last_gpu_seconds = gpu;
    return BC_OK;
}

}  // namespace

// Free everything the sequence holds on the device. Also called by bc_backend_close for sequences
// that outlive their backend, which are left as empty shells for bc_seq_free.
void bc_seq::release() {
    if (backend) {
        cudaSetDevice(backend->device);
        cudaStreamSynchronize(backend->stream);
        backend->seqs.erase(this);
    }
    k_pages.reset();
    v_pages.reset();
    cudaFree(arena);
    cudaFree(trace_embedding);
    cudaFree(trace_layers);
    cudaFree(trace_final);
    cudaFree(trace_routes);
    arena = nullptr;
    trace_embedding = trace_layers = trace_final = nullptr;
    trace_routes = nullptr;
    if (readback) cudaFreeHost(readback);
    readback = nullptr;
    if (generate_graph) cudaGraphExecDestroy(generate_graph);
    if (stream_graph) cudaGraphExecDestroy(stream_graph);
    generate_graph = stream_graph = nullptr;
    for (cudaEvent_t& e : slot_done) {
        if (e) cudaEventDestroy(e);
        e = nullptr;
    }
    if (timing_start) cudaEventDestroy(timing_start);
    if (timing_end) cudaEventDestroy(timing_end);
    timing_start = timing_end = nullptr;
    backend = nullptr;
}

bc_seq::~bc_seq() { release(); }

bc_prefix::~bc_prefix() {
    if (state || tail) cudaSetDevice(device);
    cudaFree(state);
    cudaFree(tail);
}

void release_seq(bc_seq* seq) { seq->release(); }

namespace {

// A sequence on `backend`; with `tp` its weights are the communicator rank's tensor-parallel shard
// and its shapes the rank's share.
bc_status seq_new(bc_model* model, bc_backend* backend, bc_comm* tp, uint32_t n_ctx, int32_t kv_half, bool paged, bc_seq** out) {
    if (!model || !backend || !out) return fail(BC_ERR_ARGUMENT, "model, backend and out must be non-null");
    if (n_ctx == 0) return fail(BC_ERR_ARGUMENT, "the context must hold a token");
    BC_TRY(model_check_supported(*model));
    BC_TRY(backend->activate());
    std::unique_ptr<bc_seq> s(new bc_seq());
    s->model = model;
    s->backend = backend;
    s->n_ctx = n_ctx;
    s->kv_half = kv_half != 0;
    s->batch = std::min(n_ctx, kPrefillBatch);
    s->hp = model->hp;
    if (tp && tp->world > 1) {
        BC_TRY(model->device_model_tp(backend, tp->rank, tp->world, &s->weights));
        s->hp = tensor_parallel_hparams(model->hp, tp->rank, tp->world);
        s->tp = tp;
    } else {
        BC_TRY(model->device_model(backend, &s->weights));
    }

    const bc_hparams& hp = s->hp;
    const size_t n_embd = hp.n_embd, rows = s->batch;
    const size_t kv_dim = (size_t)hp.n_kv_heads * hp.head_dim, q_dim = (size_t)hp.n_heads * hp.head_dim;
    const size_t q_width = hp.architecture == BC_ARCH_QWEN35 ? 2 * q_dim : q_dim;  // Qwen's q holds [q | gate]
    // Paged caches live in their own mapped ranges, whose layers start on page boundaries.
    s->kv_stride = n_ctx;
    if (paged && hp.n_attention_layers) {
        PageGeometry geometry;
        geometry.kv_dim = (uint32_t)kv_dim;
        geometry.element_bytes = s->kv_half ? 2 : 4;
        geometry.page_positions = page_positions_for(backend->device, geometry.kv_dim, geometry.element_bytes);
        if (geometry.page_positions == 0)
            return fail(BC_ERR_UNSUPPORTED, "KV rows of %zu elements do not divide this device's page size (or it has no virtual memory management)", kv_dim);
        geometry.stride = (uint32_t)round_up(n_ctx, geometry.page_positions);
        geometry.n_layers = hp.n_attention_layers;
        s->kv_stride = geometry.stride;
        s->k_pages.reset(new PagedCache());
        s->v_pages.reset(new PagedCache());
        BC_TRY(s->k_pages->create(backend->device, geometry));
        BC_TRY(s->v_pages->create(backend->device, geometry));
    }
    const size_t cache_bytes = s->k_pages ? 0 : (size_t)hp.n_attention_layers * n_ctx * kv_dim * (s->kv_half ? 2 : 4);
    const size_t key_dim = (size_t)hp.n_k_heads * hp.k_head_dim, value_dim = (size_t)hp.n_v_heads * hp.v_head_dim;
    const size_t conv_dim = 2 * key_dim + value_dim;
    const bool qwen = hp.architecture == BC_ARCH_QWEN35;
    // LFM2: [conv layer][K - 1][n_embd] of B*X products. Qwen3.5: [delta layer][channel][K - 1] raw inputs.
    s->conv_floats = qwen ? (size_t)hp.n_delta_layers * conv_dim * (hp.conv_kernel - 1) : (size_t)hp.n_conv_layers * (hp.conv_kernel - 1) * n_embd;
    s->delta_floats = (size_t)hp.n_delta_layers * hp.n_v_heads * hp.k_head_dim * hp.v_head_dim;
    const size_t ffn_width = std::max<size_t>(hp.n_ff, (size_t)hp.n_experts_used * hp.n_ff_expert);
    const size_t scratch_floats = hp.n_attention_layers ? k::attention_scratch_floats(hp.n_heads, hp.head_dim, n_ctx, s->batch) : 0;

    // Plan the arena: (pointer slot, bytes) pairs, each aligned to 256 bytes.
    struct Item { void** slot; size_t bytes; };
    std::vector<Item> items = {
        {&s->k_cache, cache_bytes},
        {&s->v_cache, cache_bytes},
        {(void**)&s->k, rows * kv_dim * 4},
        {(void**)&s->v, rows * kv_dim * 4},
        {(void**)&s->conv_state, s->conv_floats * 4},
        {(void**)&s->hidden, rows * n_embd * 4},
        {(void**)&s->normed, rows * n_embd * 4},
        {(void**)&s->bcx, rows * 3 * n_embd * 4},
        {(void**)&s->conv_out, rows * n_embd * 4},
        {(void**)&s->q, rows * q_width * 4},
        {(void**)&s->attn, rows * q_dim * 4},
        {(void**)&s->scores, scratch_floats * 4},
        {(void**)&s->ffn, rows * ffn_width * 4},
        {(void**)&s->logits, (size_t)hp.n_vocab * 4},
        {(void**)&s->tokens, ((size_t)n_ctx + 1) * 4},
        {(void**)&s->greedy_token, 4},
        {(void**)&s->route, rows * 2 * hp.n_experts_used * 4},
        {(void**)&s->expert_offsets, ((size_t)hp.n_experts + 1) * 4},
        {(void**)&s->expert_entries, rows * hp.n_experts_used * 4},
        {(void**)&s->expert_out, rows * hp.n_experts_used * n_embd * 4},
        {(void**)&s->delta_state, s->delta_floats * 4},
        {(void**)&s->gdn_qkv, rows * conv_dim * 4},
        {(void**)&s->gdn_conv_out, rows * conv_dim * 4},
        {(void**)&s->gdn_z, rows * value_dim * 4},
        {(void**)&s->gdn_beta, rows * hp.n_v_heads * 4},
        {(void**)&s->gdn_alpha, rows * hp.n_v_heads * 4},
        {(void**)&s->gdn_out, rows * value_dim * 4},
        {(void**)&s->q_rot, qwen ? rows * q_dim * 4 : 0},
        {(void**)&s->step_pos, 4},
        {(void**)&s->partial, s->tp ? rows * n_embd * 4 : 0},
        {(void**)&s->rope_table, hp.n_attention_layers && !qwen ? (size_t)n_ctx * (hp.n_rot / 2) * sizeof(float2) : 0},
    };
    const char* no_graph = getenv("BOBCAT_NO_GRAPH");
    s->use_graphs = !(no_graph && no_graph[0] == '1');
    // A tensor-parallel step holds collectives (the peer-memory sums and NCCL's gather of the
    // logits, which records into a capture as well); BOBCAT_TP_GRAPH=0 launches it kernel by kernel.
    if (s->tp) {
        const char* tp_graph = getenv("BOBCAT_TP_GRAPH");
        if (tp_graph && tp_graph[0] == '0') s->use_graphs = false;
    }
    // Kernels whose input vector outgrows the default shared-memory limit get their limit raised
    // now, so no launch inside a capture has to.
    uint32_t widest = std::max({hp.n_embd, hp.n_ff, hp.n_ff_expert, (uint32_t)q_dim, hp.n_v_heads * hp.v_head_dim});
    BC_CUDA(k::matvec_prepare(widest));
    size_t total = 0;
    for (Item& it : items) total += round_up(std::max<size_t>(it.bytes, 4), 256);
    cudaError_t e = cudaMalloc(&s->arena, total);
    if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate %zu bytes of sequence state: %s", total, cudaGetErrorString(e));
    s->arena_bytes = total;
    BC_CUDA(cudaMemsetAsync(s->arena, 0, total, backend->stream));
    char* p = static_cast<char*>(s->arena);
    for (Item& it : items) {
        *it.slot = p;
        p += round_up(std::max<size_t>(it.bytes, 4), 256);
    }
    if (s->k_pages) {
        s->k_cache = s->k_pages->base();
        s->v_cache = s->v_pages->base();
    }
    if (hp.n_attention_layers && !qwen) BC_CUDA(k::rope_table(backend->stream, s->rope_table, n_ctx, hp.n_rot, hp.rope_theta));
    BC_TRY(ensure_trace_rows(s.get(), 1));
    e = cudaHostAlloc((void**)&s->readback, sizeof(uint32_t) * kGenerateInFlight, cudaHostAllocMapped);
    if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate the token readback: %s", cudaGetErrorString(e));
    for (int i = 0; i < kGenerateInFlight; ++i) BC_CUDA(cudaEventCreateWithFlags(&s->slot_done[i], cudaEventDisableTiming));
    BC_CUDA(cudaEventCreate(&s->timing_start));
    BC_CUDA(cudaEventCreate(&s->timing_end));
    BC_CUDA(cudaStreamSynchronize(backend->stream));
    backend->seqs.insert(s.get());
    *out = s.release();
    return BC_OK;
}

}  // namespace

extern "C" {

bc_status bc_seq_new(bc_model* model, bc_backend* backend, uint32_t n_ctx, int32_t kv_half, bc_seq** out) {
    return seq_new(model, backend, nullptr, n_ctx, kv_half, false, out);
}

bc_status bc_seq_new_paged(bc_model* model, bc_backend* backend, uint32_t n_ctx, int32_t kv_half, bc_seq** out) {
    return seq_new(model, backend, nullptr, n_ctx, kv_half, true, out);
}

bc_status bc_seq_new_tensor_parallel(bc_model* model, bc_backend* backend, bc_comm* comm, uint32_t n_ctx, int32_t kv_half, bc_seq** out) {
    if (!comm) return fail(BC_ERR_ARGUMENT, "comm must be non-null");
    if (comm->backend != backend) return fail(BC_ERR_FOREIGN_BUFFER, "the communicator belongs to another backend");
    return seq_new(model, backend, comm, n_ctx, kv_half, false, out);
}

void bc_seq_free(bc_seq* seq) { delete seq; }
uint32_t bc_seq_n_past(const bc_seq* seq) { return seq ? seq->n_past : 0; }
uint64_t bc_seq_launches(const bc_seq* seq) { return seq ? seq->launches : 0; }

}  // extern "C"

namespace {
bc_status step_impl(bc_seq* s, uint32_t token, float* logits, size_t logits_len, bc_trace* trace, bool device_logits);
}

extern "C" {

bc_status bc_seq_step(bc_seq* s, uint32_t token, float* logits, size_t logits_len, bc_trace* trace) {
    return step_impl(s, token, logits, logits_len, trace, false);
}

bc_status bc_seq_step_on_device(bc_seq* s, uint32_t token) { return step_impl(s, token, nullptr, 0, nullptr, true); }

}  // extern "C"

namespace {

bc_status step_impl(bc_seq* s, uint32_t token, float* logits, size_t logits_len, bc_trace* trace, bool device_logits) {
    if (!s || !s->backend) return fail(BC_ERR_ARGUMENT, "seq must be non-null and its backend open");
    const bc_hparams& hp = s->hp;
    uint32_t pos = s->n_past;
    if (pos >= s->n_ctx) return fail(BC_ERR_CONTEXT_FULL, "context full: 1 token requested, 0 remaining");
    if (token >= hp.n_vocab) return fail(BC_ERR_TOKEN, "token %u outside the vocabulary of %u", token, hp.n_vocab);
    if (logits && logits_len != hp.n_vocab) return fail(BC_ERR_ARGUMENT, "logits must hold n_vocab floats");
    BC_TRY(check_trace(s, trace, 1, "the trace must hold one token"));
    if (s->backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;

    BC_CUDA(cudaMemcpyAsync(s->tokens + pos, &token, 4, cudaMemcpyHostToDevice, stream));
    auto encode_start = Clock::now();
    BC_TRY(timing_begin(s));
    Recorder r(*s);
    r.step(pos, logits != nullptr || device_logits, trace != nullptr);
    double encode = since(encode_start);
    double gpu = 0;
    bc_status finish = timing_end(s, &gpu);
    if (r.status != BC_OK) return r.status;
    BC_TRY(finish);
    if (logits) BC_TRY(read_floats(s, s->logits, logits, hp.n_vocab));
    if (trace) {
        BC_TRY(read_floats(s, s->trace_embedding, trace->embedding, hp.n_embd));
        BC_TRY(read_floats(s, s->trace_layers, trace->layers, (size_t)hp.n_layers * hp.n_embd));
        BC_TRY(read_floats(s, s->trace_final, trace->final_norm, hp.n_embd));
    }
    BC_CUDA(cudaStreamSynchronize(stream));
    s->n_past += 1;
    s->last_encode_seconds = encode;
    s->last_gpu_seconds = gpu;
    return BC_OK;
}

}  // namespace

extern "C" {

bc_status bc_seq_prefill(bc_seq* s, const uint32_t* tokens, size_t n_tokens, float* logits, size_t logits_len, float* final_norm,
                         size_t final_norm_len, bc_trace* trace) {
    if (!s || !s->backend || (!tokens && n_tokens)) return fail(BC_ERR_ARGUMENT, "seq and tokens must be non-null and the backend open");
    const bc_hparams& hp = s->hp;
    if (n_tokens > UINT32_MAX) return fail(BC_ERR_ARGUMENT, "too many tokens");
    uint32_t n = (uint32_t)n_tokens, remaining = s->n_ctx - s->n_past;
    if (n == 0) return fail(BC_ERR_ARGUMENT, "the prompt must hold a token");
    if (n > remaining) return fail(BC_ERR_CONTEXT_FULL, "context full: %u tokens requested, %u remaining", n, remaining);
    for (uint32_t i = 0; i < n; ++i)
        if (tokens[i] >= hp.n_vocab) return fail(BC_ERR_TOKEN, "token %u outside the vocabulary of %u", tokens[i], hp.n_vocab);
    if (logits && logits_len != hp.n_vocab) return fail(BC_ERR_ARGUMENT, "logits must hold n_vocab floats");
    if (final_norm && final_norm_len != hp.n_embd) return fail(BC_ERR_ARGUMENT, "final_norm must hold n_embd floats");
    BC_TRY(check_trace(s, trace, n, "the trace must hold every prompt token"));
    if (s->backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;
    const size_t n_embd = hp.n_embd;

    BC_CUDA(cudaMemcpyAsync(s->tokens + s->n_past, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, stream));
    // Qwen's final_norm output comes from the trace buffer of the last batch.
    bool traced = trace != nullptr;
    if (traced || final_norm) BC_TRY(ensure_trace_rows(s, s->batch));

    double encode = 0, gpu = 0;
    BC_TRY(timing_begin(s));
    uint32_t done = 0;
    while (done < n) {
        uint32_t count = std::min(n - done, s->batch);
        uint32_t pos = s->n_past + done;
        bool last = done + count == n;
        auto encode_start = Clock::now();
        Recorder r(*s);
        size_t layer_stride = (size_t)s->trace_rows * n_embd;
        r.batch(pos, count, last, traced || (final_norm && last), layer_stride);
        encode += since(encode_start);
        if (r.status != BC_OK) {
            cudaStreamSynchronize(stream);
            return r.status;
        }
        if (traced) {
            // A traced batch is copied out before the next batch overwrites the trace buffers.
            size_t start = (size_t)done * n_embd, row_floats = (size_t)count * n_embd;
            BC_TRY(read_floats(s, s->trace_embedding, trace->embedding + start, row_floats));
            BC_TRY(read_floats(s, s->trace_final, trace->final_norm + start, row_floats));
            for (uint32_t il = 0; il < hp.n_layers; ++il)
                BC_TRY(read_floats(s, s->trace_layers + il * layer_stride, trace->layers + ((size_t)il * n + done) * n_embd, row_floats));
            BC_CUDA(cudaStreamSynchronize(stream));
        }
        if (final_norm && last) BC_TRY(read_floats(s, s->trace_final + (size_t)(count - 1) * n_embd, final_norm, n_embd));
        done += count;
    }
    BC_TRY(timing_end(s, &gpu));
    if (logits) BC_TRY(read_floats(s, s->logits, logits, hp.n_vocab));
    BC_CUDA(cudaStreamSynchronize(stream));
    s->n_past += n;
    s->last_encode_seconds = encode;
    s->last_gpu_seconds = gpu;
    return BC_OK;
}

bc_status bc_seq_greedy_token(bc_seq* s, uint32_t* token) {
    if (!s || !s->backend || !token) return fail(BC_ERR_ARGUMENT, "seq and token must be non-null and the backend open");
    if (s->n_past == 0) return fail(BC_ERR_ARGUMENT, "generation needs a prompt first");
    if (s->backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(s->backend->activate());
    auto start = Clock::now();
    BC_TRY(timing_begin(s));
    Recorder r(*s);
    r.argmax(s->logits, s->greedy_token, nullptr);
    double encode = since(start), gpu = 0;
    bc_status finish = timing_end(s, &gpu);
    if (r.status != BC_OK) return r.status;
    BC_TRY(finish);
    BC_CUDA(cudaMemcpyAsync(token, s->greedy_token, 4, cudaMemcpyDeviceToHost, s->backend->stream));
    BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    s->last_encode_seconds = encode;
    s->last_gpu_seconds = gpu;
    return BC_OK;
}

bc_status bc_seq_sample(bc_seq* s, const bc_sampling* settings, float uniform, const uint32_t* recent, size_t n_recent, uint32_t* token) {
    if (!s || !s->backend || !settings || !token) return fail(BC_ERR_ARGUMENT, "seq, settings and token must be non-null and the backend open");
    if (!recent && n_recent) return fail(BC_ERR_ARGUMENT, "recent must be non-null");
    if (s->n_past == 0) return fail(BC_ERR_ARGUMENT, "sampling needs a prompt first");
    if (!(uniform >= 0.f && uniform < 1.f)) return fail(BC_ERR_ARGUMENT, "the draw must lie in [0, 1)");
    if (s->backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;
    // Only the window the penalty looks at goes to the device; the token slots past the context's
    // end (unused by a full context's decode) would be too few, so a scratch of the trace buffer serves.
    const size_t window = std::min<size_t>(n_recent, 64);
    uint32_t* device_recent = reinterpret_cast<uint32_t*>(s->trace_final);  // at least n_embd floats, idle outside traced passes
    if (window > s->hp.n_embd) return fail(BC_ERR_ARGUMENT, "the model is narrower than the penalty window");
    if (window) BC_CUDA(cudaMemcpyAsync(device_recent, recent + (n_recent - window), window * 4, cudaMemcpyHostToDevice, stream));
    k::Sampling k_settings{settings->temperature, settings->top_k, settings->top_p, settings->min_p, settings->repeat_penalty};
    Recorder r(*s);
    r.run("sample", 1, s->hp.n_vocab, 0, 1, [&] {
        return k::sample(stream, s->logits, s->hp.n_vocab, window ? device_recent : nullptr, (uint32_t)window, k_settings, uniform, s->greedy_token, nullptr);
    });
    if (r.status != BC_OK) return r.status;
    BC_CUDA(cudaMemcpyAsync(token, s->greedy_token, 4, cudaMemcpyDeviceToHost, stream));
    BC_CUDA(cudaStreamSynchronize(stream));
    return BC_OK;
}

bc_status bc_seq_generate(bc_seq* s, uint32_t* out, size_t n) { return generate_inner(s, out, n, false); }
bc_status bc_seq_generate_next(bc_seq* s, uint32_t* out, size_t n) { return generate_inner(s, out, n, true); }

bc_status bc_seq_generate_stream(bc_seq* s, uint32_t max_tokens, bc_emit_fn emit, void* user, uint32_t* gained, size_t gained_cap,
                                 size_t* n_gained) {
    if (!s || !s->backend || !emit || !n_gained) return fail(BC_ERR_ARGUMENT, "seq, emit and n_gained must be non-null and the backend open");
    *n_gained = 0;
    if (max_tokens == 0) return BC_OK;
    uint32_t first = 0;
    BC_TRY(bc_seq_greedy_token(s, &first));
    if (!emit(first, user)) return BC_OK;
    // Each step runs one token and selects the next, so the first token needs no step.
    uint32_t steps = std::min(max_tokens - 1, s->n_ctx - s->n_past);
    if (gained_cap < steps && !(gained == nullptr && steps == 0))
        if (gained_cap < steps) return fail(BC_ERR_ARGUMENT, "gained must hold %u tokens", steps);
    uint32_t start = s->n_past;
    cudaStream_t stream = s->backend->stream;
    bool emitting = true;
    uint32_t committed = 0;
    bool pending[kGenerateInFlight] = {};
    double encode = 0;
    bc_status result = BC_OK;
    BC_TRY(timing_begin(s));

    auto finish_slot = [&](int slot) -> bc_status {
        cudaError_t e = cudaEventSynchronize(s->slot_done[slot]);
        pending[slot] = false;
        if (e != cudaSuccess) return cuda_fail(e, "generation step");
        if (emitting) emitting = emit(s->readback[slot], user) != 0;
        return BC_OK;
    };
    const bool replay = replay_enabled(s);
    if (replay && steps > 0) {
        Recorder first_pick(*s);
        first_pick.argmax(s->logits, s->tokens + start, nullptr);
        if (first_pick.status != BC_OK) return first_pick.status;
        BC_TRY(prepare_replay(s, /*stream_variant=*/true, start));
    }

    for (uint32_t step = 0; step < steps; ++step) {
        // The slot's previous step selected the token that goes out next. A step at position p
        // uses slot p % kGenerateInFlight, which is also where the replayed argmax writes.
        uint32_t pos = start + step;
        int slot = (int)(pos % kGenerateInFlight);
        if (pending[slot] && (result = finish_slot(slot)) != BC_OK) break;
        if (!emitting) break;
        auto encode_start = Clock::now();
        Recorder r(*s);
        if (replay) {
            cudaError_t ge = cudaGraphLaunch(s->stream_graph, stream);
            if (ge != cudaSuccess) r.status = cuda_fail(ge, "cudaGraphLaunch");
            else s->launches += s->stream_graph_kernels;
        } else {
            if (step == 0) r.argmax(s->logits, s->tokens + pos, nullptr);
            r.step(pos, true, false);
            // tokens has n_ctx + 1 slots, so the pick at the last position has a place to go.
            r.argmax(s->logits, s->tokens + pos + 1, s->readback + slot);
        }
        if (r.status != BC_OK) {
            result = r.status;
            break;
        }
        cudaError_t e = cudaEventRecord(s->slot_done[slot], stream);
        if (e != cudaSuccess) {
            result = cuda_fail(e, "cudaEventRecord");
            break;
        }
        pending[slot] = true;
        ++committed;
        encode += since(encode_start);
    }
    // Finish the steps still in flight in submission order, which is the order of their tokens.
    for (int offset = 0; offset < kGenerateInFlight; ++offset) {
        int slot = (int)((start + committed + offset) % kGenerateInFlight);
        if (!pending[slot]) continue;
        bc_status st = finish_slot(slot);
        if (st != BC_OK && result == BC_OK) result = st;
    }
    double gpu = 0;
    bc_status finish = timing_end(s, &gpu);
    s->n_past += committed;
    s->last_encode_seconds = encode;
    s->last_gpu_seconds = gpu;
    if (result != BC_OK) return result;
    BC_TRY(finish);
    if (committed) {
        BC_CUDA(cudaMemcpyAsync(gained, s->tokens + start, (size_t)committed * 4, cudaMemcpyDeviceToHost, stream));
        BC_CUDA(cudaStreamSynchronize(stream));
    }
    *n_gained = committed;
    return BC_OK;
}

bc_status bc_seq_reset(bc_seq* s) {
    if (!s || !s->backend) return fail(BC_ERR_ARGUMENT, "seq must be non-null and its backend open");
    BC_TRY(s->backend->activate());
    // A new sequence starts from zero convolution history (and zero DeltaNet state). The KV cache
    // needs no clearing, because attention reads only the positions a sequence has written.
    if (s->conv_floats) BC_CUDA(cudaMemsetAsync(s->conv_state, 0, s->conv_floats * 4, s->backend->stream));
    if (s->delta_floats) BC_CUDA(cudaMemsetAsync(s->delta_state, 0, s->delta_floats * 4, s->backend->stream));
    BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    // A sequence that started from a cached prefix shares the prefix's pages; a new sequence
    // writes from position zero again, so it takes pages of its own back first.
    if (s->k_pages && s->shared_positions) {
        const PageGeometry& g = s->k_pages->geometry();
        for (uint32_t slot = 0; slot < g.n_layers * g.pages_per_layer(); ++slot) {
            BC_TRY(s->k_pages->make_private(slot));
            BC_TRY(s->v_pages->make_private(slot));
        }
    }
    s->shared_positions = 0;
    s->n_past = 0;
    s->resets += 1;
    return BC_OK;
}

bc_status bc_seq_checkpoint(bc_seq* s, bc_checkpoint** out) {
    if (!s || !s->backend || !out) return fail(BC_ERR_ARGUMENT, "seq and out must be non-null and the backend open");
    BC_TRY(s->backend->activate());
    std::unique_ptr<bc_checkpoint> c(new bc_checkpoint());
    c->owner = s;
    c->resets = s->resets;
    c->n_past = s->n_past;
    c->conv_state.resize(s->conv_floats);
    c->logits.resize(s->hp.n_vocab);
    cudaStream_t stream = s->backend->stream;
    if (s->conv_floats) BC_CUDA(cudaMemcpyAsync(c->conv_state.data(), s->conv_state, s->conv_floats * 4, cudaMemcpyDeviceToHost, stream));
    c->delta_state.resize(s->delta_floats);
    if (s->delta_floats) BC_CUDA(cudaMemcpyAsync(c->delta_state.data(), s->delta_state, s->delta_floats * 4, cudaMemcpyDeviceToHost, stream));
    BC_CUDA(cudaMemcpyAsync(c->logits.data(), s->logits, c->logits.size() * 4, cudaMemcpyDeviceToHost, stream));
    BC_CUDA(cudaStreamSynchronize(stream));
    *out = c.release();
    return BC_OK;
}

bc_status bc_seq_restore(bc_seq* s, const bc_checkpoint* c) {
    if (!s || !s->backend || !c) return fail(BC_ERR_ARGUMENT, "seq and checkpoint must be non-null and the backend open");
    // A checkpoint holds the recurrent state only; the KV rows of its prefix live in the cache of
    // the sequence that took it, so no other sequence can continue from it.
    if (c->owner != s) return fail(BC_ERR_ARGUMENT, "the checkpoint belongs to another sequence");
    if (c->resets != s->resets) return fail(BC_ERR_ARGUMENT, "the checkpoint predates a reset");
    if (c->n_past < s->shared_positions) return fail(BC_ERR_ARGUMENT, "the checkpoint lies inside the shared prefix of %u positions", s->shared_positions);
    if (c->conv_state.size() != s->conv_floats || c->delta_state.size() != s->delta_floats || c->logits.size() != s->hp.n_vocab || c->n_past > s->n_ctx)
        return fail(BC_ERR_ARGUMENT, "the checkpoint comes from a different model or context");
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;
    if (s->conv_floats) BC_CUDA(cudaMemcpyAsync(s->conv_state, c->conv_state.data(), s->conv_floats * 4, cudaMemcpyHostToDevice, stream));
    if (s->delta_floats) BC_CUDA(cudaMemcpyAsync(s->delta_state, c->delta_state.data(), s->delta_floats * 4, cudaMemcpyHostToDevice, stream));
    BC_CUDA(cudaMemcpyAsync(s->logits, c->logits.data(), c->logits.size() * 4, cudaMemcpyHostToDevice, stream));
    BC_CUDA(cudaStreamSynchronize(stream));
    s->n_past = c->n_past;
    return BC_OK;
}

void bc_checkpoint_free(bc_checkpoint* c) { delete c; }

bc_status bc_seq_prefix_save(bc_seq* s, bc_prefix** out) {
    if (!s || !s->backend || !out) return fail(BC_ERR_ARGUMENT, "seq and out must be non-null and the backend open");
    if (s->n_past == 0) return fail(BC_ERR_ARGUMENT, "a prefix holds at least one token");
    // A tensor-parallel rank saves its own share (its heads' rows and state); every rank does the same.
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;
    const bc_hparams& hp = s->hp;
    std::unique_ptr<bc_prefix> p(new bc_prefix());
    p->model = s->model;
    p->device = s->backend->device;
    p->kv_half = s->kv_half;
    p->hp = hp;
    p->n_past = s->n_past;
    p->conv_floats = s->conv_floats;
    p->delta_floats = s->delta_floats;
    const size_t state_floats = s->conv_floats + s->delta_floats + hp.n_vocab;
    cudaError_t e = cudaMalloc(&p->state, state_floats * 4);
    if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate %zu bytes for the prefix state: %s", state_floats * 4, cudaGetErrorString(e));
    if (s->conv_floats) BC_CUDA(cudaMemcpyAsync(p->state, s->conv_state, s->conv_floats * 4, cudaMemcpyDeviceToDevice, stream));
    if (s->delta_floats) BC_CUDA(cudaMemcpyAsync(p->state + s->conv_floats, s->delta_state, s->delta_floats * 4, cudaMemcpyDeviceToDevice, stream));
    BC_CUDA(cudaMemcpyAsync(p->state + s->conv_floats + s->delta_floats, s->logits, (size_t)hp.n_vocab * 4, cudaMemcpyDeviceToDevice, stream));
    // KV rows: full pages by reference, the rest by copy.
    const size_t kv_dim = (size_t)hp.n_kv_heads * hp.head_dim, element = s->kv_half ? 2 : 4;
    uint32_t first_copied = 0;
    if (s->k_pages) {
        p->paged = true;
        p->geometry = s->k_pages->geometry();
        p->full_pages = s->n_past / p->geometry.page_positions;
        first_copied = p->full_pages * p->geometry.page_positions;
        for (uint32_t layer = 0; layer < hp.n_attention_layers; ++layer)
            for (uint32_t page = 0; page < p->full_pages; ++page) {
                p->k_pages.push_back(s->k_pages->page(layer * p->geometry.pages_per_layer() + page));
                p->v_pages.push_back(s->v_pages->page(layer * p->geometry.pages_per_layer() + page));
            }
        // The source goes on writing past n_past only, which lies beyond the full pages.
        s->shared_positions = std::max(s->shared_positions, first_copied);
    }
    p->tail_rows = s->n_past - first_copied;
    if (p->tail_rows && hp.n_attention_layers) {
        const size_t layer_bytes = (size_t)p->tail_rows * kv_dim * element;
        e = cudaMalloc(&p->tail, 2 * hp.n_attention_layers * layer_bytes);
        if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate the prefix's KV rows: %s", cudaGetErrorString(e));
        for (int which = 0; which < 2; ++which)
            for (uint32_t layer = 0; layer < hp.n_attention_layers; ++layer) {
                const char* cache = static_cast<const char*>(which == 0 ? s->k_cache : s->v_cache);
                const char* src = cache + ((size_t)layer * s->kv_stride + first_copied) * kv_dim * element;
                char* dst = static_cast<char*>(p->tail) + ((size_t)which * hp.n_attention_layers + layer) * layer_bytes;
                BC_CUDA(cudaMemcpyAsync(dst, src, layer_bytes, cudaMemcpyDeviceToDevice, stream));
            }
    }
    BC_CUDA(cudaStreamSynchronize(stream));
    *out = p.release();
    return BC_OK;
}

bc_status bc_seq_prefix_load(bc_seq* s, const bc_prefix* p) {
    if (!s || !s->backend || !p) return fail(BC_ERR_ARGUMENT, "seq and prefix must be non-null and the backend open");
    if (p->hp.n_kv_heads != s->hp.n_kv_heads || p->hp.n_v_heads != s->hp.n_v_heads)
        return fail(BC_ERR_ARGUMENT, "the prefix comes from another tensor-parallel split");
    if (p->model != s->model || p->device != s->backend->device || p->kv_half != s->kv_half || p->conv_floats != s->conv_floats ||
        p->delta_floats != s->delta_floats)
        return fail(BC_ERR_ARGUMENT, "the prefix comes from a different model, device or cache type");
    if (p->n_past > s->n_ctx) return fail(BC_ERR_CONTEXT_FULL, "context full: a prefix of %u tokens, %u positions", p->n_past, s->n_ctx);
    if (s->backend->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    const bc_hparams& hp = s->hp;
    if (p->paged && p->full_pages) {
        if (!s->k_pages) return fail(BC_ERR_ARGUMENT, "a prefix of a paged sequence loads into paged sequences (bc_seq_new_paged)");
        const PageGeometry& g = s->k_pages->geometry();
        if (g.page_positions != p->geometry.page_positions || g.kv_dim != p->geometry.kv_dim || g.element_bytes != p->geometry.element_bytes)
            return fail(BC_ERR_ARGUMENT, "the prefix's pages have another shape");
    }
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;
    // Remapping pages needs the stream idle.
    BC_CUDA(cudaStreamSynchronize(stream));
    const size_t kv_dim = (size_t)hp.n_kv_heads * hp.head_dim, element = s->kv_half ? 2 : 4;
    uint32_t first_copied = 0;
    if (p->paged && p->full_pages) {
        const PageGeometry& g = s->k_pages->geometry();
        for (uint32_t layer = 0; layer < hp.n_attention_layers; ++layer)
            for (uint32_t page = 0; page < p->full_pages; ++page) {
                BC_TRY(s->k_pages->share(layer * g.pages_per_layer() + page, p->k_pages[(size_t)layer * p->full_pages + page]));
                BC_TRY(s->v_pages->share(layer * g.pages_per_layer() + page, p->v_pages[(size_t)layer * p->full_pages + page]));
            }
        first_copied = p->full_pages * g.page_positions;
    }
    // Pages past the shared ones may still be shared from an earlier prefix: this sequence writes there.
    if (s->k_pages) {
        const PageGeometry& g = s->k_pages->geometry();
        const uint32_t shared = p->paged ? p->full_pages : 0;
        for (uint32_t layer = 0; layer < hp.n_attention_layers; ++layer)
            for (uint32_t page = shared; page < g.pages_per_layer(); ++page) {
                BC_TRY(s->k_pages->make_private(layer * g.pages_per_layer() + page));
                BC_TRY(s->v_pages->make_private(layer * g.pages_per_layer() + page));
            }
    }
    if (p->tail_rows && hp.n_attention_layers) {
        const size_t layer_bytes = (size_t)p->tail_rows * kv_dim * element;
        for (int which = 0; which < 2; ++which)
            for (uint32_t layer = 0; layer < hp.n_attention_layers; ++layer) {
                char* cache = static_cast<char*>(which == 0 ? s->k_cache : s->v_cache);
                char* dst = cache + ((size_t)layer * s->kv_stride + first_copied) * kv_dim * element;
                const char* src = static_cast<const char*>(p->tail) + ((size_t)which * hp.n_attention_layers + layer) * layer_bytes;
                BC_CUDA(cudaMemcpyAsync(dst, src, layer_bytes, cudaMemcpyDeviceToDevice, stream));
            }
    }
    if (s->conv_floats) BC_CUDA(cudaMemcpyAsync(s->conv_state, p->state, s->conv_floats * 4, cudaMemcpyDeviceToDevice, stream));
    if (s->delta_floats) BC_CUDA(cudaMemcpyAsync(s->delta_state, p->state + s->conv_floats, s->delta_floats * 4, cudaMemcpyDeviceToDevice, stream));
    BC_CUDA(cudaMemcpyAsync(s->logits, p->state + s->conv_floats + s->delta_floats, (size_t)hp.n_vocab * 4, cudaMemcpyDeviceToDevice, stream));
    BC_CUDA(cudaStreamSynchronize(stream));
    s->shared_positions = first_copied;
    s->n_past = p->n_past;
    return BC_OK;
}

void bc_prefix_free(bc_prefix* p) { delete p; }

uint32_t bc_prefix_n_past(const bc_prefix* p) { return p ? p->n_past : 0; }

bc_status bc_seq_kv_pages(const bc_seq* s, uint32_t* page_positions, uint32_t* pages, uint32_t* shared_pages) {
    if (!s) return fail(BC_ERR_ARGUMENT, "seq must be non-null");
    const bool paged = s->k_pages != nullptr;
    if (page_positions) *page_positions = paged ? s->k_pages->geometry().page_positions : 0;
    if (pages) *pages = paged ? 2 * s->k_pages->geometry().n_layers * s->k_pages->geometry().pages_per_layer() : 0;
    if (shared_pages) *shared_pages = paged ? s->k_pages->shared_pages() + s->v_pages->shared_pages() : 0;
    return BC_OK;
}

bc_status bc_seq_timings(const bc_seq* s, double* encode_seconds, double* gpu_seconds) {
    if (!s || !s->backend) return fail(BC_ERR_ARGUMENT, "seq must be non-null and its backend open");
    if (encode_seconds) *encode_seconds = s->last_encode_seconds;
    if (gpu_seconds) *gpu_seconds = s->last_gpu_seconds;
    return BC_OK;
}

bc_status bc_seq_set_skip(bc_seq* s, const char* name, uint32_t n_rows, uint32_t n_cols) {
    if (!s || !s->backend) return fail(BC_ERR_ARGUMENT, "seq must be non-null and its backend open");
    BC_TRY(s->backend->activate());
    BC_CUDA(cudaStreamSynchronize(s->backend->stream));
    s->skip_name = name ? name : "";
    s->skip_rows = n_rows;
    s->skip_cols = n_cols;
    // The captured steps hold the old launch list.
    if (s->generate_graph) cudaGraphExecDestroy(s->generate_graph);
    if (s->stream_graph) cudaGraphExecDestroy(s->stream_graph);
    s->generate_graph = s->stream_graph = nullptr;
    return BC_OK;
}

bc_status bc_seq_read_state(bc_seq* s, int32_t which, uint32_t layer, float* out, size_t cap, size_t* n) {
    if (!s || !s->backend || !n) return fail(BC_ERR_ARGUMENT, "seq and n must be non-null and the backend open");
    const bc_hparams& hp = s->hp;
    BC_TRY(s->backend->activate());
    cudaStream_t stream = s->backend->stream;
    if (which == 0) {
        *n = s->conv_floats;
        if (!out) return BC_OK;
        if (cap < *n) return fail(BC_ERR_ARGUMENT, "out must hold %zu floats", *n);
        if (*n) BC_CUDA(cudaMemcpyAsync(out, s->conv_state, *n * 4, cudaMemcpyDeviceToHost, stream));
        BC_CUDA(cudaStreamSynchronize(stream));
        return BC_OK;
    }
    if (which == 1 || which == 2) {
        if (layer >= hp.n_attention_layers) return fail(BC_ERR_ARGUMENT, "no attention layer %u", layer);
        size_t count = (size_t)s->n_ctx * hp.n_kv_heads * hp.head_dim, layer_stride = (size_t)s->kv_stride * hp.n_kv_heads * hp.head_dim;
        *n = count;
        if (!out) return BC_OK;
        if (cap < count) return fail(BC_ERR_ARGUMENT, "out must hold %zu floats", count);
        const char* cache = static_cast<const char*>(which == 1 ? s->k_cache : s->v_cache);
        if (s->kv_half) {
            std::vector<uint16_t> halfs(count);
            BC_CUDA(cudaMemcpyAsync(halfs.data(), cache + (size_t)layer * layer_stride * 2, count * 2, cudaMemcpyDeviceToHost, stream));
            BC_CUDA(cudaStreamSynchronize(stream));
            for (size_t i = 0; i < count; ++i) {
                out[i] = __half2float(__half(__half_raw{halfs[i]}));
            }
        } else {
            BC_CUDA(cudaMemcpyAsync(out, cache + (size_t)layer * layer_stride * 4, count * 4, cudaMemcpyDeviceToHost, stream));
            BC_CUDA(cudaStreamSynchronize(stream));
        }
        return BC_OK;
    }
    if (which == 3) {
        if (layer >= hp.n_delta_layers) return fail(BC_ERR_ARGUMENT, "no DeltaNet layer %u", layer);
        size_t count = (size_t)hp.n_v_heads * hp.k_head_dim * hp.v_head_dim;
        *n = count;
        if (!out) return BC_OK;
        if (cap < count) return fail(BC_ERR_ARGUMENT, "out must hold %zu floats", count);
        BC_CUDA(cudaMemcpyAsync(out, s->delta_state + (size_t)layer * count, count * 4, cudaMemcpyDeviceToHost, stream));
        BC_CUDA(cudaStreamSynchronize(stream));
        return BC_OK;
    }
    if (which == 4) {
        // The routes the last traced pass recorded, [layer][trace row][2 * n_used] 32-bit words (ids,
        // then weights as float bits), copied out bit for bit.
        size_t count = (size_t)s->trace_rows * hp.n_layers * 2 * hp.n_experts_used;
        *n = count;
        if (!out) return BC_OK;
        if (cap < count) return fail(BC_ERR_ARGUMENT, "out must hold %zu words", count);
        if (count) BC_CUDA(cudaMemcpyAsync(out, s->trace_routes, count * 4, cudaMemcpyDeviceToHost, stream));
        BC_CUDA(cudaStreamSynchronize(stream));
        return BC_OK;
    }
    return fail(BC_ERR_ARGUMENT, "unknown state %d", which);
}

}  // extern "C"
