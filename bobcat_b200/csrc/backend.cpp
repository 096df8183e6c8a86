// The backend handle: device, stream, buffers, recordings, profiling, and the bounds-checked op
// wrappers. Stands in for `Metal` in crates/bobcat-metal/src/backend.rs.

#include "backend.h"

#include <cstdarg>
#include <cstring>
#include <initializer_list>

namespace bc {

std::string& last_error() {
    static thread_local std::string message;
    return message;
}

bc_status fail(bc_status status, const char* format, ...) {
    char buffer[1024];
    va_list args;
    va_start(args, format);
    vsnprintf(buffer, sizeof buffer, format, args);
    va_end(args);
    last_error() = buffer;
    return status;
}

bc_status cuda_fail(cudaError_t error, const char* what, bc_status status) {
    return fail(status, "CUDA error in %s: %s", what, cudaGetErrorString(error));
}

bc_status check_range(const bc_backend* backend, const bc_buffer* buffer, size_t offset, size_t needed, const char* op) {
    if (!buffer) return fail(BC_ERR_ARGUMENT, "the %s launch got a null buffer", op);
    if (buffer->backend != backend) return fail(BC_ERR_FOREIGN_BUFFER, "the buffer belongs to another backend");
    if (offset > buffer->len || needed > buffer->len - offset)
        return fail(BC_ERR_OUT_OF_BOUNDS, "the %s launch needs %zu bytes at offset %zu of a %zu-byte buffer", op, needed, offset,
                    buffer->len);
    return BC_OK;
}

// A kernel whose bounded wait ran out leaves a flag rather than hanging the device. Reading a flag
// clears it, so one failure is reported once and later healthy work is not blamed for it.
bc_status kernel_wait_status() {
    if (int flag = k::matvec_error_flag()) return fail(BC_ERR_EXECUTION, "a decode kernel gave up waiting for its weight stream or its input (code %d)", flag);
    if (int flag = k::matmul_error_flag()) return fail(BC_ERR_EXECUTION, "a prefill kernel gave up waiting on its pipeline (code %d)", flag);
    if (int flag = k::matmul_few_error_flag()) return fail(BC_ERR_EXECUTION, "a few-token product gave up waiting for its weights (code %d)", flag);
    if (int flag = k::peer_error_flag()) return fail(BC_ERR_EXECUTION, "a sum over ranks gave up waiting for rank %d", flag - 1);
    return BC_OK;
}

}  // namespace bc

// Defined with the sequence (seq.cpp): frees its device state and detaches it from its backend.
void release_seq(bc_seq* seq);

using namespace bc;

bc_status bc_backend::activate() {
    BC_CUDA(cudaSetDevice(device));
    return BC_OK;
}

bc_status bc_backend::pack_scratch(size_t bytes, void** out) {
    if (bytes > pack_len) {
        // Launches that read the old scratch may still be queued: drain the stream before freeing it.
        BC_CUDA(cudaStreamSynchronize(stream));
        if (pack) cudaFree(pack);
        pack = nullptr;
        pack_len = 0;
        size_t want = bytes + bytes / 2;
        BC_CUDA(cudaMalloc(&pack, want));
        pack_len = want;
    }
    *out = pack;
    return BC_OK;
}

bc_status bc_backend::partial_scratch(size_t bytes, void** out) {
    if (bytes > partials_len) {
        BC_CUDA(cudaStreamSynchronize(stream));
        if (partials) cudaFree(partials);
        partials = nullptr;
        partials_len = 0;
        size_t want = bytes + bytes / 2;
        BC_CUDA(cudaMalloc(&partials, want));
        partials_len = want;
    }
    *out = partials;
    return BC_OK;
}

namespace {

bc_status need_recording(bc_backend* b) {
    if (!b) return fail(BC_ERR_ARGUMENT, "backend must be non-null");
    if (!b->recording) return fail(BC_ERR_NOT_RECORDING, "no recording is open");
    return b->activate();
}

char* at(bc_buffer* buffer, size_t offset) { return static_cast<char*>(buffer->ptr) + offset; }

// The matrix a (buffer, GGUF byte offset) view names: whole rows from the offset's row onward.
bc_status matrix_view(bc_backend* b, bc_buffer* buffer, size_t offset, int32_t format, uint32_t n_rows, uint32_t n_cols,
                      const char* op, k::Mat* out) {
    if (!buffer) return fail(BC_ERR_ARGUMENT, "the %s launch got a null buffer", op);
    if (buffer->backend != b) return fail(BC_ERR_FOREIGN_BUFFER, "the buffer belongs to another backend");
    if (!buffer->is_matrix) return fail(BC_ERR_ARGUMENT, "the %s launch needs weights from bc_matrix_upload", op);
    const k::Mat& m = buffer->matrix;
    if (m.format != format || m.n_cols != n_cols) return fail(BC_ERR_ARGUMENT, "the %s launch names a different format or width than the upload", op);
    uint64_t row_bytes = type_row_bytes((uint32_t)format, n_cols);
    if (row_bytes == 0 || offset % row_bytes != 0) return fail(BC_ERR_ARGUMENT, "the %s weight offset must be a whole number of rows", op);
    uint64_t first = offset / row_bytes;
    if (first > m.n_rows || n_rows > m.n_rows - first)
        return fail(BC_ERR_OUT_OF_BOUNDS, "the %s launch needs %llu bytes at offset %zu of a %llu-byte matrix", op,
                    (unsigned long long)(n_rows * row_bytes), offset, (unsigned long long)(m.n_rows * row_bytes));
    *out = m.rows((uint32_t)first, n_rows);
    return BC_OK;
}

// The vectorised kernels read activations 16 bytes at a time: views of activation vectors must
// start on a 16-byte boundary (cudaMalloc bases are 256-byte aligned, so only the offset matters).
// Checked before any launch, because a misaligned vector load is a device fault, not a status code.
bc_status check_aligned(const char* op, std::initializer_list<size_t> offsets) {
    for (size_t offset : offsets)
        if (offset % 16 != 0) return fail(BC_ERR_ARGUMENT, "the %s launch needs 16-byte aligned activation offsets, got %zu", op, offset);
    return BC_OK;
}

bool known_format(int32_t format) { return format == BC_F32 || format == BC_F16 || format == BC_Q4_0 || format == BC_Q8_0 || format == BC_Q6_K; }

}  // namespace

extern "C" {

const char* bc_last_error(void) { return last_error().c_str(); }
const char* bc_version(void) { return "bobcat-cuda 0.1 (sm_100a)"; }

bc_status bc_backend_open(int32_t device, void* stream, bc_backend** out) {
    if (!out) return fail(BC_ERR_ARGUMENT, "out must be non-null");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) return fail(BC_ERR_NO_DEVICE, "no CUDA device: %s", e == cudaSuccess ? "none visible" : cudaGetErrorString(e));
    if (device < 0 || device >= count) return fail(BC_ERR_NO_DEVICE, "no CUDA device %d (of %d)", device, count);
    std::unique_ptr<bc_backend> b(new bc_backend());
    b->device = device;
    BC_TRY(b->activate());
    if (stream) {
        b->stream = static_cast<cudaStream_t>(stream);
    } else {
        BC_CUDA(cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking));
        b->owns_stream = true;
    }
    *out = b.release();
    return BC_OK;
}

void bc_backend_close(bc_backend* b) {
    if (!b) return;
    cudaSetDevice(b->device);
    cudaStreamSynchronize(b->stream);
    // Sequences that outlive their backend give up their device state now and stay behind as
    // handles that only bc_seq_free may still be called on.
    while (!b->seqs.empty()) release_seq(*b->seqs.begin());
    for (auto& t : b->tickets) cudaEventDestroy(t.second);
    for (auto& t : b->ticket_starts) cudaEventDestroy(t.second);
    if (b->record_start) cudaEventDestroy(b->record_start);
    // Buffers that outlive their backend are orphaned; their frees become no-ops on the pointer.
    for (bc_buffer* buffer : b->buffers) {
        cudaFree(buffer->ptr);
        buffer->ptr = nullptr;
        buffer->backend = nullptr;
    }
    if (b->pack) cudaFree(b->pack);
    if (b->partials) cudaFree(b->partials);
    if (b->owns_stream) cudaStreamDestroy(b->stream);
    delete b;
}

void* bc_backend_stream(bc_backend* b) { return b ? b->stream : nullptr; }

bc_status bc_buffer_new(bc_backend* b, size_t len, bc_buffer** out) {
    if (!b || !out) return fail(BC_ERR_ARGUMENT, "backend and out must be non-null");
    BC_TRY(b->activate());
    std::unique_ptr<bc_buffer> buffer(new bc_buffer());
    buffer->backend = b;
    buffer->len = len;
    if (len) {
        cudaError_t e = cudaMalloc(&buffer->ptr, len);
        if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate a device buffer of %zu bytes: %s", len, cudaGetErrorString(e));
        e = cudaMemsetAsync(buffer->ptr, 0, len, b->stream);
        if (e != cudaSuccess) {
            cudaFree(buffer->ptr);
            return cuda_fail(e, "cudaMemsetAsync");
        }
    }
    b->buffers.insert(buffer.get());
    *out = buffer.release();
    return BC_OK;
}

void bc_buffer_free(bc_buffer* buffer) {
    if (!buffer) return;
    if (buffer->backend) {
        cudaSetDevice(buffer->backend->device);
        // Work that reads the buffer may still be queued; the reference keeps a dropped buffer alive
        // until its command buffers complete (crates/bobcat/tests/metal_commands.rs).
        cudaStreamSynchronize(buffer->backend->stream);
        buffer->backend->buffers.erase(buffer);
        cudaFree(buffer->ptr);
    }
    delete buffer;
}

size_t bc_buffer_len(const bc_buffer* buffer) { return buffer ? buffer->len : 0; }
void* bc_buffer_device_ptr(bc_buffer* buffer) { return buffer ? buffer->ptr : nullptr; }

bc_status bc_buffer_write(bc_buffer* buffer, size_t offset, const void* data, size_t len) {
    if (!buffer || !buffer->backend || (!data && len)) return fail(BC_ERR_ARGUMENT, "buffer and data must be non-null");
    bc_backend* b = buffer->backend;
    if (b->recording) return fail(BC_ERR_BUSY, "the CPU cannot access a buffer while a recording is open");
    if (offset > buffer->len || len > buffer->len - offset)
        return fail(BC_ERR_OUT_OF_BOUNDS, "CPU access of %zu bytes at offset %zu exceeds a %zu-byte buffer", len, offset, buffer->len);
    if (!len) return BC_OK;
    BC_TRY(b->activate());
    BC_CUDA(cudaMemcpyAsync(at(buffer, offset), data, len, cudaMemcpyHostToDevice, b->stream));
    BC_CUDA(cudaStreamSynchronize(b->stream));
    return BC_OK;
}

bc_status bc_buffer_read(bc_buffer* buffer, size_t offset, void* out, size_t len) {
    if (!buffer || !buffer->backend || (!out && len)) return fail(BC_ERR_ARGUMENT, "buffer and out must be non-null");
    bc_backend* b = buffer->backend;
    if (b->recording) return fail(BC_ERR_BUSY, "the CPU cannot access a buffer while a recording is open");
    if (offset > buffer->len || len > buffer->len - offset)
        return fail(BC_ERR_OUT_OF_BOUNDS, "CPU access of %zu bytes at offset %zu exceeds a %zu-byte buffer", len, offset, buffer->len);
    if (!len) return BC_OK;
    BC_TRY(b->activate());
    BC_CUDA(cudaMemcpyAsync(out, at(buffer, offset), len, cudaMemcpyDeviceToHost, b->stream));
    BC_CUDA(cudaStreamSynchronize(b->stream));
    return BC_OK;
}

bc_status bc_matrix_upload(bc_backend* b, int32_t format, const void* data, uint32_t n_rows, uint32_t n_cols, bc_buffer** out) {
    if (!b || !data || !out) return fail(BC_ERR_ARGUMENT, "backend, data and out must be non-null");
    if (!known_format(format)) return fail(BC_ERR_UNSUPPORTED, "matrices in format %d", format);
    if (n_rows == 0 || n_cols == 0 || n_cols % 32 != 0) return fail(BC_ERR_ARGUMENT, "a matrix has rows of a multiple of 32 columns");
    if (format == BC_Q6_K && n_cols % 256 != 0) return fail(BC_ERR_ARGUMENT, "Q6_K rows hold whole super-blocks of 256");
    BC_TRY(b->activate());
    uint64_t raw_bytes = (uint64_t)n_rows * type_row_bytes((uint32_t)format, n_cols);
    // Q4_0 matrices also get the tile layout of the tensor-core decode kernel, after the split one.
    const bool tiled = format == BC_Q4_0 && k::tiles_supported(n_cols);
    const uint64_t split_bytes = round_up(raw_bytes, 256);
    bc_buffer* buffer = nullptr;
    BC_TRY(bc_buffer_new(b, tiled ? split_bytes + k::tiles_bytes(n_rows, n_cols) : raw_bytes, &buffer));
    buffer->is_matrix = true;
    buffer->matrix.format = format;
    buffer->matrix.n_rows = n_rows;
    buffer->matrix.n_cols = n_cols;
    buffer->matrix.data = buffer->ptr;
    bc_status status = BC_OK;
    if (format == BC_Q4_0) {
        uint64_t n_blocks = (uint64_t)n_rows * (n_cols / 32);
        buffer->matrix.scales = reinterpret_cast<const __half*>(static_cast<char*>(buffer->ptr) + n_blocks * 16);
        void* raw = nullptr;
        cudaError_t e = cudaMalloc(&raw, raw_bytes);
        if (e != cudaSuccess) status = fail(BC_ERR_ALLOCATION, "cannot allocate %llu staging bytes", (unsigned long long)raw_bytes);
        if (status == BC_OK && (e = cudaMemcpyAsync(raw, data, raw_bytes, cudaMemcpyHostToDevice, b->stream)) != cudaSuccess) status = cuda_fail(e, "upload");
        if (status == BC_OK && (e = k::repack_q4_0(b->stream, static_cast<const uint8_t*>(raw), n_blocks, buffer->ptr,
                                                    const_cast<__half*>(buffer->matrix.scales))) != cudaSuccess)
            status = cuda_fail(e, "repack_q4_0");
        if (status == BC_OK && tiled) {
            buffer->matrix.tiles = static_cast<char*>(buffer->ptr) + split_bytes;
            if ((e = k::repack_tiles(b->stream, buffer->ptr, buffer->matrix.scales, n_rows, n_cols, const_cast<void*>(buffer->matrix.tiles))) != cudaSuccess)
                status = cuda_fail(e, "repack_tiles");
        }
        if (status == BC_OK && (e = cudaStreamSynchronize(b->stream)) != cudaSuccess) status = cuda_fail(e, "repack_q4_0");
        if (raw) cudaFree(raw);
    } else {
        cudaError_t e = cudaMemcpyAsync(buffer->ptr, data, raw_bytes, cudaMemcpyHostToDevice, b->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(b->stream);
        if (e != cudaSuccess) status = cuda_fail(e, "upload");
    }
    if (status != BC_OK) {
        bc_buffer_free(buffer);
        return status;
    }
    *out = buffer;
    return BC_OK;
}

bc_status bc_begin(bc_backend* b) {
    if (!b) return fail(BC_ERR_ARGUMENT, "backend must be non-null");
    if (b->recording) return fail(BC_ERR_ALREADY_RECORDING, "a recording is already open");
    BC_TRY(b->activate());
    if (!b->record_start) BC_CUDA(cudaEventCreate(&b->record_start));
    cudaEvent_t start;
    BC_CUDA(cudaEventCreate(&start));
    BC_CUDA(cudaEventRecord(start, b->stream));
    b->ticket_starts[b->next_ticket] = start;
    b->recording = true;
    return BC_OK;
}

bc_status bc_barrier(bc_backend* b) {
    if (!b) return fail(BC_ERR_ARGUMENT, "backend must be non-null");
    if (!b->recording) return fail(BC_ERR_NOT_RECORDING, "no recording is open");
    return BC_OK;  // launches on one stream already run in order
}

bc_status bc_commit(bc_backend* b, bc_ticket* ticket) {
    BC_TRY(need_recording(b));
    cudaEvent_t end;
    BC_CUDA(cudaEventCreate(&end));
    BC_CUDA(cudaEventRecord(end, b->stream));
    uint64_t id = b->next_ticket++;
    b->tickets[id] = end;
    b->recording = false;
    if (ticket) *ticket = id;
    return BC_OK;
}

bc_status bc_wait(bc_backend* b, bc_ticket ticket, double* seconds) {
    if (!b) return fail(BC_ERR_ARGUMENT, "backend must be non-null");
    BC_TRY(b->activate());
    auto end = b->tickets.find(ticket);
    if (end == b->tickets.end()) {
        // Completed and collected earlier, or never issued.
        if (ticket == 0 || ticket >= b->next_ticket) return fail(BC_ERR_ARGUMENT, "unknown ticket");
        if (seconds) *seconds = 0.0;
        return BC_OK;
    }
    cudaError_t e = cudaEventSynchronize(end->second);
    if (e != cudaSuccess) return cuda_fail(e, "recorded work");
    float ms = 0.f;
    auto start = b->ticket_starts.find(ticket);
    if (start != b->ticket_starts.end()) {
        cudaEventElapsedTime(&ms, start->second, end->second);
        cudaEventDestroy(start->second);
        b->ticket_starts.erase(start);
    }
    cudaEventDestroy(end->second);
    b->tickets.erase(end);
    if (seconds) *seconds = ms * 1e-3;
    return kernel_wait_status();
}

bc_status bc_end(bc_backend* b, double* seconds) {
    bc_ticket ticket = 0;
    BC_TRY(bc_commit(b, &ticket));
    return bc_wait(b, ticket, seconds);
}

void bc_discard(bc_backend* b) {
    if (!b || !b->recording) return;
    // Launches already queued cannot be recalled from a stream; let them drain, then close.
    cudaSetDevice(b->device);
    cudaStreamSynchronize(b->stream);
    auto start = b->ticket_starts.find(b->next_ticket);
    if (start != b->ticket_starts.end()) {
        cudaEventDestroy(start->second);
        b->ticket_starts.erase(start);
    }
    b->recording = false;
}

bc_status bc_set_profiling(bc_backend* b, int32_t enabled) {
    if (!b) return fail(BC_ERR_ARGUMENT, "backend must be non-null");
    b->profiling = enabled != 0;
    if (enabled) b->profile.clear();
    return BC_OK;
}

bc_status bc_profile(bc_backend* b, bc_profile_entry* out, size_t capacity, size_t* count) {
    if (!b || !count) return fail(BC_ERR_ARGUMENT, "backend and count must be non-null");
    *count = b->profile.size();
    b->profile_names.clear();
    b->profile_names.reserve(b->profile.size());
    size_t i = 0;
    for (auto& entry : b->profile) {
        if (i >= capacity || !out) break;
        b->profile_names.push_back(entry.first.name);
        out[i] = bc_profile_entry{b->profile_names.back().c_str(), entry.first.n_rows, entry.first.n_cols, entry.second.calls,
                                  entry.second.seconds, entry.second.bytes};
        ++i;
    }
    return BC_OK;
}

// ------------------------------------------------------------------------------------------ ops

bc_status bc_op_matvec(bc_backend* b, int32_t format, bc_buffer* weights, size_t w_off, uint32_t n_rows, uint32_t n_cols,
                       bc_buffer* x, size_t x_off, bc_buffer* y, size_t y_off, bc_buffer* norm, size_t norm_off, float eps,
                       int32_t accumulate) {
    BC_TRY(need_recording(b));
    k::MatvecSegment seg;
    BC_TRY(matrix_view(b, weights, w_off, format, n_rows, n_cols, "matvec", &seg.w));
    BC_TRY(check_range(b, x, x_off, (size_t)n_cols * 4, "matvec"));
    BC_TRY(check_range(b, y, y_off, (size_t)n_rows * 4, "matvec"));
    BC_TRY(check_aligned("matvec", {x_off, y_off, norm ? norm_off : 0}));
    k::Norm nm;
    if (norm) {
        BC_TRY(check_range(b, norm, norm_off, (size_t)n_cols * 4, "matvec"));
        nm.weight = reinterpret_cast<const float*>(at(norm, norm_off));
        nm.eps = eps;
    }
    seg.y = reinterpret_cast<float*>(at(y, y_off));
    const float* xp = reinterpret_cast<const float*>(at(x, x_off));
    return b->run("matvec", n_rows, n_cols, seg.w.bytes(), 1,
                  [&] { return k::matvec(b->stream, &seg, 1, xp, nm, accumulate != 0); });
}

bc_status bc_op_matvec_swiglu(bc_backend* b, int32_t format, bc_buffer* gate, size_t gate_off, bc_buffer* up, size_t up_off,
                              uint32_t n_rows, uint32_t n_cols, bc_buffer* x, size_t x_off, bc_buffer* norm, size_t norm_off,
                              float eps, bc_buffer* y, size_t y_off) {
    BC_TRY(need_recording(b));
    k::Mat g, u;
    BC_TRY(matrix_view(b, gate, gate_off, format, n_rows, n_cols, "matvec_swiglu", &g));
    BC_TRY(matrix_view(b, up, up_off, format, n_rows, n_cols, "matvec_swiglu", &u));
    BC_TRY(check_range(b, x, x_off, (size_t)n_cols * 4, "matvec_swiglu"));
    BC_TRY(check_range(b, y, y_off, (size_t)n_rows * 4, "matvec_swiglu"));
    if (!norm) return fail(BC_ERR_ARGUMENT, "matvec_swiglu needs a norm");
    BC_TRY(check_range(b, norm, norm_off, (size_t)n_cols * 4, "matvec_swiglu"));
    BC_TRY(check_aligned("matvec_swiglu", {x_off, y_off, norm_off}));
    k::Norm nm{reinterpret_cast<const float*>(at(norm, norm_off)), eps};
    return b->run("matvec_swiglu", n_rows, n_cols, g.bytes() * 2, 1, [&] {
        return k::matvec_swiglu(b->stream, g, u, reinterpret_cast<const float*>(at(x, x_off)), nm, reinterpret_cast<float*>(at(y, y_off)));
    });
}

bc_status bc_op_matvec_conv(bc_backend* b, int32_t format, bc_buffer* in_proj, size_t w_off, uint32_t n_cols, bc_buffer* x,
                            size_t x_off, bc_buffer* norm, size_t norm_off, float eps, bc_buffer* taps, size_t taps_off,
                            bc_buffer* history, size_t hist_off, bc_buffer* out, size_t out_off, uint32_t n_embd, uint32_t kernel) {
    BC_TRY(need_recording(b));
    if (kernel < 2 || kernel > 9) return fail(BC_ERR_UNSUPPORTED, "a convolution of 2 to 9 taps, got %u", kernel);
    k::Mat w;
    BC_TRY(matrix_view(b, in_proj, w_off, format, 3 * n_embd, n_cols, "matvec_conv", &w));
    BC_TRY(check_range(b, x, x_off, (size_t)n_cols * 4, "matvec_conv"));
    BC_TRY(check_range(b, taps, taps_off, (size_t)n_embd * kernel * 4, "matvec_conv"));
    BC_TRY(check_range(b, history, hist_off, (size_t)n_embd * (kernel - 1) * 4, "matvec_conv"));
    BC_TRY(check_range(b, out, out_off, (size_t)n_embd * 4, "matvec_conv"));
    BC_TRY(check_aligned("matvec_conv", {x_off, out_off, norm ? norm_off : 0}));
    k::Norm nm;
    if (norm) {
        BC_TRY(check_range(b, norm, norm_off, (size_t)n_cols * 4, "matvec_conv"));
        nm = k::Norm{reinterpret_cast<const float*>(at(norm, norm_off)), eps};
    }
    return b->run("matvec_conv", 3 * n_embd, n_cols, w.bytes(), 1, [&] {
        return k::matvec_conv(b->stream, w, reinterpret_cast<const float*>(at(x, x_off)), nm,
                              reinterpret_cast<const float*>(at(taps, taps_off)), reinterpret_cast<float*>(at(history, hist_off)),
                              reinterpret_cast<float*>(at(out, out_off)), n_embd, kernel);
    });
}

bc_status bc_op_short_conv(bc_backend* b, bc_buffer* bcx, size_t bcx_off, bc_buffer* taps, size_t taps_off, bc_buffer* history,
                           size_t hist_off, bc_buffer* out, size_t out_off, uint32_t n_embd, uint32_t kernel, uint32_t n_tokens) {
    BC_TRY(need_recording(b));
    if (kernel < 2 || kernel > 9) return fail(BC_ERR_UNSUPPORTED, "a convolution of 2 to 9 taps, got %u", kernel);
    BC_TRY(check_range(b, bcx, bcx_off, (size_t)n_tokens * 3 * n_embd * 4, "short_conv"));
    BC_TRY(check_range(b, taps, taps_off, (size_t)n_embd * kernel * 4, "short_conv"));
    BC_TRY(check_range(b, history, hist_off, (size_t)n_embd * (kernel - 1) * 4, "short_conv"));
    BC_TRY(check_range(b, out, out_off, (size_t)n_tokens * n_embd * 4, "short_conv"));
    return b->run("short_conv", n_tokens, n_embd, 0, 2, [&] {
        return k::short_conv(b->stream, reinterpret_cast<const float*>(at(bcx, bcx_off)), reinterpret_cast<const float*>(at(taps, taps_off)),
                             reinterpret_cast<float*>(at(history, hist_off)), reinterpret_cast<float*>(at(out, out_off)), n_embd, kernel,
                             n_tokens);
    });
}

bc_status bc_op_matmul(bc_backend* b, int32_t format, bc_buffer* weights, size_t w_off, uint32_t n_rows, uint32_t n_cols,
                       bc_buffer* x, size_t x_off, bc_buffer* y, size_t y_off, uint32_t n_tokens, int32_t store) {
    BC_TRY(need_recording(b));
    if (store < BC_STORE_OVERWRITE || store > BC_STORE_SWIGLU) return fail(BC_ERR_ARGUMENT, "unknown store mode %d", store);
    k::Mat w;
    BC_TRY(matrix_view(b, weights, w_off, format, n_rows, n_cols, "matmul", &w));
    BC_TRY(check_range(b, x, x_off, (size_t)n_tokens * n_cols * 4, "matmul"));
    BC_TRY(check_range(b, y, y_off, (size_t)n_tokens * n_rows * 4, "matmul"));
    BC_TRY(check_aligned("matmul", {x_off, y_off}));
    void* pack = nullptr;
    if (k::matmul_umma_supported(w, n_tokens)) BC_TRY(b->pack_scratch(k::matmul_scratch_bytes(w, n_tokens), &pack));
    return b->run("matmul", n_rows, n_cols, w.bytes(), pack ? k::matmul_umma_launches(w, n_tokens) : 1, [&] {
        return k::matmul(b->stream, w, reinterpret_cast<const float*>(at(x, x_off)), reinterpret_cast<float*>(at(y, y_off)), n_tokens,
                         n_rows, store, pack);
    });
}

bc_status bc_op_expand(bc_backend* b, int32_t format, bc_buffer* weights, size_t w_off, bc_buffer* out, size_t out_off,
                       uint32_t n_rows, uint32_t n_cols, int32_t out_half) {
    BC_TRY(need_recording(b));
    k::Mat w;
    BC_TRY(matrix_view(b, weights, w_off, format, n_rows, n_cols, "expand", &w));
    BC_TRY(check_range(b, out, out_off, (size_t)n_rows * n_cols * (out_half ? 2 : 4), "expand"));
    return b->run("expand", n_rows, n_cols, w.bytes(), 1, [&] { return k::expand(b->stream, w, at(out, out_off), out_half != 0); });
}

bc_status bc_op_embed(bc_backend* b, int32_t format, bc_buffer* weights, size_t w_off, uint32_t n_vocab, bc_buffer* tokens,
                      size_t tok_off, bc_buffer* out, size_t out_off, uint32_t n_embd, uint32_t n_tokens) {
    BC_TRY(need_recording(b));
    k::Mat w;
    BC_TRY(matrix_view(b, weights, w_off, format, n_vocab, n_embd, "embed", &w));
    BC_TRY(check_range(b, tokens, tok_off, (size_t)n_tokens * 4, "embed"));
    BC_TRY(check_range(b, out, out_off, (size_t)n_tokens * n_embd * 4, "embed"));
    return b->run("embed", n_tokens, n_embd, 0, 1, [&] {
        return k::embed(b->stream, w, reinterpret_cast<const uint32_t*>(at(tokens, tok_off)), k::Pos{}, reinterpret_cast<float*>(at(out, out_off)),
                        n_tokens);
    });
}

bc_status bc_op_rms_norm(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* weight, size_t w_off, bc_buffer* out, size_t out_off,
                         uint32_t n_cols, uint32_t n_rows, float eps) {
    BC_TRY(need_recording(b));
    BC_TRY(check_range(b, x, x_off, (size_t)n_rows * n_cols * 4, "rms_norm"));
    BC_TRY(check_range(b, weight, w_off, (size_t)n_cols * 4, "rms_norm"));
    BC_TRY(check_range(b, out, out_off, (size_t)n_rows * n_cols * 4, "rms_norm"));
    return b->run("rms_norm", n_rows, n_cols, 0, 1, [&] {
        return k::rms_norm(b->stream, reinterpret_cast<const float*>(at(x, x_off)), reinterpret_cast<const float*>(at(weight, w_off)),
                           reinterpret_cast<float*>(at(out, out_off)), n_cols, n_rows, eps);
    });
}

bc_status bc_op_norm_rope(bc_backend* b, bc_buffer* src, size_t src_off, bc_buffer* dst, size_t dst_off, int32_t dst_half,
                          bc_buffer* weight, size_t w_off, uint32_t n_heads, uint32_t head_dim, uint32_t head_stride, uint32_t n_rot,
                          uint32_t first_pos, uint32_t n_tokens, uint32_t src_stride, uint32_t dst_stride, float theta, float eps) {
    BC_TRY(need_recording(b));
    if (head_dim == 0 || head_dim % 32 != 0 || head_dim > 256 || n_rot % 2 != 0 || n_rot > head_dim || n_heads == 0)
        return fail(BC_ERR_ATTENTION_LIMITS, "norm_rope needs heads of a multiple of 32 up to 256 elements and an even rotation, got %u and %u",
                    head_dim, n_rot);
    if (n_tokens == 0) return BC_OK;
    size_t src_need = ((size_t)(n_tokens - 1) * src_stride + (size_t)(n_heads - 1) * head_stride + head_dim) * 4;
    size_t dst_need = ((size_t)(n_tokens - 1) * dst_stride + (size_t)n_heads * head_dim) * (dst_half ? 2 : 4);
    BC_TRY(check_range(b, src, src_off, src_need, "norm_rope"));
    BC_TRY(check_range(b, dst, dst_off, dst_need, "norm_rope"));
    BC_TRY(check_range(b, weight, w_off, (size_t)head_dim * 4, "norm_rope"));
    return b->run("norm_rope", n_heads * n_tokens, head_dim, 0, 1, [&] {
        return k::norm_rope(b->stream, reinterpret_cast<const float*>(at(src, src_off)), at(dst, dst_off), dst_half != 0,
                            reinterpret_cast<const float*>(at(weight, w_off)), n_heads, head_dim, head_stride, n_rot, first_pos, n_tokens,
                            src_stride, dst_stride, theta, eps);
    });
}

bc_status bc_op_convert_half(bc_backend* b, bc_buffer* src, size_t src_off, bc_buffer* dst, size_t dst_off, uint32_t n) {
    BC_TRY(need_recording(b));
    BC_TRY(check_range(b, src, src_off, (size_t)n * 4, "convert_half"));
    BC_TRY(check_range(b, dst, dst_off, (size_t)n * 2, "convert_half"));
    return b->run("convert_half", 1, n, 0, 1, [&] {
        return k::convert_half(b->stream, reinterpret_cast<const float*>(at(src, src_off)), reinterpret_cast<__half*>(at(dst, dst_off)), n);
    });
}

bc_status bc_op_copy(bc_backend* b, bc_buffer* src, size_t src_off, bc_buffer* dst, size_t dst_off, uint32_t n) {
    BC_TRY(need_recording(b));
    BC_TRY(check_range(b, src, src_off, (size_t)n * 4, "copy"));
    BC_TRY(check_range(b, dst, dst_off, (size_t)n * 4, "copy"));
    return b->run("copy", 1, n, 0, 0, [&] {
        return k::copy_floats(b->stream, reinterpret_cast<const float*>(at(src, src_off)), reinterpret_cast<float*>(at(dst, dst_off)), n);
    });
}

size_t bc_attention_scratch_floats(uint32_t n_heads, uint32_t head_dim, uint32_t n_ctx, uint32_t n_queries) {
    return (size_t)k::attention_scratch_floats(n_heads, head_dim, n_ctx, n_queries);
}

bc_status bc_op_attention(bc_backend* b, bc_buffer* q, size_t q_off, bc_buffer* k_cache, size_t k_off, bc_buffer* v_cache, size_t v_off,
                          int32_t kv_half, bc_buffer* scratch, size_t s_off, bc_buffer* out, size_t out_off, uint32_t n_heads,
                          uint32_t n_kv_heads, uint32_t head_dim, uint32_t first_pos, uint32_t n_queries, uint32_t n_ctx) {
    BC_TRY(need_recording(b));
    if (n_kv_heads == 0 || n_heads % n_kv_heads != 0 || n_heads / n_kv_heads > 8 || head_dim == 0 || head_dim % 32 != 0 || head_dim > 256 ||
        n_queries == 0 || (uint64_t)first_pos + n_queries > n_ctx)
        return fail(BC_ERR_ATTENTION_LIMITS,
                    "attention needs heads of a multiple of 32 up to 256 elements, at most 8 query heads per KV head and queries inside the "
                    "context, got head_dim %u, %u/%u heads, positions %u..%u of %u",
                    head_dim, n_heads, n_kv_heads, first_pos, first_pos + n_queries, n_ctx);
    size_t kv_bytes = (size_t)(first_pos + n_queries) * n_kv_heads * head_dim * (kv_half ? 2 : 4);
    BC_TRY(check_range(b, q, q_off, (size_t)n_queries * n_heads * head_dim * 4, "attention"));
    BC_TRY(check_range(b, k_cache, k_off, kv_bytes, "attention"));
    BC_TRY(check_range(b, v_cache, v_off, kv_bytes, "attention"));
    BC_TRY(check_range(b, scratch, s_off, bc_attention_scratch_floats(n_heads, head_dim, n_ctx, n_queries) * 4, "attention"));
    BC_TRY(check_range(b, out, out_off, (size_t)n_queries * n_heads * head_dim * 4, "attention"));
    k::AttentionShape shape{n_heads, n_kv_heads, head_dim, first_pos, n_queries, n_ctx, n_heads * head_dim, head_dim};
    int launches = k::attention_launches(kv_half != 0, shape);
    return b->run("attention", n_queries, first_pos + n_queries, kv_bytes * 2, launches, [&] {
        return k::attention(b->stream, reinterpret_cast<const float*>(at(q, q_off)), at(k_cache, k_off), at(v_cache, v_off), kv_half != 0,
                            reinterpret_cast<float*>(at(scratch, s_off)), reinterpret_cast<float*>(at(out, out_off)), shape);
    });
}

bc_status bc_op_argmax(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* out, size_t out_off, uint32_t n) {
    BC_TRY(need_recording(b));
    if (n == 0) return fail(BC_ERR_ARGUMENT, "argmax needs at least one value");
    BC_TRY(check_range(b, x, x_off, (size_t)n * 4, "argmax"));
    BC_TRY(check_range(b, out, out_off, 4, "argmax"));
    return b->run("argmax", 1, n, 0, 1, [&] {
        return k::argmax(b->stream, reinterpret_cast<const float*>(at(x, x_off)), n, reinterpret_cast<uint32_t*>(at(out, out_off)), nullptr);
    });
}

bc_status bc_op_sample(bc_backend* b, bc_buffer* logits, size_t logits_off, uint32_t n, bc_buffer* recent, size_t recent_off, uint32_t n_recent,
                       const bc_sampling* settings, float uniform, bc_buffer* out, size_t out_off) {
    BC_TRY(need_recording(b));
    if (!settings) return fail(BC_ERR_ARGUMENT, "settings must be non-null");
    if (n == 0) return fail(BC_ERR_ARGUMENT, "sampling needs at least one logit");
    if (!(uniform >= 0.f && uniform < 1.f)) return fail(BC_ERR_ARGUMENT, "the draw must lie in [0, 1)");
    if (settings->temperature > 0.f && (!(settings->top_p > 0.f) || settings->min_p < 0.f || settings->min_p > 1.f || !(settings->repeat_penalty > 0.f)))
        return fail(BC_ERR_ARGUMENT, "top_p must be positive, min_p in [0, 1] and the repetition penalty positive");
    BC_TRY(check_range(b, logits, logits_off, (size_t)n * 4, "sample"));
    BC_TRY(check_range(b, out, out_off, 4, "sample"));
    const uint32_t* recent_ptr = nullptr;
    if (n_recent) {
        BC_TRY(check_range(b, recent, recent_off, (size_t)n_recent * 4, "sample"));
        recent_ptr = reinterpret_cast<const uint32_t*>(at(recent, recent_off));
    }
    k::Sampling s{settings->temperature, settings->top_k, settings->top_p, settings->min_p, settings->repeat_penalty};
    return b->run("sample", 1, n, 0, 1, [&] {
        return k::sample(b->stream, reinterpret_cast<float*>(at(logits, logits_off)), n, recent_ptr, n_recent, s, uniform,
                         reinterpret_cast<uint32_t*>(at(out, out_off)), nullptr);
    });
}

bc_status bc_readback_new(bc_backend* b, size_t slots, bc_readback** out) {
    if (!b || !out) return fail(BC_ERR_ARGUMENT, "backend and out must be non-null");
    BC_TRY(b->activate());
    std::unique_ptr<bc_readback> r(new bc_readback());
    r->backend = b;
    r->writers.assign(slots, 0);
    cudaError_t e = cudaHostAlloc((void**)&r->words, sizeof(uint32_t) * std::max<size_t>(slots, 1), cudaHostAllocMapped);
    if (e != cudaSuccess) return fail(BC_ERR_ALLOCATION, "cannot allocate %zu readback slots: %s", slots, cudaGetErrorString(e));
    *out = r.release();
    return BC_OK;
}

void bc_readback_free(bc_readback* r) {
    if (!r) return;
    if (r->words) {
        // A recorded argmax may still be about to write a slot.
        if (r->backend) {
            cudaSetDevice(r->backend->device);
            cudaStreamSynchronize(r->backend->stream);
        }
        cudaFreeHost(r->words);
    }
    delete r;
}

bc_status bc_op_argmax_readback(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* out, size_t out_off, bc_readback* readback, size_t slot,
                                uint32_t n) {
    BC_TRY(need_recording(b));
    if (!readback || readback->backend != b) return fail(BC_ERR_FOREIGN_BUFFER, "the readback belongs to another backend");
    if (slot >= readback->writers.size())
        return fail(BC_ERR_OUT_OF_BOUNDS, "CPU access of 4 bytes at offset %zu exceeds a %zu-byte buffer", slot * 4, readback->writers.size() * 4);
    if (n == 0) return fail(BC_ERR_ARGUMENT, "argmax needs at least one value");
    BC_TRY(check_range(b, x, x_off, (size_t)n * 4, "argmax"));
    BC_TRY(check_range(b, out, out_off, 4, "argmax"));
    // The open recording becomes the slot's writer; the slot is readable once that ticket finished.
    readback->writers[slot] = b->next_ticket;
    return b->run("argmax", 1, n, 0, 1, [&] {
        return k::argmax(b->stream, reinterpret_cast<const float*>(at(x, x_off)), n, reinterpret_cast<uint32_t*>(at(out, out_off)),
                         readback->words + slot);
    });
}

bc_status bc_read_readback(bc_backend* b, const bc_readback* readback, size_t slot, uint32_t* token) {
    if (!b || !readback || !token) return fail(BC_ERR_ARGUMENT, "backend, readback and token must be non-null");
    if (slot >= readback->writers.size() || readback->writers[slot] == 0)
        return fail(BC_ERR_OUT_OF_BOUNDS, "CPU access of 4 bytes at offset %zu exceeds a %zu-byte buffer", slot * 4, readback->writers.size() * 4);
    uint64_t writer = readback->writers[slot];
    // Finished: collected by bc_wait, or its end event has completed. An open or unfinished
    // recording still owns the slot.
    if (writer >= b->next_ticket) return fail(BC_ERR_BUSY, "the recording that writes this slot has not been committed");
    auto end = b->tickets.find(writer);
    if (end != b->tickets.end()) {
        cudaError_t e = cudaEventQuery(end->second);
        if (e == cudaErrorNotReady) return fail(BC_ERR_BUSY, "the recording that writes this slot is still running");
        if (e != cudaSuccess) return cuda_fail(e, "recorded work");
    }
    *token = *(volatile uint32_t*)(readback->words + slot);
    return BC_OK;
}

bc_status bc_op_silu_mul(bc_backend* b, bc_buffer* x, size_t x_off, bc_buffer* gate, size_t g_off, uint32_t n) {
    BC_TRY(need_recording(b));
    BC_TRY(check_range(b, x, x_off, (size_t)n * 4, "silu_mul"));
    BC_TRY(check_range(b, gate, g_off, (size_t)n * 4, "silu_mul"));
    return b->run("silu_mul", 1, n, 0, 1, [&] {
        return k::silu_mul(b->stream, reinterpret_cast<float*>(at(x, x_off)), reinterpret_cast<const float*>(at(gate, g_off)), n);
    });
}

}  // extern "C"
