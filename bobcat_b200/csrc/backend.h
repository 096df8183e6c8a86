// Internal definitions behind the opaque handles of the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "common.h"
#include "gguf.h"
#include "kernels.h"

struct bc_seq;

struct bc_buffer {
    bc_backend* backend = nullptr;
    void* ptr = nullptr;
    size_t len = 0;
    // Set by bc_matrix_upload: the matrix this buffer holds in the device layout.
    bool is_matrix = false;
    bc::k::Mat matrix;
};

// Token slots in host-mapped memory that argmax launches write and the CPU reads once the
// recording that wrote a slot has finished (Readback, crates/bobcat-metal/src/backend.rs:324-333).
struct bc_readback {
    bc_backend* backend = nullptr;
    uint32_t* words = nullptr;
    std::vector<uint64_t> writers;  // per slot: ticket of the recording that last wrote it, 0 = never
};

struct ProfileKey {
    std::string name;
    uint32_t n_rows, n_cols;
    bool operator<(const ProfileKey& o) const {
        if (name != o.name) return name < o.name;
        if (n_rows != o.n_rows) return n_rows < o.n_rows;
        return n_cols < o.n_cols;
    }
};

struct ProfileTotals {
    uint64_t calls = 0;
    double seconds = 0;
    uint64_t bytes = 0;
};

struct bc_backend {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    bool recording = false;
    uint64_t next_ticket = 1;
    cudaEvent_t record_start = nullptr;
    std::map<uint64_t, cudaEvent_t> tickets;  // ticket -> end-of-recording event
    std::map<uint64_t, cudaEvent_t> ticket_starts;
    std::set<bc_buffer*> buffers;
    std::set<bc_seq*> seqs;  // sequences recording onto this backend; closing the backend releases them
    uint64_t launches = 0;  // kernels launched through this backend
    // Scratch of the tensor-core prefill kernel: the fp16 operand-layout copy of a matmul's inputs.
    // Grown on demand; only launches of this backend's stream touch it, one after another.
    void* pack = nullptr;
    size_t pack_len = 0;
    bc_status pack_scratch(size_t bytes, void** out);
    // Partial products of split-K launches, apart from the packed inputs: they may outlive the
    // launch that wrote them until the next normalisation adds them up.
    void* partials = nullptr;
    size_t partials_len = 0;
    bc_status partial_scratch(size_t bytes, void** out);

    bool profiling = false;
    std::map<ProfileKey, ProfileTotals> profile;
    std::vector<std::string> profile_names;  // keeps c_str() pointers handed out alive

    // Run `launch` on the stream, counting it and, in profiling mode, timing it with events.
    template <typename F>
    bc_status run(const char* name, uint32_t n_rows, uint32_t n_cols, uint64_t bytes, int kernels, F&& launch);
    bc_status activate();
};

namespace bc {

// Check that [offset, offset + needed) lies inside `buffer`, which must belong to `backend`
// (check_range, crates/bobcat-metal/src/backend.rs:2772-2790).
bc_status check_range(const bc_backend* backend, const bc_buffer* buffer, size_t offset, size_t needed, const char* op);
// BC_ERR_EXECUTION when a kernel's bounded wait ran out since the last call; clears the record.
bc_status kernel_wait_status();

}  // namespace bc

template <typename F>
bc_status bc_backend::run(const char* name, uint32_t n_rows, uint32_t n_cols, uint64_t bytes, int kernels, F&& launch) {
    launches += (uint64_t)kernels;
    if (!profiling) {
        cudaError_t e = launch();
        if (e != cudaSuccess) return bc::cuda_fail(e, name);
        return BC_OK;
    }
    cudaEvent_t a, b;
    BC_CUDA(cudaEventCreate(&a));
    BC_CUDA(cudaEventCreate(&b));
    BC_CUDA(cudaEventRecord(a, stream));
    cudaError_t e = launch();
    if (e != cudaSuccess) {
        cudaEventDestroy(a);
        cudaEventDestroy(b);
        return bc::cuda_fail(e, name);
    }
    BC_CUDA(cudaEventRecord(b, stream));
    BC_CUDA(cudaEventSynchronize(b));
    float ms = 0.f;
    cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    ProfileTotals& t = profile[ProfileKey{name, n_rows, n_cols}];
    t.calls += 1;
    t.seconds += ms * 1e-3;
    t.bytes += bytes;
    return BC_OK;
}
