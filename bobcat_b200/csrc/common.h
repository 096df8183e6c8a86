// Shared host-side helpers: status codes, the thread-local error message, CUDA call checks.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/bobcat_cuda.h"
#include "../../include/bobcat_cuda_test.h"

namespace bc {

// The calling thread's latest failure message.
std::string& last_error();

// Record a failure message and return `status`, so call sites read `return fail(BC_ERR_X, ...)`.
bc_status fail(bc_status status, const char* format, ...) __attribute__((format(printf, 2, 3)));

// Turn a CUDA error into BC_ERR_EXECUTION (or `status`) with the call site in the message.
bc_status cuda_fail(cudaError_t error, const char* what, bc_status status = BC_ERR_EXECUTION);

#define BC_CUDA(call)                                                   \
    do {                                                                \
        cudaError_t bc_cuda_error_ = (call);                            \
        if (bc_cuda_error_ != cudaSuccess) return ::bc::cuda_fail(bc_cuda_error_, #call); \
    } while (0)

#define BC_TRY(call)                         \
    do {                                     \
        bc_status bc_status_ = (call);       \
        if (bc_status_ != BC_OK) return bc_status_; \
    } while (0)

inline uint64_t div_up(uint64_t a, uint64_t b) { return (a + b - 1) / b; }
inline uint64_t round_up(uint64_t a, uint64_t b) { return div_up(a, b) * b; }

}  // namespace bc
