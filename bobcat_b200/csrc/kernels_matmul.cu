// Batched multiply for prefill: Y[t][r] (store) sum_c W[r][c] X[t][c] over n_tokens rows of X.
//
// This file holds the SIMT tile kernel: f32 inputs, weights dequantised to f32 in shared memory,
// f32 accumulation. It serves every format and every shape (ragged row and token counts) and is
// the in-library cross-check of the tensor-core kernel. Counterpart: matmul_q / matmul_tile in
// crates/bobcat-metal/src/matmul.metal:249-470 with the three stores of backend.rs:361-370.

#include "async_utils.cuh"
#include "device_utils.cuh"
#include "kernels.h"
#include "../../include/bobcat_cuda.h"

namespace bc {
namespace k {

namespace {

constexpr int kTileRows = 64;    // weight rows per CTA
constexpr int kTileTokens = 64;  // tokens per CTA
constexpr int kTileK = 32;       // columns per step: one Q4_0 block per row
constexpr int kThreads = 256;    // each thread owns a 4 x 4 patch of the 64 x 64 tile

struct MatmulParams {
    Mat w;
    const float* x;
    float* y;
    uint32_t n_tokens, y_stride;
    int store;
};

__global__ void __launch_bounds__(kThreads) matmul_simt_kernel(MatmulParams p) {
    __shared__ float ws[kTileK][kTileRows + 4];    // [k][row]
    __shared__ float xs[kTileK][kTileTokens + 4];  // [k][token]
    const uint32_t row0 = blockIdx.y * kTileRows, tok0 = blockIdx.x * kTileTokens;
    const uint32_t n_rows = p.w.n_rows, n_cols = p.w.n_cols;
    const int tid = threadIdx.x;
    const int tr = (tid % 16) * 4, tt = (tid / 16) * 4;
    float acc[4][4] = {};

    for (uint32_t k0 = 0; k0 < n_cols; k0 += kTileK) {
        // Weights: 64 rows x 32 columns. Threads 0..63 dequantise one Q4_0 block each; other
        // formats spread the 2048 elements over the CTA.
        if (p.w.format == BC_Q4_0) {
            if (tid < kTileRows) {
                uint32_t row = row0 + tid;
                if (row < n_rows) {
                    uint64_t block = (uint64_t)row * (n_cols >> 5) + (k0 >> 5);
                    uint4 q = static_cast<const uint4*>(p.w.data)[block];
                    float d = __half2float(p.w.scales[block]);
                    uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t byte = (words[w] >> (8 * i)) & 0xffu;
                            ws[4 * w + i][tid] = (float)((int)(byte & 0xfu) - 8) * d;
                            ws[16 + 4 * w + i][tid] = (float)((int)(byte >> 4) - 8) * d;
                        }
                    }
                } else {
                    for (int kk = 0; kk < kTileK; ++kk) ws[kk][tid] = 0.f;
                }
            }
        } else {
            for (int i = tid; i < kTileRows * kTileK; i += kThreads) {
                int r = i / kTileK, kk = i % kTileK;
                uint32_t row = row0 + r;
                float v = 0.f;
                if (row < n_rows) {
                    uint64_t at = (uint64_t)row * n_cols + k0 + kk;
                    if (p.w.format == BC_Q8_0) v = q8_0_at(static_cast<const uint8_t*>(p.w.data) + (uint64_t)row * (n_cols >> 5) * kQ8_0BlockBytes, k0 + kk);
                    else if (p.w.format == BC_Q6_K) v = q6k_at(static_cast<const uint8_t*>(p.w.data) + (uint64_t)row * (n_cols >> 8) * kQ6KBlockBytes, k0 + kk);
                    else v = p.w.format == BC_F16 ? __half2float(static_cast<const __half*>(p.w.data)[at])
                                                  : static_cast<const float*>(p.w.data)[at];
                }
                ws[kk][r] = v;
            }
        }
        for (int i = tid; i < kTileTokens * kTileK; i += kThreads) {
            int t = i / kTileK, kk = i % kTileK;
            uint32_t tok = tok0 + t;
            xs[kk][t] = tok < p.n_tokens ? p.x[(uint64_t)tok * n_cols + k0 + kk] : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kTileK; ++kk) {
            float4 wv = *reinterpret_cast<const float4*>(&ws[kk][tr]);
            float4 xv = *reinterpret_cast<const float4*>(&xs[kk][tt]);
            float wr[4] = {wv.x, wv.y, wv.z, wv.w}, xt[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] += xt[a] * wr[b];
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        uint32_t tok = tok0 + tt + a;
        if (tok >= p.n_tokens) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            uint32_t row = row0 + tr + b;
            if (row >= n_rows) continue;
            float* y = p.y + (uint64_t)tok * p.y_stride + row;
            float v = acc[a][b];
            if (p.store == BC_STORE_ACCUMULATE) v += *y;
            else if (p.store == BC_STORE_SWIGLU) {
                float g = *y;
                v = g / (1.f + expf(-g)) * v;
            }
            *y = v;
        }
    }
}

// An f32 matrix against at most 32 rows of X (the logits of a pass over several sequences: the
// output matrix is the model's largest and is kept in f32): Y[t][r] = sum_c W[r][c] X[t][c], f32
// throughout, every sum one chain of fused multiply-adds over the columns in order. The tile kernel
// above spends a pass over a 65536 x 2048 matrix mostly on loads of single elements (0.97 ms for 32
// rows). Here a CTA is ONE warp with 64 weight rows to itself: 1024 such warps spread evenly over
// the SMs (seven on most), and none waits for another. A lane holds an 8 x 8 block of sums (rows
// lane/4 + 8i, tokens lane%4 + 4j), so a step of four columns costs 16 vector reads of shared
// memory for 256 multiply-adds; the bytes stream in by cp.async, 32 columns per stage, two stages
// (deeper or narrower stages measured the same: the kernel is bound by instruction issue, at 0.25
// ms for that matrix).
constexpr int kFewRows = 64, kFewThreads = 32;
template <int kFewStep, int kStages>
constexpr size_t few_smem_bytes() { return (size_t)kStages * (kFewRows + 32) * (kFewStep + 4) * sizeof(float); }

template <int kFewStep, int kStages>
__global__ void __launch_bounds__(kFewThreads) matmul_f32_few_kernel(const float* __restrict__ w, const float* __restrict__ x, float* __restrict__ y,
                                                                     uint32_t n_rows, uint32_t n_cols, uint32_t n_tokens, uint32_t y_stride) {
    constexpr int kFewPitch = kFewStep + 4;
    extern __shared__ __align__(16) float few_smem[];
    float (*ws)[kFewRows][kFewPitch] = reinterpret_cast<float (*)[kFewRows][kFewPitch]>(few_smem);
    float (*xs)[32][kFewPitch] = reinterpret_cast<float (*)[32][kFewPitch]>(few_smem + kStages * kFewRows * kFewPitch);
    pdl_launch_dependents();
    const uint32_t lane = threadIdx.x, row0 = blockIdx.x * kFewRows, rg = lane >> 2, tg = lane & 3;
    constexpr uint32_t kPieces = kFewStep / 4;
    // Rows and tokens past the end are zeros, written once: no copy ever lands there.
    for (uint32_t i = lane; i < kStages * (kFewRows + 32) * kPieces; i += kFewThreads) {
        const uint32_t buf = i / ((kFewRows + 32) * kPieces), r = i / kPieces % (kFewRows + 32), piece = i % kPieces;
        if (r < kFewRows ? row0 + r >= n_rows : r - kFewRows >= n_tokens)
            *reinterpret_cast<float4*>(r < kFewRows ? &ws[buf][r][4 * piece] : &xs[buf][r - kFewRows][4 * piece]) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    auto bring_w = [&](uint32_t step, uint32_t buf) {
        const float* src = w + (uint64_t)row0 * n_cols + step * kFewStep;
#pragma unroll 4
        for (uint32_t i = lane; i < kFewRows * kPieces; i += kFewThreads) {
            const uint32_t r = i / kPieces, piece = i % kPieces;
            if (row0 + r < n_rows) async::cp_async_16(async::smem_u32(&ws[buf][r][4 * piece]), src + (uint64_t)r * n_cols + 4 * piece);
        }
    };
    auto bring_x = [&](uint32_t step, uint32_t buf) {
        const float* src = x + step * kFewStep;
#pragma unroll 4
        for (uint32_t i = lane; i < 32 * kPieces; i += kFewThreads) {
            const uint32_t t = i / kPieces, piece = i % kPieces;
            if (t < n_tokens) async::cp_async_16(async::smem_u32(&xs[buf][t][4 * piece]), src + (uint64_t)t * n_cols + 4 * piece);
        }
    };
    const uint32_t steps = n_cols / kFewStep;
    bring_w(0, 0);  // the weights are nobody's output
    pdl_wait();
    bring_x(0, 0);
    async::cp_async_commit();
    for (uint32_t s = 1; s + 1 < kStages; ++s) {  // a group per stage, empty past the end
        if (s < steps) {
            bring_w(s, s);
            bring_x(s, s);
        }
        async::cp_async_commit();
    }
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    for (uint32_t step = 0; step < steps; ++step) {
        const uint32_t buf = step % kStages, ahead = step + kStages - 1;
        if (ahead < steps) {
            bring_w(ahead, ahead % kStages);
            bring_x(ahead, ahead % kStages);
        }
        async::cp_async_commit();
        async::cp_async_wait<kStages - 1>();
        __syncwarp();
#pragma unroll 2
        for (int kk = 0; kk < kFewStep; kk += 4) {
            float4 xv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) xv[j] = *reinterpret_cast<const float4*>(&xs[buf][tg + 4 * j][kk]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 wv = *reinterpret_cast<const float4*>(&ws[buf][rg + 8 * i][kk]);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float a = acc[i][j];
                    a = fmaf(wv.x, xv[j].x, a);
                    a = fmaf(wv.y, xv[j].y, a);
                    a = fmaf(wv.z, xv[j].z, a);
                    a = fmaf(wv.w, xv[j].w, a);
                    acc[i][j] = a;
                }
            }
        }
        __syncwarp();  // the stage is read before the copy after next lands in it
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t t = tg + 4 * j;
        if (t >= n_tokens) continue;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t r = row0 + rg + 8 * i;
            if (r < n_rows) y[(uint64_t)t * y_stride + r] = acc[i][j];
        }
    }
}

}  // namespace

cudaError_t matmul(cudaStream_t stream, const Mat& w, const float* x, float* y, uint32_t n_tokens, uint32_t y_stride,
                   int32_t store, void* pack) {
    if (n_tokens == 0 || w.n_rows == 0) return cudaSuccess;
    if (w.format == BC_F32 && n_tokens <= 32 && store == BC_STORE_OVERWRITE && w.n_cols % 32 == 0 && w.n_cols > 0 &&
        ((reinterpret_cast<uintptr_t>(w.data) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
        constexpr size_t bytes = few_smem_bytes<32, 2>();
        cudaError_t e = ensure_dynamic_smem((const void*)matmul_f32_few_kernel<32, 2>, bytes);
        if (e != cudaSuccess) return e;
        return launch_dependent(matmul_f32_few_kernel<32, 2>, dim3((w.n_rows + kFewRows - 1) / kFewRows), dim3(kFewThreads), bytes, stream,
                                static_cast<const float*>(w.data), x, y, w.n_rows, w.n_cols, n_tokens, y_stride);
    }
    if (pack && matmul_umma_supported(w, n_tokens)) {
        cudaError_t e = matmul_pack(stream, x, n_tokens, w.n_cols, pack);
        if (e != cudaSuccess) return e;
        return matmul_umma(stream, w, pack, y, n_tokens, y_stride, store);
    }
    MatmulParams p{w, x, y, n_tokens, y_stride, store};
    dim3 grid((n_tokens + kTileTokens - 1) / kTileTokens, (w.n_rows + kTileRows - 1) / kTileRows);
    matmul_simt_kernel<<<grid, kThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace k
}  // namespace bc
