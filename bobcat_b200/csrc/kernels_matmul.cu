// Batched multiply for prefill: Y[t][r] (store) sum_c W[r][c] X[t][c] over n_tokens rows of X.
//
// This file holds the SIMT tile kernel: f32 inputs, weights dequantised to f32 in shared memory,
// f32 accumulation. It serves every format and every shape (ragged row and token counts) and is
// the in-library cross-check of the tensor-core kernel. Counterpart: matmul_q / matmul_tile in
// crates/bobcat-metal/src/matmul.metal:249-470 with the three stores of backend.rs:361-370.

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

}  // namespace

cudaError_t matmul(cudaStream_t stream, const Mat& w, const float* x, float* y, uint32_t n_tokens, uint32_t y_stride,
                   int32_t store, void* pack) {
    if (n_tokens == 0 || w.n_rows == 0) return cudaSuccess;
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
