// Device code shared by the SIMT matrix-vector kernels: row addressing in the device layouts, the
// L2 prefetch of a row, staging of the input vector in shared memory, and the per-lane dot product
// of a few rows with the staged input.
#pragma once

#include "device_utils.cuh"
#include "kernels.h"
#include "../../include/bobcat_cuda.h"

namespace bc {
namespace k {

struct RowPtr {
    const void* data;      // first byte of the row's weights
    const __half* scales;  // first scale of the row (Q4_0 only)
};

__device__ __forceinline__ RowPtr row_of(const Mat& m, uint32_t row) {
    RowPtr p;
    if (m.format == BC_Q4_0) {
        uint64_t nb = m.n_cols >> 5;
        p.data = static_cast<const uint4*>(m.data) + row * nb;
        p.scales = m.scales + row * nb;
    } else if (m.format == BC_F16) {
        p.data = static_cast<const __half*>(m.data) + (uint64_t)row * m.n_cols;
        p.scales = nullptr;
    } else if (m.format == BC_Q8_0) {
        p.data = static_cast<const uint8_t*>(m.data) + (uint64_t)row * (m.n_cols >> 5) * kQ8_0BlockBytes;
        p.scales = nullptr;
    } else if (m.format == BC_Q6_K) {
        p.data = static_cast<const uint8_t*>(m.data) + (uint64_t)row * (m.n_cols >> 8) * kQ6KBlockBytes;
        p.scales = nullptr;
    } else {
        p.data = static_cast<const float*>(m.data) + (uint64_t)row * m.n_cols;
        p.scales = nullptr;
    }
    return p;
}

// Ask the L2 to fetch [p, p + bytes); both must be multiples of 16.
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

template <int FORMAT>
__device__ __forceinline__ void prefetch_row(const RowPtr& r, uint32_t n_cols) {
    if (FORMAT == BC_Q4_0) {
        uint32_t nb = n_cols >> 5;
        prefetch_l2(r.data, nb * 16);
        if ((reinterpret_cast<uintptr_t>(r.scales) & 15) == 0 && (nb & 7) == 0) prefetch_l2(r.scales, nb * 2);
    } else if (FORMAT == BC_F16 || FORMAT == BC_F32) {
        prefetch_l2(r.data, n_cols * (FORMAT == BC_F16 ? 2u : 4u));
    }
    // Rows of the byte-layout formats are only 2-byte aligned: no bulk prefetch for them.
}

// Stage x into shared memory in the rotated chunk layout, times the norm weight when given.
// Returns the factor the finished row sums are multiplied by (1 without a norm).
__device__ inline float stage_input(const float* __restrict__ x, const float* __restrict__ norm_weight, float eps,
                             uint32_t n_cols, float4* xs, float* reduce_scratch) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const float4* w4 = reinterpret_cast<const float4*>(norm_weight);
    float sumsq = 0.f;
    for (uint32_t ci = threadIdx.x; ci < n_cols / 4; ci += blockDim.x) {
        float4 v = x4[ci];
        if (norm_weight) {
            sumsq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            float4 w = __ldg(w4 + ci);
            v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
        }
        xs[x_slot(ci >> 3, ci & 7)] = v;
    }
    float scale = 1.f;
    if (norm_weight) {
        float total = block_sum(sumsq, reduce_scratch);
        scale = rsqrtf(total / (float)n_cols + eps);
    } else {
        __syncthreads();
    }
    return scale;
}

// Partial dot products of R rows with the staged input over this warp's share of the columns:
// part `kpart` of `ksplit` interleaved parts, each a stride of 32 lanes.
template <int FORMAT, int R>
__device__ __forceinline__ void dot_rows(const RowPtr (&rows)[R], uint32_t n_cols, const float4* __restrict__ xs, int lane,
                                         int kpart, int ksplit, float (&acc)[R]) {
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    const int step = 32 * ksplit;
    if (FORMAT == BC_Q4_0) {
        const int nb = n_cols >> 5;
#pragma unroll 2
        for (int b0 = kpart * 32; b0 < nb; b0 += step) {
            int b = b0 + lane;
            bool live = b < nb;
            int bc_ = live ? b : nb - 1;
            uint4 q[R];
            float d[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                q[r] = ldg_stream(static_cast<const uint4*>(rows[r].data) + bc_);
                d[r] = live ? __half2float(rows[r].scales[bc_]) : 0.f;
            }
            float sum[R];
#pragma unroll
            for (int r = 0; r < R; ++r) sum[r] = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                float4 xl = xs[x_slot(bc_, w)];
                float4 xh = xs[x_slot(bc_, 4 + w)];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    uint32_t word = w == 0 ? q[r].x : w == 1 ? q[r].y : w == 2 ? q[r].z : q[r].w;
                    float lo[4], hi[4];
                    unpack_q4_word(word, lo, hi);
                    sum[r] += lo[0] * xl.x + lo[1] * xl.y + lo[2] * xl.z + lo[3] * xl.w;
                    sum[r] += hi[0] * xh.x + hi[1] * xh.y + hi[2] * xh.z + hi[3] * xh.w;
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] += d[r] * sum[r];
        }
    } else if (FORMAT == BC_F32) {
        const int nc = n_cols >> 2;
#pragma unroll 4
        for (int c0 = kpart * 32; c0 < nc; c0 += step) {
            int c = c0 + lane;
            bool live = c < nc;
            int cc = live ? c : nc - 1;
            float4 xv = xs[x_slot(cc >> 3, cc & 7)];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float4 w = ldg_stream(static_cast<const float4*>(rows[r].data) + cc);
                float s = w.x * xv.x + w.y * xv.y + w.z * xv.z + w.w * xv.w;
                acc[r] += live ? s : 0.f;
            }
        }
    } else if (FORMAT == BC_Q8_0) {
        // A lane owns whole blocks: 32 int8 quants (read as 16 aligned byte pairs) and one scale.
        const int nb = n_cols >> 5;
        for (int b0 = kpart * 32; b0 < nb; b0 += step) {
            const int b = b0 + lane;
            if (b >= nb) continue;
            float xv[32];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float4 v = xs[x_slot(b, c)];
                xv[4 * c] = v.x; xv[4 * c + 1] = v.y; xv[4 * c + 2] = v.z; xv[4 * c + 3] = v.w;
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint8_t* block = static_cast<const uint8_t*>(rows[r].data) + (uint64_t)b * kQ8_0BlockBytes;
                const unsigned short* pairs = reinterpret_cast<const unsigned short*>(block + 2);
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const unsigned short two = pairs[i];
                    sum += (float)(int)(signed char)(two & 0xff) * xv[2 * i] + (float)(int)(signed char)(two >> 8) * xv[2 * i + 1];
                }
                acc[r] += half_at(block) * sum;
            }
        }
    } else if (FORMAT == BC_Q6_K) {
        // Item (super-block, half, l) yields the four elements l + 32 k of that half; lanes take
        // consecutive l, so their byte reads are contiguous.
        const int items = (n_cols >> 8) * 64;
        const float* xf = reinterpret_cast<const float*>(xs);
        for (int j0 = kpart * 32; j0 < items; j0 += step) {
            const int j = j0 + lane;
            if (j >= items) continue;
            const int sb = j >> 6, half_index = (j >> 5) & 1, l = j & 31;
            float xv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int e = sb * 256 + half_index * 128 + l + 32 * k;
                xv[k] = xf[x_slot(e >> 5, (e & 31) >> 2) * 4 + (e & 3)];
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint8_t* block = static_cast<const uint8_t*>(rows[r].data) + (uint64_t)sb * kQ6KBlockBytes;
                const uint8_t* low = block + half_index * 64;
                const uint8_t hb = block[128 + half_index * 32 + l];
                const signed char* scales = reinterpret_cast<const signed char*>(block + 192 + half_index * 8);
                const float d = half_at(block + 208);
                const uint8_t b0 = low[l], b1 = low[l + 32];
                const int q[4] = {(int)((b0 & 0xfu) | ((hb & 3u) << 4)) - 32, (int)((b1 & 0xfu) | (((hb >> 2) & 3u) << 4)) - 32,
                                  (int)((b0 >> 4) | (((hb >> 4) & 3u) << 4)) - 32, (int)((b1 >> 4) | (((hb >> 6) & 3u) << 4)) - 32};
                float sum = 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) sum += (d * (float)(int)scales[(l >> 4) + 2 * k]) * (float)q[k] * xv[k];
                acc[r] += sum;
            }
        }
    } else {  // BC_F16
        const int nc = n_cols >> 3;
#pragma unroll 2
        for (int c0 = kpart * 32; c0 < nc; c0 += step) {
            int c = c0 + lane;
            bool live = c < nc;
            int cc = live ? c : nc - 1;
            float4 x0 = xs[x_slot(cc >> 2, (2 * cc) & 7)];
            float4 x1 = xs[x_slot(cc >> 2, (2 * cc + 1) & 7)];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                uint4 w = ldg_stream(static_cast<const uint4*>(rows[r].data) + cc);
                float2 a = __half22float2(*reinterpret_cast<__half2*>(&w.x));
                float2 b = __half22float2(*reinterpret_cast<__half2*>(&w.y));
                float2 c2 = __half22float2(*reinterpret_cast<__half2*>(&w.z));
                float2 e = __half22float2(*reinterpret_cast<__half2*>(&w.w));
                float s = a.x * x0.x + a.y * x0.y + b.x * x0.z + b.y * x0.w + c2.x * x1.x + c2.y * x1.y + e.x * x1.z +
                          e.y * x1.w;
                acc[r] += live ? s : 0.f;
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
}

}  // namespace k
}  // namespace bc
