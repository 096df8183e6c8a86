// Kernels of the multi-sequence decode step: one token of each of n_seqs independent sequences
// per pass. The weight products of such a pass are the batched products of the prefill path (every
// weight is read once for all sequences); what is per sequence - the position, the KV cache, the
// convolution history - is reached here through arrays of per-sequence pointers and positions, so
// the sequences need neither a common position nor one allocation.
//
// The reference runs one sequence per runner (crates/bobcat/src/lfm2_metal.rs:103-105); each row of
// a pass here computes what Lfm2Metal::step (lfm2_metal.rs:308) computes for that sequence.

#include <cfloat>

#include "device_utils.cuh"
#include "kernels.h"

namespace bc {
namespace k {

namespace {

// One warp per head of one sequence. Blocks [0, n_heads) treat q (normalised and rotated in place),
// [n_heads, n_heads + n_kv) treat k (into the sequence's cache row), the rest copy v. grid
// (n_heads + 2 n_kv, n_seqs), 32 threads. The arithmetic is rope_store's (norm weight * (x * scale),
// NeoX pairs i, i + n_rot / 2, angle in f32).
__global__ void rope_store_seqs_kernel(RopeStore p, SeqTable seqs, uint32_t q_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x;
    const uint32_t b = blockIdx.y;
    const uint32_t pos = seqs.pos[b];
    const uint32_t hd = p.head_dim, kv_dim = p.n_kv_heads * hd;
    const size_t element = p.kv_half ? 2 : 4;
    char* k_cache = static_cast<char*>(seqs.k_cache[b]) + seqs.layer_offset * element;
    char* v_cache = static_cast<char*>(seqs.v_cache[b]) + seqs.layer_offset * element;
    uint32_t block = blockIdx.x;
    if (block >= p.n_heads + p.n_kv_heads) {
        uint32_t head = block - p.n_heads - p.n_kv_heads;
        const float* src = p.v + (uint64_t)b * kv_dim + (uint64_t)head * hd;
        uint64_t at = (uint64_t)pos * kv_dim + (uint64_t)head * hd;
        for (uint32_t e = lane; e < hd; e += 32) {
            if (p.kv_half) reinterpret_cast<__half*>(v_cache)[at + e] = __float2half_rn(src[e]);
            else reinterpret_cast<float*>(v_cache)[at + e] = src[e];
        }
        return;
    }
    const bool is_q = block < p.n_heads;
    const uint32_t head = is_q ? block : block - p.n_heads;
    float* q_row = p.q + (uint64_t)b * q_stride + (uint64_t)head * p.q_head_stride;
    const float* src = is_q ? q_row : p.k + (uint64_t)b * kv_dim + (uint64_t)head * hd;
    const float* weight = is_q ? p.q_norm : p.k_norm;
    __shared__ float values[256];
    float sumsq = 0.f;
    for (uint32_t e = lane; e < hd; e += 32) {
        float v = src[e];
        values[e] = v;
        sumsq += v * v;
    }
    sumsq = warp_sum(sumsq);
    const float scale = rsqrtf(sumsq / (float)hd + p.eps);
    __syncwarp();
    for (uint32_t e = lane; e < hd; e += 32) values[e] = weight[e] * (values[e] * scale);
    __syncwarp();
    const uint32_t half_rot = p.n_rot / 2;
    for (uint32_t e = lane; e < hd; e += 32) {
        float result = values[e];
        if (e < p.n_rot) {
            uint32_t i = e < half_rot ? e : e - half_rot;
            float inv_freq = 1.0f / powf(p.theta, (float)(2 * i) / (float)p.n_rot);
            float angle = (float)pos * inv_freq;
            float s, c;
            sincosf(angle, &s, &c);
            float a = values[i], bb = values[i + half_rot];
            result = e < half_rot ? a * c - bb * s : bb * c + a * s;
        }
        if (is_q) {
            q_row[e] = result;
        } else {
            uint64_t at = (uint64_t)pos * kv_dim + (uint64_t)head * hd + e;
            if (p.kv_half) reinterpret_cast<__half*>(k_cache)[at] = __float2half_rn(result);
            else reinterpret_cast<float*>(k_cache)[at] = result;
        }
    }
}

template <typename T>
__device__ __forceinline__ float kv_value(const T* p);
template <>
__device__ __forceinline__ float kv_value<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float kv_value<__half>(const __half* p) { return __half2float(*p); }

constexpr int kSeqAttentionWarps = 8;
constexpr int kSeqMaxGroup = 8;

// Attention of one new token per sequence: a CTA per (KV head, sequence) walks positions
// [0, pos] of that sequence's cache, every warp taking every kSeqAttentionWarps-th position with a
// running (maximum, sum, weighted values) per query head of the group; the warps' results are
// merged in warp order. EPL = head_dim / 32 elements per lane. grid (n_kv_heads, n_seqs).
template <typename T, int EPL>
__global__ void __launch_bounds__(kSeqAttentionWarps * 32) attention_seqs_kernel(const float* __restrict__ q, float* __restrict__ out, SeqTable seqs,
                                                                                   uint32_t n_heads, uint32_t n_kv_heads, uint32_t q_stride,
                                                                                   uint32_t q_head_stride) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int HD = EPL * 32;
    const uint32_t kv_head = blockIdx.x, b = blockIdx.y;
    const uint32_t group = n_heads / n_kv_heads, kv_dim = n_kv_heads * HD;
    const uint32_t pos = seqs.pos[b];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* kc = static_cast<const T*>(seqs.k_cache[b]) + seqs.layer_offset + (uint64_t)kv_head * HD;
    const T* vc = static_cast<const T*>(seqs.v_cache[b]) + seqs.layer_offset + (uint64_t)kv_head * HD;
    const float scale = 1.0f / sqrtf((float)HD);

    __shared__ float merged_max[kSeqAttentionWarps][kSeqMaxGroup], merged_sum[kSeqAttentionWarps][kSeqMaxGroup];
    __shared__ float merged_acc[kSeqAttentionWarps][HD];

    for (uint32_t g0 = 0; g0 < group; g0 += 2) {
        // Two query heads at a time keep the running sums in registers for heads of up to 256 elements.
        const uint32_t heads_now = min(2u, group - g0);
        float qv[2][EPL], acc[2][EPL], m[2], l[2];
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            m[g] = -FLT_MAX;
            l[g] = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                acc[g][e] = 0.f;
                qv[g][e] = (uint32_t)g < heads_now
                               ? q[(uint64_t)b * q_stride + (uint64_t)(kv_head * group + g0 + g) * q_head_stride + lane + 32 * e] * scale
                               : 0.f;
            }
        }
        for (uint32_t t = warp; t <= pos; t += kSeqAttentionWarps) {
            float kvals[EPL], vvals[EPL];
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                kvals[e] = kv_value<T>(kc + (uint64_t)t * kv_dim + lane + 32 * e);
                vvals[e] = kv_value<T>(vc + (uint64_t)t * kv_dim + lane + 32 * e);
            }
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                float dot = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) dot += kvals[e] * qv[g][e];
                dot = warp_sum(dot);
                const float m_new = fmaxf(m[g], dot);
                const float keep = expf(m[g] - m_new), w = expf(dot - m_new);
                l[g] = l[g] * keep + w;
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * keep + w * vvals[e];
                m[g] = m_new;
            }
        }
        // Merge the warps, one query head at a time.
        for (uint32_t g = 0; g < heads_now; ++g) {
            __syncthreads();
            if (lane == 0) {
                merged_max[warp][0] = g == 0 ? m[0] : m[1];
                merged_sum[warp][0] = g == 0 ? l[0] : l[1];
            }
#pragma unroll
            for (int e = 0; e < EPL; ++e) merged_acc[warp][lane + 32 * e] = g == 0 ? acc[0][e] : acc[1][e];
            __syncthreads();
            if (warp == 0) {
                float top = -FLT_MAX;
                for (int w = 0; w < kSeqAttentionWarps; ++w) top = fmaxf(top, merged_max[w][0]);
                float total = 0.f, sum[EPL];
#pragma unroll
                for (int e = 0; e < EPL; ++e) sum[e] = 0.f;
                for (int w = 0; w < kSeqAttentionWarps; ++w) {
                    // A warp that saw no position holds the maximum -FLT_MAX and sums of zero.
                    const float f = merged_sum[w][0] > 0.f ? expf(merged_max[w][0] - top) : 0.f;
                    total += merged_sum[w][0] * f;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) sum[e] += merged_acc[w][lane + 32 * e] * f;
                }
                float* o = out + (uint64_t)b * n_heads * HD + (uint64_t)(kv_head * group + g0 + g) * HD;
#pragma unroll
                for (int e = 0; e < EPL; ++e) o[lane + 32 * e] = sum[e] / total;
            }
        }
    }
}

// The gated short convolution of one token per sequence (crates/bobcat/src/lfm2.rs:456-475): row b
// of bcx is the sequence's B | C | X projection, its history [kernel - 1][n_embd] is shifted in
// place. One thread per (channel, sequence).
__global__ void short_conv_seqs_kernel(const float* __restrict__ bcx, const float* __restrict__ taps, SeqTable seqs, float* __restrict__ out,
                                       uint32_t n_embd, uint32_t kernel) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t ch = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (ch >= n_embd) return;
    const float* row = bcx + (uint64_t)b * 3 * n_embd;
    float* history = seqs.conv_state[b] + seqs.conv_offset;
    const float bv = row[ch], c = row[n_embd + ch], x = row[2 * n_embd + ch];
    const float bx = bv * x;
    float sum = taps[(uint64_t)ch * kernel + kernel - 1] * bx;
    for (uint32_t kk = 0; kk + 1 < kernel; ++kk) sum += taps[(uint64_t)ch * kernel + kk] * history[(uint64_t)kk * n_embd + ch];
    for (uint32_t kk = 0; kk + 2 < kernel; ++kk) history[(uint64_t)kk * n_embd + ch] = history[(uint64_t)(kk + 1) * n_embd + ch];
    history[(uint64_t)(kernel - 2) * n_embd + ch] = bx;
    out[(uint64_t)b * n_embd + ch] = c * sum;
}

// argmax of each row (ties to the lowest index): a CTA per sequence. picked[b] takes the index and,
// when `record` is non-null, so does record[b * record_stride + record_at].
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float* __restrict__ x, uint32_t n, uint32_t* __restrict__ picked,
                                                           uint32_t* __restrict__ record, uint32_t record_stride, uint32_t record_at) {
    __shared__ float best_value[32];
    __shared__ uint32_t best_index[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = x + (uint64_t)blockIdx.x * n;
    float value = -INFINITY;
    uint32_t index = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = row[i];
        if (v > value || index == 0xffffffffu) {
            value = v;
            index = i;
        }
    }
    auto better = [](float v, uint32_t i, float bv, uint32_t bi) { return i != 0xffffffffu && (bi == 0xffffffffu || v > bv || (v == bv && i < bi)); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, value, o);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, index, o);
        if (better(ov, oi, value, index)) {
            value = ov;
            index = oi;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        best_value[warp] = value;
        best_index[warp] = index;
    }
    __syncthreads();
    if (warp == 0) {
        value = best_value[lane];
        index = best_index[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, value, o);
            uint32_t oi = __shfl_xor_sync(0xffffffffu, index, o);
            if (better(ov, oi, value, index)) {
                value = ov;
                index = oi;
            }
        }
        if (lane == 0) {
            picked[blockIdx.x] = index;
            if (record) record[(uint64_t)blockIdx.x * record_stride + record_at] = index;
        }
    }
}

__global__ void advance_seqs_kernel(uint32_t* pos, uint32_t n_seqs) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < n_seqs) pos[b] += 1;
}

}  // namespace

cudaError_t rope_store_seqs(cudaStream_t stream, const RopeStore& p, const SeqTable& seqs, uint32_t q_stride, uint32_t n_seqs) {
    RopeStore params = p;
    SeqTable table = seqs;
    void* args[] = {&params, &table, &q_stride};
    return launch_kernel((const void*)rope_store_seqs_kernel, dim3(p.n_heads + 2 * p.n_kv_heads, n_seqs), dim3(32), 0, stream, args);
}

bool attention_seqs_supported(uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim) {
    return n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_heads / n_kv_heads <= (uint32_t)kSeqMaxGroup &&
           (head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256);
}

cudaError_t attention_seqs(cudaStream_t stream, const float* q, float* out, const SeqTable& seqs, bool kv_half, uint32_t n_heads,
                           uint32_t n_kv_heads, uint32_t head_dim, uint32_t q_stride, uint32_t q_head_stride, uint32_t n_seqs) {
    if (!attention_seqs_supported(n_heads, n_kv_heads, head_dim)) return cudaErrorInvalidValue;
    SeqTable table = seqs;
    void* args[] = {&q, &out, &table, &n_heads, &n_kv_heads, &q_stride, &q_head_stride};
    const void* kernel = nullptr;
    if (kv_half) {
        kernel = head_dim == 32 ? (const void*)attention_seqs_kernel<__half, 1> : head_dim == 64 ? (const void*)attention_seqs_kernel<__half, 2>
               : head_dim == 128 ? (const void*)attention_seqs_kernel<__half, 4> : (const void*)attention_seqs_kernel<__half, 8>;
    } else {
        kernel = head_dim == 32 ? (const void*)attention_seqs_kernel<float, 1> : head_dim == 64 ? (const void*)attention_seqs_kernel<float, 2>
               : head_dim == 128 ? (const void*)attention_seqs_kernel<float, 4> : (const void*)attention_seqs_kernel<float, 8>;
    }
    return launch_kernel(kernel, dim3(n_kv_heads, n_seqs), dim3(kSeqAttentionWarps * 32), 0, stream, args);
}

cudaError_t short_conv_seqs(cudaStream_t stream, const float* bcx, const float* taps, const SeqTable& seqs, float* out, uint32_t n_embd,
                            uint32_t kernel, uint32_t n_seqs) {
    SeqTable table = seqs;
    void* args[] = {&bcx, &taps, &table, &out, &n_embd, &kernel};
    return launch_kernel((const void*)short_conv_seqs_kernel, dim3((n_embd + 255) / 256, n_seqs), dim3(256), 0, stream, args);
}

cudaError_t argmax_rows(cudaStream_t stream, const float* x, uint32_t n, uint32_t n_rows, uint32_t* picked, uint32_t* record,
                        uint32_t record_stride, uint32_t record_at) {
    void* args[] = {&x, &n, &picked, &record, &record_stride, &record_at};
    return launch_kernel((const void*)argmax_rows_kernel, dim3(n_rows), dim3(1024), 0, stream, args);
}

cudaError_t advance_seqs(cudaStream_t stream, uint32_t* pos, uint32_t n_seqs) {
    void* args[] = {&pos, &n_seqs};
    return launch_kernel((const void*)advance_seqs_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, stream, args);
}

}  // namespace k
}  // namespace bc
