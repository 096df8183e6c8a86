// The small kernels of the decode and prefill graphs: weight repack and expansion, embedding
// gather, RMSNorm, per-head norm + rotary embedding + cache store, conversions, the batched short
// convolution, and argmax. Counterparts: crates/bobcat-metal/src/norm.metal, conv.metal,
// quant.metal:279-330 (expand).

#include "device_utils.cuh"
#include "kernels.h"
#include "../../include/bobcat_cuda.h"

namespace bc {
namespace k {

namespace {

constexpr int kThreads = 256;

inline int blocks_for(uint64_t n, int per_block = kThreads) {
    uint64_t b = (n + per_block - 1) / per_block;
    return (int)(b < 1 ? 1 : b);
}

// GGUF Q4_0 block = 2 bytes of fp16 scale + 16 bytes of quants, 18 bytes, so blocks are only
// 2-byte aligned. One thread moves one block.
__global__ void repack_q4_0_kernel(const uint8_t* __restrict__ raw, uint64_t n_blocks, uint4* __restrict__ quants,
                                   __half* __restrict__ scales) {
    uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const uint16_t* p = reinterpret_cast<const uint16_t*>(raw + 18 * b);
    uint16_t h[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) h[i] = p[i];
    scales[b] = __ushort_as_half(h[0]);
    uint4 q;
    q.x = h[1] | ((uint32_t)h[2] << 16);
    q.y = h[3] | ((uint32_t)h[4] << 16);
    q.z = h[5] | ((uint32_t)h[6] << 16);
    q.w = h[7] | ((uint32_t)h[8] << 16);
    quants[b] = q;
}

// One thread per Q4_0 block: value = f32(q - 8) * f32(d), the single multiply of
// scalar::dequantize_q4_0 (crates/bobcat/src/scalar.rs:98-105), so the f32 output is bit-identical.
template <typename Out>
__global__ void expand_q4_0_kernel(const uint4* __restrict__ quants, const __half* __restrict__ scales,
                                   uint64_t n_blocks, Out* __restrict__ out) {
    uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint4 q = quants[b];
    float d = __half2float(scales[b]);
    uint32_t words[4] = {q.x, q.y, q.z, q.w};
    Out* o = out + 32 * b;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t byte = (words[w] >> (8 * i)) & 0xffu;
            float lo = (float)((int)(byte & 0xfu) - 8) * d;
            float hi = (float)((int)(byte >> 4) - 8) * d;
            o[4 * w + i] = (Out)lo;
            o[16 + 4 * w + i] = (Out)hi;
        }
    }
}

template <typename In, typename Out>
__global__ void convert_kernel(const In* __restrict__ src, Out* __restrict__ dst, uint64_t n) {
    pdl_launch_dependents();
    pdl_wait();
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = (Out)(float)src[i];
}

__global__ void silu_mul_kernel(float* __restrict__ x, const float* __restrict__ gate, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float g = gate[i];
        x[i] = g / (1.f + expf(-g)) * x[i];
    }
}

// Dequantise a matrix kept in its GGUF byte layout (Q8_0, Q6_K), one thread per element.
template <typename Out>
__global__ void expand_bytes_kernel(Mat w, Out* __restrict__ out) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)w.n_rows * w.n_cols) return;
    const uint32_t row = (uint32_t)(i / w.n_cols), col = (uint32_t)(i % w.n_cols);
    float v;
    if (w.format == BC_Q8_0) v = q8_0_at(static_cast<const uint8_t*>(w.data) + (uint64_t)row * (w.n_cols >> 5) * kQ8_0BlockBytes, col);
    else v = q6k_at(static_cast<const uint8_t*>(w.data) + (uint64_t)row * (w.n_cols >> 8) * kQ6KBlockBytes, col);
    out[i] = (Out)v;
}

// grid (ceil(n_embd / threads), n_tokens)
__global__ void embed_kernel(Mat w, const uint32_t* __restrict__ tokens, Pos pos, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    uint32_t token = tokens[(pos.ptr ? *pos.ptr : 0u) + pos.value + blockIdx.y];
    uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= w.n_cols) return;
    float v;
    if (w.format == BC_Q4_0) {
        uint64_t block = (uint64_t)token * (w.n_cols >> 5) + (c >> 5);
        const uint8_t* q = reinterpret_cast<const uint8_t*>(static_cast<const uint4*>(w.data) + block);
        uint32_t i = c & 31;
        uint8_t byte = q[i & 15];
        int n = i < 16 ? (byte & 0xf) : (byte >> 4);
        v = (float)(n - 8) * __half2float(w.scales[block]);
    } else if (w.format == BC_F16) {
        v = __half2float(static_cast<const __half*>(w.data)[(uint64_t)token * w.n_cols + c]);
    } else if (w.format == BC_Q8_0) {
        v = q8_0_at(static_cast<const uint8_t*>(w.data) + (uint64_t)token * (w.n_cols >> 5) * kQ8_0BlockBytes, c);
    } else if (w.format == BC_Q6_K) {
        v = q6k_at(static_cast<const uint8_t*>(w.data) + (uint64_t)token * (w.n_cols >> 8) * kQ6KBlockBytes, c);
    } else {
        v = static_cast<const float*>(w.data)[(uint64_t)token * w.n_cols + c];
    }
    out[(uint64_t)blockIdx.y * w.n_cols + c] = v;
}

// One CTA per row: out = w * (x * rsqrt(mean(x^2) + eps)), the order of scalar::rms_norm
// (crates/bobcat/src/scalar.rs:224-229).
__global__ void __launch_bounds__(kThreads) rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                             float* __restrict__ out, uint32_t n_cols, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = x + (uint64_t)blockIdx.x * n_cols;
    float* o = out + (uint64_t)blockIdx.x * n_cols;
    float sumsq = 0.f;
    for (uint32_t c = threadIdx.x; c < n_cols; c += blockDim.x) sumsq += row[c] * row[c];
    float total = block_sum(sumsq, scratch);
    float scale = rsqrtf(total / (float)n_cols + eps);
    for (uint32_t c = threadIdx.x; c < n_cols; c += blockDim.x) o[c] = weight[c] * (row[c] * scale);
}

struct NormRopeParams {
    const float* src;
    void* dst;
    const float* weight;
    uint32_t n_heads, head_dim, head_stride, n_rot, first_pos, src_stride, dst_stride;
    float theta, eps;
    int dst_half;
};

// One warp per (head, token): RMSNorm over head_dim with the shared weight, then the NeoX rotation
// of the first n_rot elements (pairs i, i + n_rot / 2; inverse frequency 1 / theta^(2i / n_rot)
// and angle in f32, as scalar::rope_neox does, crates/bobcat/src/scalar.rs:253-266), then the
// store as f32 or half. grid (n_heads, n_tokens), 32 threads.
__global__ void norm_rope_kernel(NormRopeParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x;
    const uint32_t head = blockIdx.x, token = blockIdx.y;
    const float* src = p.src + (uint64_t)token * p.src_stride + (uint64_t)head * p.head_stride;
    const uint64_t dst_index = (uint64_t)token * p.dst_stride + (uint64_t)head * p.head_dim;
    // head_dim <= 256: each lane holds up to 8 elements, element e = lane + 32 j.
    float v[8];
    float sumsq = 0.f;
    const int per_lane = p.head_dim / 32;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[j] = 0.f;
        if (j < per_lane) {
            v[j] = src[lane + 32 * j];
            sumsq += v[j] * v[j];
        }
    }
    sumsq = warp_sum(sumsq);
    float scale = rsqrtf(sumsq / (float)p.head_dim + p.eps);
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if (j < per_lane) v[j] = p.weight[lane + 32 * j] * (v[j] * scale);
    // Rotation: element e < n_rot / 2 pairs with e + n_rot / 2. n_rot / 2 is a multiple of 16 here
    // only when n_rot is a multiple of 32; handle any even n_rot through shared memory.
    __shared__ float head_values[256];
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if (j < per_lane) head_values[lane + 32 * j] = v[j];
    __syncwarp();
    const uint32_t half_rot = p.n_rot / 2;
    const float pos = (float)(p.first_pos + token);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (j >= per_lane) continue;
        uint32_t e = lane + 32 * j;
        float result = v[j];
        if (e < p.n_rot) {
            uint32_t i = e < half_rot ? e : e - half_rot;
            float inv_freq = 1.0f / powf(p.theta, (float)(2 * i) / (float)p.n_rot);
            float angle = pos * inv_freq;
            float s, c;
            sincosf(angle, &s, &c);
            float a = head_values[i], b = head_values[i + half_rot];
            result = e < half_rot ? a * c - b * s : b * c + a * s;
        }
        if (p.dst_half) static_cast<__half*>(p.dst)[dst_index + e] = __float2half_rn(result);
        else static_cast<float*>(p.dst)[dst_index + e] = result;
    }
}

// The gated short convolution over a batch (crates/bobcat/src/lfm2.rs:456-475): bx = B * X, the
// taps over bx of this token and the kernel - 1 before it (from the batch, or from the history for
// the first tokens), times C. bcx is [n_tokens][3 n_embd], out is [n_tokens][n_embd], history is
// [kernel - 1][n_embd], oldest first. kernel <= 9. One thread per (token, channel); the sum runs in
// the order of the token-by-token recurrence, so batches of any split give the same bits. The
// history is only read here; short_conv_history_kernel rewrites it afterwards.
__device__ __forceinline__ float short_conv_token(const float* __restrict__ bcx, const float* __restrict__ taps,
                                                  const float* __restrict__ history, uint32_t n_embd, uint32_t kernel, uint32_t t, uint32_t ch) {
    const float* row = bcx + (uint64_t)t * 3 * n_embd;
    const float b = row[ch], c = row[n_embd + ch], x = row[2 * n_embd + ch];
    float sum = taps[(uint64_t)ch * kernel + kernel - 1] * (b * x);
    // Tap kk meets the product of token t - (kernel - 1) + kk.
    for (uint32_t kk = 0; kk + 1 < kernel; ++kk) {
        int64_t src = (int64_t)t - (int64_t)(kernel - 1) + kk;
        float past;
        if (src >= 0) {
            const float* r = bcx + (uint64_t)src * 3 * n_embd;
            past = r[ch] * r[2 * n_embd + ch];
        } else {
            past = history[(uint64_t)(src + (int64_t)(kernel - 1)) * n_embd + ch];
        }
        sum += taps[(uint64_t)ch * kernel + kk] * past;
    }
    return c * sum;
}

// With `packed`, the results go out as the fp16 operand of the product that consumes them
// (rows up to the next multiple of 16 tokens zero) instead of as f32 rows.
__global__ void __launch_bounds__(256) short_conv_kernel(const float* __restrict__ bcx, const float* __restrict__ taps,
                                                         const float* __restrict__ history, float* __restrict__ out, __half* __restrict__ packed,
                                                         uint32_t n_embd, uint32_t kernel, uint32_t n_tokens) {
    pdl_launch_dependents();  // the output projection that reads the packed results may set itself up meanwhile
    pdl_wait();
    const uint32_t ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= n_embd) return;
    if (packed) {
        const uint32_t padded = (n_tokens + 15u) & ~15u;
        for (uint32_t t = blockIdx.y; t < padded; t += gridDim.y) {
            const float v = t < n_tokens ? short_conv_token(bcx, taps, history, n_embd, kernel, t, ch) : 0.f;
            packed[packed_operand_index(t, ch, padded / 8)] = __float2half_rn(v);
        }
        return;
    }
    for (uint32_t t = blockIdx.y; t < n_tokens; t += gridDim.y) out[(uint64_t)t * n_embd + ch] = short_conv_token(bcx, taps, history, n_embd, kernel, t, ch);
}

// The history after the batch: slot kk holds the product of token n_tokens - (kernel - 1) + kk, or
// an older slot when the batch is shorter than the history. One thread per channel.
__global__ void short_conv_history_kernel(const float* __restrict__ bcx, float* __restrict__ history, uint32_t n_embd, uint32_t kernel,
                                          uint32_t n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= n_embd) return;
    float next[8];
    for (uint32_t kk = 0; kk + 1 < kernel; ++kk) {
        int64_t src = (int64_t)n_tokens - (int64_t)(kernel - 1) + kk;
        if (src >= 0) {
            const float* r = bcx + (uint64_t)src * 3 * n_embd;
            next[kk] = r[ch] * r[2 * n_embd + ch];
        } else {
            next[kk] = history[(uint64_t)(src + (int64_t)(kernel - 1)) * n_embd + ch];
        }
    }
    for (uint32_t kk = 0; kk + 1 < kernel; ++kk) history[(uint64_t)kk * n_embd + ch] = next[kk];
}

// One CTA of 1024 threads scans the vocabulary; ties go to the lowest index.
struct ArgmaxOut {
    uint32_t* out;       // direct mode: the word to write
    uint32_t* readback;  // direct mode: optional host-mapped copy
    uint32_t* counter;   // step mode (non-null): position counter
    int advance;
    uint32_t* tokens;
    uint32_t offset;
    uint32_t* ring;
    uint32_t ring_slots;
};

__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ x, uint32_t n, ArgmaxOut o) {
    __shared__ float best_value[32];
    __shared__ uint32_t best_index[32];
    pdl_launch_dependents();
    pdl_wait();
    float value = -INFINITY;
    uint32_t index = 0xffffffffu;
    auto consider = [&](float v, uint32_t i) {
        if (v > value || index == 0xffffffffu) {
            value = v;
            index = i;
        }
    };
    // Eight 16-byte loads in flight per thread, visited in increasing index order so the first
    // maximum wins; whatever does not fill a float4 goes one by one.
    const uint32_t n4 = (reinterpret_cast<uintptr_t>(x) & 15) == 0 ? n / 4 : 0;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (uint32_t base = threadIdx.x; base < n4; base += blockDim.x * 8) {
        float4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            uint32_t i = base + k * blockDim.x;
            v[k] = i < n4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            uint32_t i = base + k * blockDim.x;
            if (i < n4) {
                consider(v[k].x, 4 * i);
                consider(v[k].y, 4 * i + 1);
                consider(v[k].z, 4 * i + 2);
                consider(v[k].w, 4 * i + 3);
            }
        }
    }
    for (uint32_t i = 4 * n4 + threadIdx.x; i < n; i += blockDim.x) consider(x[i], i);
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
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        best_value[warp] = value;
        best_index[warp] = index;
    }
    __syncthreads();
    if (warp == 0) {
        value = best_value[lane];
        index = best_index[lane];
#pragma unroll
        for (int step = 16; step > 0; step >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, value, step);
            uint32_t oi = __shfl_xor_sync(0xffffffffu, index, step);
            if (better(ov, oi, value, index)) {
                value = ov;
                index = oi;
            }
        }
        if (lane == 0) {
            if (o.counter) {
                uint32_t pos = *o.counter;
                if (o.advance) {
                    pos += 1;
                    *o.counter = pos;
                }
                o.tokens[pos + o.offset] = index;
                if (o.ring) o.ring[pos % o.ring_slots] = index;
            } else {
                *o.out = index;
                if (o.readback) *o.readback = index;
            }
        }
    }
}

// One warp per head. Blocks [0, n_heads) treat q, [n_heads, n_heads + n_kv) treat k, the rest copy v.
__global__ void rope_store_kernel(RopeStore p, Pos pos_ref) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x;
    const uint32_t pos = (pos_ref.ptr ? *pos_ref.ptr : 0u) + pos_ref.value;
    const uint32_t hd = p.head_dim, kv_dim = p.n_kv_heads * hd;
    uint32_t block = blockIdx.x;
    if (block >= p.n_heads + p.n_kv_heads) {
        uint32_t head = block - p.n_heads - p.n_kv_heads;
        const float* src = p.v + (uint64_t)head * hd;
        uint64_t at = (uint64_t)pos * kv_dim + (uint64_t)head * hd;
        for (uint32_t e = lane; e < hd; e += 32) {
            if (p.kv_half) static_cast<__half*>(p.v_cache)[at + e] = __float2half_rn(src[e]);
            else static_cast<float*>(p.v_cache)[at + e] = src[e];
        }
        return;
    }
    const bool is_q = block < p.n_heads;
    const uint32_t head = is_q ? block : block - p.n_heads;
    const float* src = is_q ? p.q + (uint64_t)head * p.q_head_stride : p.k + (uint64_t)head * hd;
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
            float a = values[i], b = values[i + half_rot];
            result = e < half_rot ? a * c - b * s : b * c + a * s;
        }
        if (is_q) {
            p.q[(uint64_t)head * p.q_head_stride + e] = result;
        } else {
            uint64_t at = (uint64_t)pos * kv_dim + (uint64_t)head * hd + e;
            if (p.kv_half) static_cast<__half*>(p.k_cache)[at] = __float2half_rn(result);
            else static_cast<float*>(p.k_cache)[at] = result;
        }
    }
}

__global__ void rope_table_kernel(float2* table, uint32_t n_positions, uint32_t n_rot, float theta) {
    const uint32_t half_rot = n_rot / 2;
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)n_positions * half_rot) return;
    const uint32_t pos = (uint32_t)(i / half_rot), pair = (uint32_t)(i % half_rot);
    const float inv_freq = 1.0f / powf(theta, (float)(2 * pair) / (float)n_rot);
    float s, c;
    sincosf((float)pos * inv_freq, &s, &c);
    table[i] = make_float2(c, s);
}

// y[i] += x[i].
__global__ void add_floats_kernel(float* __restrict__ y, const float* __restrict__ x, uint64_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] += x[i];
}

__global__ void advance_kernel(uint32_t* counter) {
    pdl_launch_dependents();
    pdl_wait();
    *counter += 1;
}

}  // namespace

cudaError_t repack_q4_0(cudaStream_t stream, const uint8_t* raw, uint64_t n_blocks, void* quants, __half* scales) {
    if (n_blocks == 0) return cudaSuccess;
    repack_q4_0_kernel<<<blocks_for(n_blocks), kThreads, 0, stream>>>(raw, n_blocks, static_cast<uint4*>(quants), scales);
    return cudaGetLastError();
}

cudaError_t expand(cudaStream_t stream, const Mat& w, void* out, bool out_half) {
    uint64_t n = (uint64_t)w.n_rows * w.n_cols;
    if (n == 0) return cudaSuccess;
    if (w.format == BC_Q4_0) {
        uint64_t nb = n / 32;
        if (out_half)
            expand_q4_0_kernel<__half><<<blocks_for(nb), kThreads, 0, stream>>>(static_cast<const uint4*>(w.data), w.scales, nb, static_cast<__half*>(out));
        else
            expand_q4_0_kernel<float><<<blocks_for(nb), kThreads, 0, stream>>>(static_cast<const uint4*>(w.data), w.scales, nb, static_cast<float*>(out));
    } else if (w.format == BC_Q8_0 || w.format == BC_Q6_K) {
        if (out_half) expand_bytes_kernel<__half><<<blocks_for(n), kThreads, 0, stream>>>(w, static_cast<__half*>(out));
        else expand_bytes_kernel<float><<<blocks_for(n), kThreads, 0, stream>>>(w, static_cast<float*>(out));
    } else if (w.format == BC_F16) {
        if (out_half) convert_kernel<__half, __half><<<blocks_for(n), kThreads, 0, stream>>>(static_cast<const __half*>(w.data), static_cast<__half*>(out), n);
        else convert_kernel<__half, float><<<blocks_for(n), kThreads, 0, stream>>>(static_cast<const __half*>(w.data), static_cast<float*>(out), n);
    } else {
        if (out_half) convert_kernel<float, __half><<<blocks_for(n), kThreads, 0, stream>>>(static_cast<const float*>(w.data), static_cast<__half*>(out), n);
        else convert_kernel<float, float><<<blocks_for(n), kThreads, 0, stream>>>(static_cast<const float*>(w.data), static_cast<float*>(out), n);
    }
    return cudaGetLastError();
}

cudaError_t embed(cudaStream_t stream, const Mat& w, const uint32_t* tokens, Pos pos, float* out, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    dim3 grid(blocks_for(w.n_cols), n_tokens);
    Mat wm = w;
    void* args[] = {&wm, &tokens, &pos, &out};
    return launch_kernel((const void*)embed_kernel, grid, dim3(kThreads), 0, stream, args);
}

cudaError_t rms_norm(cudaStream_t stream, const float* x, const float* weight, float* out, uint32_t n_cols, uint32_t n_rows,
                     float eps) {
    if (n_rows == 0) return cudaSuccess;
    {
        cudaError_t launched = launch_dependent(rms_norm_kernel, dim3(n_rows), dim3(kThreads), 0, stream, x, weight, out, n_cols, eps);
        if (launched != cudaSuccess) return launched;
    }
    return cudaGetLastError();
}

cudaError_t norm_rope(cudaStream_t stream, const float* src, void* dst, bool dst_half, const float* weight, uint32_t n_heads,
                      uint32_t head_dim, uint32_t head_stride, uint32_t n_rot, uint32_t first_pos, uint32_t n_tokens,
                      uint32_t src_stride, uint32_t dst_stride, float theta, float eps) {
    if (n_tokens == 0 || n_heads == 0) return cudaSuccess;
    NormRopeParams p{src, dst, weight, n_heads, head_dim, head_stride, n_rot, first_pos, src_stride, dst_stride, theta, eps, dst_half ? 1 : 0};
    dim3 grid(n_heads, n_tokens);
    {
        cudaError_t launched = launch_dependent(norm_rope_kernel, grid, dim3(32), 0, stream, p);
        if (launched != cudaSuccess) return launched;
    }
    return cudaGetLastError();
}

cudaError_t convert_half(cudaStream_t stream, const float* src, __half* dst, uint64_t n) {
    if (n == 0) return cudaSuccess;
    {
        cudaError_t launched = launch_dependent(convert_kernel<float, __half>, dim3(blocks_for(n)), dim3(kThreads), 0, stream, src, dst, n);
        if (launched != cudaSuccess) return launched;
    }
    return cudaGetLastError();
}

cudaError_t copy_floats(cudaStream_t stream, const float* src, float* dst, uint64_t n) {
    if (n == 0) return cudaSuccess;
    return cudaMemcpyAsync(dst, src, n * sizeof(float), cudaMemcpyDeviceToDevice, stream);
}

cudaError_t silu_mul(cudaStream_t stream, float* x, const float* gate, uint64_t n) {
    if (n == 0) return cudaSuccess;
    silu_mul_kernel<<<blocks_for(n), kThreads, 0, stream>>>(x, gate, n);
    return cudaGetLastError();
}

cudaError_t short_conv(cudaStream_t stream, const float* bcx, const float* taps, float* history, float* out, uint32_t n_embd,
                       uint32_t kernel, uint32_t n_tokens, void* packed) {
    if (n_tokens == 0) return cudaSuccess;
    if (packed && n_embd % 64 != 0) return cudaErrorInvalidValue;
    const uint32_t rows = packed ? ((n_tokens + 15u) & ~15u) : n_tokens;
    cudaError_t e = launch_dependent(short_conv_kernel, dim3(blocks_for(n_embd, 256), rows < 65535u ? rows : 65535u), dim3(256), 0, stream, bcx, taps,
                                     static_cast<const float*>(history), out, static_cast<__half*>(packed), n_embd, kernel, n_tokens);
    if (e != cudaSuccess) return e;
    return launch_dependent(short_conv_history_kernel, dim3(blocks_for(n_embd, 128)), dim3(128), 0, stream, bcx, history, n_embd, kernel, n_tokens);
}

cudaError_t argmax(cudaStream_t stream, const float* x, uint32_t n, uint32_t* out, uint32_t* readback) {
    ArgmaxOut o{out, readback, nullptr, 0, nullptr, 0, nullptr, 1};
    void* args[] = {&x, &n, &o};
    return launch_kernel((const void*)argmax_kernel, dim3(1), dim3(1024), 0, stream, args);
}

cudaError_t argmax_step(cudaStream_t stream, const float* x, uint32_t n, uint32_t* counter, bool advance, uint32_t* tokens,
                        uint32_t offset, uint32_t* ring, uint32_t ring_slots) {
    ArgmaxOut o{nullptr, nullptr, counter, advance ? 1 : 0, tokens, offset, ring, ring_slots ? ring_slots : 1};
    void* args[] = {&x, &n, &o};
    return launch_kernel((const void*)argmax_kernel, dim3(1), dim3(1024), 0, stream, args);
}

cudaError_t add_floats(cudaStream_t stream, float* y, const float* x, uint64_t n) {
    if (n == 0) return cudaSuccess;
    void* args[] = {&y, &x, &n};
    return launch_kernel((const void*)add_floats_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, args);
}

cudaError_t advance(cudaStream_t stream, uint32_t* counter) {
    void* args[] = {&counter};
    return launch_kernel((const void*)advance_kernel, dim3(1), dim3(1), 0, stream, args);
}

cudaError_t rope_table(cudaStream_t stream, float2* table, uint32_t n_positions, uint32_t n_rot, float theta) {
    const uint64_t items = (uint64_t)n_positions * (n_rot / 2);
    if (items == 0) return cudaSuccess;
    rope_table_kernel<<<(unsigned)((items + 255) / 256), 256, 0, stream>>>(table, n_positions, n_rot, theta);
    return cudaGetLastError();
}

cudaError_t rope_store(cudaStream_t stream, const RopeStore& p, Pos pos) {
    RopeStore params = p;
    void* args[] = {&params, &pos};
    return launch_kernel((const void*)rope_store_kernel, dim3(p.n_heads + 2 * p.n_kv_heads), dim3(32), 0, stream, args);
}

}  // namespace k
}  // namespace bc
