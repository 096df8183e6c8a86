// Causal grouped-query attention over a contiguous KV cache, split over 64-position chunks with a
// combine pass (the structure of attention_chunk / attention_wide / attention_combine in
// crates/bobcat-metal/src/attention.metal:26-265, :496-540; host side backend.rs:2150-2320).
//
// Chunk pass: one CTA per (KV head, chunk, query). The query heads of the group that shares the KV
// head are scored together, so each key and value row is read from the cache once per group.
// Each CTA writes, per query head, the chunk's score maximum, the sum of exponentials and the
// unnormalised weighted value sum. Combine pass: one CTA per (query head, query) rescales the
// chunk partials by exp(max_c - max) and divides. A decode step over a half-precision cache takes
// attention_decode_kernel for its chunk pass: the same partials from 16-byte cache loads with the
// group's running sums in registers.

#include "common.h"
#include "device_utils.cuh"
#include "kernels.h"

namespace bc {
namespace k {

namespace {

constexpr int kChunk = 64;         // positions per chunk of a batch
constexpr int kDecodeChunk = 16;   // positions per chunk when only a few queries run: more, smaller CTAs fill the device
// Longer contexts take longer chunks: the chunk count (and with it the partials the combine pass
// reads back, head_dim + 2 floats per chunk and head) stays a small fraction of the cache traffic,
// and a replayed step, whose grid covers the whole context, launches a few thousand CTAs at most.
inline uint32_t decode_chunk(uint32_t n_ctx) { return n_ctx <= 4096 ? (uint32_t)kDecodeChunk : n_ctx <= 32768 ? 64u : 256u; }
constexpr int kDecodeQueries = 4;  // up to this many queries use the small chunks
constexpr int kMaxGroup = 8;       // query heads per KV head
constexpr int kQueryBatch = 64;    // queries per launch, which bounds the scratch
constexpr int kChunkThreads = 256;

template <typename T>
__device__ __forceinline__ float load_kv(const T* p);
template <>
__device__ __forceinline__ float load_kv<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_kv<__half>(const __half* p) { return __half2float(*p); }

struct ChunkParams {
    const float* q;
    const void* k_cache;
    const void* v_cache;
    float* scratch;
    uint32_t n_heads, n_kv_heads, head_dim, first_pos, n_ctx, q_stride, q_head_stride;
    uint32_t query0;      // first query of this launch
    uint32_t max_chunks;  // chunks the scratch holds per (query, head)
    const uint32_t* pos_ptr;  // when set, added to first_pos at run time
    uint32_t chunk;           // positions per chunk
    // The fused decode step: q is the raw projection, and the new position's key and value rows
    // come from raw_k and raw_v instead of the caches, which this launch also fills.
    const float* raw_k;
    const float* raw_v;
    const float* q_norm;
    const float* k_norm;
    float eps, theta;
    const float2* rope_table;  // [position][HD / 2] (cos, sin), or null to compute them here
};

// Scratch layout: [query in batch][head][chunk][head_dim + 2] = (max, sum, acc[head_dim]).
template <typename T>
__global__ void __launch_bounds__(kChunkThreads) attention_chunk_kernel(ChunkParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t kv_head = blockIdx.x, chunk = blockIdx.y, qi = blockIdx.z;
    const uint32_t query = p.query0 + qi;
    const uint32_t pos = p.first_pos + (p.pos_ptr ? *p.pos_ptr : 0u) + query;  // the query attends to positions 0..pos
    const uint32_t start = chunk * p.chunk;
    if (start > pos) return;
    const uint32_t count = min(p.chunk, pos + 1 - start);
    const uint32_t hd = p.head_dim, group = p.n_heads / p.n_kv_heads;
    const uint32_t kv_dim = p.n_kv_heads * hd;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = kChunkThreads / 32;

    extern __shared__ float smem[];
    float* qs = smem;                         // [group][hd], pre-scaled
    float* scores = qs + group * hd;           // [group][chunk]
    float* partial = scores + group * p.chunk; // [slices][group][hd]
    __shared__ float head_max[kMaxGroup], head_sum[kMaxGroup];

    const float scale = 1.0f / sqrtf((float)hd);
    for (uint32_t i = tid; i < group * hd; i += kChunkThreads) {
        uint32_t g = i / hd, d = i % hd;
        uint32_t head = kv_head * group + g;
        qs[i] = p.q[(uint64_t)query * p.q_stride + (uint64_t)head * p.q_head_stride + d] * scale;
    }
    __syncthreads();

    const T* kc = static_cast<const T*>(p.k_cache) + (uint64_t)start * kv_dim + (uint64_t)kv_head * hd;
    const T* vc = static_cast<const T*>(p.v_cache) + (uint64_t)start * kv_dim + (uint64_t)kv_head * hd;

    // Scores: a warp per position, lanes across the head.
    for (uint32_t t = warp; t < count; t += n_warps) {
        float dot[kMaxGroup];
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) dot[g] = 0.f;
        for (uint32_t d = lane; d < hd; d += 32) {
            float kv = load_kv<T>(kc + (uint64_t)t * kv_dim + d);
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g)
                if (g < group) dot[g] += kv * qs[g * hd + d];
        }
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            if (g < group) {
                float s = warp_sum(dot[g]);
                if (lane == 0) scores[g * p.chunk + t] = s;
            }
        }
    }
    __syncthreads();

    // Per head: chunk maximum, exponentials, their sum. A warp per head.
    for (uint32_t g = warp; g < group; g += n_warps) {
        float m = -INFINITY;
        for (uint32_t t = lane; t < count; t += 32) m = fmaxf(m, scores[g * p.chunk + t]);
        m = warp_max(m);
        float sum = 0.f;
        for (uint32_t t = lane; t < count; t += 32) {
            float e = expf(scores[g * p.chunk + t] - m);
            scores[g * p.chunk + t] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        if (lane == 0) {
            head_max[g] = m;
            head_sum[g] = sum;
        }
    }
    __syncthreads();

    // Weighted value sums: thread (slice, d) walks every n_slices-th position of the chunk.
    const uint32_t n_slices = kChunkThreads / hd;  // hd <= 256 and divides 256
    const uint32_t d = tid % hd, slice = tid / hd;
    float acc[kMaxGroup];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) acc[g] = 0.f;
    if (slice < n_slices) {
        for (uint32_t t = slice; t < count; t += n_slices) {
            float v = load_kv<T>(vc + (uint64_t)t * kv_dim + d);
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g)
                if (g < group) acc[g] += scores[g * p.chunk + t] * v;
        }
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g)
            if (g < group) partial[(slice * group + g) * hd + d] = acc[g];
    }
    __syncthreads();
    for (uint32_t i = tid; i < group * hd; i += kChunkThreads) {
        uint32_t g = i / hd, dd = i % hd;
        float total = 0.f;
        for (uint32_t s = 0; s < n_slices; ++s) total += partial[(s * group + g) * hd + dd];
        uint32_t head = kv_head * group + g;
        float* out = p.scratch + (((uint64_t)qi * p.n_heads + head) * p.max_chunks + chunk) * (hd + 2);
        out[2 + dd] = total;
        if (dd == 0) {
            out[0] = head_max[g];
            out[1] = head_sum[g];
        }
    }
}

// Decode form of the chunk pass for a half-precision cache: the same partials as
// attention_chunk_kernel, computed with 16-byte cache loads. A lane owns 8 consecutive elements of a
// row, HD / 8 lanes cover a row and a warp reads 256 / HD rows with one load per lane; the query
// heads of the group and their running (max, sum, weighted values) stay in registers. The rows of
// a warp are merged with shuffles and the four warps through shared memory.
constexpr int kDecodeThreads = 128;

__device__ __forceinline__ void unpack_row(const uint4& raw, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 v = __half22float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}

// Per-head RMSNorm, norm weights and NeoX rotation of the 8 elements d0..d0+7 a lane holds of a
// head (the lanes of a row hold the whole head); the same arithmetic as rope_store_kernel, with the
// rotation over the whole head. `rot[i]` is (cos, sin) of pair i at this position.
template <int HD>
__device__ __forceinline__ void norm_rotate(float (&v)[8], const float* __restrict__ weight, float eps, int d0, const float2* rot) {
    constexpr int kLanesPerRow = HD / 8;
    float sumsq = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sumsq += v[i] * v[i];
#pragma unroll
    for (int o = 1; o < kLanesPerRow; o <<= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
    const float scale = rsqrtf(sumsq / (float)HD + eps);
    const bool low = d0 < HD / 2;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = weight[d0 + i] * (v[i] * scale);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, v[i], kLanesPerRow / 2);  // element d0 + i +- HD / 2
        const float2 cs = rot[(d0 % (HD / 2)) + i];
        v[i] = low ? v[i] * cs.x - other * cs.y : v[i] * cs.x + other * cs.y;
    }
}

__device__ __forceinline__ uint4 pack_row(const float (&f)[8]) {
    uint4 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return raw;
}

template <int HD, int GROUP, bool FUSED>
__global__ void __launch_bounds__(kDecodeThreads) attention_decode_kernel(ChunkParams p) {
    constexpr int kLanesPerRow = HD / 8, kRowsPerLoad = 32 / kLanesPerRow, kWarps = kDecodeThreads / 32;
    pdl_launch_dependents();
    const uint32_t kv_head = blockIdx.x, chunk = blockIdx.y, qi = blockIdx.z;
    const uint32_t query = p.query0 + qi;
    const uint32_t start = chunk * p.chunk;
    const uint32_t group = p.n_heads / p.n_kv_heads, kv_dim = p.n_kv_heads * HD;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane / kLanesPerRow, d0 = (lane % kLanesPerRow) * 8;

    __shared__ float merged[kWarps][GROUP][HD + 2];

    const __half* kc = static_cast<const __half*>(p.k_cache) + (uint64_t)start * kv_dim + (uint64_t)kv_head * HD + d0;
    const __half* vc = static_cast<const __half*>(p.v_cache) + (uint64_t)start * kv_dim + (uint64_t)kv_head * HD + d0;

    // The first row's loads go out before the query arrives. `base` is the same for the whole
    // warp, so the shuffles below run with every lane present; rows past the chunk's end only skip
    // the update. In the fused step the cache rows of earlier positions were written by earlier
    // tokens' launches, long finished, so these loads also go out before the wait for the
    // predecessor, for every row of the chunk inside the context: which rows count is known
    // after the wait, and the new position's row is replaced below. They bypass L1, which must
    // not keep a row read before it was written.
    uint32_t base = warp * kRowsPerLoad;
    uint4 k_raw = make_uint4(0, 0, 0, 0), v_raw = make_uint4(0, 0, 0, 0);
    if (FUSED && base + sub < p.chunk && start + base + sub < p.n_ctx) {
        k_raw = __ldcg(reinterpret_cast<const uint4*>(kc + (uint64_t)(base + sub) * kv_dim));
        v_raw = __ldcg(reinterpret_cast<const uint4*>(vc + (uint64_t)(base + sub) * kv_dim));
    }
    pdl_wait();
    const uint32_t pos = p.first_pos + (p.pos_ptr ? *p.pos_ptr : 0u) + query;
    if (start > pos) return;
    const uint32_t count = min(p.chunk, pos + 1 - start);
    if (!FUSED && base + sub < count) {
        k_raw = __ldg(reinterpret_cast<const uint4*>(kc + (uint64_t)(base + sub) * kv_dim));
        v_raw = __ldg(reinterpret_cast<const uint4*>(vc + (uint64_t)(base + sub) * kv_dim));
    }

    // Fused step: the rotation's cosines and sines for this position, one pair per thread; the
    // CTA whose chunk ends at the new position prepares that position's key and value rows,
    // rounds them to the cache's precision, stores them, and uses them in place of the cache.
    __shared__ float2 rot[HD / 2];
    const uint32_t new_row = pos - start;  // the new position's row, when it lies in this chunk
    const bool holds_new = FUSED && new_row < p.chunk;
    uint4 k_new = make_uint4(0, 0, 0, 0), v_new = make_uint4(0, 0, 0, 0);
    if (FUSED) {
        if (tid < HD / 2) {
            if (p.rope_table) {
                rot[tid] = p.rope_table[(uint64_t)pos * (HD / 2) + tid];
            } else {
                const float inv_freq = 1.0f / powf(p.theta, (float)(2 * tid) / (float)HD);
                float sn, cs;
                sincosf((float)pos * inv_freq, &sn, &cs);
                rot[tid] = make_float2(cs, sn);
            }
        }
        __syncthreads();
        if (holds_new) {
            const float* kp = p.raw_k + (uint64_t)kv_head * HD + d0;
            const float* vp = p.raw_v + (uint64_t)kv_head * HD + d0;
            const float4 ka = *reinterpret_cast<const float4*>(kp), kb = *reinterpret_cast<const float4*>(kp + 4);
            const float4 va = *reinterpret_cast<const float4*>(vp), vb = *reinterpret_cast<const float4*>(vp + 4);
            float kf[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
            const float vf[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
            norm_rotate<HD>(kf, p.k_norm, p.eps, d0, rot);
            k_new = pack_row(kf);
            v_new = pack_row(vf);
            if (warp == 0 && sub == 0) {
                const uint64_t at = (uint64_t)pos * kv_dim + (uint64_t)kv_head * HD + d0;
                *reinterpret_cast<uint4*>(static_cast<__half*>(const_cast<void*>(p.k_cache)) + at) = k_new;
                *reinterpret_cast<uint4*>(static_cast<__half*>(const_cast<void*>(p.v_cache)) + at) = v_new;
            }
            if (base + sub == new_row) {
                k_raw = k_new;
                v_raw = v_new;
            }
        }
    }

    const float scale = 1.0f / sqrtf((float)HD);
    float qv[GROUP][8], acc[GROUP][8], top[GROUP], sum[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
        top[g] = -INFINITY;
        sum[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
        if (g < (int)group) {
            const float* qp = p.q + (uint64_t)query * p.q_stride + (uint64_t)(kv_head * group + g) * p.q_head_stride + d0;
            float4 a = *reinterpret_cast<const float4*>(qp), b = *reinterpret_cast<const float4*>(qp + 4);
            float raw[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            if (FUSED) norm_rotate<HD>(raw, p.q_norm, p.eps, d0, rot);
#pragma unroll
            for (int i = 0; i < 8; ++i) qv[g][i] = raw[i] * scale;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) qv[g][i] = 0.f;
        }
    }

    while (base < count) {
        float kf[8], vf[8];
        unpack_row(k_raw, kf);
        unpack_row(v_raw, vf);
        const bool valid = base + sub < count;
        const uint32_t next = base + kWarps * kRowsPerLoad;
        if (holds_new && next + sub == new_row) {
            k_raw = k_new;  // not in the cache when this launch began: never read it from there
            v_raw = v_new;
        } else if (next + sub < count) {
            k_raw = __ldg(reinterpret_cast<const uint4*>(kc + (uint64_t)(next + sub) * kv_dim));
            v_raw = __ldg(reinterpret_cast<const uint4*>(vc + (uint64_t)(next + sub) * kv_dim));
        }
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) dot += kf[i] * qv[g][i];
#pragma unroll
            for (int o = 1; o < kLanesPerRow; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (valid) {
                const float m = fmaxf(top[g], dot);
                const float keep = expf(top[g] - m), w = expf(dot - m);  // exp(-inf) = 0 on the first row
                sum[g] = sum[g] * keep + w;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * keep + w * vf[i];
                top[g] = m;
            }
        }
        base = next;
    }

    // Merge the rows of the warp: lanes that hold the same elements of different rows.
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
#pragma unroll
        for (int o = kLanesPerRow; o < 32; o <<= 1) {
            const float other_top = __shfl_xor_sync(0xffffffffu, top[g], o);
            const float other_sum = __shfl_xor_sync(0xffffffffu, sum[g], o);
            const float m = fmaxf(top[g], other_top);
            const float mine = top[g] == -INFINITY ? 0.f : expf(top[g] - m);
            const float theirs = other_top == -INFINITY ? 0.f : expf(other_top - m);
            sum[g] = sum[g] * mine + other_sum * theirs;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, acc[g][i], o);
                acc[g][i] = acc[g][i] * mine + other * theirs;
            }
            top[g] = m;
        }
        if (sub == 0 && g < (int)group) {
            float* out = merged[warp][g];
            if (d0 == 0) {
                out[0] = top[g];
                out[1] = sum[g];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) out[2 + d0 + i] = acc[g][i];
        }
    }
    __syncthreads();

    // Merge the warps and write the chunk's partial.
    for (uint32_t i = tid; i < group * HD; i += kDecodeThreads) {
        const uint32_t g = i / HD, d = i % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) m = fmaxf(m, merged[w][g][0]);
        float total = 0.f, weight = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float t = merged[w][g][0];
            const float f = t == -INFINITY ? 0.f : expf(t - m);
            weight += merged[w][g][1] * f;
            total += merged[w][g][2 + d] * f;
        }
        const uint32_t head = kv_head * group + g;
        float* out = p.scratch + (((uint64_t)qi * p.n_heads + head) * p.max_chunks + chunk) * (HD + 2);
        out[2 + d] = total;
        if (d == 0) {
            out[0] = m;
            out[1] = weight;
        }
    }
}

template <int HD>
const void* decode_kernel_for(uint32_t group, bool fused) {
    if (fused) {
        if (group <= 2) return (const void*)attention_decode_kernel<HD, 2, true>;
        if (group <= 4) return (const void*)attention_decode_kernel<HD, 4, true>;
        return (const void*)attention_decode_kernel<HD, 8, true>;
    }
    if (group <= 2) return (const void*)attention_decode_kernel<HD, 2, false>;
    if (group <= 4) return (const void*)attention_decode_kernel<HD, 4, false>;
    return (const void*)attention_decode_kernel<HD, 8, false>;
}

// The decode form covers a half-precision cache, heads of 64, 128 or 256 elements and 16-byte aligned
// query rows; everything else takes the general kernel.
bool decode_shape(bool kv_half, const AttentionShape& s) {
    return kv_half && s.n_queries <= (uint32_t)kDecodeQueries && s.q_stride % 4 == 0 && s.q_head_stride % 4 == 0 &&
           (s.head_dim == 64 || s.head_dim == 128 || s.head_dim == 256);
}

const void* decode_kernel(bool kv_half, const AttentionShape& s, const float* q, const void* k_cache, const void* v_cache, bool fused = false) {
    if (!decode_shape(kv_half, s) || ((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16 != 0) return nullptr;
    const uint32_t group = s.n_heads / s.n_kv_heads;
    switch (s.head_dim) {
        case 64: return decode_kernel_for<64>(group, fused);
        case 128: return decode_kernel_for<128>(group, fused);
        default: return decode_kernel_for<256>(group, fused);
    }
}

struct CombineParams {
    const float* scratch;
    float* out;
    uint32_t n_heads, head_dim, first_pos, query0, max_chunks;
    const uint32_t* pos_ptr;
    uint32_t chunk;
};

// grid (n_heads, queries in batch), kCombineParts * head_dim threads. The threads first share out
// the chunks' maxima and sums (so the exponentials are computed once, in parallel); then part r
// of the threads adds up every kCombineParts-th chunk, each thread one element of the head with
// independent loads, and the parts are added in order.
constexpr int kCombineParts = 4;
constexpr int kCombineSlice = 512;  // chunks whose weights shared memory holds at a time

__global__ void attention_combine_kernel(CombineParams p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float weights[kCombineSlice];  // exp(max_c - max) of a slice of chunks
    __shared__ float across[32];
    extern __shared__ float parts[];           // [kCombineParts][head_dim]
    const uint32_t head = blockIdx.x, qi = blockIdx.y, tid = threadIdx.x, hd = p.head_dim;
    const uint32_t d = tid % hd, part = tid / hd, n_warps = blockDim.x / 32;
    const uint32_t query = p.query0 + qi, pos = p.first_pos + (p.pos_ptr ? *p.pos_ptr : 0u) + query;
    const uint32_t n_chunks = pos / p.chunk + 1;
    const float* base = p.scratch + ((uint64_t)qi * p.n_heads + head) * p.max_chunks * (hd + 2);
    // With up to kCombineParts * kCombineHeld chunks a thread's share of the weighted values is
    // read now, together with the maxima, so the combine costs one trip to L2 instead of three.
    constexpr int kCombineHeld = 16;
    const bool held = n_chunks <= (uint32_t)(kCombineParts * kCombineHeld);
    float mine[kCombineHeld];
    if (held) {
#pragma unroll
        for (int j = 0; j < kCombineHeld; ++j) {
            const uint32_t c = part + (uint32_t)j * kCombineParts;
            mine[j] = c < n_chunks ? base[(uint64_t)c * (hd + 2) + 2 + d] : 0.f;
        }
    }
    float m = -INFINITY;
    for (uint32_t c = tid; c < n_chunks; c += blockDim.x) m = fmaxf(m, base[(uint64_t)c * (hd + 2)]);
    m = warp_max(m);
    if ((tid & 31) == 0) across[tid >> 5] = m;
    __syncthreads();
    m = across[0];
    for (uint32_t w = 1; w < n_warps; ++w) m = fmaxf(m, across[w]);
    float sum = 0.f, acc = 0.f;
    for (uint32_t c0 = 0; c0 < n_chunks; c0 += kCombineSlice) {
        const uint32_t count = min((uint32_t)kCombineSlice, n_chunks - c0);
        __syncthreads();
        for (uint32_t c = tid; c < count; c += blockDim.x) {
            const float* at = base + (uint64_t)(c0 + c) * (hd + 2);
            const float w = expf(at[0] - m);
            weights[c] = w;
            sum += w * at[1];
        }
        __syncthreads();
        if (held) {
#pragma unroll
            for (int j = 0; j < kCombineHeld; ++j) {
                const uint32_t c = part + (uint32_t)j * kCombineParts;
                if (c < count) acc += weights[c] * mine[j];
            }
        } else {
#pragma unroll 8
            for (uint32_t c = part; c < count; c += kCombineParts) acc += weights[c] * base[(uint64_t)(c0 + c) * (hd + 2) + 2 + d];
        }
    }
    sum = warp_sum(sum);
    __syncthreads();  // the maxima in `across` have been read
    if ((tid & 31) == 0) across[tid >> 5] = sum;
    parts[part * hd + d] = acc;
    __syncthreads();
    if (part == 0) {
        float total = 0.f, all = 0.f;
        for (uint32_t w = 0; w < n_warps; ++w) total += across[w];
#pragma unroll
        for (int r = 0; r < kCombineParts; ++r) all += parts[r * hd + d];
        p.out[(uint64_t)query * p.n_heads * hd + (uint64_t)head * hd + d] = all / total;
    }
}

}  // namespace

uint64_t attention_scratch_floats(uint32_t n_heads, uint32_t head_dim, uint32_t n_ctx, uint32_t n_queries) {
    // A buffer sized for n queries also serves any smaller count, which may use the small chunks.
    uint64_t queries = n_queries < (uint32_t)kQueryBatch ? n_queries : (uint32_t)kQueryBatch;
    uint64_t few = n_queries < (uint32_t)kDecodeQueries ? n_queries : (uint32_t)kDecodeQueries;
    uint64_t batch = queries * (((uint64_t)n_ctx + kChunk - 1) / kChunk);
    uint64_t decode = few * (((uint64_t)n_ctx + kDecodeChunk - 1) / kDecodeChunk);
    return (batch > decode ? batch : decode) * n_heads * (head_dim + 2);
}

int attention_launches(bool kv_half, const AttentionShape& s) {
    if (attention_flash_supported(kv_half, s)) return 1;
    return 2 * (int)((s.n_queries + kQueryBatch - 1) / kQueryBatch);
}

cudaError_t attention(cudaStream_t stream, const float* q, const void* k_cache, const void* v_cache, bool kv_half,
                      float* scratch, float* out, const AttentionShape& s) {
    if (s.n_queries == 0) return cudaSuccess;
    // The tensor-core kernel reads q and out 8 bytes and the caches 16 bytes at a time; views that
    // do not start on those boundaries take the chunk kernels, whose loads are scalar.
    const bool flash_aligned = ((uintptr_t)q | (uintptr_t)out) % 8 == 0 && ((uintptr_t)k_cache | (uintptr_t)v_cache) % 16 == 0;
    if (flash_aligned && attention_flash_supported(kv_half, s)) return attention_flash(stream, q, k_cache, v_cache, out, s);
    const uint32_t group = s.n_heads / s.n_kv_heads;
    const uint32_t chunk = s.n_queries <= (uint32_t)kDecodeQueries ? decode_chunk(s.n_ctx) : (uint32_t)kChunk;
    const uint32_t max_chunks = (s.n_ctx + chunk - 1) / chunk;
    const uint32_t n_slices = kChunkThreads / s.head_dim;
    size_t smem = ((size_t)group * s.head_dim + (size_t)group * chunk + (size_t)n_slices * group * s.head_dim) * sizeof(float);
    cudaError_t e;
    if (kv_half) e = ensure_dynamic_smem(reinterpret_cast<const void*>(attention_chunk_kernel<__half>), smem);
    else e = ensure_dynamic_smem(reinterpret_cast<const void*>(attention_chunk_kernel<float>), smem);
    if (e != cudaSuccess) return e;
    for (uint32_t q0 = 0; q0 < s.n_queries; q0 += kQueryBatch) {
        uint32_t nq = s.n_queries - q0 < (uint32_t)kQueryBatch ? s.n_queries - q0 : (uint32_t)kQueryBatch;
        uint32_t last_pos = s.first_pos + q0 + nq - 1;
        ChunkParams cp{q, k_cache, v_cache, scratch, s.n_heads, s.n_kv_heads, s.head_dim, s.first_pos, s.n_ctx,
                       s.q_stride, s.q_head_stride, q0, max_chunks, s.pos_ptr, chunk, nullptr, nullptr, nullptr, nullptr, 0.f, 0.f, nullptr};
        // With a run-time position the grid covers every chunk of the context; CTAs past the position exit at once.
        dim3 grid(s.n_kv_heads, s.pos_ptr ? max_chunks : last_pos / chunk + 1, nq);
        void* chunk_args[] = {&cp};
        const void* fast = decode_kernel(kv_half, s, q, k_cache, v_cache);
        if (fast) {
            if ((e = launch_kernel(fast, grid, dim3(kDecodeThreads), 0, stream, chunk_args)) != cudaSuccess) return e;
        } else {
            const void* chunk_kernel = kv_half ? (const void*)attention_chunk_kernel<__half> : (const void*)attention_chunk_kernel<float>;
            if ((e = launch_kernel(chunk_kernel, grid, dim3(kChunkThreads), smem, stream, chunk_args)) != cudaSuccess) return e;
        }
        CombineParams mp{scratch, out, s.n_heads, s.head_dim, s.first_pos, q0, max_chunks, s.pos_ptr, chunk};
        void* combine_args[] = {&mp};
        if ((e = launch_kernel((const void*)attention_combine_kernel, dim3(s.n_heads, nq), dim3(kCombineParts * s.head_dim),
                               (size_t)kCombineParts * s.head_dim * sizeof(float), stream, combine_args)) != cudaSuccess)
            return e;
    }
    return cudaSuccess;
}

bool attention_step_supported(const RopeStore& r, const AttentionShape& s) {
    return r.kv_half && s.n_queries == 1 && decode_shape(true, s) && r.n_rot == s.head_dim && r.q_head_stride == s.q_head_stride &&
           ((uintptr_t)r.q | (uintptr_t)r.k | (uintptr_t)r.v | (uintptr_t)r.k_cache | (uintptr_t)r.v_cache) % 16 == 0;
}

cudaError_t attention_step(cudaStream_t stream, const RopeStore& r, float* scratch, float* out, const AttentionShape& s) {
    const uint32_t chunk = decode_chunk(s.n_ctx), max_chunks = (s.n_ctx + chunk - 1) / chunk;
    ChunkParams cp{r.q, r.k_cache, r.v_cache, scratch, s.n_heads, s.n_kv_heads, s.head_dim, s.first_pos, s.n_ctx,
                   s.q_stride, s.q_head_stride, 0, max_chunks, s.pos_ptr, chunk, r.k, r.v, r.q_norm, r.k_norm, r.eps, r.theta, r.table};
    dim3 grid(s.n_kv_heads, s.pos_ptr ? max_chunks : s.first_pos / chunk + 1, 1);
    void* chunk_args[] = {&cp};
    const void* kernel = decode_kernel(true, s, r.q, r.k_cache, r.v_cache, true);
    if (!kernel) return cudaErrorInvalidValue;
    cudaError_t e = launch_kernel(kernel, grid, dim3(kDecodeThreads), 0, stream, chunk_args);
    if (e != cudaSuccess) return e;
    CombineParams mp{scratch, out, s.n_heads, s.head_dim, s.first_pos, 0, max_chunks, s.pos_ptr, chunk};
    void* combine_args[] = {&mp};
    return launch_kernel((const void*)attention_combine_kernel, dim3(s.n_heads, 1), dim3(kCombineParts * s.head_dim),
                         (size_t)kCombineParts * s.head_dim * sizeof(float), stream, combine_args);
}

}  // namespace k
}  // namespace bc

// ------------------------------------------------------------------------------------------------
// Attention without any allocation.
//
// Some embedders may not allocate device memory at all while they decode: an engine whose device
// memory is one pool planned up front and owned by its own allocator hands a plugin only the
// tensors of the call, and a serving loop that must not stall cannot afford cudaMalloc, which
// synchronises the whole device. For them the chunk partials live in the fixed array below, which
// every GPU that loads this library holds from load until exit.
// ------------------------------------------------------------------------------------------------

// 2 Mi floats = 8 MiB. A call needs ceil(positions / chunk) * queries in a pass * n_heads *
// (head_dim + 2) floats, positions = first_pos + n_queries, chunk = 16 positions for up to 4
// queries and 64 for more (at most 64 queries in a pass): one query over 32 heads of 64 elements
// fits up to 15 872 positions, a 64-query pass of the same heads up to 960 positions.
#define BC_STATIC_ATTENTION_SCRATCH_FLOATS (2u << 20)
static __device__ __align__(256) float bc_static_attention_scratch[BC_STATIC_ATTENTION_SCRATCH_FLOATS];

extern "C" bc_status bc_attention_static(void* stream, const float* q, const void* k_cache, const void* v_cache, int32_t kv_half,
                                         float* out, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t first_pos,
                                         uint32_t n_queries, uint32_t n_ctx) {
    using namespace bc;
    if (!q || !k_cache || !v_cache || !out) return fail(BC_ERR_ARGUMENT, "q, the caches and out must be non-null");
    if (n_kv_heads == 0 || n_heads % n_kv_heads != 0 || n_heads / n_kv_heads > 8 || head_dim == 0 || head_dim % 32 != 0 || head_dim > 256 ||
        n_queries == 0 || (uint64_t)first_pos + n_queries > n_ctx)
        return fail(BC_ERR_ATTENTION_LIMITS,
                    "attention needs heads of a multiple of 32 up to 256 elements, at most 8 query heads per KV head and queries inside the "
                    "context, got head_dim %u, %u/%u heads, positions %u..%u of %u",
                    head_dim, n_heads, n_kv_heads, first_pos, first_pos + n_queries, n_ctx);
    // The partials are laid out for the positions in use, not for the cache's capacity: positions
    // are known here (no device-side position), so no chunk past the last query is ever written.
    const uint32_t positions = first_pos + n_queries;
    uint64_t need = k::attention_scratch_floats(n_heads, head_dim, positions, n_queries);
    if (need > BC_STATIC_ATTENTION_SCRATCH_FLOATS)
        return fail(BC_ERR_ARGUMENT,
                    "this shape needs %llu floats of chunk partials and the built-in scratch holds %u; use bc_op_attention with a scratch "
                    "buffer of your own, or fewer positions",
                    (unsigned long long)need, (unsigned)BC_STATIC_ATTENTION_SCRATCH_FLOATS);
    // The array's name is only a host-side handle; the kernels need its address on the current
    // device, looked up once per device.
    static float* address_on_device[64] = {};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (device < 0 || device >= 64) return fail(BC_ERR_ARGUMENT, "device index %d is outside the table of 64", device);
    float* scratch = address_on_device[device];
    if (!scratch) {
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), bc_static_attention_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(bc_static_attention_scratch)");
        address_on_device[device] = scratch;
    }
    (void)n_ctx;
    k::AttentionShape shape{n_heads, n_kv_heads, head_dim, first_pos, n_queries, positions, n_heads * head_dim, head_dim};
    e = k::attention(static_cast<cudaStream_t>(stream), q, k_cache, v_cache, kv_half != 0, scratch, out, shape);
    if (e != cudaSuccess) return cuda_fail(e, "attention");
    return BC_OK;
}

