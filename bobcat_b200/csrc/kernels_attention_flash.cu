// Prefill attention for heads of 64, 128 or 256 elements over an f16 cache: one CTA per (64
// queries, head), 64-key tiles, online softmax, the two products on tensor cores. Counterpart of
// attention_flash (crates/bobcat-metal/src/attention.metal:290-480), which the reference uses for
// head_dim == 64 and at least 32 queries (backend.rs:2185-2225); the wider heads (Qwen3.5's
// attention layers have 256 elements) take the same path here instead of the chunk kernels.
//
// Arithmetic. Keys and values are the cache's fp16 values, exactly. The scaled query and the
// probabilities are each split into two fp16 halves (value = hi + lo, about 22 bits), so neither
// is rounded to fp16: every product is fp16 x fp16 accumulated in f32, and the result differs from
// an f32 evaluation only by summation order. The row maximum, exponentials (expf) and row sums are
// f32, as in the chunk kernels.
//
// A warp owns 16 queries. Scores S = Q K^T come from mma.m16n8k16 with the query fragments held in
// registers (heads of 64; wider heads re-read them from the staged queries at every step, their
// registers hold the output instead) and key fragments read with ldmatrix from the staged tile; the accumulator layout of S
// is the A-fragment layout of the second product, so probabilities go from registers straight into
// P V, whose value fragments are ldmatrix.trans reads of the staged tile.

#include "device_utils.cuh"
#include "kernels.h"

namespace bc {
namespace k {

namespace {

constexpr int kQueries = 64;   // queries per CTA: 4 warps x 16
constexpr int kKeys = 64;      // keys per tile
constexpr int kFlashThreads = 128;
// Halves per staged row: 16 bytes more than the head, so the 8 rows of an ldmatrix fall in distinct banks.
template <int HD>
constexpr int flash_pitch() { return HD + 8; }
template <int HD>
constexpr size_t flash_smem_bytes() { return (size_t)(2 * kQueries + 2 * kKeys) * flash_pitch<HD>() * 2; }

struct FlashParams {
    const float* q;
    const __half* k_cache;
    const __half* v_cache;
    float* out;
    uint32_t n_heads, n_kv_heads, first_pos, n_queries, q_stride, q_head_stride;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (x, y) as half2 bits of the high parts, and of what the high parts left over.
__device__ __forceinline__ void split_half2(float x, float y, uint32_t& hi, uint32_t& lo) {
    __half2 h = __floats2half2_rn(x, y);
    float2 back = __half22float2(h);
    __half2 l = __floats2half2_rn(x - back.x, y - back.y);
    hi = *reinterpret_cast<uint32_t*>(&h);
    lo = *reinterpret_cast<uint32_t*>(&l);
}

template <int HD>
__global__ void __launch_bounds__(kFlashThreads) attention_flash_kernel(FlashParams p) {
    constexpr int kHead = HD, kPitch = flash_pitch<HD>();
    constexpr bool kQueriesInRegisters = HD == 64;
    extern __shared__ __align__(16) uint8_t flash_smem[];
    __half (*q_hi)[kPitch] = reinterpret_cast<__half (*)[kPitch]>(flash_smem);
    __half (*q_lo)[kPitch] = q_hi + kQueries;
    __half (*k_tile)[kPitch] = q_lo + kQueries;
    __half (*v_tile)[kPitch] = k_tile + kKeys;

    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t q0 = blockIdx.x * kQueries, head = blockIdx.y;
    const uint32_t kv_head = head / (p.n_heads / p.n_kv_heads);
    const uint32_t kv_dim = p.n_kv_heads * kHead;
    const uint32_t kv_len = p.first_pos + p.n_queries;  // cache rows that exist
    const float scale = 1.0f / sqrtf((float)kHead);

    // Stage the scaled queries as hi + lo halves; rows past the batch are zero.
    for (int i = tid; i < kQueries * (kHead / 2); i += kFlashThreads) {
        int row = i / (kHead / 2), pair = i % (kHead / 2);
        float2 v = make_float2(0.f, 0.f);
        if (q0 + row < p.n_queries) {
            const float* src = p.q + (uint64_t)(q0 + row) * p.q_stride + (uint64_t)head * p.q_head_stride + 2 * pair;
            v = *reinterpret_cast<const float2*>(src);
        }
        uint32_t hi, lo;
        split_half2(v.x * scale, v.y * scale, hi, lo);
        *reinterpret_cast<uint32_t*>(&q_hi[row][2 * pair]) = hi;
        *reinterpret_cast<uint32_t*>(&q_lo[row][2 * pair]) = lo;
    }
    __syncthreads();

    // Query fragments: k-steps of 16 elements, hi and lo.
    constexpr int kHeld = kQueriesInRegisters ? kHead / 16 : 1;
    uint32_t qa_hi[kHeld][4], qa_lo[kHeld][4];
    auto query_fragments = [&](int ks, uint32_t (&hi)[4], uint32_t (&lo)[4]) {
        const int m = lane >> 3, r = lane & 7;
        const int row = warp * 16 + (m & 1) * 8 + r, col = ks * 16 + (m >> 1) * 8;
        ldmatrix_x4(hi, (uint32_t)__cvta_generic_to_shared(&q_hi[row][col]));
        ldmatrix_x4(lo, (uint32_t)__cvta_generic_to_shared(&q_lo[row][col]));
    };
    if (kQueriesInRegisters) {
#pragma unroll
        for (int ks = 0; ks < kHeld; ++ks) query_fragments(ks, qa_hi[ks], qa_lo[ks]);
    }

    float o[kHead / 8][4];
#pragma unroll
    for (int n = 0; n < kHead / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};

    // The position of this thread's two rows (g and g + 8 of the warp's 16 queries).
    const uint32_t pos_a = p.first_pos + q0 + warp * 16 + g, pos_b = pos_a + 8;
    // Keys up to the position of the CTA's last query.
    const uint32_t last_query = min(q0 + kQueries, p.n_queries) - 1;
    const uint32_t n_tiles = (p.first_pos + last_query) / kKeys + 1;
    // A warp whose queries all lie before a tile has nothing to add from it.
    const uint32_t warp_last_pos = p.first_pos + q0 + warp * 16 + 15;

    const __half* kc = p.k_cache + (uint64_t)kv_head * kHead;
    const __half* vc = p.v_cache + (uint64_t)kv_head * kHead;

    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        const uint32_t key0 = tile * kKeys;
        __syncthreads();  // the previous tile has been read
        for (int i = tid; i < kKeys * (kHead / 8); i += kFlashThreads) {
            int row = i / (kHead / 8), piece = i % (kHead / 8);
            uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
            if (key0 + row < kv_len) {
                kv = *reinterpret_cast<const uint4*>(kc + (uint64_t)(key0 + row) * kv_dim + 8 * piece);
                vv = *reinterpret_cast<const uint4*>(vc + (uint64_t)(key0 + row) * kv_dim + 8 * piece);
            }
            *reinterpret_cast<uint4*>(&k_tile[row][8 * piece]) = kv;
            *reinterpret_cast<uint4*>(&v_tile[row][8 * piece]) = vv;
        }
        __syncthreads();
        if (key0 > warp_last_pos) continue;  // warp-uniform

        // S = Q K^T: 8 tiles of 8 keys.
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
        {
            const int m = lane >> 3, r = lane & 7;
#pragma unroll
            for (int ks = 0; ks < kHead / 16; ++ks) {
                if (!kQueriesInRegisters) query_fragments(ks, qa_hi[0], qa_lo[0]);
                const uint32_t (&a_hi)[4] = qa_hi[kQueriesInRegisters ? ks : 0];
                const uint32_t (&a_lo)[4] = qa_lo[kQueriesInRegisters ? ks : 0];
#pragma unroll
                for (int np = 0; np < 4; ++np) {  // pairs of key tiles
                    uint32_t b[4];
                    ldmatrix_x4(b, (uint32_t)__cvta_generic_to_shared(&k_tile[np * 16 + (m >> 1) * 8 + r][ks * 16 + (m & 1) * 8]));
                    mma_f16(s[2 * np], a_hi, b[0], b[1]);
                    mma_f16(s[2 * np], a_lo, b[0], b[1]);
                    mma_f16(s[2 * np + 1], a_hi, b[2], b[3]);
                    mma_f16(s[2 * np + 1], a_lo, b[2], b[3]);
                }
            }
        }
        // Causal mask (only tiles that reach past a query's position need it).
        if (key0 + kKeys - 1 > p.first_pos + q0 + warp * 16) {
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const uint32_t key = key0 + n * 8 + 2 * t;
                if (key > pos_a) s[n][0] = -INFINITY;
                if (key + 1 > pos_a) s[n][1] = -INFINITY;
                if (key > pos_b) s[n][2] = -INFINITY;
                if (key + 1 > pos_b) s[n][3] = -INFINITY;
            }
        }
        // Online softmax. Key 0 is visible to every query, so after the first tile the maxima are finite.
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            tile_max[0] = fmaxf(tile_max[0], fmaxf(s[n][0], s[n][1]));
            tile_max[1] = fmaxf(tile_max[1], fmaxf(s[n][2], s[n][3]));
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
            tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
        }
        float correction[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float m_new = fmaxf(row_max[h], tile_max[h]);
            correction[h] = expf(row_max[h] - m_new);  // exp(-inf) = 0 on the first tile
            row_max[h] = m_new;
        }
        float tile_sum[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            s[n][0] = expf(s[n][0] - row_max[0]);
            s[n][1] = expf(s[n][1] - row_max[0]);
            s[n][2] = expf(s[n][2] - row_max[1]);
            s[n][3] = expf(s[n][3] - row_max[1]);
            tile_sum[0] += s[n][0] + s[n][1];
            tile_sum[1] += s[n][2] + s[n][3];
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            tile_sum[h] += __shfl_xor_sync(0xffffffffu, tile_sum[h], 1);
            tile_sum[h] += __shfl_xor_sync(0xffffffffu, tile_sum[h], 2);
            row_sum[h] = row_sum[h] * correction[h] + tile_sum[h];
        }
#pragma unroll
        for (int n = 0; n < kHead / 8; ++n) {
            o[n][0] *= correction[0];
            o[n][1] *= correction[0];
            o[n][2] *= correction[1];
            o[n][3] *= correction[1];
        }
        // O += P V: 4 k-steps of 16 keys; the scores' accumulator layout is the A-fragment layout.
        {
            const int m = lane >> 3, r = lane & 7;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t pa_hi[4], pa_lo[4];
                split_half2(s[2 * kk][0], s[2 * kk][1], pa_hi[0], pa_lo[0]);
                split_half2(s[2 * kk][2], s[2 * kk][3], pa_hi[1], pa_lo[1]);
                split_half2(s[2 * kk + 1][0], s[2 * kk + 1][1], pa_hi[2], pa_lo[2]);
                split_half2(s[2 * kk + 1][2], s[2 * kk + 1][3], pa_hi[3], pa_lo[3]);
#pragma unroll
                for (int np = 0; np < kHead / 16; ++np) {  // pairs of 8-element output tiles
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, (uint32_t)__cvta_generic_to_shared(&v_tile[kk * 16 + (m & 1) * 8 + r][np * 16 + (m >> 1) * 8]));
                    mma_f16(o[2 * np], pa_hi, b[0], b[1]);
                    mma_f16(o[2 * np], pa_lo, b[0], b[1]);
                    mma_f16(o[2 * np + 1], pa_hi, b[2], b[3]);
                    mma_f16(o[2 * np + 1], pa_lo, b[2], b[3]);
                }
            }
        }
    }

    // Normalise and store: row g holds columns 2t, 2t + 1 of each 8-element tile.
    const uint32_t query_a = q0 + warp * 16 + g, query_b = query_a + 8;
    const float inv_a = 1.f / row_sum[0], inv_b = 1.f / row_sum[1];
#pragma unroll
    for (int n = 0; n < kHead / 8; ++n) {
        const uint32_t col = head * kHead + n * 8 + 2 * t;
        if (query_a < p.n_queries)
            *reinterpret_cast<float2*>(p.out + (uint64_t)query_a * p.n_heads * kHead + col) = make_float2(o[n][0] * inv_a, o[n][1] * inv_a);
        if (query_b < p.n_queries)
            *reinterpret_cast<float2*>(p.out + (uint64_t)query_b * p.n_heads * kHead + col) = make_float2(o[n][2] * inv_b, o[n][3] * inv_b);
    }
}

}  // namespace

bool attention_flash_supported(bool kv_half, const AttentionShape& s) {
    return kv_half && (s.head_dim == 64 || s.head_dim == 128 || s.head_dim == 256) && s.n_queries >= 32 && s.pos_ptr == nullptr &&
           s.n_kv_heads > 0 && s.n_heads % s.n_kv_heads == 0 && s.q_stride % 2 == 0 && s.q_head_stride % 2 == 0;
}

cudaError_t attention_flash(cudaStream_t stream, const float* q, const void* k_cache, const void* v_cache, float* out,
                            const AttentionShape& s) {
    FlashParams p{q, static_cast<const __half*>(k_cache), static_cast<const __half*>(v_cache), out, s.n_heads, s.n_kv_heads,
                  s.first_pos, s.n_queries, s.q_stride, s.q_head_stride};
    dim3 grid((s.n_queries + kQueries - 1) / kQueries, s.n_heads);
    cudaError_t e;
    switch (s.head_dim) {
        case 64:
            if ((e = ensure_dynamic_smem((const void*)attention_flash_kernel<64>, flash_smem_bytes<64>())) != cudaSuccess) return e;
            return launch_dependent(attention_flash_kernel<64>, grid, dim3(kFlashThreads), flash_smem_bytes<64>(), stream, p);
        case 128:
            if ((e = ensure_dynamic_smem((const void*)attention_flash_kernel<128>, flash_smem_bytes<128>())) != cudaSuccess) return e;
            return launch_dependent(attention_flash_kernel<128>, grid, dim3(kFlashThreads), flash_smem_bytes<128>(), stream, p);
        default:
            if ((e = ensure_dynamic_smem((const void*)attention_flash_kernel<256>, flash_smem_bytes<256>())) != cudaSuccess) return e;
            return launch_dependent(attention_flash_kernel<256>, grid, dim3(kFlashThreads), flash_smem_bytes<256>(), stream, p);
    }
}

}  // namespace k
}  // namespace bc
