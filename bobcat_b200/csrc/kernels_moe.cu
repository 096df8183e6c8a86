// Mixture-of-experts kernels: the router (with its top-k pick), the per-token expert
// matrix-vector products of decode, and the grouped multiply and combine of prefill.
// Counterparts: crates/bobcat-metal/src/moe.metal (moe_route :22, moe_group :131, moe_combine :182,
// matvec_experts_swiglu :211, matvec_experts_down :246) and matmul_experts in matmul.metal:473-506;
// the arithmetic they must reproduce is lfm2.rs:413-440 (moe_block) and :691-709 (route).
//
// A token's route is 2 * n_used 32-bit words: the picked expert ids, then their weights as float
// bits (moe.metal:4-6).

#include "matvec_common.cuh"

namespace bc {
namespace k {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxExperts = 128;

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct RouteParams {
    const float* x;
    const float* norm_weight;  // null: x is already normalised
    float eps;
    float* normed;             // receives the normalised tokens when norm_weight is set
    const float* router;       // [n_experts][n_cols] f32
    const float* bias;
    uint32_t* route;
    uint32_t n_cols, n_experts, n_used;
};

constexpr int kRouteThreads = 1024;
constexpr int kRouteWarps = kRouteThreads / 32;

// One CTA per token, a warp per expert. The token's norm and the router's dot products accumulate
// in f64, as the scalar reference does (scalar.rs:240-249, :292-304), so the scores - and with them
// the picked expert ids - do not depend on the order a parallel sum happens to take. Each lane
// keeps four independent sums so the f64 adds do not wait on one another.
__global__ void __launch_bounds__(kRouteThreads) moe_route_kernel(RouteParams p) {
    extern __shared__ float xs[];  // the normalised token
    __shared__ double reduce[kRouteWarps];
    __shared__ float scores[kMaxExperts];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t token = blockIdx.x, n_cols = p.n_cols;
    const float* x = p.x + (uint64_t)token * n_cols;
    if (p.norm_weight) {
        double sumsq = 0.0;
        for (uint32_t c = tid; c < n_cols; c += kRouteThreads) sumsq += (double)x[c] * (double)x[c];
        sumsq = warp_sum_f64(sumsq);
        if (lane == 0) reduce[warp] = sumsq;
        __syncthreads();
        double total = 0.0;
        for (int w = 0; w < kRouteWarps; ++w) total += reduce[w];
        float scale = (float)(1.0 / sqrt(total / (double)n_cols + (double)p.eps));
        float* normed = p.normed + (uint64_t)token * n_cols;
        for (uint32_t c = tid; c < n_cols; c += kRouteThreads) {
            float v = p.norm_weight[c] * (x[c] * scale);
            xs[c] = v;
            normed[c] = v;
        }
    } else {
        for (uint32_t c = tid; c < n_cols; c += kRouteThreads) xs[c] = x[c];
    }
    __syncthreads();
    for (uint32_t e = warp; e < p.n_experts; e += kRouteWarps) {
        const float* row = p.router + (uint64_t)e * n_cols;
        double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
        uint32_t c = 0;
        if ((n_cols & 3u) == 0 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
            // Four 16-byte loads in flight per lane and trip, so a row costs a few round trips to L2, not one per element.
            const float4* row4 = reinterpret_cast<const float4*>(row);
            const float4* x4 = reinterpret_cast<const float4*>(xs);
            const uint32_t n4 = n_cols / 4;
            uint32_t i = lane;
            for (; i + 96 < n4; i += 128) {
                const float4 a = __ldg(row4 + i), b = __ldg(row4 + i + 32), cc = __ldg(row4 + i + 64), d = __ldg(row4 + i + 96);
                const float4 xa = x4[i], xb = x4[i + 32], xc = x4[i + 64], xd = x4[i + 96];
                s0 += (double)a.x * xa.x + (double)a.y * xa.y + (double)a.z * xa.z + (double)a.w * xa.w;
                s1 += (double)b.x * xb.x + (double)b.y * xb.y + (double)b.z * xb.z + (double)b.w * xb.w;
                s2 += (double)cc.x * xc.x + (double)cc.y * xc.y + (double)cc.z * xc.z + (double)cc.w * xc.w;
                s3 += (double)d.x * xd.x + (double)d.y * xd.y + (double)d.z * xd.z + (double)d.w * xd.w;
            }
            for (; i < n4; i += 32) {
                const float4 a = __ldg(row4 + i);
                const float4 xa = x4[i];
                s0 += (double)a.x * xa.x + (double)a.y * xa.y + (double)a.z * xa.z + (double)a.w * xa.w;
            }
            c = n_cols;
        }
        for (c += lane; c < n_cols; c += 32) s0 += (double)row[c] * (double)xs[c];
        double sum = warp_sum_f64((s0 + s1) + (s2 + s3));
        if (lane == 0) scores[e] = 1.0f / (1.0f + expf(-(float)sum));
    }
    __syncthreads();
    if (warp == 0) {
        // Top n_used by repeated argmax of score + bias, ties to the lower id; the weights are the
        // unbiased scores over their f32 sum plus 1e-6 (lfm2.rs:698-708). Lane l looks after experts
        // l, l + 32, l + 64, l + 96; a round is a lane-local scan and a warp-wide compare.
        float value[kMaxExperts / 32];
        bool taken[kMaxExperts / 32];
#pragma unroll
        for (int k = 0; k < kMaxExperts / 32; ++k) {
            const uint32_t e = lane + 32 * k;
            value[k] = e < p.n_experts ? scores[e] + p.bias[e] : 0.f;
            taken[k] = e >= p.n_experts;
        }
        uint32_t picked = 0;   // lane i < n_used ends up holding the i-th pick
        float picked_score = 0.f, sum = 0.f;
        for (uint32_t i = 0; i < p.n_used; ++i) {
            float best_value = 0.f;
            uint32_t best = 0xffffffffu;
#pragma unroll
            for (int k = 0; k < kMaxExperts / 32; ++k) {
                if (!taken[k] && (best == 0xffffffffu || value[k] > best_value)) {
                    best_value = value[k];
                    best = lane + 32 * k;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float other_value = __shfl_xor_sync(0xffffffffu, best_value, o);
                const uint32_t other = __shfl_xor_sync(0xffffffffu, best, o);
                if (other != 0xffffffffu && (best == 0xffffffffu || other_value > best_value || (other_value == best_value && other < best))) {
                    best_value = other_value;
                    best = other;
                }
            }
#pragma unroll
            for (int k = 0; k < kMaxExperts / 32; ++k)
                if (best == lane + 32 * k) taken[k] = true;
            const float score = scores[best];
            sum += score;  // in pick order, as the scalar code adds them
            if (lane == i) {
                picked = best;
                picked_score = score;
            }
        }
        const float norm = sum + 1e-6f;
        uint32_t* route = p.route + (uint64_t)token * 2 * p.n_used;
        if (lane < p.n_used) {
            route[lane] = picked;
            route[p.n_used + lane] = __float_as_uint(picked_score / norm);
        }
    }
}

// One CTA: counting sort of the (token, slot) entries by expert. offsets[e] is the first entry of
// expert e (offsets[n_experts] the total); entries hold token * n_used + slot in token order.
//
// With a range (first_expert, n_experts of them) only the entries of those experts are kept, under
// the local index expert - first_expert: the grouping an expert-parallel rank multiplies.
__global__ void __launch_bounds__(1024) moe_group_kernel(const uint32_t* __restrict__ route, uint32_t* __restrict__ offsets,
                                                          uint32_t* __restrict__ entries, uint32_t n_experts, uint32_t n_used, uint32_t n_tokens,
                                                          uint32_t first_expert) {
    __shared__ uint32_t counts[kMaxExperts + 1];
    const uint32_t total = n_tokens * n_used;
    for (uint32_t e = threadIdx.x; e <= n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < total; i += blockDim.x) {
        uint32_t token = i / n_used, slot = i % n_used;
        uint32_t local = route[(uint64_t)token * 2 * n_used + slot] - first_expert;  // wraps for experts below the range
        if (local < n_experts) atomicAdd(&counts[local], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t running = 0;
        for (uint32_t e = 0; e < n_experts; ++e) {
            uint32_t c = counts[e];
            counts[e] = running;
            running += c;
        }
        counts[n_experts] = running;
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e <= n_experts; e += blockDim.x) offsets[e] = counts[e];
    __syncthreads();
    // A warp per expert walks the entries 32 at a time in token order; a ballot and a count of the
    // lower lanes give each of the expert's entries its place, which keeps the order stable.
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (uint32_t e = warp; e < n_experts; e += n_warps) {
        uint32_t at = counts[e];
        for (uint32_t base = 0; base < total; base += 32) {
            const uint32_t i = base + lane;
            bool mine = false;
            if (i < total) {
                uint32_t token = i / n_used, slot = i % n_used;
                mine = route[(uint64_t)token * 2 * n_used + slot] == e + first_expert;
            }
            const uint32_t votes = __ballot_sync(0xffffffffu, mine);
            if (mine) entries[at + __popc(votes & ((1u << lane) - 1u))] = i;
            at += __popc(votes);
        }
    }
}

struct ExpertsParams {
    Mat gate, up;            // stacked experts: expert e owns rows [e * n_rows, (e + 1) * n_rows)
    const float* x;          // swiglu: [n_tokens][n_cols]; down: [n_tokens][n_used][n_cols]
    const uint32_t* route;
    float* y;                // swiglu: [n_tokens][n_used][n_rows]; down: [n_tokens][n_rows], accumulated
    uint32_t n_rows, n_used;
};

// grid (row groups, n_used, n_tokens): SwiGLU of the picked expert's gate and up rows.
template <int FORMAT>
__global__ void __launch_bounds__(kThreads) experts_swiglu_kernel(ExpertsParams p) {
    extern __shared__ float4 xs4[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t slot = blockIdx.y, token = blockIdx.z, n_cols = p.gate.n_cols;
    const uint32_t expert = p.route[(uint64_t)token * 2 * p.n_used + slot];
    stage_input(p.x + (uint64_t)token * n_cols, nullptr, 0.f, n_cols, xs4, scratch);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* y = p.y + ((uint64_t)token * p.n_used + slot) * p.n_rows;
    for (uint32_t row = blockIdx.x * kWarps + warp; row < p.n_rows; row += gridDim.x * kWarps) {
        RowPtr rows[2] = {row_of(p.gate, expert * p.n_rows + row), row_of(p.up, expert * p.n_rows + row)};
        float acc[2];
        dot_rows<FORMAT, 2>(rows, n_cols, xs4, lane, 0, 1, acc);
        if (lane == 0) y[row] = acc[0] / (1.f + expf(-acc[0])) * acc[1];
    }
}

// grid (row groups, n_tokens): y[token][row] += sum over slots of weight * (down row of the
// slot's expert . that slot's activations), slots in route order as lfm2.rs:429-439 adds them.
template <int FORMAT>
__global__ void __launch_bounds__(kThreads) experts_down_kernel(ExpertsParams p) {
    extern __shared__ float4 xs4[];  // n_used staged inputs, one after another
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t token = blockIdx.y, n_cols = p.gate.n_cols;
    const uint32_t* route = p.route + (uint64_t)token * 2 * p.n_used;
    for (uint32_t s = 0; s < p.n_used; ++s)
        stage_input(p.x + ((uint64_t)token * p.n_used + s) * n_cols, nullptr, 0.f, n_cols, xs4 + (uint64_t)s * (n_cols / 4), scratch);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* y = p.y + (uint64_t)token * p.n_rows;
    for (uint32_t row = blockIdx.x * kWarps + warp; row < p.n_rows; row += gridDim.x * kWarps) {
        float total = 0.f;
        for (uint32_t s = 0; s < p.n_used; ++s) {
            uint32_t expert = route[s];
            float weight = __uint_as_float(route[p.n_used + s]);
            RowPtr rows[1] = {row_of(p.gate, expert * p.n_rows + row)};
            float acc[1];
            dot_rows<FORMAT, 1>(rows, n_cols, xs4 + (uint64_t)s * (n_cols / 4), lane, 0, 1, acc);
            total += weight * acc[0];
        }
        if (lane == 0) y[row] += total;
    }
}

// y[t] += sum over slots of weight[t, s] * expert_out[t * n_used + s]
__global__ void moe_combine_kernel(const float* __restrict__ expert_out, const uint32_t* __restrict__ route, float* __restrict__ y,
                                   uint32_t n_embd, uint32_t n_used) {
    uint32_t token = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n_embd) return;
    const uint32_t* r = route + (uint64_t)token * 2 * n_used;
    float total = 0.f;
    for (uint32_t s = 0; s < n_used; ++s) total += __uint_as_float(r[n_used + s]) * expert_out[((uint64_t)token * n_used + s) * n_embd + c];
    y[(uint64_t)token * n_embd + c] += total;
}

// Grouped multiply for prefill: for each expert, the entries routed to it times that expert's
// rows. 64 entries x 64 rows per CTA, K in steps of 32, f32 throughout (the tile of
// kernels_matmul.cu with row indirection). With `up`, the store is silu(gate) * up.
struct GroupedParams {
    Mat w, up;
    bool paired;
    const float* x;
    bool gather;  // true: input row = entry / n_used (the token's row); false: input row = entry
    const uint32_t* offsets;
    const uint32_t* entries;
    float* y;     // [entry][n_rows]
    uint32_t n_rows, n_used;
};

__device__ __forceinline__ void load_weight_tile(const Mat& w, uint32_t row0, uint32_t rows_here, uint32_t k0, float (*ws)[68], int tid) {
    const uint32_t n_cols = w.n_cols;
    if (w.format == BC_Q4_0) {
        if (tid < 64) {
            if ((uint32_t)tid < rows_here) {
                uint64_t block = (uint64_t)(row0 + tid) * (n_cols >> 5) + (k0 >> 5);
                uint4 q = static_cast<const uint4*>(w.data)[block];
                float d = __half2float(w.scales[block]);
                uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int wi = 0; wi < 4; ++wi)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t byte = (words[wi] >> (8 * i)) & 0xffu;
                        ws[4 * wi + i][tid] = (float)((int)(byte & 0xfu) - 8) * d;
                        ws[16 + 4 * wi + i][tid] = (float)((int)(byte >> 4) - 8) * d;
                    }
            } else {
                for (int kk = 0; kk < 32; ++kk) ws[kk][tid] = 0.f;
            }
        }
    } else {
        for (int i = tid; i < 64 * 32; i += kThreads) {
            int r = i / 32, kk = i % 32;
            float v = 0.f;
            if ((uint32_t)r < rows_here) {
                uint64_t at = (uint64_t)(row0 + r) * n_cols + k0 + kk;
                v = w.format == BC_F16 ? __half2float(static_cast<const __half*>(w.data)[at]) : static_cast<const float*>(w.data)[at];
            }
            ws[kk][r] = v;
        }
    }
}

__global__ void __launch_bounds__(kThreads) matmul_experts_kernel(GroupedParams p) {
    __shared__ float ws[32][68], us[32][68], xs[32][68];
    const uint32_t expert = blockIdx.z;
    const uint32_t first = p.offsets[expert], count = p.offsets[expert + 1] - first;
    const uint32_t e0 = blockIdx.x * 64, row0 = blockIdx.y * 64;
    if (e0 >= count) return;
    const uint32_t n_cols = p.w.n_cols, rows_here = min(64u, p.n_rows - row0), entries_here = min(64u, count - e0);
    const int tid = threadIdx.x, tr = (tid % 16) * 4, tt = (tid / 16) * 4;
    float acc[4][4] = {}, acc_up[4][4] = {};
    for (uint32_t k0 = 0; k0 < n_cols; k0 += 32) {
        load_weight_tile(p.w, expert * p.n_rows + row0, rows_here, k0, ws, tid);
        if (p.paired) load_weight_tile(p.up, expert * p.n_rows + row0, rows_here, k0, us, tid);
        for (int i = tid; i < 64 * 32; i += kThreads) {
            int t = i / 32, kk = i % 32;
            float v = 0.f;
            if ((uint32_t)t < entries_here) {
                uint32_t entry = p.entries[first + e0 + t];
                uint32_t in_row = p.gather ? entry / p.n_used : entry;
                v = p.x[(uint64_t)in_row * n_cols + k0 + kk];
            }
            xs[kk][t] = v;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
            float4 wv = *reinterpret_cast<const float4*>(&ws[kk][tr]);
            float4 xv = *reinterpret_cast<const float4*>(&xs[kk][tt]);
            float wr[4] = {wv.x, wv.y, wv.z, wv.w}, xt[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] += xt[a] * wr[b];
            if (p.paired) {
                float4 uv = *reinterpret_cast<const float4*>(&us[kk][tr]);
                float ur[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) acc_up[a][b] += xt[a] * ur[b];
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        if ((uint32_t)(tt + a) >= entries_here) continue;
        uint32_t entry = p.entries[first + e0 + tt + a];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            if ((uint32_t)(tr + b) >= rows_here) continue;
            float v = acc[a][b];
            if (p.paired) v = v / (1.f + expf(-v)) * acc_up[a][b];
            p.y[(uint64_t)entry * p.n_rows + row0 + tr + b] = v;
        }
    }
}

template <typename Kernel>
cudaError_t launch_experts(Kernel kernel, dim3 grid, size_t smem, cudaStream_t stream, ExpertsParams& p) {
    cudaError_t e = ensure_dynamic_smem((const void*)kernel, smem);
    if (e != cudaSuccess) return e;
    void* args[] = {&p};
    return launch_kernel((const void*)kernel, grid, dim3(kThreads), smem, stream, args);
}

}  // namespace

cudaError_t moe_route(cudaStream_t stream, const float* x, Norm norm, float* normed, const float* router, const float* bias,
                      uint32_t* route, uint32_t n_cols, uint32_t n_experts, uint32_t n_used, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    RouteParams p{x, norm.weight, norm.eps, normed, router, bias, route, n_cols, n_experts, n_used};
    size_t smem = (size_t)n_cols * 4;
    cudaError_t e = ensure_dynamic_smem((const void*)moe_route_kernel, smem);
    if (e != cudaSuccess) return e;
    void* args[] = {&p};
    return launch_kernel((const void*)moe_route_kernel, dim3(n_tokens), dim3(kRouteThreads), smem, stream, args);
}

cudaError_t moe_group(cudaStream_t stream, const uint32_t* route, uint32_t* offsets, uint32_t* entries, uint32_t n_experts,
                      uint32_t n_used, uint32_t n_tokens, uint32_t first_expert) {
    moe_group_kernel<<<1, 1024, 0, stream>>>(route, offsets, entries, n_experts, n_used, n_tokens, first_expert);
    return cudaGetLastError();
}

cudaError_t matvec_experts_swiglu(cudaStream_t stream, const Mat& gate, const Mat& up, uint32_t n_rows, const float* x,
                                  const uint32_t* route, uint32_t n_used, float* y, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    if (n_tokens == 1 && matvec_experts_mma_supported(gate, n_rows, n_used) && up.tiles)
        return matvec_experts_swiglu_mma(stream, gate, up, n_rows, x, route, n_used, y);
    ExpertsParams p{gate, up, x, route, y, n_rows, n_used};
    unsigned groups = (n_rows + kWarps - 1) / kWarps;
    unsigned cap = (unsigned)sm_count() * 8 / (n_used * n_tokens) + 1;
    dim3 grid(groups < cap ? groups : cap, n_used, n_tokens);
    size_t smem = (size_t)gate.n_cols * 4;
    switch (gate.format) {
        case BC_Q4_0: return launch_experts(experts_swiglu_kernel<BC_Q4_0>, grid, smem, stream, p);
        case BC_F16: return launch_experts(experts_swiglu_kernel<BC_F16>, grid, smem, stream, p);
        default: return launch_experts(experts_swiglu_kernel<BC_F32>, grid, smem, stream, p);
    }
}

int matvec_experts_down_launches(const Mat& down, uint32_t n_rows, uint32_t n_used, uint32_t n_tokens, bool has_scratch) {
    return n_tokens == 1 && has_scratch && matvec_experts_mma_supported(down, n_rows, n_used) ? 2 : 1;
}

cudaError_t matvec_experts_down(cudaStream_t stream, const Mat& down, uint32_t n_rows, const float* x, const uint32_t* route,
                                uint32_t n_used, float* y, uint32_t n_tokens, float* expert_out) {
    if (n_tokens == 0) return cudaSuccess;
    if (n_tokens == 1 && expert_out && matvec_experts_mma_supported(down, n_rows, n_used)) {
        cudaError_t e = matvec_experts_down_mma(stream, down, n_rows, x, route, n_used, expert_out);
        if (e != cudaSuccess) return e;
        return moe_combine(stream, expert_out, route, y, n_rows, n_used, 1);
    }
    ExpertsParams p{down, down, x, route, y, n_rows, n_used};
    unsigned groups = (n_rows + kWarps - 1) / kWarps;
    unsigned cap = (unsigned)sm_count() * 8 / n_tokens + 1;
    dim3 grid(groups < cap ? groups : cap, n_tokens);
    size_t smem = (size_t)down.n_cols * 4 * n_used;
    switch (down.format) {
        case BC_Q4_0: return launch_experts(experts_down_kernel<BC_Q4_0>, grid, smem, stream, p);
        case BC_F16: return launch_experts(experts_down_kernel<BC_F16>, grid, smem, stream, p);
        default: return launch_experts(experts_down_kernel<BC_F32>, grid, smem, stream, p);
    }
}

cudaError_t matmul_experts(cudaStream_t stream, const Mat& w, const Mat* up, uint32_t n_rows, uint32_t n_experts, const float* x,
                           bool gather, const uint32_t* offsets, const uint32_t* entries, uint32_t n_used, float* y, uint32_t n_tokens,
                           void* scratch) {
    if (n_tokens == 0) return cudaSuccess;
    if (scratch && matmul_experts_umma_supported(w, up, n_tokens))
        return matmul_experts_umma(stream, w, up, n_rows, n_experts, x, gather, offsets, entries, n_used, y, n_tokens, scratch);
    GroupedParams p{w, up ? *up : w, up != nullptr, x, gather, offsets, entries, y, n_rows, n_used};
    // Any one expert can receive up to n_tokens entries (a token picks an expert at most once).
    dim3 grid((n_tokens + 63) / 64, (n_rows + 63) / 64, n_experts);
    matmul_experts_kernel<<<grid, kThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t moe_combine(cudaStream_t stream, const float* expert_out, const uint32_t* route, float* y, uint32_t n_embd,
                        uint32_t n_used, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    dim3 grid((n_embd + 255) / 256, n_tokens);
    moe_combine_kernel<<<grid, 256, 0, stream>>>(expert_out, route, y, n_embd, n_used);
    return cudaGetLastError();
}

}  // namespace k
}  // namespace bc
