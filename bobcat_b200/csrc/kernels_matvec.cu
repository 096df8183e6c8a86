// Decode-time matrix-vector kernels: y = W x with optional fused RMSNorm of x, residual
// accumulate, SwiGLU of a gate/up pair, and the LFM2 gated short convolution.
//
// Shape of every kernel here: a CTA stages the input vector once in shared memory (multiplied by
// the norm weight when a norm is fused, with the sum of squares reduced on the way), then its warps
// walk rows. A lane owns whole 32-weight blocks: one 128-bit load brings a block's quants, the
// block's 32 inputs come from shared memory once and are reused for every row the warp has in
// flight, and the block's scale multiplies the finished block sum. A warp's loads are contiguous
// 512-byte runs of the weight stream, which is the only HBM traffic that matters here.
//
// Counterparts in the reference: matvec_k / matvec_q / swiglu_rows / matvec_conv in
// crates/bobcat-metal/src/matvec.metal:151-585, lane layout q4_0_lanes in quant.metal:587-656.

#include <map>
#include <mutex>
#include <utility>

#include "device_utils.cuh"
#include "kernels.h"
#include "../../include/bobcat_cuda.h"

namespace bc {
namespace k {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

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
    } else {
        p.data = static_cast<const float*>(m.data) + (uint64_t)row * m.n_cols;
        p.scales = nullptr;
    }
    return p;
}

// Stage x into shared memory in the rotated chunk layout, times the norm weight when given.
// Returns the factor the finished row sums are multiplied by (1 without a norm).
__device__ float stage_input(const float* __restrict__ x, const float* __restrict__ norm_weight, float eps,
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

// Partial dot products of R rows with the staged input, for this lane's share of the columns.
template <int FORMAT, int R>
__device__ __forceinline__ void dot_rows(const RowPtr (&rows)[R], uint32_t n_cols, const float4* __restrict__ xs, int lane,
                                         float (&acc)[R]) {
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    if (FORMAT == BC_Q4_0) {
        const int nb = n_cols >> 5;
#pragma unroll 2
        for (int b0 = 0; b0 < nb; b0 += 32) {
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
        for (int c0 = 0; c0 < nc; c0 += 32) {
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
    } else {  // BC_F16
        const int nc = n_cols >> 3;
#pragma unroll 2
        for (int c0 = 0; c0 < nc; c0 += 32) {
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

struct MatvecParams {
    MatvecSegment seg[3];
    int n_segments;
    uint32_t total_rows;
    const float* x;
    const float* norm_weight;
    float eps;
    int accumulate;
};

template <int FORMAT>
__global__ void __launch_bounds__(kThreads) matvec_kernel(MatvecParams p) {
    extern __shared__ float4 xs[];
    __shared__ float reduce_scratch[32];
    const uint32_t n_cols = p.seg[0].w.n_cols;
    float scale = stage_input(p.x, p.norm_weight, p.eps, n_cols, xs, reduce_scratch);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int R = 2;
    // Row pairs are dealt round-robin to warps across the grid.
    const uint32_t n_pairs = (p.total_rows + R - 1) / R;
    for (uint32_t pair = blockIdx.x * kWarps + warp; pair < n_pairs; pair += gridDim.x * kWarps) {
        RowPtr rows[R];
        float* out[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            uint32_t row = pair * R + r;
            bool valid = row < p.total_rows;
            if (!valid) row = p.total_rows - 1;
            int s = 0;
            uint32_t local = row;
            while (s + 1 < p.n_segments && local >= p.seg[s].w.n_rows) {
                local -= p.seg[s].w.n_rows;
                ++s;
            }
            rows[r] = row_of(p.seg[s].w, local);
            out[r] = valid ? p.seg[s].y + local : nullptr;
        }
        float acc[R];
        dot_rows<FORMAT, R>(rows, n_cols, xs, lane, acc);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (out[r]) {
                    float v = acc[r] * scale;
                    *out[r] = p.accumulate ? *out[r] + v : v;
                }
            }
        }
    }
}

struct SwigluParams {
    Mat gate, up;
    const float* x;
    const float* norm_weight;
    float eps;
    float* y;
};

template <int FORMAT>
__global__ void __launch_bounds__(kThreads) matvec_swiglu_kernel(SwigluParams p) {
    extern __shared__ float4 xs[];
    __shared__ float reduce_scratch[32];
    const uint32_t n_cols = p.gate.n_cols, n_rows = p.gate.n_rows;
    float scale = stage_input(p.x, p.norm_weight, p.eps, n_cols, xs, reduce_scratch);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t row = blockIdx.x * kWarps + warp; row < n_rows; row += gridDim.x * kWarps) {
        RowPtr rows[2] = {row_of(p.gate, row), row_of(p.up, row)};
        float acc[2];
        dot_rows<FORMAT, 2>(rows, n_cols, xs, lane, acc);
        if (lane == 0) {
            float g = acc[0] * scale, u = acc[1] * scale;
            p.y[row] = g / (1.f + expf(-g)) * u;
        }
    }
}

struct ConvParams {
    Mat in_proj;
    const float* x;
    const float* norm_weight;
    float eps;
    const float* taps;
    float* history;
    float* out;
    uint32_t n_embd, kernel;
};

// One warp per channel: rows ch, n_embd + ch and 2 n_embd + ch of in_proj give B, C and X; lane 0
// then runs the taps over B*X and the channel's history, shifts the history and writes C * conv
// (the arithmetic of crates/bobcat/src/lfm2.rs:456-475 with f32 sums).
template <int FORMAT>
__global__ void __launch_bounds__(kThreads) matvec_conv_kernel(ConvParams p) {
    extern __shared__ float4 xs[];
    __shared__ float reduce_scratch[32];
    const uint32_t n_cols = p.in_proj.n_cols;
    float scale = stage_input(p.x, p.norm_weight, p.eps, n_cols, xs, reduce_scratch);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t ch = blockIdx.x * kWarps + warp; ch < p.n_embd; ch += gridDim.x * kWarps) {
        RowPtr rows[3] = {row_of(p.in_proj, ch), row_of(p.in_proj, p.n_embd + ch), row_of(p.in_proj, 2 * p.n_embd + ch)};
        float acc[3];
        dot_rows<FORMAT, 3>(rows, n_cols, xs, lane, acc);
        if (lane == 0) {
            float b = acc[0] * scale, c = acc[1] * scale, xv = acc[2] * scale;
            float bx = b * xv;
            const float* taps = p.taps + (uint64_t)ch * p.kernel;
            float sum = taps[p.kernel - 1] * bx;
            for (uint32_t kk = 0; kk + 1 < p.kernel; ++kk) sum += taps[kk] * p.history[(uint64_t)kk * p.n_embd + ch];
            for (uint32_t kk = 0; kk + 2 < p.kernel; ++kk)
                p.history[(uint64_t)kk * p.n_embd + ch] = p.history[(uint64_t)(kk + 1) * p.n_embd + ch];
            p.history[(uint64_t)(p.kernel - 2) * p.n_embd + ch] = bx;
            p.out[ch] = c * sum;
        }
    }
}

int sm_count_impl() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
        if (count <= 0) count = 148;
    }
    return count;
}

}  // namespace

// Raise a kernel's dynamic shared-memory limit when a launch needs more than the 48 KB default.
// The setting is per device and per function; remember what was granted so steady-state launches
// (and launches under stream capture) make no extra runtime calls.
cudaError_t ensure_dynamic_smem(const void* kernel, size_t smem) {
    if (smem <= 48 * 1024) return cudaSuccess;
    static std::mutex mutex;
    static std::map<std::pair<int, const void*>, size_t> granted;
    int device = 0;
    cudaGetDevice(&device);
    std::lock_guard<std::mutex> lock(mutex);
    size_t& have = granted[{device, kernel}];
    if (have >= smem) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) have = smem;
    return e;
}

namespace {

template <typename Kernel>
cudaError_t prepare(Kernel kernel, size_t smem) {
    return ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
}

// CTAs for `units` warp-sized pieces of work: enough to fill the machine a few times over, never
// more than the work.
int grid_for(uint64_t units) {
    uint64_t ctas = (units + kWarps - 1) / kWarps;
    uint64_t cap = (uint64_t)sm_count_impl() * 8;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    return (int)ctas;
}

}  // namespace

int sm_count() { return sm_count_impl(); }

Mat Mat::rows(uint32_t first, uint32_t count) const {
    Mat m = *this;
    m.n_rows = count;
    if (format == BC_Q4_0) {
        uint64_t nb = n_cols >> 5;
        m.data = static_cast<const uint4*>(data) + first * nb;
        m.scales = scales + first * nb;
    } else if (format == BC_F16) {
        m.data = static_cast<const __half*>(data) + (uint64_t)first * n_cols;
    } else {
        m.data = static_cast<const float*>(data) + (uint64_t)first * n_cols;
    }
    return m;
}

uint64_t Mat::bytes() const {
    uint64_t n = (uint64_t)n_rows * n_cols;
    if (format == BC_Q4_0) return n / 32 * 18;
    if (format == BC_F16) return n * 2;
    return n * 4;
}

cudaError_t matvec(cudaStream_t stream, const MatvecSegment* segments, int n_segments, const float* x, Norm norm,
                   bool accumulate) {
    MatvecParams p{};
    p.n_segments = n_segments;
    p.total_rows = 0;
    for (int i = 0; i < n_segments; ++i) {
        p.seg[i] = segments[i];
        p.total_rows += segments[i].w.n_rows;
    }
    p.x = x;
    p.norm_weight = norm.weight;
    p.eps = norm.eps;
    p.accumulate = accumulate;
    size_t smem = (size_t)segments[0].w.n_cols * 4;
    int grid = grid_for((p.total_rows + 1) / 2);
    cudaError_t e;
    switch (segments[0].w.format) {
        case BC_Q4_0:
            if ((e = prepare(matvec_kernel<BC_Q4_0>, smem)) != cudaSuccess) return e;
            matvec_kernel<BC_Q4_0><<<grid, kThreads, smem, stream>>>(p);
            break;
        case BC_F16:
            if ((e = prepare(matvec_kernel<BC_F16>, smem)) != cudaSuccess) return e;
            matvec_kernel<BC_F16><<<grid, kThreads, smem, stream>>>(p);
            break;
        default:
            if ((e = prepare(matvec_kernel<BC_F32>, smem)) != cudaSuccess) return e;
            matvec_kernel<BC_F32><<<grid, kThreads, smem, stream>>>(p);
            break;
    }
    return cudaGetLastError();
}

cudaError_t matvec_swiglu(cudaStream_t stream, const Mat& gate, const Mat& up, const float* x, Norm norm, float* y) {
    SwigluParams p{gate, up, x, norm.weight, norm.eps, y};
    size_t smem = (size_t)gate.n_cols * 4;
    int grid = grid_for(gate.n_rows);
    cudaError_t e;
    switch (gate.format) {
        case BC_Q4_0:
            if ((e = prepare(matvec_swiglu_kernel<BC_Q4_0>, smem)) != cudaSuccess) return e;
            matvec_swiglu_kernel<BC_Q4_0><<<grid, kThreads, smem, stream>>>(p);
            break;
        case BC_F16:
            if ((e = prepare(matvec_swiglu_kernel<BC_F16>, smem)) != cudaSuccess) return e;
            matvec_swiglu_kernel<BC_F16><<<grid, kThreads, smem, stream>>>(p);
            break;
        default:
            if ((e = prepare(matvec_swiglu_kernel<BC_F32>, smem)) != cudaSuccess) return e;
            matvec_swiglu_kernel<BC_F32><<<grid, kThreads, smem, stream>>>(p);
            break;
    }
    return cudaGetLastError();
}

cudaError_t matvec_conv(cudaStream_t stream, const Mat& in_proj, const float* x, Norm norm, const float* taps,
                        float* history, float* out, uint32_t n_embd, uint32_t kernel) {
    ConvParams p{in_proj, x, norm.weight, norm.eps, taps, history, out, n_embd, kernel};
    size_t smem = (size_t)in_proj.n_cols * 4;
    int grid = grid_for(n_embd);
    cudaError_t e;
    switch (in_proj.format) {
        case BC_Q4_0:
            if ((e = prepare(matvec_conv_kernel<BC_Q4_0>, smem)) != cudaSuccess) return e;
            matvec_conv_kernel<BC_Q4_0><<<grid, kThreads, smem, stream>>>(p);
            break;
        case BC_F16:
            if ((e = prepare(matvec_conv_kernel<BC_F16>, smem)) != cudaSuccess) return e;
            matvec_conv_kernel<BC_F16><<<grid, kThreads, smem, stream>>>(p);
            break;
        default:
            if ((e = prepare(matvec_conv_kernel<BC_F32>, smem)) != cudaSuccess) return e;
            matvec_conv_kernel<BC_F32><<<grid, kThreads, smem, stream>>>(p);
            break;
    }
    return cudaGetLastError();
}

}  // namespace k
}  // namespace bc
