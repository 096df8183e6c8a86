// Decode-time matrix-vector kernels: y = W x with optional fused RMSNorm of x, residual
// accumulate, SwiGLU of a gate/up pair, and the LFM2 gated short convolution.
//
// One kernel template serves all of them. A CTA stages the input vector once in shared memory
// (multiplied by the norm weight when a norm is fused, with the sum of squares reduced on the
// way), then its warps walk "units" of two or three rows that share the staged input. A lane owns
// whole 32-weight blocks: one 128-bit load brings a block's quants, the block's 32 inputs come from
// shared memory once and are reused for every row of the unit, and the block's scale multiplies the
// finished block sum. A warp's loads are contiguous 512-byte runs of the weight stream. Rows too
// wide for one warp to finish quickly are split across 2, 4 or 8 warps whose partial sums meet in
// shared memory.
//
// A decode step is a chain of such launches, each depending on the one before through a few
// kilobytes of activations, while the weights - the only real HBM traffic - depend on nothing. So
// every kernel here is written for programmatic dependent launch: it first lets its successor
// start, then asks the L2 to fetch the weights its CTA will read, and only then waits for its
// predecessor's results. The weight stream of launch N+1 overlaps the tail of launch N.
//
// Counterparts in the reference: matvec_k / matvec_q / swiglu_rows / matvec_conv in
// crates/bobcat-metal/src/matvec.metal:151-585, lane layout q4_0_lanes in quant.metal:587-656.

#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "matvec_common.cuh"

namespace bc {
namespace k {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
// Bytes of weights one CTA asks the L2 to fetch ahead of its dependency wait.
constexpr uint32_t kPrefetchCap = 96 * 1024;

enum Mode { kPlain = 0, kSwiglu = 1, kConv = 2 };

struct Params {
    // kPlain: up to three matrices that share x; kSwiglu: seg[0] = gate, seg[1] = up;
    // kConv: seg[0] = in_proj.
    MatvecSegment seg[4];
    int n_segments;
    uint32_t total_rows;  // kPlain: rows over all segments
    uint32_t units;       // kPlain: row pairs; kSwiglu: rows; kConv: channels
    int ksplit;           // warps that share one unit: 1, 2, 4 or 8
    uint32_t prefetch_bytes;  // weight bytes each CTA asks the L2 for ahead of its dependency wait
    const float* x;
    const float* norm_weight;
    float eps;
    int accumulate;
    // kConv
    const float* taps;
    float* history;
    uint32_t n_embd, conv_kernel;
};

template <int MODE>
__device__ __forceinline__ constexpr int rows_per_unit() { return MODE == kConv ? 3 : 2; }

// The rows of unit `unit` (clamped into range by the caller) and, for kPlain, where each result goes.
template <int MODE>
__device__ __forceinline__ void unit_rows(const Params& p, uint32_t unit, RowPtr (&rows)[rows_per_unit<MODE>()], float* (&out)[rows_per_unit<MODE>()]) {
    if (MODE == kPlain) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            uint32_t row = unit * 2 + r;
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
    } else if (MODE == kSwiglu) {
        rows[0] = row_of(p.seg[0].w, unit);
        rows[1] = row_of(p.seg[1].w, unit);
        out[0] = p.seg[0].y + unit;
        out[1] = nullptr;
    } else {
        rows[0] = row_of(p.seg[0].w, unit);
        rows[1] = row_of(p.seg[0].w, p.n_embd + unit);
        rows[2] = row_of(p.seg[0].w, 2 * p.n_embd + unit);
        out[0] = p.seg[0].y + unit;
        out[1] = out[2] = nullptr;
    }
}

template <int FORMAT, int MODE>
__global__ void __launch_bounds__(kThreads) matvec_kernel(Params p) {
    constexpr int R = rows_per_unit<MODE>();
    extern __shared__ float4 xs[];
    __shared__ float reduce_scratch[32];
    __shared__ float partial[2][kWarps][3];
    const uint32_t n_cols = p.seg[0].w.n_cols;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ksplit = p.ksplit, units_per_pass = kWarps / ksplit;
    const int kpart = warp % ksplit, slot = warp / ksplit;

    // Let the next launch of the stream start, fetch this CTA's weights toward the L2, and only
    // then wait for the launches before this one: their results (x, and y when accumulating) are
    // first touched below the wait.
    pdl_launch_dependents();
    {
        const uint32_t row_bytes = FORMAT == BC_Q4_0 ? (n_cols >> 5) * 18 : FORMAT == BC_Q8_0 ? (n_cols >> 5) * 34 : FORMAT == BC_Q6_K ? (n_cols >> 8) * 210
                                 : n_cols * (FORMAT == BC_F16 ? 2u : 4u);
        const uint32_t rows_per_pass = (uint32_t)units_per_pass * R;
        uint32_t max_rows = p.prefetch_bytes / (row_bytes ? row_bytes : 1);
        for (uint32_t t = threadIdx.x; t < max_rows; t += blockDim.x) {
            uint32_t pass = t / rows_per_pass, within = t % rows_per_pass;
            uint64_t unit = ((uint64_t)blockIdx.x + (uint64_t)pass * gridDim.x) * units_per_pass + within / R;
            if (unit >= p.units) break;
            RowPtr rows[R];
            float* out[R];
            unit_rows<MODE>(p, (uint32_t)unit, rows, out);
            prefetch_row<FORMAT>(rows[within % R], n_cols);
        }
    }
    pdl_wait();

    const float scale = stage_input(p.x, p.norm_weight, p.eps, n_cols, xs, reduce_scratch);
    int parity = 0;
    for (uint64_t first = (uint64_t)blockIdx.x * units_per_pass; first < p.units; first += (uint64_t)gridDim.x * units_per_pass) {
        uint64_t wanted = first + slot;
        const bool valid = wanted < p.units;
        const uint32_t unit = valid ? (uint32_t)wanted : p.units - 1;
        RowPtr rows[R];
        float* out[R];
        unit_rows<MODE>(p, unit, rows, out);
        float acc[R];
        dot_rows<FORMAT, R>(rows, n_cols, xs, lane, kpart, ksplit, acc);
        if (ksplit > 1) {
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r) partial[parity][warp][r] = acc[r];
            }
            __syncthreads();
            if (kpart == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float total = 0.f;
                    for (int kk = 0; kk < ksplit; ++kk) total += partial[parity][warp + kk][r];
                    acc[r] = total;
                }
            }
            parity ^= 1;
        }
        if (lane == 0 && kpart == 0 && valid) {
            if (MODE == kPlain) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    if (out[r]) {
                        float v = acc[r] * scale;
                        *out[r] = p.accumulate ? *out[r] + v : v;
                    }
                }
            } else if (MODE == kSwiglu) {
                float g = acc[0] * scale, u = acc[1] * scale;
                *out[0] = g / (1.f + expf(-g)) * u;
            } else {
                // Rows ch, n_embd + ch and 2 n_embd + ch of in_proj gave B, C and X; run the taps over
                // B*X and the channel's history, shift the history, write C * conv (the arithmetic
                // of crates/bobcat/src/lfm2.rs:456-475 with f32 sums).
                float b = acc[0] * scale, c = acc[1] * scale, xv = acc[2] * scale;
                float bx = b * xv;
                const uint32_t ch = unit, K = p.conv_kernel;
                const float* taps = p.taps + (uint64_t)ch * K;
                float sum = taps[K - 1] * bx;
                for (uint32_t kk = 0; kk + 1 < K; ++kk) sum += taps[kk] * p.history[(uint64_t)kk * p.n_embd + ch];
                for (uint32_t kk = 0; kk + 2 < K; ++kk) p.history[(uint64_t)kk * p.n_embd + ch] = p.history[(uint64_t)(kk + 1) * p.n_embd + ch];
                p.history[(uint64_t)(K - 2) * p.n_embd + ch] = bx;
                *out[0] = c * sum;
            }
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

// How many warps share a unit: split rows that would take one warp more than three trips when the
// launch has too few units to fill the machine anyway.
int choose_ksplit(int format, uint32_t n_cols, uint64_t units) {
    uint32_t per_trip = format == BC_Q4_0 || format == BC_Q8_0 ? 1024 : format == BC_F16 ? 256 : 128;
    uint32_t trips = (n_cols + per_trip - 1) / per_trip;
    if (units >= (uint64_t)sm_count_impl() * kWarps * 2) return 1;
    int ksplit = 1;
    while (ksplit < kWarps && (trips + ksplit - 1) / ksplit > 3) ksplit *= 2;
    return ksplit;
}

template <int MODE>
const void* kernel_for(int format) {
    switch (format) {
        case BC_Q4_0: return (const void*)matvec_kernel<BC_Q4_0, MODE>;
        case BC_F16: return (const void*)matvec_kernel<BC_F16, MODE>;
        case BC_Q8_0: return (const void*)matvec_kernel<BC_Q8_0, MODE>;
        case BC_Q6_K: return (const void*)matvec_kernel<BC_Q6_K, MODE>;
        default: return (const void*)matvec_kernel<BC_F32, MODE>;
    }
}

cudaError_t launch(const void* kernel, cudaStream_t stream, Params& p) {
    size_t smem = (size_t)p.seg[0].w.n_cols * 4;
    cudaError_t e = ensure_dynamic_smem(kernel, smem);
    if (e != cudaSuccess) return e;
    p.ksplit = choose_ksplit(p.seg[0].w.format, p.seg[0].w.n_cols, p.units);
    uint64_t per_cta = (uint64_t)(kWarps / p.ksplit);
    uint64_t ctas = (p.units + per_cta - 1) / per_cta;
    uint64_t cap = (uint64_t)sm_count_impl() * 8;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    // Keep the whole launch's prefetch well inside the L2.
    uint64_t budget = (48ull << 20) / ctas;
    p.prefetch_bytes = (uint32_t)(budget < kPrefetchCap ? budget : kPrefetchCap);
    void* args[] = {&p};
    return launch_kernel(kernel, dim3((unsigned)ctas), dim3(kThreads), smem, stream, args);
}

bool g_pdl = [] {
    const char* v = getenv("BOBCAT_NO_PDL");
    return !(v && v[0] == '1');
}();

}  // namespace

bool pdl_enabled() { return g_pdl; }

cudaError_t launch_kernel(const void* kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, void** args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = g_pdl ? 1 : 0;
    return cudaLaunchKernelExC(&config, kernel, args);
}

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

int sm_count() { return sm_count_impl(); }

Mat Mat::rows(uint32_t first, uint32_t count) const {
    Mat m = *this;
    m.n_rows = count;
    if (format == BC_Q4_0) {
        uint64_t nb = n_cols >> 5;
        m.data = static_cast<const uint4*>(data) + first * nb;
        m.scales = scales + first * nb;
        // Tiles hold 16 rows each, so only a tile-aligned row range keeps its tile copy.
        m.tiles = (tiles && first % 16 == 0) ? static_cast<const uint8_t*>(tiles) + (uint64_t)(first / 16) * nb * 288 : nullptr;
    } else if (format == BC_F16) {
        m.data = static_cast<const __half*>(data) + (uint64_t)first * n_cols;
    } else if (format == BC_Q8_0) {
        m.data = static_cast<const uint8_t*>(data) + (uint64_t)first * (n_cols >> 5) * 34;
    } else if (format == BC_Q6_K) {
        m.data = static_cast<const uint8_t*>(data) + (uint64_t)first * (n_cols >> 8) * 210;
    } else {
        m.data = static_cast<const float*>(data) + (uint64_t)first * n_cols;
    }
    return m;
}

uint64_t Mat::bytes() const {
    uint64_t n = (uint64_t)n_rows * n_cols;
    if (format == BC_Q4_0) return n / 32 * 18;
    if (format == BC_F16) return n * 2;
    if (format == BC_Q8_0) return n / 32 * 34;
    if (format == BC_Q6_K) return n / 256 * 210;
    return n * 4;
}

cudaError_t matvec_prepare(uint32_t widest_cols) {
    size_t smem = (size_t)widest_cols * 4;
    cudaError_t prepared = matvec_mma_prepare(widest_cols);
    if (prepared != cudaSuccess) return prepared;
    for (int format : {BC_Q4_0, BC_F16, BC_F32, BC_Q8_0, BC_Q6_K}) {
        for (const void* kernel : {kernel_for<kPlain>(format), kernel_for<kSwiglu>(format), kernel_for<kConv>(format)}) {
            cudaError_t e = ensure_dynamic_smem(kernel, smem);
            if (e != cudaSuccess) return e;
        }
    }
    return cudaSuccess;
}

cudaError_t matvec(cudaStream_t stream, const MatvecSegment* segments, int n_segments, const float* x, Norm norm,
                   bool accumulate) {
    bool tiled = segments[0].w.format == BC_Q4_0;
    for (int i = 0; i < n_segments; ++i) tiled = tiled && segments[i].w.tiles != nullptr;
    if (tiled) return matvec_mma(stream, segments, n_segments, x, norm, accumulate);
    Params p{};
    p.n_segments = n_segments;
    for (int i = 0; i < n_segments; ++i) {
        p.seg[i] = segments[i];
        p.total_rows += segments[i].w.n_rows;
    }
    p.units = (p.total_rows + 1) / 2;
    p.x = x;
    p.norm_weight = norm.weight;
    p.eps = norm.eps;
    p.accumulate = accumulate;
    return launch(kernel_for<kPlain>(segments[0].w.format), stream, p);
}

cudaError_t matvec_swiglu(cudaStream_t stream, const Mat& gate, const Mat& up, const float* x, Norm norm, float* y) {
    if (gate.format == BC_Q4_0 && gate.tiles && up.tiles) return matvec_swiglu_mma(stream, gate, up, x, norm, y);
    Params p{};
    p.n_segments = 2;
    p.seg[0] = MatvecSegment{gate, y};
    p.seg[1] = MatvecSegment{up, nullptr};
    p.total_rows = gate.n_rows;
    p.units = gate.n_rows;
    p.x = x;
    p.norm_weight = norm.weight;
    p.eps = norm.eps;
    return launch(kernel_for<kSwiglu>(gate.format), stream, p);
}

cudaError_t matvec_conv(cudaStream_t stream, const Mat& in_proj, const float* x, Norm norm, const float* taps,
                        float* history, float* out, uint32_t n_embd, uint32_t kernel) {
    if (in_proj.format == BC_Q4_0 && in_proj.tiles && n_embd % 16 == 0) return matvec_conv_mma(stream, in_proj, x, norm, taps, history, out, n_embd, kernel);
    Params p{};
    p.n_segments = 1;
    p.seg[0] = MatvecSegment{in_proj, out};
    p.total_rows = in_proj.n_rows;
    p.units = n_embd;
    p.x = x;
    p.norm_weight = norm.weight;
    p.eps = norm.eps;
    p.taps = taps;
    p.history = history;
    p.n_embd = n_embd;
    p.conv_kernel = kernel;
    return launch(kernel_for<kConv>(in_proj.format), stream, p);
}

}  // namespace k
}  // namespace bc
