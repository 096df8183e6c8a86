// Qwen3.5 kernels: the Gated DeltaNet layer (causal convolution, gates, the delta-rule recurrence,
// the gated output norm) and the sigmoid output gate of Qwen's attention layers.
// Counterparts: crates/bobcat-metal/src/gdn.metal (gdn_conv :14, gdn_gated_norm :106, gdn_gates :132,
// gdn_qk_norm :181, gdn_recurrence :222, attention_gate :307); the arithmetic they must reproduce is
// crates/bobcat/src/qwen35.rs:430-516 and :754-778, f32 throughout and in the reference's order.

#include <cstdlib>

#include "async_utils.cuh"
#include "device_utils.cuh"
#include "kernels.h"

namespace bc {
namespace k {

namespace {

constexpr uint32_t kConvSerialTokens = 4;  // up to this many tokens one launch walks them serially

// One thread per (token, channel). x and out are [n_tokens][conv_dim]; taps are [conv_dim][K],
// oldest first; history is [conv_dim][K - 1] raw inputs, oldest first. The sum starts from the
// newest tap's term and adds the earlier inputs oldest first (qwen35.rs:449-461), from the batch or,
// for its first tokens, from the history, so any split into batches gives the same bits. K <= 8.
// The history is only read here; gdn_conv_history_kernel rewrites it afterwards.
__global__ void __launch_bounds__(256) gdn_conv_kernel(const float* __restrict__ x, const float* __restrict__ taps,
                                                       const float* __restrict__ history, float* __restrict__ out, uint32_t conv_dim,
                                                       uint32_t kernel, uint32_t n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= conv_dim) return;
    const uint32_t H = kernel - 1;
    float tap[8];
    for (uint32_t i = 0; i < kernel; ++i) tap[i] = taps[(uint64_t)c * kernel + i];
    for (uint32_t t = blockIdx.y; t < n_tokens; t += gridDim.y) {
        float sum = tap[H] * x[(uint64_t)t * conv_dim + c];
        for (uint32_t i = 0; i < H; ++i) {
            int64_t src = (int64_t)t - (int64_t)H + i;  // tap i meets the input of token t - H + i
            float past = src >= 0 ? x[(uint64_t)src * conv_dim + c] : history[(uint64_t)c * H + (uint32_t)(src + (int64_t)H)];
            sum += tap[i] * past;
        }
        out[(uint64_t)t * conv_dim + c] = sum / (1.f + expf(-sum));
    }
}

// The history after the batch: slot i holds the input of token n_tokens - H + i, or an older slot
// when the batch is shorter than the history. One thread per channel.
__global__ void gdn_conv_history_kernel(const float* __restrict__ x, float* __restrict__ history, uint32_t conv_dim, uint32_t kernel,
                                        uint32_t n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= conv_dim) return;
    const uint32_t H = kernel - 1;
    float next[7];
    for (uint32_t i = 0; i < H; ++i) {
        int64_t src = (int64_t)n_tokens - (int64_t)H + i;
        next[i] = src >= 0 ? x[(uint64_t)src * conv_dim + c] : history[(uint64_t)c * H + (uint32_t)(src + (int64_t)H)];
    }
    for (uint32_t i = 0; i < H; ++i) history[(uint64_t)c * H + i] = next[i];
}

// The same for a few tokens (a decode step): one thread per channel walks the tokens and
// updates the history itself, so one launch does it all. Same order of additions, same bits.
__global__ void gdn_conv_serial_kernel(const float* __restrict__ x, const float* __restrict__ taps, float* __restrict__ history,
                                       float* __restrict__ out, uint32_t conv_dim, uint32_t kernel, uint32_t n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= conv_dim) return;
    const uint32_t H = kernel - 1;
    float tap[8], past[7];
    for (uint32_t i = 0; i < kernel; ++i) tap[i] = taps[(uint64_t)c * kernel + i];
    for (uint32_t i = 0; i < H; ++i) past[i] = history[(uint64_t)c * H + i];
    for (uint32_t t = 0; t < n_tokens; ++t) {
        float input = x[(uint64_t)t * conv_dim + c];
        float sum = tap[H] * input;
        for (uint32_t i = 0; i < H; ++i) sum += tap[i] * past[i];
        out[(uint64_t)t * conv_dim + c] = sum / (1.f + expf(-sum));
        for (uint32_t i = 0; i + 1 < H; ++i) past[i] = past[i + 1];
        past[H - 1] = input;
    }
    for (uint32_t i = 0; i < H; ++i) history[(uint64_t)c * H + i] = past[i];
}

// beta = sigmoid(beta); decay = exp(a * softplus(alpha + dt_bias)), softplus(x) = x above 20
// (qwen35.rs:479-481, :776-778). In place over [n_tokens][n_v_heads]; alpha receives the decay.
__global__ void gdn_gates_kernel(float* __restrict__ beta, float* __restrict__ alpha, const float* __restrict__ a,
                                 const float* __restrict__ dt_bias, uint32_t n_v_heads, uint32_t n) {
    pdl_launch_dependents();
    pdl_wait();
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t head = i % n_v_heads;
    beta[i] = 1.f / (1.f + expf(-beta[i]));
    float v = alpha[i] + dt_bias[head];
    float sp = v > 20.f ? v : log1pf(expf(v));
    alpha[i] = expf(a[head] * sp);
}

struct RecurrenceParams {
    const float* qkv;    // [n_tokens][2 * key_dim + value_dim]: q heads, k heads, v heads (after the conv)
    const float* beta;   // [n_tokens][n_v_heads]
    const float* decay;  // [n_tokens][n_v_heads]
    float* state;        // [n_v_heads][k_dim][v_dim]
    float* out;          // [n_tokens][n_v_heads * v_dim]
    uint32_t n_k_heads, n_v_heads, k_dim, v_dim, n_tokens;
    int normalize;       // L2-normalise q (times 1/sqrt(k_dim)) and k here, as decode does
};

// l2_normalize of one head's q or k (qwen35.rs:762-768), element e * 32 + lane in `x[e]`: the sum of
// squares is taken per run of 32 elements across the warp and the runs are added in order, which
// is the order gdn_step_kernel takes (there a warp holds one run), so a batch and single steps
// normalise to the same bits. Returns the factor 1 / sqrt(sum + 1e-6).
template <int PER>
__device__ __forceinline__ float l2_factor(const float (&x)[PER]) {
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < PER; ++e) sum += warp_sum(x[e] * x[e]);
    return 1.0f / sqrtf(sum + 1e-6f);
}

// The q and k heads of a batch normalised in place, q also scaled by 1 / sqrt(k_dim): one warp
// per (token, q or k, key head). Run before the recurrence so that its token loop does not carry
// the reductions.
template <int KDIM>
__global__ void __launch_bounds__(256) gdn_qk_norm_kernel(float* __restrict__ qkv, uint32_t n_k_heads, uint32_t conv_dim, uint32_t n_tokens) {
    constexpr int PER = KDIM / 32;
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31, item = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
    if (item >= n_tokens * 2 * n_k_heads) return;
    const uint32_t t = item / (2 * n_k_heads), which = (item / n_k_heads) & 1, head = item % n_k_heads;
    float* x = qkv + (uint64_t)t * conv_dim + (uint64_t)which * n_k_heads * KDIM + head * KDIM;
    float v[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) v[e] = x[e * 32 + lane];
    const float factor = l2_factor<PER>(v);
    const float scale = which == 0 ? (1.0f / sqrtf((float)KDIM)) * factor : factor;
#pragma unroll
    for (int e = 0; e < PER; ++e) x[e * 32 + lane] = v[e] * scale;
}

// The delta rule over a run of tokens. One warp (a CTA of its own) per 8 state columns of a value
// head; four neighbouring lanes share a column, each holding a quarter of its k_dim state values in
// registers for the whole run. Per token (qwen35.rs:483-506): S *= decay; r = sum_i S[i] k_i;
// delta = (v - r) beta; S[i] += k_i delta; o = sum_i S[i] q_i. A lane sums its quarter as two
// interleaved partial sums and the quarters are added in order - the arithmetic of
// gdn_step_kernel, so a batch and single steps walk the same values. Value head h reads key head
// h % n_k_heads. A column's recurrence needs nothing of the other columns, so the warps share no
// state and meet at no barrier: each stages (and, when asked, normalises) the token's q and k for
// itself. A head spreads over v_dim / 8 warps, and a token is a chain of k_dim / 4 multiply-adds;
// the earlier form (a CTA per head, a thread per column with all k_dim values, two block barriers
// per token) took 1.45 us per token.
constexpr uint32_t kRecurrenceWarps = 4;  // independent warps per CTA, one per SM partition

template <int KDIM>
__global__ void __launch_bounds__(32 * kRecurrenceWarps) gdn_recurrence_kernel(RecurrenceParams p) {
    constexpr int PER = KDIM / 32;   // elements of q and of k a lane brings in
    constexpr int MINE = KDIM / 4;   // state values of its column a lane holds
    static_assert(KDIM % 32 == 0 && MINE % 4 == 0, "k_dim");
    // A token's inputs come through a ring of kAhead + 1 slots of shared memory, copied
    // (cp.async) kAhead tokens ahead: a token that loaded its successor's inputs into registers
    // and handed them on lasted one trip to memory, however little it computed.
    constexpr int kAhead = 7, kSlots = kAhead + 1;
    // A quarter of q (of k) is followed by four floats of padding, so the four quarters that a
    // warp's lanes read at once lie in different banks.
    struct Slot {
        float q[KDIM + 16], k[KDIM + 16], v[8], beta, decay, pad[2];
    };
    auto at = [](uint32_t e) { return e + 4 * (e / MINE); };
    __shared__ __align__(16) Slot rings[kRecurrenceWarps][kSlots];
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t vd = p.v_dim, groups = (vd + 7) / 8;
    const uint32_t unit = blockIdx.x * kRecurrenceWarps + (threadIdx.x >> 5);  // (head, group of 8 columns)
    if (unit >= p.n_v_heads * groups) return;  // whole warps; the warps of a CTA never meet
    Slot* ring = rings[threadIdx.x >> 5];
    const uint32_t head = unit / groups, lane = threadIdx.x & 31, part = lane & 3, first_lane = lane & ~3u;
    const uint32_t column = lane >> 2, j = (unit % groups) * 8 + column;
    const uint32_t key_head = head % p.n_k_heads;
    const uint32_t key_dim = p.n_k_heads * KDIM, conv_dim = 2 * key_dim + p.n_v_heads * vd;
    float* state = p.state + (uint64_t)head * KDIM * vd + (uint64_t)part * MINE * vd;
    float S[MINE];
    if (j < vd) {
#pragma unroll
        for (int i = 0; i < MINE; ++i) S[i] = state[(uint64_t)i * vd + j];
    }
    // Lane l brings elements e * 32 + l of q and of k; the first lane of a column its v; lanes 1 and 2 the gates.
    auto bring = [&](uint32_t t) {
        if (t < p.n_tokens) {
            Slot& slot = ring[t % kSlots];
            const float* row = p.qkv + (uint64_t)t * conv_dim;
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                async::cp_async_4(async::smem_u32(&slot.q[at(e * 32 + lane)]), row + key_head * KDIM + e * 32 + lane);
                async::cp_async_4(async::smem_u32(&slot.k[at(e * 32 + lane)]), row + key_dim + key_head * KDIM + e * 32 + lane);
            }
            if (part == 0 && j < vd) async::cp_async_4(async::smem_u32(&slot.v[column]), row + 2 * key_dim + head * vd + j);
            if (lane == 1) async::cp_async_4(async::smem_u32(&slot.beta), p.beta + (uint64_t)t * p.n_v_heads + head);
            if (lane == 2) async::cp_async_4(async::smem_u32(&slot.decay), p.decay + (uint64_t)t * p.n_v_heads + head);
        }
        async::cp_async_commit();
    };
#pragma unroll
    for (int t = 0; t < kAhead; ++t) bring((uint32_t)t);
    for (uint32_t t = 0; t < p.n_tokens; ++t) {
        __syncwarp();  // every lane is through with the slot the next copy overwrites (the previous token's)
        bring(t + kAhead);
        async::cp_async_wait<kAhead>();  // all but the newest kAhead groups: this token's bytes are in
        __syncwarp();
        Slot& slot = ring[t % kSlots];
        if (p.normalize) {
            float q[PER], k[PER];
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                q[e] = slot.q[at(e * 32 + lane)];
                k[e] = slot.k[at(e * 32 + lane)];
            }
            const float q_scale = (1.0f / sqrtf((float)KDIM)) * l2_factor<PER>(q), k_scale = l2_factor<PER>(k);
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                slot.q[at(e * 32 + lane)] = q[e] * q_scale;
                slot.k[at(e * 32 + lane)] = k[e] * k_scale;
            }
            __syncwarp();
        }
        const float decay = slot.decay, beta = slot.beta, v = j < vd ? slot.v[column] : 0.f;
        // Every lane takes part in the shuffles; lanes past the last column carry zeros.
        const float4* k4 = reinterpret_cast<const float4*>(slot.k + part * (MINE + 4));
        const float4* q4 = reinterpret_cast<const float4*>(slot.q + part * (MINE + 4));
        float r0 = 0.f, r1 = 0.f;
        if (j < vd) {
#pragma unroll
            for (int i = 0; i < MINE / 4; ++i) {
                const float4 kk = k4[i];
                S[4 * i] *= decay;
                S[4 * i + 1] *= decay;
                S[4 * i + 2] *= decay;
                S[4 * i + 3] *= decay;
                r0 += S[4 * i] * kk.x + S[4 * i + 2] * kk.z;
                r1 += S[4 * i + 1] * kk.y + S[4 * i + 3] * kk.w;
            }
        }
        const float r_part = r0 + r1;
        float r = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) r += __shfl_sync(0xffffffffu, r_part, first_lane + q);  // the quarters in order
        const float delta = (v - r) * beta;
        float o0 = 0.f, o1 = 0.f;
        if (j < vd) {
#pragma unroll
            for (int i = 0; i < MINE / 4; ++i) {
                const float4 kk = k4[i], qq = q4[i];
                S[4 * i] += kk.x * delta;
                S[4 * i + 1] += kk.y * delta;
                S[4 * i + 2] += kk.z * delta;
                S[4 * i + 3] += kk.w * delta;
                o0 += S[4 * i] * qq.x + S[4 * i + 2] * qq.z;
                o1 += S[4 * i + 1] * qq.y + S[4 * i + 3] * qq.w;
            }
        }
        const float o_part = o0 + o1;
        float out = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) out += __shfl_sync(0xffffffffu, o_part, first_lane + q);
        if (j < vd && part == 0) p.out[(uint64_t)t * p.n_v_heads * vd + head * vd + j] = out;
    }
    async::cp_async_wait<0>();
    if (j < vd) {
#pragma unroll
        for (int i = 0; i < MINE; ++i) state[(uint64_t)i * vd + j] = S[i];
    }
}

// One warp per (token, value head): x = RMSNorm(x) * weight * silu(z) (qwen35.rs:508-513).
__global__ void gdn_gated_norm_kernel(float* __restrict__ x, const float* __restrict__ z, const float* __restrict__ weight,
                                      uint32_t v_dim, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x;
    float* row = x + (uint64_t)blockIdx.x * v_dim;
    const float* gate = z + (uint64_t)blockIdx.x * v_dim;
    float sumsq = 0.f;
    for (uint32_t d = lane; d < v_dim; d += 32) sumsq += row[d] * row[d];
    sumsq = warp_sum(sumsq);
    const float scale = rsqrtf(sumsq / (float)v_dim + eps);
    for (uint32_t d = lane; d < v_dim; d += 32) {
        float g = gate[d];
        row[d] = weight[d] * (row[d] * scale) * (g / (1.f + expf(-g)));
    }
}

// ---- One token through a whole DeltaNet mixer in one launch (decode): the causal convolution
// with SiLU and its history shift, the gates, the L2 norms of q and k, the delta rule on the state
// and the gated RMSNorm of the output, i.e. gdn_conv + gdn_gates + gdn_recurrence + gdn_gated_norm
// for n_tokens == 1 (qwen35.rs:430-516). One CTA per key head; it serves the value heads that read
// that key head (h = key_head + m * n_k_heads), one thread per state column of each, so the
// convolution of q and k happens once and nothing races on its history.
struct StepParams {
    const float* qkv;      // [conv_dim] projections before the convolution: q heads, k heads, v heads
    const float* taps;     // [conv_dim][kernel]
    float* history;        // [conv_dim][kernel - 1]
    const float* beta;     // [n_v_heads] before the sigmoid
    const float* alpha;    // [n_v_heads] before the softplus
    const float* a;        // [n_v_heads]
    const float* dt_bias;  // [n_v_heads]
    float* state;          // [n_v_heads][k_dim][v_dim]
    const float* z;        // [n_v_heads * v_dim]
    const float* norm_weight;  // [v_dim]
    float* out;            // [n_v_heads * v_dim]
    uint32_t n_k_heads, n_v_heads, k_dim, v_dim, kernel;
    float eps;
};

// The convolution of one channel for one token, and the history shift (same order of additions as gdn_conv).
__device__ __forceinline__ float conv_step(const StepParams& p, uint32_t channel) {
    const uint32_t H = p.kernel - 1;
    const float* tap = p.taps + (uint64_t)channel * p.kernel;
    float* hist = p.history + (uint64_t)channel * H;
    const float input = p.qkv[channel];
    float sum = tap[H] * input;
    float past[7];
    for (uint32_t i = 0; i < H; ++i) {
        past[i] = hist[i];
        sum += tap[i] * past[i];
    }
    for (uint32_t i = 0; i + 1 < H; ++i) hist[i] = past[i + 1];
    hist[H - 1] = input;
    return sum / (1.f + expf(-sum));
}

constexpr int kStepParts = 4;  // threads that share a state column, each holding a quarter of its rows

template <int KDIM>
__global__ void __launch_bounds__(1024) gdn_step_kernel(StepParams p) {
    // Thread (part, m, j): rows [part * KDIM / 4, (part + 1) * KDIM / 4) of column j of the state of
    // value head key_head + m * n_k_heads. The quarter column is loaded into registers first of
    // all, so that read overlaps the convolution; the quarters' partial dot products meet in shared memory.
    constexpr int kRows = KDIM / kStepParts;
    __shared__ __align__(16) float qs[KDIM], ks[KDIM];
    __shared__ float scratch[96];
    __shared__ float r_part[kStepParts][256], o_part[kStepParts][256], o_full[256];
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t key_head = blockIdx.x, tid = threadIdx.x, vd = p.v_dim;
    const uint32_t lane = tid & 31, warp = tid >> 5;
    const uint32_t key_dim = p.n_k_heads * KDIM, ratio = p.n_v_heads / p.n_k_heads;
    const uint32_t column_id = tid % (ratio * vd), part = tid / (ratio * vd);  // blockDim.x == kStepParts * ratio * v_dim
    const uint32_t m = column_id / vd, j = column_id % vd, head = key_head + m * p.n_k_heads;
    float* column = p.state + (uint64_t)head * KDIM * vd + (uint64_t)(part * kRows) * vd + j;
    float S[kRows];
#pragma unroll
    for (int i = 0; i < kRows; ++i) S[i] = column[(uint64_t)i * vd];
    // q and k of this key head: threads below KDIM convolve one channel of each.
    float qv = 0.f, kv = 0.f;
    if (tid < KDIM) {
        qv = conv_step(p, key_head * KDIM + tid);
        kv = conv_step(p, key_dim + key_head * KDIM + tid);
    }
    // l2_normalize (qwen35.rs:762-768): f32 sum of squares, x *= scale / sqrt(sum + 1e-6).
    float q2 = warp_sum(qv * qv), k2 = warp_sum(kv * kv);
    if (lane == 0) {
        scratch[warp] = q2;
        scratch[32 + warp] = k2;
    }
    __syncthreads();
    if (tid < KDIM) {
        float qsum = 0.f, ksum = 0.f;
        for (uint32_t w = 0; w < (KDIM + 31) / 32; ++w) {
            qsum += scratch[w];
            ksum += scratch[32 + w];
        }
        qs[tid] = qv * ((1.0f / sqrtf((float)KDIM)) / sqrtf(qsum + 1e-6f));
        ks[tid] = kv * (1.0f / sqrtf(ksum + 1e-6f));
    }
    // The column's element of v (convolved once, by the part-0 thread) and the head's gates.
    float v = 0.f;
    if (part == 0) v = conv_step(p, 2 * key_dim + head * vd + j);
    // beta = sigmoid(beta); decay = exp(a * softplus(alpha + dt_bias)), softplus(x) = x above 20.
    const float braw = p.beta[head], araw = p.alpha[head] + p.dt_bias[head];
    const float beta = 1.f / (1.f + expf(-braw));
    const float decay = expf(p.a[head] * (araw > 20.f ? araw : log1pf(expf(araw))));
    __syncthreads();
    const float4* k4 = reinterpret_cast<const float4*>(ks + part * kRows);
    const float4* q4 = reinterpret_cast<const float4*>(qs + part * kRows);
    float r0 = 0.f, r1 = 0.f;
#pragma unroll
    for (int i = 0; i < kRows / 4; ++i) {
        const float4 kk = k4[i];
        S[4 * i] *= decay;
        S[4 * i + 1] *= decay;
        S[4 * i + 2] *= decay;
        S[4 * i + 3] *= decay;
        r0 += S[4 * i] * kk.x + S[4 * i + 2] * kk.z;
        r1 += S[4 * i + 1] * kk.y + S[4 * i + 3] * kk.w;
    }
    r_part[part][column_id] = r0 + r1;
    if (part == 0) o_full[column_id] = v;  // parks v where every part can read it
    __syncthreads();
    float r = 0.f;
#pragma unroll
    for (int q = 0; q < kStepParts; ++q) r += r_part[q][column_id];  // every part adds them in the same order
    const float delta = (o_full[column_id] - r) * beta;
    float o0 = 0.f, o1 = 0.f;
#pragma unroll
    for (int i = 0; i < kRows / 4; ++i) {
        const float4 kk = k4[i], qq = q4[i];
        S[4 * i] += kk.x * delta;
        S[4 * i + 1] += kk.y * delta;
        S[4 * i + 2] += kk.z * delta;
        S[4 * i + 3] += kk.w * delta;
        o0 += S[4 * i] * qq.x + S[4 * i + 2] * qq.z;
        o1 += S[4 * i + 1] * qq.y + S[4 * i + 3] * qq.w;
    }
#pragma unroll
    for (int i = 0; i < kRows; ++i) column[(uint64_t)i * vd] = S[i];
    o_part[part][column_id] = o0 + o1;
    __syncthreads();
    // Gated RMSNorm over each value head's v_dim outputs, by the part-0 threads (v_dim is a multiple
    // of 32, so a warp belongs to one head): out = weight * (o * scale) * silu(z).
    float o = 0.f;
    if (part == 0) {
#pragma unroll
        for (int q = 0; q < kStepParts; ++q) o += o_part[q][column_id];
    }
    const float sq = warp_sum(o * o);
    if (lane == 0) scratch[64 + warp] = sq;
    __syncthreads();
    if (part == 0) {
        const uint32_t warps_per_head = vd / 32, first = m * warps_per_head;
        float sumsq = 0.f;
        for (uint32_t w = 0; w < warps_per_head; ++w) sumsq += scratch[64 + first + w];
        const float scale = rsqrtf(sumsq / (float)vd + p.eps);
        const float g = p.z[head * vd + j];
        p.out[head * vd + j] = p.norm_weight[j] * (o * scale) * (g / (1.f + expf(-g)));
    }
}

// out[t][h][d] *= sigmoid(gate) with the gate read from the interleaved q projection:
// q_gate[t][h][head_dim + d] of [n_tokens][n_heads][2 * head_dim] (qwen35.rs:383-390, :422-424).
__global__ void attention_gate_kernel(float* __restrict__ out, const float* __restrict__ q_gate, uint32_t n_heads, uint32_t head_dim,
                                      uint64_t n) {
    pdl_launch_dependents();
    pdl_wait();
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t d = i % head_dim;
    uint64_t th = i / head_dim;  // token * n_heads + head
    float g = q_gate[th * 2 * head_dim + head_dim + d];
    out[i] *= 1.f / (1.f + expf(-g));
}

}  // namespace

int gdn_conv_launches(uint32_t n_tokens) { return n_tokens <= kConvSerialTokens ? 1 : 2; }

cudaError_t gdn_conv(cudaStream_t stream, const float* x, const float* taps, float* history, float* out, uint32_t conv_dim,
                     uint32_t kernel, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    if (n_tokens <= kConvSerialTokens) {
        void* args[] = {&x, &taps, &history, &out, &conv_dim, &kernel, &n_tokens};
        return launch_kernel((const void*)gdn_conv_serial_kernel, dim3((conv_dim + 127) / 128), dim3(128), 0, stream, args);
    }
    const float* read_history = history;
    void* args[] = {&x, &taps, &read_history, &out, &conv_dim, &kernel, &n_tokens};
    cudaError_t e = launch_kernel((const void*)gdn_conv_kernel, dim3((conv_dim + 255) / 256, n_tokens < 65535u ? n_tokens : 65535u), dim3(256), 0,
                                  stream, args);
    if (e != cudaSuccess) return e;
    void* history_args[] = {&x, &history, &conv_dim, &kernel, &n_tokens};
    return launch_kernel((const void*)gdn_conv_history_kernel, dim3((conv_dim + 127) / 128), dim3(128), 0, stream, history_args);
}

cudaError_t gdn_gates(cudaStream_t stream, float* beta, float* alpha, const float* a, const float* dt_bias, uint32_t n_v_heads,
                      uint32_t n_tokens) {
    uint32_t n = n_v_heads * n_tokens;
    if (n == 0) return cudaSuccess;
    void* args[] = {&beta, &alpha, &a, &dt_bias, &n_v_heads, &n};
    return launch_kernel((const void*)gdn_gates_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, args);
}

cudaError_t gdn_recurrence(cudaStream_t stream, const float* qkv, const float* beta, const float* decay, float* state, float* out,
                           uint32_t n_k_heads, uint32_t n_v_heads, uint32_t k_dim, uint32_t v_dim, uint32_t n_tokens, bool normalize) {
    if (n_tokens == 0) return cudaSuccess;
    RecurrenceParams p{qkv, beta, decay, state, out, n_k_heads, n_v_heads, k_dim, v_dim, n_tokens, normalize ? 1 : 0};
    void* args[] = {&p};
    // A warp per 8 state columns of a head.
    const void* kernel = k_dim == 32 ? (const void*)gdn_recurrence_kernel<32> : k_dim == 64 ? (const void*)gdn_recurrence_kernel<64>
                       : k_dim == 96 ? (const void*)gdn_recurrence_kernel<96> : (const void*)gdn_recurrence_kernel<128>;
    const uint32_t units = n_v_heads * ((v_dim + 7) / 8);
    return launch_kernel(kernel, dim3((units + kRecurrenceWarps - 1) / kRecurrenceWarps), dim3(32 * kRecurrenceWarps), 0, stream, args);
}

cudaError_t gdn_qk_norm(cudaStream_t stream, float* qkv, uint32_t n_k_heads, uint32_t n_v_heads, uint32_t k_dim, uint32_t v_dim, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    uint32_t conv_dim = 2 * n_k_heads * k_dim + n_v_heads * v_dim;
    const uint32_t items = n_tokens * 2 * n_k_heads;
    void* args[] = {&qkv, &n_k_heads, &conv_dim, &n_tokens};
    const void* kernel = k_dim == 32 ? (const void*)gdn_qk_norm_kernel<32> : k_dim == 64 ? (const void*)gdn_qk_norm_kernel<64>
                       : k_dim == 96 ? (const void*)gdn_qk_norm_kernel<96> : (const void*)gdn_qk_norm_kernel<128>;
    return launch_kernel(kernel, dim3((items + 7) / 8), dim3(256), 0, stream, args);
}

bool gdn_step_supported(uint32_t n_k_heads, uint32_t n_v_heads, uint32_t k_dim, uint32_t v_dim, uint32_t kernel) {
    if (n_k_heads == 0 || n_v_heads % n_k_heads != 0 || kernel < 2 || kernel > 8) return false;
    if (k_dim != 32 && k_dim != 64 && k_dim != 96 && k_dim != 128) return false;
    const uint32_t columns = (n_v_heads / n_k_heads) * v_dim;  // state columns a CTA serves
    return v_dim % 32 == 0 && columns <= 256 && kStepParts * columns >= k_dim;
}

cudaError_t gdn_step(cudaStream_t stream, const float* qkv, const float* taps, float* history, const float* beta, const float* alpha,
                     const float* a, const float* dt_bias, float* state, const float* z, const float* norm_weight, float* out,
                     uint32_t n_k_heads, uint32_t n_v_heads, uint32_t k_dim, uint32_t v_dim, uint32_t kernel, float eps) {
    StepParams p{qkv, taps, history, beta, alpha, a, dt_bias, state, z, norm_weight, out, n_k_heads, n_v_heads, k_dim, v_dim, kernel, eps};
    void* args[] = {&p};
    const uint32_t threads = kStepParts * (n_v_heads / n_k_heads) * v_dim;
    const void* kernel_fn = k_dim == 32 ? (const void*)gdn_step_kernel<32> : k_dim == 64 ? (const void*)gdn_step_kernel<64>
                          : k_dim == 96 ? (const void*)gdn_step_kernel<96> : (const void*)gdn_step_kernel<128>;
    return launch_kernel(kernel_fn, dim3(n_k_heads), dim3(threads), 0, stream, args);
}

cudaError_t gdn_gated_norm(cudaStream_t stream, float* x, const float* z, const float* weight, uint32_t v_dim, uint32_t n_rows,
                           float eps) {
    if (n_rows == 0) return cudaSuccess;
    void* args[] = {&x, &z, &weight, &v_dim, &eps};
    return launch_kernel((const void*)gdn_gated_norm_kernel, dim3(n_rows), dim3(32), 0, stream, args);
}

cudaError_t attention_gate(cudaStream_t stream, float* out, const float* q_gate, uint32_t n_heads, uint32_t head_dim, uint32_t n_tokens) {
    uint64_t n = (uint64_t)n_tokens * n_heads * head_dim;
    if (n == 0) return cudaSuccess;
    void* args[] = {&out, &q_gate, &n_heads, &head_dim, &n};
    return launch_kernel((const void*)attention_gate_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, args);
}

}  // namespace k
}  // namespace bc
