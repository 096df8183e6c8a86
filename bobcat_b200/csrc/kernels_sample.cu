// Token sampling on the device: the steps of the reference's Sampler::sample
// (crates/bobcat-cli/src/sampler.rs:45-112, llama.cpp's order) without sorting the vocabulary and
// without bringing the logits to the host: repetition penalty, top-k, top-p, min-p, temperature,
// then the draw.
//
// The reference sorts the candidates by logit and walks them in that order three times (the
// top-p cut, the min-p floor, the draw). Walking a sorted list until a running sum crosses a
// target is a selection problem: it needs the key at which the sum crosses, not the order of
// everything else. Logits map to 32-bit keys that sort the same way (descending logit = ascending
// key), and a key is found eight bits at a time: a histogram of the summed weight per value of the
// next eight bits (over the candidates that match the bits decided so far), a walk over its 256
// buckets to the one where the running sum crosses, four rounds. So every step is a few passes
// over the logits by one CTA:
//   top-k   - the key of the k-th largest logit (weights 1),
//   top-p   - the key where the softmax at temperature one, summed from the largest logit down,
//             reaches top_p,
//   min-p   - a plain threshold, logit >= largest + ln(min_p),
//   draw    - the key where the softmax of the survivors at the temperature, summed from the
//             largest logit down, passes the uniform draw; equal logits are told apart by index.
// Where the reference's unstable sort breaks ties between equal logits arbitrarily at a cut, every
// logit equal to the cut value is kept here. The uniform draw comes from the caller (the
// reference draws it from fastrand, whose stream is the host's business), so the kernel is a
// function of its inputs; its histogram sums are taken in whatever order the threads arrive, so a
// draw that lands within rounding of a boundary between two tokens may fall either way.

#include <cfloat>

#include "device_utils.cuh"
#include "kernels.h"

namespace bc {
namespace k {

namespace {

constexpr int kSampleThreads = 1024;
constexpr uint32_t kRepeatLastN = 64;  // REPEAT_LAST_N, sampler.rs:9-10

// Ascending key = descending logit. NaNs sort last.
__device__ __forceinline__ uint32_t descending_key(float v) {
    uint32_t bits = __float_as_uint(v);
    uint32_t ascending = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    return ~ascending;
}

struct SampleParams {
    float* logits;
    uint32_t n;
    const uint32_t* recent;
    uint32_t n_recent;
    Sampling settings;
    float uniform;
    uint32_t* out;
    uint32_t* readback;
};

struct Shared {
    float hist[256];
    float reduce[32];
    uint32_t reduce_index[32];
    uint32_t counts[kSampleThreads / 32];
    uint32_t prefix;   // key bits decided so far
    float below;       // weight of keys below the decided prefix
    float scalar;
    uint32_t word;
};

__device__ float block_max(float v, Shared& sh) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh.reduce[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = sh.reduce[0];
    for (int w = 1; w < kSampleThreads / 32; ++w) m = fmaxf(m, sh.reduce[w]);
    return m;
}

__device__ float block_total(float v, Shared& sh) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh.reduce[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < kSampleThreads / 32; ++w) total += sh.reduce[w];
    return total;
}

// The smallest key K among the candidates (keys <= limit) at which the weight summed over keys
// <= K passes `target` (exceeds it, or reaches it when `inclusive`). `weight(logit)` gives a
// candidate's weight. Returns K; sh.below then holds the weight of the candidates with smaller keys.
// When the target lies beyond the total (rounding), the largest candidate key is returned.
template <typename W>
__device__ uint32_t select_key(const SampleParams& p, uint32_t limit, float target, bool inclusive, W weight, Shared& sh) {
    if (threadIdx.x == 0) {
        sh.prefix = 0;
        sh.below = 0.f;
    }
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x; b < 256; b += kSampleThreads) sh.hist[b] = 0.f;
        __syncthreads();
        const uint32_t prefix = sh.prefix;
        for (uint32_t i = threadIdx.x; i < p.n; i += kSampleThreads) {
            const float v = p.logits[i];
            const uint32_t key = descending_key(v);
            if (key > limit) continue;
            if (shift < 24 && (key >> (shift + 8)) != prefix) continue;
            atomicAdd(&sh.hist[(key >> shift) & 255u], weight(v));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float running = sh.below;
            int chosen = -1, last_filled = -1;
            for (int b = 0; b < 256; ++b) {
                const float h = sh.hist[b];
                if (h <= 0.f) continue;
                last_filled = b;
                const float with = running + h;
                if (inclusive ? with >= target : with > target) {
                    chosen = b;
                    break;
                }
                running = with;
            }
            if (chosen < 0) {
                // Past the end: settle on the last filled bucket, with everything before it below.
                chosen = last_filled < 0 ? 0 : last_filled;
                running = sh.below;
                for (int b = 0; b < chosen; ++b) running += sh.hist[b];
            }
            sh.below = running;
            sh.prefix = (prefix << 8) | (uint32_t)chosen;
        }
        __syncthreads();
    }
    return sh.prefix;
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(SampleParams p) {
    __shared__ Shared sh;
    pdl_launch_dependents();
    pdl_wait();
    const Sampling s = p.settings;
    const int tid = threadIdx.x;

    // Repetition penalty: each distinct token among the last 64 takes it once (sampler.rs:47-63).
    if (fabsf(s.repeat_penalty - 1.0f) > FLT_EPSILON && p.n_recent) {
        const uint32_t window = min(p.n_recent, kRepeatLastN);
        const uint32_t* recent = p.recent + (p.n_recent - window);
        if ((uint32_t)tid < window) {
            const uint32_t token = recent[tid];
            bool first = token < p.n;
            for (int j = 0; j < tid && first; ++j) first = recent[j] != token;
            if (first) {
                const float logit = p.logits[token];
                p.logits[token] = logit > 0.f ? logit / s.repeat_penalty : logit * s.repeat_penalty;
            }
        }
        __syncthreads();
    }

    // The largest logit and its lowest index.
    float best = -INFINITY;
    uint32_t best_index = 0xffffffffu;
    for (uint32_t i = tid; i < p.n; i += kSampleThreads) {
        const float v = p.logits[i];
        if (v > best || best_index == 0xffffffffu) {
            best = v;
            best_index = i;
        }
    }
    const float top = block_max(best, sh);
    if (s.temperature <= 0.f) {
        // Greedy: the first maximum (sampler.rs:70-76).
        uint32_t candidate = best == top ? best_index : 0xffffffffu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) candidate = min(candidate, __shfl_xor_sync(0xffffffffu, candidate, o));
        __syncthreads();
        if ((tid & 31) == 0) sh.reduce_index[tid >> 5] = candidate;
        __syncthreads();
        if (tid == 0) {
            uint32_t index = 0xffffffffu;
            for (int w = 0; w < kSampleThreads / 32; ++w) index = min(index, sh.reduce_index[w]);
            *p.out = index;
            if (p.readback) *p.readback = index;
        }
        return;
    }

    uint32_t limit = 0xffffffffu;  // candidates are the logits whose key is <= limit
    if (s.top_k > 0 && s.top_k < p.n) limit = select_key(p, limit, (float)s.top_k - 0.5f, false, [](float) { return 1.0f; }, sh);
    auto unit_softmax = [top](float v) { return expf(v - top); };
    if (s.top_p < 1.0f) {
        float mine = 0.f;
        for (uint32_t i = tid; i < p.n; i += kSampleThreads) {
            const float v = p.logits[i];
            if (descending_key(v) <= limit) mine += unit_softmax(v);
        }
        const float total = block_total(mine, sh);
        limit = select_key(p, limit, s.top_p * total, true, unit_softmax, sh);
    }
    if (s.min_p > 0.f) {
        // p >= p_first * min_p, with p proportional to exp(logit - top) (sampler.rs:98-99).
        const uint32_t floor_key = descending_key(top + logf(s.min_p));
        limit = min(limit, floor_key);
    }

    // The draw over the survivors at the temperature (sampler.rs:101-111).
    const float inv_t = 1.0f / s.temperature;
    auto tempered = [top, inv_t](float v) { return expf((v - top) * inv_t); };
    float mine = 0.f;
    for (uint32_t i = tid; i < p.n; i += kSampleThreads) {
        const float v = p.logits[i];
        if (descending_key(v) <= limit) mine += tempered(v);
    }
    const float total = block_total(mine, sh);
    const float target = p.uniform * total;
    const uint32_t picked_key = select_key(p, limit, target, false, tempered, sh);

    // Equal logits share the key: the draw's remainder picks among them by index.
    const uint32_t per_thread = (p.n + kSampleThreads - 1) / kSampleThreads;
    const uint32_t first = tid * per_thread, last = min(p.n, first + per_thread);
    uint32_t ties = 0;
    float tie_weight = 0.f;
    for (uint32_t i = first; i < last; ++i) {
        const float v = p.logits[i];
        if (descending_key(v) == picked_key) {
            ++ties;
            tie_weight = tempered(v);
        }
    }
    // Exclusive scan of the per-thread tie counts.
    uint32_t inclusive_scan = ties;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t other = __shfl_up_sync(0xffffffffu, inclusive_scan, o);
        if ((tid & 31) >= o) inclusive_scan += other;
    }
    __syncthreads();
    if ((tid & 31) == 31) sh.counts[tid >> 5] = inclusive_scan;
    if (tid == 0) sh.scalar = 0.f;
    __syncthreads();
    uint32_t before = inclusive_scan - ties;
    for (int w = 0; w < (tid >> 5); ++w) before += sh.counts[w];
    uint32_t all_ties = 0;
    for (int w = 0; w < kSampleThreads / 32; ++w) all_ties += sh.counts[w];
    if (ties) sh.scalar = tie_weight;  // the same value from every thread that has one
    __syncthreads();
    const float w = sh.scalar;
    uint32_t wanted = 0;
    if (w > 0.f && all_ties > 1) {
        const float remainder = fmaxf(target - sh.below, 0.f);
        wanted = min((uint32_t)(remainder / w), all_ties - 1);
    }
    if (ties && wanted >= before && wanted < before + ties) {
        uint32_t seen = before;
        for (uint32_t i = first; i < last; ++i) {
            if (descending_key(p.logits[i]) != picked_key) continue;
            if (seen == wanted) {
                *p.out = i;
                if (p.readback) *p.readback = i;
                break;
            }
            ++seen;
        }
    }
}

}  // namespace

cudaError_t sample(cudaStream_t stream, float* logits, uint32_t n, const uint32_t* recent, uint32_t n_recent, const Sampling& settings,
                   float uniform, uint32_t* out, uint32_t* readback) {
    SampleParams p{logits, n, recent, n_recent, settings, uniform, out, readback};
    void* args[] = {&p};
    return launch_kernel((const void*)sample_kernel, dim3(1), dim3(kSampleThreads), 0, stream, args);
}

}  // namespace k
}  // namespace bc
