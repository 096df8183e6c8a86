// The decode Q4_0 matrix-vector kernel: a persistent, TMA-fed weight stream with the dot products
// on the tensor cores.
//
// Why it looks like this. At batch 1 a Q4_0 multiply moves 18 bytes per 32 weights and nothing
// else of size, so the only goal is to keep HBM streaming. Two things stand in the way. (1) A lane
// that turns nibbles into floats and multiplies them one by one spends about 3.5 instructions per
// weight, more than an SM can issue at the rate HBM delivers weights (40 per clock per SM). Here
// the multiply-adds run on the tensor cores in integers, which keeps them exact: four nibbles of
// a word become the signed bytes 16 * (q - 8) with two logic ops, the 16-row weight tile is the A
// operand of an mma.m16n8k32 (one per block of 32 weights), and the input vector, each block of 32
// values scaled by its own power of two to 31-bit integers and split into four signed base-256
// digits, fills four of the eight columns of B. The digit sums are joined in integers and the
// block's two scales (the fp16 weight scale, the input's power of two) multiply the per-block
// result in f32: about 0.6 instructions per weight.
// (2) A decode step is a chain of small dependent launches, and a launch that starts its loads
// only after its input exists idles HBM for microseconds at every link. Here every warp streams
// its own share of the matrix into its slot of a shared-memory ring with bulk async copies
// (lane 0 issues them, an mbarrier per slot reports their arrival, every wait is bounded), and the
// first copies go out before the kernel waits for its predecessor (programmatic dependent launch):
// the weights depend on nothing, only the few kilobytes of activations do. A slot is refilled by
// the warp that has just read it, so there is no producer to hand it back to. A CTA is 16 warps,
// one CTA per SM, and a warp has one slot of 32 blocks (9 KB): 147 KB in flight per SM. Measured on
// the 2.6B shape with every warp issuing its own copies: two 8-warp CTAs per SM with two 16-block
// slots per warp 1 170 tok/s, this CTA with two 16-block slots 1 184, with one 16-block slot 1 195,
// with one 32-block slot 1 226 - fewer, larger copies and fewer bytes queued ahead of the input's
// loads, which wait behind the ring's copies once the dependency wait releases. (A single thread
// issuing all of a CTA's copies was the largest cost of this kernel once the multiplies were
// cheap: the sixteenth copy left more than a microsecond after the first. A lane per warp: +9 %.)
//
// Layout ("tiles"): rows in tiles of 16, columns in chunks of 32 blocks. A chunk of a tile is
// contiguous: for each pair of blocks 512 bytes ordered by lane - lane (g, t) = (lane / 4, lane % 4)
// holds word t of the quants of rows g and g + 8 for both blocks, exactly its A-fragment share -
// then the chunk's fp16 scales, 8 bytes per (block pair, g): rows g and g + 8 of the first block,
// then of the second. A tile's chunks follow one another, 288 bytes per block, so a tile is one
// contiguous run and the matrix is the tiles in order. Values are the GGUF values bit for bit.
//
// Reference counterpart: matvec_k<q4_0_lanes> (crates/bobcat-metal/src/matvec.metal:298-365,
// quant.metal:587-656) and its swiglu / conv variants (:386-585).

#include <cstdlib>

#include "device_utils.cuh"
#include "kernels.h"
#include "../../include/bobcat_cuda.h"

namespace bc {
namespace k {

namespace {

constexpr int kConsumers = 16;                   // warps per CTA
constexpr int kThreads = kConsumers * 32;
constexpr int kDepth = 1;                        // ring slots per warp
constexpr uint32_t kCtasPerSm = 1;               // CTAs a launch may put on one SM
constexpr int kStages = kConsumers * kDepth;
constexpr int kChunkBlocks = 32;                 // blocks of 32 weights per chunk of a tile
constexpr int kBlockBytes = 288;                 // 16 rows x 18 bytes
constexpr int kStageBytes = kChunkBlocks * kBlockBytes;
constexpr uint32_t kSpinLimit = 1u << 22;        // bounded waits: give up rather than hang

__device__ int g_error_flag;

// ---- mbarrier and bulk-copy wrappers (shared::cta addresses as 32-bit integers)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Returns false when the wait ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}

// d = a * b over 16 rows, 8 columns and 32 signed bytes of depth, from a zero accumulator.
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// d += a * b.
__device__ __forceinline__ void mma_s8_add(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The four low (high) nibbles q of a word as signed bytes 16 * (q - 8): the nibble moves to the top
// of its byte and flipping the byte's sign bit takes off 128.
__device__ __forceinline__ uint32_t low_nibbles_s8(uint32_t w) { return ((w << 4) & 0xf0f0f0f0u) ^ 0x80808080u; }
__device__ __forceinline__ uint32_t high_nibbles_s8(uint32_t w) { return (w & 0xf0f0f0f0u) ^ 0x80808080u; }

// An integer as four signed base-256 digits, one per byte, least significant first: adding 128 at
// every byte position makes each byte digit + 128, and flipping the sign bits takes it off again.
__device__ __forceinline__ uint32_t signed_digits(int v) { return ((uint32_t)v + 0x80808080u) ^ 0x80808080u; }

enum Mode { kPlain = 0, kSwiglu = 1, kConv = 2 };

struct Params {
    // Tile streams. kPlain: up to three matrices sharing x, one job per tile of their
    // concatenation. kSwiglu: gate, up; one job per tile pair. kConv: in_proj; a job is the tiles
    // of 16 channels' B, C and X rows.
    const uint8_t* tiles[4];
    float* y[4];
    uint32_t seg_tiles[4];  // tiles per segment
    uint32_t seg_rows[4];   // rows per segment (the last tile may be padded)
    int n_segments;
    uint32_t n_jobs, n_blocks;  // blocks per row
    const float* x;
    const float* norm_weight;
    float eps;
    int accumulate;
    const float* taps;
    float* history;
    uint32_t n_embd, conv_kernel;
    // Mixture of experts: the matrices are stacks of n_experts matrices of tiles_per_expert tiles
    // and route[slot] names the expert of a slot. kSwiglu: job j is tile j % tiles_per_expert of
    // slot j / tiles_per_expert, all slots read x. kPlain: CTA c works for slot c % n_used on the
    // tiles of that slot's expert, reads x + slot * n_cols and writes y + slot * rows.
    const uint32_t* route;
    uint32_t tiles_per_expert, n_used;
};

template <int MODE>
__device__ __forceinline__ constexpr int segments_per_job() { return MODE == kPlain ? 1 : MODE == kSwiglu ? 2 : 3; }

// The tile stream of segment `s` of job `job`.
template <int MODE>
__device__ __forceinline__ const uint8_t* job_tiles(const Params& p, uint32_t job, int s, uint32_t tile_bytes) {
    if (MODE == kPlain) {
        int seg = 0;
        uint32_t local = job;
        while (seg + 1 < p.n_segments && local >= p.seg_tiles[seg]) {
            local -= p.seg_tiles[seg];
            ++seg;
        }
        return p.tiles[seg] + (uint64_t)local * tile_bytes;
    }
    if (MODE == kSwiglu) {
        if (p.route) job = p.route[job / p.tiles_per_expert] * p.tiles_per_expert + job % p.tiles_per_expert;
        return p.tiles[s] + (uint64_t)job * tile_bytes;
    }
    return p.tiles[0] + ((uint64_t)s * (p.n_embd / 16) + job) * tile_bytes;
}

// Warps per group: the warps of a group share one job, taking its chunks in turn, so a CTA with only
// a few jobs still keeps all its warps busy. The smallest power of two that covers the job's
// chunks, at most all warps.
__device__ __forceinline__ uint32_t group_size(uint32_t q_per_job) {
    uint32_t gs = 1;
    while (gs < (uint32_t)kConsumers && gs < q_per_job) gs *= 2;
    return gs;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) matvec_mma_kernel(Params p) {
    constexpr int S = segments_per_job<MODE>();
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;                                                   // kStages * kStageBytes
    uint4* xs = reinterpret_cast<uint4*>(smem + kStages * kStageBytes);     // [block][digit][t]: 16 x 8 bytes per block
    float* x_scale = reinterpret_cast<float*>(smem + kStages * kStageBytes + (size_t)p.n_blocks * 128);  // [block]
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ float reduce_scratch[64];
    __shared__ uint2 zero_columns[kChunkBlocks * 16];  // a chunk's worth of B operand that is all zero
    __shared__ float partial[2][kConsumers][3 * 16];  // [job parity][warp][segment * 16 + row in tile]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t nb = p.n_blocks;
    const uint32_t tile_bytes = nb * kBlockBytes;
    const uint32_t chunks = (nb + kChunkBlocks - 1) / kChunkBlocks;  // per tile
    const uint32_t q_per_job = S * chunks;
    const uint32_t gs = group_size(q_per_job), groups = kConsumers / gs;
    // Jobs of this CTA: cta, cta + n_ctas, ... Job m goes to group m % groups. A routed plain
    // product splits the grid among the slots, and a CTA's jobs are the tiles of its slot's expert.
    const bool slotted = MODE == kPlain && p.route != nullptr;
    const uint32_t slot = slotted ? blockIdx.x % p.n_used : 0u;
    const uint32_t cta = slotted ? blockIdx.x / p.n_used : blockIdx.x, n_ctas = slotted ? gridDim.x / p.n_used : gridDim.x;
    const uint32_t my_jobs = p.n_jobs > cta ? (p.n_jobs - cta + n_ctas - 1) / n_ctas : 0;

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(smem_u32(&full_bar[i]), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    // ---- Every warp streams its own chunks: lane 0 copies the warp's next chunk into the slot
    // the warp has just finished reading, in the order the warp takes them (its group's jobs round
    // by round, every gs-th chunk of a job). The first kDepth copies go out now, before the wait
    // for the predecessor, unless the routing (a predecessor's output) picks the weights.
    const uint32_t grp = warp / gs, rank = warp % gs;
    uint32_t first_tile = 0;
    if (p.route) {
        pdl_wait();
        if (slotted) first_tile = p.route[slot] * p.tiles_per_expert;
    }
    uint32_t ahead_r = 0, ahead_q = rank, issued = 0;  // the next chunk to copy and how many were
    auto copy_next = [&]() {
        if (ahead_q >= q_per_job || ahead_r * groups + grp >= my_jobs) return;  // a group may have more warps than a job has chunks
        if (lane == 0) {
            const uint32_t job = cta + n_ctas * (ahead_r * groups + grp);
            const uint32_t seg = ahead_q / chunks, chunk = ahead_q % chunks;
            const uint32_t cb = min((uint32_t)kChunkBlocks, nb - chunk * kChunkBlocks);
            const uint32_t stage = warp * kDepth + issued % kDepth;
            const uint8_t* src = job_tiles<MODE>(p, first_tile + job, (int)seg, tile_bytes) + (uint64_t)chunk * kStageBytes;
            const uint32_t bytes = cb * kBlockBytes;
            mbar_arrive_expect(smem_u32(&full_bar[stage]), bytes);
            bulk_load(smem_u32(ring + stage * kStageBytes), src, bytes, smem_u32(&full_bar[stage]));
        }
        ++issued;
        ahead_q += gs;
        if (ahead_q >= q_per_job) {
            ahead_q = rank;
            ++ahead_r;
        }
    };
#pragma unroll
    for (int d = 0; d < kDepth; ++d) copy_next();

    // Everything above touched only weights; the input vector (and y, the conv history) belong
    // to earlier launches.
    // The norm's weights are the model's, not a predecessor's: a thread's share of them is on its
    // way before the wait, so the input's loads after the wait are the only trip to L2 the
    // staging waits for (inputs of up to one item per thread; longer inputs load them in the loop).
    float4 early_wl = make_float4(1.f, 1.f, 1.f, 1.f), early_wh = early_wl;
    const bool norm_early = p.norm_weight != nullptr && p.n_blocks * 4 <= (uint32_t)kThreads;
    if (norm_early && (uint32_t)threadIdx.x < p.n_blocks * 4) {
        const float4* w4e = reinterpret_cast<const float4*>(p.norm_weight);
        early_wl = __ldg(w4e + (threadIdx.x >> 2) * 8 + (threadIdx.x & 3));
        early_wh = __ldg(w4e + (threadIdx.x >> 2) * 8 + 4 + (threadIdx.x & 3));
    }
    if (!p.route) pdl_wait();

    // Stage x as the B operand in one pass over global memory: RMSNorm weights applied, every
    // block of 32 values scaled by its own power of two so that its largest magnitude lands in
    // [2^29, 2^30), rounded to integers (no change for a value of at least 2^-7 of the block's
    // largest, an absolute error below 2^-30 of it for the rest) and split into four signed
    // base-256 digits, one digit per column of B. Thread (b, t) holds elements 4t..4t+3 and
    // 16+4t..16+4t+3 of block b, so a block's maximum is two shuffles among four lanes, and the 8
    // bytes at xs8[b * 16 + j * 4 + t] take digit j (0 = most significant) of those elements.
    // The inverse of the block's power of two goes to x_scale[b] and multiplies the block's sum;
    // the norm's scalar multiplies the finished rows.
    const int ctid = tid;
    constexpr int kConsumerThreads = kConsumers * 32;
    const float4* x4 = reinterpret_cast<const float4*>(p.x) + (size_t)slot * nb * 8;
    const float4* w4 = reinterpret_cast<const float4*>(p.norm_weight);
    uint2* xs8 = reinterpret_cast<uint2*>(xs);
    float sumsq = 0.f;
    // Whole warps call this together: item i is (block, word index) = (i / 4, i % 4).
    auto stage_item = [&](uint32_t i, float4 lo4, float4 hi4) {
        const uint32_t b = i >> 2, t = i & 3;
        const bool valid = i < nb * 4;
        if (valid) {
            sumsq += (lo4.x * lo4.x + lo4.y * lo4.y + lo4.z * lo4.z + lo4.w * lo4.w) + (hi4.x * hi4.x + hi4.y * hi4.y + hi4.z * hi4.z + hi4.w * hi4.w);
            if (p.norm_weight) {
                float4 wl = early_wl, wh = early_wh;
                if (!norm_early) {
                    wl = __ldg(w4 + b * 8 + t);
                    wh = __ldg(w4 + b * 8 + 4 + t);
                }
                lo4.x *= wl.x; lo4.y *= wl.y; lo4.z *= wl.z; lo4.w *= wl.w;
                hi4.x *= wh.x; hi4.y *= wh.y; hi4.z *= wh.z; hi4.w *= wh.w;
            }
        }
        const float v[8] = {lo4.x, lo4.y, lo4.z, lo4.w, hi4.x, hi4.y, hi4.z, hi4.w};
        float top = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) top = fmaxf(top, fabsf(v[e]));
        top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
        top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
        // top lies in [2^(e - 127), 2^(e - 126)) for its exponent field e; 2^(156 - e) brings it
        // to [2^29, 2^30). Fields below 60 (and zero) share the scale 2^96.
        const uint32_t field = max(__float_as_uint(top) >> 23, 60u);
        const float up = __uint_as_float((283u - field) << 23);
        if (valid) {
            uint32_t word[2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t d[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) d[e] = signed_digits(__float2int_rn(v[h * 4 + e] * up));
                // Transpose the 4 x 4 bytes: word[h][j] = byte 3 - j of the four elements.
                const uint32_t lo01 = __byte_perm(d[0], d[1], 0x5140), hi01 = __byte_perm(d[0], d[1], 0x7362);
                const uint32_t lo23 = __byte_perm(d[2], d[3], 0x5140), hi23 = __byte_perm(d[2], d[3], 0x7362);
                word[h][3] = __byte_perm(lo01, lo23, 0x5410);
                word[h][2] = __byte_perm(lo01, lo23, 0x7632);
                word[h][1] = __byte_perm(hi01, hi23, 0x5410);
                word[h][0] = __byte_perm(hi01, hi23, 0x7632);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) xs8[b * 16 + j * 4 + t] = make_uint2(word[0][j], word[1][j]);
            if (t == 0) x_scale[b] = __uint_as_float((field - 29u) << 23);  // 1 / up
        }
    };
    if (nb * 4 <= (uint32_t)kConsumerThreads) {
        const uint32_t i = (uint32_t)ctid;
        float4 lo4 = make_float4(0.f, 0.f, 0.f, 0.f), hi4 = lo4;
        if (i < nb * 4) {
            lo4 = x4[(i >> 2) * 8 + (i & 3)];
            hi4 = x4[(i >> 2) * 8 + 4 + (i & 3)];
        }
        if ((uint32_t)(ctid & ~31) < nb * 4) stage_item(i, lo4, hi4);
    } else {
        // The loads of a thread's next item go out before it works on the current one.
        float4 next_lo = x4[((uint32_t)ctid >> 2) * 8 + (ctid & 3)], next_hi = x4[((uint32_t)ctid >> 2) * 8 + 4 + (ctid & 3)];
        for (uint32_t first = (uint32_t)(ctid & ~31); first < nb * 4; first += kConsumerThreads) {
            const uint32_t i = first + lane, ahead = i + kConsumerThreads;
            const float4 lo4 = next_lo, hi4 = next_hi;
            if (ahead < nb * 4) {
                next_lo = x4[(ahead >> 2) * 8 + (ahead & 3)];
                next_hi = x4[(ahead >> 2) * 8 + 4 + (ahead & 3)];
            }
            stage_item(i, lo4, hi4);
        }
    }
    for (int i = ctid; i < kChunkBlocks * 16; i += kConsumerThreads) zero_columns[i] = make_uint2(0u, 0u);
    sumsq = warp_sum(sumsq);
    if (lane == 0) reduce_scratch[warp] = sumsq;
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
    float total = 0.f;
    for (int i = 0; i < kConsumers; ++i) total += reduce_scratch[i];
    const float norm_scale = p.norm_weight ? rsqrtf(total / (float)(nb * 32) + p.eps) : 1.f;
    const float out_scale = norm_scale * 0.0625f;  // the weights come as 16 * (q - 8)

    const int g = lane >> 2, t = lane & 3;
    uint32_t taken = 0;  // chunks this warp has consumed
    bool dead = false;
    for (uint32_t r = 0; r * groups + grp < my_jobs; ++r) {
        const uint32_t job = cta + n_ctas * (r * groups + grp);
        // The thread that will finish a row of a plain product finds the row now and, when the
        // product adds to y, starts reading the old value, so that read overlaps the multiply.
        float* y_row = nullptr;
        float y_old = 0.f;
        if (MODE == kPlain && rank == 0 && lane < 16) {
            int seg = 0;
            uint32_t local = job;
            while (seg + 1 < p.n_segments && local >= p.seg_tiles[seg]) {
                local -= p.seg_tiles[seg];
                ++seg;
            }
            uint32_t row = local * 16 + lane;
            if (row < p.seg_rows[seg]) {
                y_row = p.y[seg] + (size_t)slot * p.seg_rows[seg] + row;
                if (p.accumulate) y_old = *y_row;
            }
        }
        // The same for the conv: the channel's taps and history (kernels of up to kMaxTaps taps)
        // are on their way while the products run.
        constexpr int kMaxTaps = 4;
        float tap[kMaxTaps], past[kMaxTaps - 1];
        const bool taps_early = MODE == kConv && p.conv_kernel <= (uint32_t)kMaxTaps && rank == 0 && lane < 16 && job * 16 + lane < p.n_embd;
        if (taps_early) {
            const uint32_t ch = job * 16 + lane;
#pragma unroll
            for (int kk = 0; kk < kMaxTaps; ++kk)
                if ((uint32_t)kk < p.conv_kernel) tap[kk] = p.taps[(uint64_t)ch * p.conv_kernel + kk];
#pragma unroll
            for (int kk = 0; kk < kMaxTaps - 1; ++kk)
                if ((uint32_t)kk + 1 < p.conv_kernel) past[kk] = p.history[(uint64_t)kk * p.n_embd + ch];
        }
        float acc[S][2];
#pragma unroll
        for (int s = 0; s < S; ++s) acc[s][0] = acc[s][1] = 0.f;
        for (uint32_t q = rank; q < q_per_job; q += gs, ++taken) {
            const uint32_t s_of_q = q / chunks, chunk = q % chunks;
            const uint32_t stage = warp * kDepth + taken % kDepth, use = taken / kDepth;
            // A wait that runs out marks the launch failed; the warp then skips its remaining chunks
            // but still meets its group at every barrier, so nothing is left waiting on it.
            if (!dead && !mbar_wait(smem_u32(&full_bar[stage]), use & 1)) {
                atomicExch(&g_error_flag, 2);
                dead = true;
            }
            if (dead) continue;
            const uint32_t cb = min((uint32_t)kChunkBlocks, nb - chunk * kChunkBlocks);
            // This lane's quants (one 16-byte group per block pair), scales and inputs. Plain loads,
            // so the compiler can run the next pair's loads ahead of this pair's arithmetic. Lanes
            // with g >= 2 hold columns of the product nobody reads; they repeat the reads of g & 1.
            const uint8_t* slot = ring + stage * kStageBytes;
            const uint4* quants = reinterpret_cast<const uint4*>(slot) + lane;
            // Two blocks share one pass over the product's columns: the first block's multiply
            // sees the digits of x in columns 0..3 and zeros in 4..7, the second block's the
            // reverse, and both add into one accumulator. Afterwards lanes t = 0, 1 hold the first
            // block's sums (high and low digit pair) and lanes t = 2, 3 the second block's, so
            // the conversion and the block scale run once per pair of blocks with every lane useful.
            // A lane supplies column g of B: real digits for one block of the pair, zeros for the other.
            const uint2* chunk_x = reinterpret_cast<const uint2*>(xs) + (size_t)chunk * kChunkBlocks * 16 + (g & 3) * 4 + t;
            const uint2* x_first = g < 4 ? chunk_x : zero_columns + (g & 3) * 4 + t;
            const uint2* x_second = g < 4 ? zero_columns + (g & 3) * 4 + t : chunk_x + 16;
            const uint32_t* scales = reinterpret_cast<const uint32_t*>(slot + cb * 256) + g * 2 + (t >> 1);
            const float* block_scale = x_scale + chunk * kChunkBlocks + (t >> 1);  // of this lane's block of each pair
            float a0 = 0.f, a1 = 0.f;
#pragma unroll 4
            for (uint32_t pair = 0; pair < cb / 2; ++pair) {
                const uint4 v = quants[pair * 32];  // rows g, g + 8 of the first block, then of the second
                const uint32_t dw = scales[pair * 16];  // the scales of rows g and g + 8 in this lane's block
                const uint2 xa = x_first[pair * 32], xb = x_second[pair * 32];
                int c[4];
                mma_s8(c, low_nibbles_s8(v.x), low_nibbles_s8(v.y), high_nibbles_s8(v.x), high_nibbles_s8(v.y), xa.x, xa.y);
                mma_s8_add(c, low_nibbles_s8(v.z), low_nibbles_s8(v.w), high_nibbles_s8(v.z), high_nibbles_s8(v.w), xb.x, xb.y);
                const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&dw));
                const float bs = block_scale[pair * 2];
                // Columns 2t and 2t + 1 are neighbouring digits of x, joined before the scales.
                a0 = fmaf((float)(c[0] * 256 + c[1]) * bs, d.x, a0);
                a1 = fmaf((float)(c[2] * 256 + c[3]) * bs, d.y, a1);
            }
            // The slot is read out: order the reads before the copy engine's writes, then refill it.
            __syncwarp();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            copy_next();
#pragma unroll
            for (int s = 0; s < S; ++s) {
                if ((uint32_t)s == s_of_q) {
                    acc[s][0] += a0;
                    acc[s][1] += a1;
                }
            }
        }
        // Lanes with even t hold sums over the two high digits of x, lanes with odd t over the two
        // low ones, each for every other block; the four lanes of a row add up to the row's sum.
        // The group's warps leave their partial sums in shared memory; after the group's barrier
        // its first warp adds them in warp order and finishes the 16 rows.
        const int parity = r & 1;
        const float digit_weight = (t & 1) ? 1.f : 65536.f;
#pragma unroll
        for (int s = 0; s < S; ++s) {
#pragma unroll
            for (int half_rows = 0; half_rows < 2; ++half_rows) {
                float v = acc[s][half_rows] * digit_weight;
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                acc[s][half_rows] = v;
            }
        }
        if (t == 0) {
#pragma unroll
            for (int s = 0; s < S; ++s) {
                partial[parity][warp][s * 16 + g] = acc[s][0];
                partial[parity][warp][s * 16 + g + 8] = acc[s][1];
            }
        }
        if (gs > 1) asm volatile("bar.sync %0, %1;" ::"r"(2 + grp), "r"(gs * 32) : "memory");
        else __syncwarp();
        if (rank == 0 && lane < 16) {
            float sum[S];
#pragma unroll
            for (int s = 0; s < S; ++s) {
                sum[s] = 0.f;
                for (uint32_t w = 0; w < gs; ++w) sum[s] += partial[parity][warp + w][s * 16 + lane];
                sum[s] *= out_scale;
            }
            const uint32_t in_tile = lane;
            if (MODE == kPlain) {
                if (y_row) *y_row = y_old + sum[0];
            } else if (MODE == kSwiglu) {
                uint32_t row = job * 16 + in_tile;
                if (row < p.seg_rows[0]) {
                    float gate = sum[0], upv = sum[S > 1 ? 1 : 0];
                    p.y[0][row] = gate / (1.f + expf(-gate)) * upv;
                }
            } else {
                // B, C and X of channel ch; the taps over B*X and the channel's history; the
                // history shift; C * conv (crates/bobcat/src/lfm2.rs:456-475, f32 sums).
                uint32_t ch = job * 16 + in_tile;
                if (ch < p.n_embd) {
                    float b = sum[0], c = sum[S > 1 ? 1 : 0], xv = sum[S > 2 ? 2 : 0];
                    float bx = b * xv;
                    const uint32_t K = p.conv_kernel;
                    if (taps_early) {
                        float last_tap = 0.f;
#pragma unroll
                        for (int kk = 0; kk < kMaxTaps; ++kk)
                            if ((uint32_t)kk + 1 == K) last_tap = tap[kk];
                        float total_taps = last_tap * bx;
#pragma unroll
                        for (int kk = 0; kk < kMaxTaps - 1; ++kk)
                            if ((uint32_t)kk + 1 < K) total_taps += tap[kk] * past[kk];
#pragma unroll
                        for (int kk = 0; kk < kMaxTaps - 2; ++kk)
                            if ((uint32_t)kk + 2 < K) p.history[(uint64_t)kk * p.n_embd + ch] = past[kk + 1];
                        p.history[(uint64_t)(K - 2) * p.n_embd + ch] = bx;
                        p.y[0][ch] = c * total_taps;
                    } else {
                        const float* taps = p.taps + (uint64_t)ch * K;
                        float total_taps = taps[K - 1] * bx;
                        for (uint32_t kk = 0; kk + 1 < K; ++kk) total_taps += taps[kk] * p.history[(uint64_t)kk * p.n_embd + ch];
                        for (uint32_t kk = 0; kk + 2 < K; ++kk) p.history[(uint64_t)kk * p.n_embd + ch] = p.history[(uint64_t)(kk + 1) * p.n_embd + ch];
                        p.history[(uint64_t)(K - 2) * p.n_embd + ch] = bx;
                        p.y[0][ch] = c * total_taps;
                    }
                }
            }
        }
    }
}

// One thread per 16 bytes of quants and one per scale: split layout -> tile layout.
__global__ void repack_tiles_kernel(const uint4* __restrict__ quants, const __half* __restrict__ scales, uint32_t n_rows, uint32_t nb,
                                    uint8_t* __restrict__ tiles) {
    const uint32_t n_tiles = (n_rows + 15) / 16;
    const uint64_t quant_items = (uint64_t)n_tiles * (nb / 2) * 32;
    const uint64_t scale_items = (uint64_t)n_tiles * nb * 16;
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < quant_items) {
        uint32_t lane = i % 32;
        uint64_t rest = i / 32;
        uint32_t pair = rest % (nb / 2), tile = rest / (nb / 2);
        uint32_t g = lane >> 2, t = lane & 3;
        uint32_t chunk = (2 * pair) / kChunkBlocks, local_pair = pair - chunk * (kChunkBlocks / 2);
        uint32_t rows[2] = {tile * 16 + g, tile * 16 + g + 8};
        uint32_t out[4];
#pragma unroll
        for (int half_pair = 0; half_pair < 2; ++half_pair) {
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                uint32_t word = 0;
                if (rows[rr] < n_rows) {
                    uint4 q = quants[(uint64_t)rows[rr] * nb + 2 * pair + half_pair];
                    word = t == 0 ? q.x : t == 1 ? q.y : t == 2 ? q.z : q.w;
                }
                out[half_pair * 2 + rr] = word;
            }
        }
        uint8_t* dst = tiles + (uint64_t)tile * nb * kBlockBytes + (uint64_t)chunk * kStageBytes + ((uint64_t)local_pair * 32 + lane) * 16;
        *reinterpret_cast<uint4*>(dst) = make_uint4(out[0], out[1], out[2], out[3]);
    } else if (i < quant_items + scale_items) {
        uint64_t j = i - quant_items;
        uint32_t in_tile = j % 16;
        uint64_t rest = j / 16;
        uint32_t block = rest % nb, tile = rest / nb;
        uint32_t chunk = block / kChunkBlocks, local = block - chunk * kChunkBlocks;
        uint32_t cb = min((uint32_t)kChunkBlocks, nb - chunk * kChunkBlocks);
        uint32_t row = tile * 16 + in_tile;
        __half d = row < n_rows ? scales[(uint64_t)row * nb + block] : __float2half(0.f);
        // 8 bytes per (block pair, g): rows g and g + 8 of the first block, then of the second.
        uint8_t* dst = tiles + (uint64_t)tile * nb * kBlockBytes + (uint64_t)chunk * kStageBytes + (uint64_t)cb * 256 +
                       ((uint64_t)(local / 2) * 8 + (in_tile & 7)) * 8 + ((local & 1) * 2 + (in_tile >> 3)) * 2;
        *reinterpret_cast<__half*>(dst) = d;
    }
}

template <int MODE>
cudaError_t launch(cudaStream_t stream, Params& p) {
    const void* kernel = (const void*)matvec_mma_kernel<MODE>;
    size_t smem = (size_t)kStages * kStageBytes + (size_t)p.n_blocks * 132;  // ring, digits, block scales
    cudaError_t e = ensure_dynamic_smem(kernel, smem);
    if (e != cudaSuccess) return e;
    uint32_t cap = kCtasPerSm * (uint32_t)sm_count();
    uint32_t ctas = p.n_jobs < cap ? p.n_jobs : cap;
    if (MODE == kPlain && p.route) {
        // The grid is split evenly among the slots; n_jobs counts the tiles of one slot.
        uint32_t per_slot = cap / p.n_used > 0 ? cap / p.n_used : 1;
        ctas = p.n_used * (p.n_jobs < per_slot ? p.n_jobs : per_slot);
    }
    void* args[] = {&p};
    return launch_kernel(kernel, dim3(ctas), dim3(kThreads), smem, stream, args);
}

bool g_enabled = [] {
    const char* v = getenv("BOBCAT_NO_MMA_MATVEC");
    return !(v && v[0] == '1');
}();

}  // namespace

uint64_t tiles_bytes(uint32_t n_rows, uint32_t n_cols) { return (uint64_t)((n_rows + 15) / 16) * (n_cols / 32) * kBlockBytes; }

bool tiles_supported(uint32_t n_cols) { return g_enabled && n_cols % 64 == 0; }

cudaError_t repack_tiles(cudaStream_t stream, const void* quants, const __half* scales, uint32_t n_rows, uint32_t n_cols, void* tiles) {
    uint32_t nb = n_cols / 32;
    uint64_t n_tiles = (n_rows + 15) / 16;
    uint64_t items = n_tiles * (nb / 2) * 32 + n_tiles * nb * 16;
    if (items == 0) return cudaSuccess;
    repack_tiles_kernel<<<(unsigned)((items + 255) / 256), 256, 0, stream>>>(static_cast<const uint4*>(quants), scales, n_rows, nb, static_cast<uint8_t*>(tiles));
    return cudaGetLastError();
}

cudaError_t matvec_mma_prepare(uint32_t widest_cols) {
    size_t smem = (size_t)kStages * kStageBytes + (size_t)(widest_cols / 32) * 132;
    for (const void* kernel : {(const void*)matvec_mma_kernel<kPlain>, (const void*)matvec_mma_kernel<kSwiglu>, (const void*)matvec_mma_kernel<kConv>}) {
        cudaError_t e = ensure_dynamic_smem(kernel, smem);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

int matvec_error_flag() {
    int flag = 0;
    cudaMemcpyFromSymbol(&flag, g_error_flag, sizeof flag);
    if (flag) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_error_flag, &zero, sizeof zero);
    }
    return flag;
}

cudaError_t matvec_mma(cudaStream_t stream, const MatvecSegment* segments, int n_segments, const float* x, Norm norm, bool accumulate) {
    Params p{};
    p.n_segments = n_segments;
    for (int i = 0; i < n_segments; ++i) {
        p.tiles[i] = static_cast<const uint8_t*>(segments[i].w.tiles);
        p.y[i] = segments[i].y;
        p.seg_rows[i] = segments[i].w.n_rows;
        p.seg_tiles[i] = (segments[i].w.n_rows + 15) / 16;
        p.n_jobs += p.seg_tiles[i];
    }
    p.n_blocks = segments[0].w.n_cols / 32;
    p.x = x;
    p.norm_weight = norm.weight;
    p.eps = norm.eps;
    p.accumulate = accumulate;
    return launch<kPlain>(stream, p);
}

cudaError_t matvec_swiglu_mma(cudaStream_t stream, const Mat& gate, const Mat& up, const float* x, Norm norm, float* y) {
    Params p{};
    p.n_segments = 2;
    p.tiles[0] = static_cast<const uint8_t*>(gate.tiles);
    p.tiles[1] = static_cast<const uint8_t*>(up.tiles);
    p.y[0] = y;
    p.seg_rows[0] = p.seg_rows[1] = gate.n_rows;
    p.seg_tiles[0] = p.seg_tiles[1] = (gate.n_rows + 15) / 16;
    p.n_jobs = p.seg_tiles[0];
    p.n_blocks = gate.n_cols / 32;
    p.x = x;
    p.norm_weight = norm.weight;
    p.eps = norm.eps;
    return launch<kSwiglu>(stream, p);
}

bool matvec_experts_mma_supported(const Mat& w, uint32_t n_rows, uint32_t n_used) {
    return w.format == BC_Q4_0 && w.tiles != nullptr && n_rows % 16 == 0 && n_used >= 1 && n_used <= 64;
}

cudaError_t matvec_experts_swiglu_mma(cudaStream_t stream, const Mat& gate, const Mat& up, uint32_t n_rows, const float* x, const uint32_t* route,
                                      uint32_t n_used, float* y) {
    Params p{};
    p.n_segments = 2;
    p.tiles[0] = static_cast<const uint8_t*>(gate.tiles);
    p.tiles[1] = static_cast<const uint8_t*>(up.tiles);
    p.y[0] = y;
    p.tiles_per_expert = n_rows / 16;
    p.n_used = n_used;
    p.route = route;
    p.seg_rows[0] = p.seg_rows[1] = n_used * n_rows;  // y holds the slots' rows one after another
    p.seg_tiles[0] = p.seg_tiles[1] = n_used * p.tiles_per_expert;
    p.n_jobs = p.seg_tiles[0];
    p.n_blocks = gate.n_cols / 32;
    p.x = x;
    return launch<kSwiglu>(stream, p);
}

cudaError_t matvec_experts_down_mma(cudaStream_t stream, const Mat& down, uint32_t n_rows, const float* x, const uint32_t* route, uint32_t n_used,
                                    float* expert_out) {
    Params p{};
    p.n_segments = 1;
    p.tiles[0] = static_cast<const uint8_t*>(down.tiles);
    p.y[0] = expert_out;
    p.tiles_per_expert = n_rows / 16;
    p.n_used = n_used;
    p.route = route;
    p.seg_rows[0] = n_rows;
    p.seg_tiles[0] = 0xffffffffu;  // one segment: a job is a tile of the stack
    p.n_jobs = p.tiles_per_expert;
    p.n_blocks = down.n_cols / 32;
    p.x = x;
    return launch<kPlain>(stream, p);
}

cudaError_t matvec_conv_mma(cudaStream_t stream, const Mat& in_proj, const float* x, Norm norm, const float* taps, float* history,
                            float* out, uint32_t n_embd, uint32_t kernel) {
    Params p{};
    p.n_segments = 1;
    p.tiles[0] = static_cast<const uint8_t*>(in_proj.tiles);
    p.y[0] = out;
    p.seg_rows[0] = in_proj.n_rows;
    p.seg_tiles[0] = (in_proj.n_rows + 15) / 16;
    p.n_jobs = n_embd / 16;
    p.n_blocks = in_proj.n_cols / 32;
    p.x = x;
    p.norm_weight = norm.weight;
    p.eps = norm.eps;
    p.taps = taps;
    p.history = history;
    p.n_embd = n_embd;
    p.conv_kernel = kernel;
    return launch<kConv>(stream, p);
}

}  // namespace k
}  // namespace bc
