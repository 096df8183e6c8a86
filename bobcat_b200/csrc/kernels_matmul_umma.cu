// The prefill Q4_0 contraction on the fifth-generation tensor cores: Y[t][r] (store) sum_c W[r][c] X[t][c]
// for a batch of tokens, with tcgen05.mma accumulating in tensor memory.
//
// Arithmetic. Weights are dequantised to fp16 ((q - 8) * d, one rounding) and inputs are rounded to
// fp16; products accumulate in f32. That is the arithmetic of the reference's prefill kernel for
// Q4_0 (crates/bobcat-metal/src/matmul.metal:249-470: half weight tiles, half inputs at :519-521,
// f32 accumulation) and of its three stores (crates/bobcat-metal/src/backend.rs:361-370).
//
// Shape of the kernel. One CTA owns 128 weight rows (the MMA's M) and up to 256 tokens (its N);
// the accumulator is 128 lanes x N columns of tensor memory. K advances 64 columns (two Q4_0
// blocks per row) per pipeline stage, four stages:
//   * producer warps in groups of four, one group per stage (four stages; three when two weight
//     matrices share the token tile). Group g takes every chunk that lands in stage g: a thread
//     loads its row's two blocks (32 bytes of quants, two scales) two turns ahead into registers,
//     turns nibbles into fp16 with logic ops on packed halves before it waits for the stage, and
//     then only stores them in the operand layout. The groups' turns overlap, which hides the
//     latency of a turn (the wait for the stage, the proxy fence, the arrival), not only that of
//     the loads;
//   * one thread brings the stage's token tile, already fp16 and already in operand layout (see
//     pack_kernel), with a single bulk copy;
//   * one thread issues four tcgen05.mma (K = 16 each) per stage and commits the stage's release;
//   * after the last stage the producer warps become the epilogue: tcgen05.ld, the store mode,
//     coalesced stores (a warp's 32 lanes are 32 consecutive rows of one token).
// Matrices with few row tiles split K over blockIdx.z so the grid fills the device; the partial
// products go to scratch and reduce_kernel adds them in a fixed order, so results do not depend on
// scheduling.
// Operand layout (both operands, K-major, no swizzle): core matrices of 8 rows x 8 halves (128
// contiguous bytes); the 8 core matrices of an 8-row group follow one another along K, and groups
// follow one another, so a tile of R rows is R / 8 groups of a kilobyte whatever R is.
// Within a Q4_0 block the K order is permuted to the order the nibbles fall out of a quant word
// (word j gives elements 4j, 4j+2, 4j+1, 4j+3, 16+4j, 16+4j+2, 16+4j+1, 16+4j+3); the packed
// inputs use the same order, and a dot product does not care.
//
// Every wait on a barrier is bounded. A wait that runs out raises a flag in shared memory that
// makes every other wait of the CTA give up, records a code the host reads, skips the stores, and
// the CTA still frees its tensor memory and returns.

#include <cstdlib>

#include "async_utils.cuh"
#include "device_utils.cuh"
#include "kernels.h"
#include "../../include/bobcat_cuda.h"

namespace bc {
namespace k {

namespace {

using namespace async;

constexpr uint32_t kRows = 128;       // weight rows per CTA: the MMA's M
constexpr uint32_t kMaxTokens = 256;  // tokens per CTA: the MMA's N, a multiple of 16
constexpr uint32_t kChunkK = 64;      // columns per stage
constexpr uint32_t kChunkBlocks = kChunkK / 32;  // Q4_0 blocks per row per stage
constexpr uint32_t kCores = kChunkK / 8;         // core matrices along K per stage
constexpr uint32_t kGroupThreads = kRows;  // a producer thread per row of the tile
constexpr uint32_t kATile = kRows * kChunkK * 2;       // 16 KB
constexpr uint32_t kGroupBytes = 8 * kChunkK * 2;      // an 8-row group of a stage: 1 KB
constexpr uint32_t kCoreBytes = 128;
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr uint32_t kMaxSplit = 8;
// The kernel multiplies one weight matrix, or two that share the token tile (gate and up of a
// SwiGLU, two accumulators): DUAL is that count. Two weight tiles per stage leave room for three
// stages instead of four. There is one producer group per stage: group g fills stage g on every
// turn, so a group is never more than one phase ahead of its stage's barrier and a parity is
// enough to tell the phases apart. (Were a stage shared by several groups, a group two uses ahead
// would see the parity of an older phase and overwrite a tile still in use.)
template <int DUAL>
struct Shape {
    static constexpr uint32_t kStages = DUAL == 2 ? 3 : 4;
    static constexpr uint32_t kGroups = kStages;
    static constexpr uint32_t kProducers = kGroups * kGroupThreads;
    static constexpr uint32_t kTmaWarp = kProducers / 32, kMmaWarp = kTmaWarp + 1;
    static constexpr uint32_t kThreads = kProducers + 64;
    static constexpr uint32_t kStageA = DUAL * kATile;
    static constexpr uint32_t kTmemColumns = DUAL * kMaxTokens;
    // With two weight matrices the producers take the Q4_0 bytes through shared memory (below), and
    // the room for that comes from the token tiles: at most 192 tokens instead of 256.
    static constexpr bool kStaged = DUAL == 2;
    static constexpr uint32_t kTileTokens = kStaged ? 192 : kMaxTokens;
    static constexpr uint32_t kStageB = kTileTokens * kChunkK * 2;
    // Staged form: per group two slots of raw bytes per matrix, 32 bytes of quants and 4 of scales per row.
    static constexpr uint32_t kRawTile = kGroupThreads * (kChunkBlocks * 18);
    static constexpr uint32_t kRawBytes = kStaged ? kGroups * 2 * DUAL * kRawTile : 0;
    static constexpr size_t kSmemBytes = kStages * (kStageA + kStageB) + kRawBytes + (2 * kStages + 1) * 8 + 16;
};

__device__ int g_matmul_error;

struct UmmaParams {
    const uint4* quants[2];   // split layout: [n_rows][n_blocks] 16-byte groups (the second matrix only when DUAL == 2)
    const __half* scales[2];  // [n_rows][n_blocks]
    const __half* packed;  // inputs in operand layout: [n_chunks][token_groups][8 cores][8 tokens][8 halves]
    float* y;              // the output, or with split > 1 the partial products [split][n_tokens][n_rows]
    uint32_t n_rows, n_blocks, n_chunks, n_tokens, y_stride, token_groups;
    uint32_t split;        // parts K is divided into (blockIdx.z)
    uint32_t tile_tokens;  // tokens per CTA, a multiple of 16 up to the shape's kTileTokens
    int store;
    // Grouped mode (mixture of experts), when offsets is set: blockIdx.z is an expert, whose weights
    // are rows [z * n_rows, (z + 1) * n_rows) of the stacked matrices, whose tokens are the entries
    // offsets[z] .. offsets[z + 1], packed from token group z * cap_groups on, and whose output
    // row for its t-th token is entries[offsets[z] + t].
    const uint32_t* offsets;
    const uint32_t* entries;
    uint32_t cap_groups;
    // DUAL == 1 only: up to three further matrices that read the same packed inputs in the same launch
    // (q, k, v; the four projections of a DeltaNet layer).
    // Row tiles [more_first[i], next) belong to matrix i + 1, which overwrites its own output of
    // more_rows[i] floats per token. No K split, no grouping.
    uint32_t n_more;
    uint32_t more_first[3], more_rows[3];
    const uint4* more_quants[3];
    const __half* more_scales[3];
    float* more_y[3];
    // DUAL == 2 only: when set, silu(gate) * up is written as the fp16 operand of the product that
    // consumes it (the layout of pack_kernel for n_rows columns and the same tokens) instead of to y.
    __half* packed_out;
};

// X [n_tokens][n_cols] f32 -> fp16 operand layout, zero rows up to the padded token count. One
// thread writes one core-matrix row (16 bytes): 8 halves of one token.
__global__ void __launch_bounds__(256) pack_kernel(const float* __restrict__ x, __half* __restrict__ packed, uint32_t n_tokens,
                                                   uint32_t n_cols, uint32_t token_groups, uint64_t total) {
    pdl_launch_dependents();  // the product that reads this packing may set itself up meanwhile
    pdl_wait();
    uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;  // index of the 16-byte output
    if (o >= total) return;
    uint32_t tr = o & 7, j = (o >> 3) & (kCores - 1);
    uint64_t group = o / (8 * kCores);  // chunk * token_groups + token group
    uint32_t tg = group % token_groups, chunk = group / token_groups;
    uint32_t token = tg * 8 + tr;
    uint4 out = make_uint4(0, 0, 0, 0);
    if (token < n_tokens) {
        const float* src = x + (uint64_t)token * n_cols + chunk * kChunkK + (j >> 2) * 32 + 4 * (j & 3);
        float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 16);
        __half2 a = __floats2half2_rn(lo.x, lo.z), b = __floats2half2_rn(lo.y, lo.w);
        __half2 c = __floats2half2_rn(hi.x, hi.z), d = __floats2half2_rn(hi.y, hi.w);
        out.x = *reinterpret_cast<uint32_t*>(&a);
        out.y = *reinterpret_cast<uint32_t*>(&b);
        out.z = *reinterpret_cast<uint32_t*>(&c);
        out.w = *reinterpret_cast<uint32_t*>(&d);
    }
    reinterpret_cast<uint4*>(packed)[o] = out;
}

// RMSNorm and packing in one pass: packed = fp16(weight * (x * scale)), scale = 1 / sqrt(mean x^2 + eps)
// per token, the arithmetic of rms_norm_kernel followed by pack_kernel. A CTA serves a group of 8
// tokens: a warp per token sums its squares, then the CTA writes the group's kilobyte of its share
// of the chunks (blockIdx.y of gridDim.y; each share repeats the cheap sums, which keeps the grid
// wide). Rows past the batch are zero.
__global__ void __launch_bounds__(256) pack_norm_kernel(const float* __restrict__ x, const float* __restrict__ weight, float eps,
                                                        __half* __restrict__ packed, uint32_t n_tokens, uint32_t n_cols, uint32_t token_groups) {
    __shared__ float scales[8];
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t tg = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    {
        const uint32_t token = tg * 8 + warp;
        float sumsq = 0.f;
        if (token < n_tokens) {
            const float4* row = reinterpret_cast<const float4*>(x + (uint64_t)token * n_cols);
            for (uint32_t i = lane; i < n_cols / 4; i += 32) {
                float4 v = row[i];
                sumsq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        sumsq = warp_sum(sumsq);
        if (lane == 0) scales[warp] = rsqrtf(sumsq / (float)n_cols + eps);
    }
    __syncthreads();
    const uint32_t tr = tid & 7, j = (tid >> 3) & (kCores - 1), sub = tid / (8 * kCores);  // 256 / 64 = 4 chunks per pass
    const uint32_t token = tg * 8 + tr, n_chunks = n_cols / kChunkK;
    const float scale = scales[tr];
    for (uint32_t chunk = blockIdx.y * (256 / (8 * kCores)) + sub; chunk < n_chunks; chunk += gridDim.y * (256 / (8 * kCores))) {
        uint4 out = make_uint4(0, 0, 0, 0);
        if (token < n_tokens) {
            const uint32_t col = chunk * kChunkK + (j >> 2) * 32 + 4 * (j & 3);
            const float* src = x + (uint64_t)token * n_cols + col;
            float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 16);
            const float4 wl = __ldg(reinterpret_cast<const float4*>(weight + col)), wh = __ldg(reinterpret_cast<const float4*>(weight + col + 16));
            lo.x = wl.x * (lo.x * scale); lo.y = wl.y * (lo.y * scale); lo.z = wl.z * (lo.z * scale); lo.w = wl.w * (lo.w * scale);
            hi.x = wh.x * (hi.x * scale); hi.y = wh.y * (hi.y * scale); hi.z = wh.z * (hi.z * scale); hi.w = wh.w * (hi.w * scale);
            __half2 a = __floats2half2_rn(lo.x, lo.z), b = __floats2half2_rn(lo.y, lo.w);
            __half2 c = __floats2half2_rn(hi.x, hi.z), d = __floats2half2_rn(hi.y, hi.w);
            out.x = *reinterpret_cast<uint32_t*>(&a);
            out.y = *reinterpret_cast<uint32_t*>(&b);
            out.z = *reinterpret_cast<uint32_t*>(&c);
            out.w = *reinterpret_cast<uint32_t*>(&d);
        }
        reinterpret_cast<uint4*>(packed)[(((uint64_t)chunk * token_groups + tg) * kCores + j) * 8 + tr] = out;
    }
}

// pack_norm_kernel for a batch whose rows still lack the sum of a split-K launch's partial
// products: a token's row first takes the `split` partial rows in index order (like
// reduce_kernel) and x keeps the sums. One CTA of 16 warps per 4 tokens (half a token group, so
// the grid is twice as wide), four warps to a token: a row is summed and written by exactly one
// CTA, which then packs its 4 tokens (64 of a group's 128 bytes per core-matrix row).
__global__ void __launch_bounds__(512) pack_norm_add_kernel(float* __restrict__ x, const float* __restrict__ weight, float eps,
                                                            __half* __restrict__ packed, uint32_t n_tokens, uint32_t n_cols, uint32_t token_groups,
                                                            const float* __restrict__ partial, uint32_t split) {
    __shared__ float sums[4][4];
    __shared__ float scales[4];
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, token0 = blockIdx.x * 4;
    {
        const uint32_t token = token0 + (warp >> 2), cols4 = n_cols / 4;
        float sumsq = 0.f;
        if (token < n_tokens) {
            float4* row = reinterpret_cast<float4*>(x + (uint64_t)token * n_cols);
            const uint64_t total4 = (uint64_t)n_tokens * cols4;
            const float4* part = reinterpret_cast<const float4*>(partial) + (uint64_t)token * cols4;
#pragma unroll 4
            for (uint32_t i = (warp & 3) * 32 + lane; i < cols4; i += 128) {
                float4 sum = __ldcg(part + i);
                for (uint32_t sp = 1; sp < split; ++sp) {
                    const float4 o = __ldcg(part + sp * total4 + i);
                    sum.x += o.x; sum.y += o.y; sum.z += o.z; sum.w += o.w;
                }
                float4 v = row[i];
                v.x += sum.x; v.y += sum.y; v.z += sum.z; v.w += sum.w;
                row[i] = v;
                sumsq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        sumsq = warp_sum(sumsq);
        if (lane == 0) sums[warp >> 2][warp & 3] = sumsq;
    }
    __syncthreads();
    if (tid < 4) scales[tid] = rsqrtf(((sums[tid][0] + sums[tid][1]) + (sums[tid][2] + sums[tid][3])) / (float)n_cols + eps);
    __syncthreads();
    const uint32_t tr = tid & 3, j = (tid >> 2) & (kCores - 1), sub = tid / (4 * kCores);  // 512 / 32 = 16 chunks per pass
    const uint32_t token = token0 + tr, n_chunks = n_cols / kChunkK, tg = token0 >> 3, in_group = (token0 & 4) + tr;
    const float scale = scales[tr];
    for (uint32_t chunk = sub; chunk < n_chunks; chunk += 512 / (4 * kCores)) {
        uint4 out = make_uint4(0, 0, 0, 0);
        if (token < n_tokens) {
            const uint32_t col = chunk * kChunkK + (j >> 2) * 32 + 4 * (j & 3);
            const float* src = x + (uint64_t)token * n_cols + col;
            float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 16);
            const float4 wl = __ldg(reinterpret_cast<const float4*>(weight + col)), wh = __ldg(reinterpret_cast<const float4*>(weight + col + 16));
            lo.x = wl.x * (lo.x * scale); lo.y = wl.y * (lo.y * scale); lo.z = wl.z * (lo.z * scale); lo.w = wl.w * (lo.w * scale);
            hi.x = wh.x * (hi.x * scale); hi.y = wh.y * (hi.y * scale); hi.z = wh.z * (hi.z * scale); hi.w = wh.w * (hi.w * scale);
            __half2 a = __floats2half2_rn(lo.x, lo.z), b = __floats2half2_rn(lo.y, lo.w);
            __half2 c = __floats2half2_rn(hi.x, hi.z), d = __floats2half2_rn(hi.y, hi.w);
            out.x = *reinterpret_cast<uint32_t*>(&a);
            out.y = *reinterpret_cast<uint32_t*>(&b);
            out.z = *reinterpret_cast<uint32_t*>(&c);
            out.w = *reinterpret_cast<uint32_t*>(&d);
        }
        reinterpret_cast<uint4*>(packed)[(((uint64_t)chunk * token_groups + tg) * kCores + j) * 8 + in_group] = out;
    }
}

// Packing for grouped mode: sorted entry i of expert e (offsets[e] <= i < offsets[e + 1]) becomes
// token i - offsets[e] of the expert's region, which starts at token group e * cap_groups; its row
// of x is the entry's token (gather: entry / n_used) or the entry itself. One thread per 16-byte
// output. Rows between an expert's last token and the end of its last group of 16 stay unwritten:
// they only reach accumulator columns nobody stores.
__global__ void __launch_bounds__(256) pack_grouped_kernel(const float* __restrict__ x, __half* __restrict__ packed, const uint32_t* __restrict__ offsets,
                                                           const uint32_t* __restrict__ entries, uint32_t n_experts, uint32_t n_used, int gather,
                                                           uint32_t n_cols, uint32_t cap_groups, uint32_t total_entries) {
    pdl_launch_dependents();
    pdl_wait();
    const uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t n_chunks = n_cols / kChunkK;
    if (o >= (uint64_t)total_entries * n_chunks * kCores) return;
    const uint32_t j = o % kCores;
    const uint32_t i = (o / kCores) % total_entries, chunk = (uint32_t)(o / ((uint64_t)kCores * total_entries));
    // A grouping over a range of experts keeps fewer entries than tokens x slots.
    if (i >= offsets[n_experts]) return;
    // The expert of sorted entry i: the last e with offsets[e] <= i.
    uint32_t lo = 0, hi = n_experts;
    while (hi - lo > 1) {
        uint32_t mid = (lo + hi) / 2;
        if (offsets[mid] <= i) lo = mid;
        else hi = mid;
    }
    const uint32_t local = i - offsets[lo], entry = entries[i];
    const uint32_t row = gather ? entry / n_used : entry;
    const float* src = x + (uint64_t)row * n_cols + chunk * kChunkK + (j >> 2) * 32 + 4 * (j & 3);
    const float4 l4 = *reinterpret_cast<const float4*>(src), h4 = *reinterpret_cast<const float4*>(src + 16);
    __half2 a = __floats2half2_rn(l4.x, l4.z), b = __floats2half2_rn(l4.y, l4.w);
    __half2 c = __floats2half2_rn(h4.x, h4.z), d = __floats2half2_rn(h4.y, h4.w);
    uint4 out = make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b), *reinterpret_cast<uint32_t*>(&c),
                           *reinterpret_cast<uint32_t*>(&d));
    const uint64_t token_groups = (uint64_t)n_experts * cap_groups, tg = (uint64_t)lo * cap_groups + local / 8;
    reinterpret_cast<uint4*>(packed)[((chunk * token_groups + tg) * kCores + j) * 8 + (local & 7)] = out;
}

__device__ __forceinline__ void give_up(volatile int* dead, int code) {
    *dead = 1;
    atomicCAS(&g_matmul_error, 0, code);
}

template <int DUAL>
__global__ void __launch_bounds__(Shape<DUAL>::kThreads, 1) matmul_umma_kernel(UmmaParams p) {
    constexpr uint32_t kStages = Shape<DUAL>::kStages, kStageA = Shape<DUAL>::kStageA, kTmemColumns = Shape<DUAL>::kTmemColumns;
    constexpr uint32_t kGroups = Shape<DUAL>::kGroups, kTmaWarp = Shape<DUAL>::kTmaWarp, kMmaWarp = Shape<DUAL>::kMmaWarp;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* a_tiles = smem;
    constexpr uint32_t kBTile = Shape<DUAL>::kStageB;
    uint8_t* b_tiles = a_tiles + kStages * kStageA;
    uint8_t* raw = b_tiles + kStages * kBTile;
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw + Shape<DUAL>::kRawBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 1);
    volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Launched with the programmatic-dependency attribute: a CTA may start while the launch before
    // it (the packing of this product's inputs, which needs next to no shared memory) still runs.
    // The weights are nobody's output, so barriers, tensor memory and the producers' first loads
    // go ahead; whatever reads or writes another launch's data waits first (the token-tile copies,
    // the epilogue, and in grouped mode everything, since the grouping decides the CTA's work).
    pdl_launch_dependents();
    if (p.offsets) pdl_wait();
    // The matrix this row tile belongs to.
    uint32_t row_tile = blockIdx.y, w_rows = p.n_rows, w_stride = p.y_stride;
    const uint4* w_quants = p.quants[0];
    const __half* w_scales = p.scales[0];
    float* w_y = p.y;
    if (DUAL == 1 && p.n_more) {
        int m = -1;
        if (row_tile >= p.more_first[0]) m = 0;
        if (p.n_more > 1 && row_tile >= p.more_first[1]) m = 1;
        if (p.n_more > 2 && row_tile >= p.more_first[2]) m = 2;
        if (m >= 0) {
            row_tile -= p.more_first[m];
            w_rows = w_stride = p.more_rows[m];
            w_quants = p.more_quants[m];
            w_scales = p.more_scales[m];
            w_y = p.more_y[m];
        }
    }
    const uint32_t tok0 = blockIdx.x * p.tile_tokens, row0 = row_tile * kRows;
    uint32_t n_tokens = p.n_tokens, group0 = 0;
    uint64_t weight0 = 0;  // first block of this CTA's matrix in the stacked weights
    const uint32_t* out_rows = nullptr;
    if (p.offsets) {
        const uint32_t first = p.offsets[blockIdx.z];
        n_tokens = p.offsets[blockIdx.z + 1] - first;
        if (tok0 >= n_tokens) return;  // the whole CTA, before it owns anything
        group0 = blockIdx.z * p.cap_groups;
        weight0 = (uint64_t)blockIdx.z * p.n_rows * p.n_blocks;
        out_rows = p.entries + first;
    }
    const uint32_t left = n_tokens - tok0;
    const uint32_t n_tile = left >= p.tile_tokens ? p.tile_tokens : ((left + 15u) & ~15u);  // the MMA's N
    // This CTA's share of K.
    const uint32_t per_part = (p.n_chunks + p.split - 1) / p.split;
    const uint32_t kc_begin = p.offsets ? 0 : blockIdx.z * per_part;
    const uint32_t kc_end = kc_begin + per_part < p.n_chunks ? kc_begin + per_part : p.n_chunks;
    const uint32_t my_chunks = kc_end > kc_begin ? kc_end - kc_begin : 0;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + kStages * 8, accum = empty0 + kStages * 8;
    const uint32_t a0 = smem_u32(a_tiles), b0 = smem_u32(b_tiles);

    if (tid == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(full0 + 8 * s, kGroupThreads / 32 + 1);  // the group's warps, plus the bulk copy's arrive.expect_tx
            mbar_init(empty0 + 8 * s, 1);                      // the MMA thread's commit
        }
        mbar_init(accum, 1);
        *dead = 0;
        mbar_init_fence();
    }
    if (warp == kMmaWarp) tmem_alloc(smem_u32(tmem_slot), kTmemColumns);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp < kTmaWarp) {
        // ---- producers: group `group` takes chunks group, group + kGroups, ...
        const uint32_t row = tid & (kRows - 1), group = tid / kGroupThreads;
        const uint32_t grow = row0 + row;
        const bool valid = grow < w_rows;
        const uint64_t first = weight0 + (uint64_t)(valid ? grow : 0) * p.n_blocks + (uint64_t)kc_begin * kChunkBlocks;
        const uint32_t a_off = (row >> 3) * kGroupBytes + (row & 7) * 16;
        // A row's share of a chunk of one matrix. Rows past the matrix keep scale zero, so their tile rows are zero.
        struct Share {
            uint4 q[kChunkBlocks];
            unsigned short d[kChunkBlocks];
        };
        auto fetch = [&](uint32_t i, int m) {
            Share r;
            const uint4* qsrc = (m == 0 ? w_quants : p.quants[1]) + first;
            const unsigned short* ssrc = reinterpret_cast<const unsigned short*>(m == 0 ? w_scales : p.scales[1]) + first;
#pragma unroll
            for (uint32_t b = 0; b < kChunkBlocks; ++b) {
                r.q[b] = make_uint4(0, 0, 0, 0);
                r.d[b] = 0;
                if (valid && i < my_chunks) {
                    r.q[b] = __ldg(qsrc + (uint64_t)i * kChunkBlocks + b);
                    r.d[b] = __ldg(ssrc + (uint64_t)i * kChunkBlocks + b);
                }
            }
            return r;
        };
        // One matrix: loads stay in flight in registers two turns ahead. Two matrices: a thread's
        // bytes come through its own two slots of shared memory by cp.async, two turns ahead as
        // well, and it reads them back itself (no other thread touches them): handing loaded
        // registers on from turn to turn waits for the youngest load, which with one turn of lead
        // made a turn as long as a trip to memory.
        constexpr bool kStaged = Shape<DUAL>::kStaged;
        constexpr uint32_t kRawTile = Shape<DUAL>::kRawTile;
        uint8_t* my_raw = raw + (size_t)group * 2 * DUAL * kRawTile;  // [slot][matrix]: quants of the 128 rows, then their scales
        auto stage_bytes = [&](uint32_t i, uint32_t slot) {
            if (valid && i < my_chunks) {
#pragma unroll
                for (int m = 0; m < DUAL; ++m) {
                    const uint4* qsrc = (m == 0 ? w_quants : p.quants[1]) + first + (uint64_t)i * kChunkBlocks;
                    const unsigned short* ssrc = reinterpret_cast<const unsigned short*>(m == 0 ? w_scales : p.scales[1]) + first + (uint64_t)i * kChunkBlocks;
                    uint8_t* tile = my_raw + (slot * DUAL + m) * kRawTile;
#pragma unroll
                    for (uint32_t b = 0; b < kChunkBlocks; ++b) cp_async_16(smem_u32(tile + row * (16 * kChunkBlocks) + 16 * b), qsrc + b);
                    cp_async_4(smem_u32(tile + kGroupThreads * (16 * kChunkBlocks) + row * (2 * kChunkBlocks)), ssrc);
                }
            }
            cp_async_commit();
        };
        auto staged = [&](uint32_t slot, int m) {
            Share r;
            const uint8_t* tile = my_raw + (slot * DUAL + m) * kRawTile;
#pragma unroll
            for (uint32_t b = 0; b < kChunkBlocks; ++b) {
                r.q[b] = make_uint4(0, 0, 0, 0);
                r.d[b] = 0;
            }
            if (valid) {
#pragma unroll
                for (uint32_t b = 0; b < kChunkBlocks; ++b) r.q[b] = *reinterpret_cast<const uint4*>(tile + row * (16 * kChunkBlocks) + 16 * b);
                const uint32_t two = *reinterpret_cast<const uint32_t*>(tile + kGroupThreads * (16 * kChunkBlocks) + row * (2 * kChunkBlocks));
                r.d[0] = (unsigned short)(two & 0xffffu);
                r.d[kChunkBlocks - 1] = (unsigned short)(two >> 16);
            }
            return r;
        };
        static_assert(!kStaged || kChunkBlocks == 2, "the staged form reads a row's two scales as one word");
        Share cur[DUAL], next[DUAL], after[DUAL];
        if (kStaged) {
            stage_bytes(group, 0);
            stage_bytes(group + kGroups, 1);
        } else {
#pragma unroll
            for (int m = 0; m < DUAL; ++m) {
                cur[m] = fetch(group, m);
                next[m] = fetch(group + kGroups, m);
            }
        }
        bool alive = true;
        const uint32_t stage = group;  // kGroups == kStages
        uint32_t phase = 1;            // the parity a free stage shows
        uint32_t slot = 0;
        for (uint32_t i = group; i < my_chunks; i += kGroups, phase ^= 1, slot ^= 1) {
            if (kStaged) {
                cp_async_wait<1>();  // all but the newest group: this turn's bytes are in
#pragma unroll
                for (int m = 0; m < DUAL; ++m) cur[m] = staged(slot, m);
            } else if (DUAL == 1) {
                after[0] = fetch(i + 2 * kGroups, 0);
            }
#pragma unroll
            for (int m = 0; m < DUAL; ++m) {
                // Dequantise before waiting for the stage, so only the stores follow the wait.
                uint4 v[kChunkBlocks * 4];
#pragma unroll
                for (uint32_t b = 0; b < kChunkBlocks; ++b) {
                    const __half d = __ushort_as_half(cur[m].d[b]);
                    const __half2 scale = __halves2half2(d, d);
                    v[4 * b + 0] = dequant_word(cur[m].q[b].x, scale);
                    v[4 * b + 1] = dequant_word(cur[m].q[b].y, scale);
                    v[4 * b + 2] = dequant_word(cur[m].q[b].z, scale);
                    v[4 * b + 3] = dequant_word(cur[m].q[b].w, scale);
                }
                if (m == 0) {
                    // Lane 0 polls for the whole warp.
                    bool ok = lane != 0 || mbar_wait(empty0 + 8 * stage, phase, kSpinLimit, dead);
                    if (!__all_sync(0xffffffffu, ok)) {
                        if (lane == 0) give_up(dead, 1);
                        alive = false;
                    }
                }
                if (alive) {
                    const uint32_t dst = a0 + stage * kStageA + m * kATile + a_off;
#pragma unroll
                    for (uint32_t j = 0; j < kChunkBlocks * 4; ++j) {
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + j * kCoreBytes), "r"(v[j].x), "r"(v[j].y), "r"(v[j].z),
                                     "r"(v[j].w)
                                     : "memory");
                    }
                }
            }
            if (!alive) break;
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(full0 + 8 * stage);
            if (kStaged) {
                stage_bytes(i + 2 * kGroups, slot);  // the slot just read takes the bytes of two turns on
            } else {
#pragma unroll
                for (int m = 0; m < DUAL; ++m) {
                    cur[m] = next[m];
                    if (DUAL == 1) next[m] = after[m];
                    else next[m] = fetch(i + 2 * kGroups, m);
                }
            }
        }
        if (kStaged) cp_async_wait<0>();

        // ---- epilogue: lanes 32 * (warp % 4).. of tensor memory, a quarter of the columns per warp
        pdl_wait();  // y, the partial products and the packed output are other launches' to read or write until now
        alive = __all_sync(0xffffffffu, alive);
        if (alive && !mbar_wait(accum, 0, kSpinLimit, dead)) {
            give_up(dead, 2);
            alive = false;
        }
        alive = __all_sync(0xffffffffu, alive);
        if (alive) {
            tc_fence_after_sync();
            const uint32_t quarter = warp & 3, part = warp >> 2, units = n_tile / 16;
            const uint32_t out_row = row0 + quarter * 32 + lane;
            float* out = w_y + (p.split > 1 ? (uint64_t)blockIdx.z * n_tokens * w_stride : 0);
            for (uint32_t u = part; u < units; u += kGroups) {
                float v[16];
                __syncwarp();
                tmem_load_16(tmem + ((quarter * 32) << 16) + u * 16, v);
                if (DUAL == 2) {
                    // silu(gate) * up, both from tensor memory.
                    float up[16];
                    tmem_load_16(tmem + ((quarter * 32) << 16) + kMaxTokens + u * 16, up);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = v[j] / (1.f + expf(-v[j])) * up[j];
                }
                if (DUAL == 2 && p.packed_out) {
                    // The warp's 32 rows are one block of 32 columns of the consuming product, its
                    // 16 tokens two groups of 8: 4 core-matrix rows of 16 bytes per token. A lane
                    // holds one column of 16 tokens and the layout wants 8 columns of one token
                    // per 16 bytes, so the values turn through shared memory (the weight tiles
                    // are idle by now; 17 rows of 16 bytes per core matrix keep both sides free of
                    // bank conflicts), and each lane stores two 16-byte rows, 8 lanes to a 128-byte line.
                    if (row0 + quarter * 32 < w_rows) {
                        __half* turn = reinterpret_cast<__half*>(a_tiles + warp * 1152);
                        const uint32_t core = (lane & 15) >> 2, e = lane & 3;
                        const uint32_t at = (lane >> 4) * 4 + (e & 1) * 2 + (e >> 1);  // the column order of pack_kernel
#pragma unroll
                        for (int j = 0; j < 16; ++j) turn[(core * 17 + j) * 8 + at] = __float2half_rn(v[j]);
                        __syncwarp();
                        const uint32_t tr = lane & 7, mm = lane >> 3;
                        const uint32_t chunk = (row0 >> 6) + (quarter >> 1), jj = (quarter & 1) * 4 + mm;
#pragma unroll
                        for (uint32_t it = 0; it < 2; ++it) {
                            const uint4 row16 = *reinterpret_cast<const uint4*>(turn + (mm * 17 + it * 8 + tr) * 8);
                            const uint32_t tg = ((tok0 + u * 16) >> 3) + it;
                            reinterpret_cast<uint4*>(p.packed_out)[(((uint64_t)chunk * p.token_groups + tg) * kCores + jj) * 8 + tr] = row16;
                        }
                    }
                    continue;
                }
                if (out_row < w_rows) {
                    // Old values first, all 16 in flight at once, so the read-modify-write stores cost one round trip.
                    float old[16];
                    // The output row of each token: itself, or in grouped mode the entry it came from.
                    uint32_t dest[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        uint32_t tok = tok0 + u * 16 + j;
                        dest[j] = tok < n_tokens ? (out_rows ? __ldg(out_rows + tok) : tok) : 0xffffffffu;
                    }
                    if (DUAL == 1 && p.store != BC_STORE_OVERWRITE) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) old[j] = dest[j] != 0xffffffffu ? __ldcg(out + (uint64_t)dest[j] * w_stride + out_row) : 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (dest[j] != 0xffffffffu) {
                            float r = my_chunks ? v[j] : 0.f;
                            if (DUAL == 1 && p.store == BC_STORE_ACCUMULATE) r += old[j];
                            else if (DUAL == 1 && p.store == BC_STORE_SWIGLU) r = old[j] / (1.f + expf(-old[j])) * r;
                            out[(uint64_t)dest[j] * w_stride + out_row] = r;
                        }
                    }
                }
            }
        }
    } else if (warp == kTmaWarp) {
        // ---- the token tiles: one bulk copy per stage
        if (lane == 0) {
            pdl_wait();  // the packed inputs are the launch before's
            const uint32_t bytes = n_tile * kChunkK * 2;
            const __half* src = p.packed + (uint64_t)(group0 + tok0 / 8) * (8 * kChunkK);
            uint32_t stage = 0, phase = 1;
            for (uint32_t i = 0; i < my_chunks; ++i, ++stage) {
                if (stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
                if (!mbar_wait(empty0 + 8 * stage, phase, kSpinLimit, dead)) {
                    give_up(dead, 3);
                    break;
                }
                mbar_arrive_expect(full0 + 8 * stage, bytes);
                bulk_load(b0 + stage * kBTile, src + (uint64_t)(kc_begin + i) * p.token_groups * (8 * kChunkK), bytes, full0 + 8 * stage);
            }
        }
    } else {
        // ---- the tensor core: kChunkK / 16 steps of K = 16 per stage and matrix
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(kRows, n_tile);
            const uint64_t a_desc0 = umma_desc(a0, kCoreBytes, kGroupBytes), b_desc0 = umma_desc(b0, kCoreBytes, kGroupBytes);
            bool alive = true;
            uint32_t stage = 0, phase = 0;
            for (uint32_t i = 0; i < my_chunks; ++i, ++stage) {
                if (stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
                if (!mbar_wait(full0 + 8 * stage, phase, kSpinLimit, dead)) {
                    give_up(dead, 4);
                    alive = false;
                    break;
                }
                tc_fence_after_sync();
                // The address field counts 16-byte units, so stepping a descriptor is an add.
                const uint64_t b_desc = b_desc0 + ((stage * kBTile) >> 4);
#pragma unroll
                for (uint32_t m = 0; m < (uint32_t)DUAL; ++m) {
                    const uint64_t a_desc = a_desc0 + ((stage * kStageA + m * kATile) >> 4);
#pragma unroll
                    for (uint32_t j = 0; j < kChunkK / 16; ++j)
                        umma_f16(tmem + m * kMaxTokens, a_desc + ((j * 2 * kCoreBytes) >> 4), b_desc + ((j * 2 * kCoreBytes) >> 4), idesc,
                                 (i | j) != 0);
                }
                umma_commit(empty0 + 8 * stage);
            }
            if (alive) umma_commit(accum);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*dead) __nanosleep(100000);  // let copies and instructions still in flight land before the CTA goes
    if (warp == kMmaWarp) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem, kTmemColumns);
    }
}

// y (store) the sum of the `split` partial products, added in index order.
__global__ void __launch_bounds__(256) reduce_kernel(const float* __restrict__ partial, float* __restrict__ y, uint32_t n_rows,
                                                     uint32_t n_tokens, uint32_t y_stride, uint32_t split, int store) {
    pdl_launch_dependents();
    pdl_wait();
    const uint64_t total = (uint64_t)n_tokens * n_rows;
    const uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= total) return;  // n_rows is a multiple of 4 here, so a float4 never straddles tokens
    float4 sum = *reinterpret_cast<const float4*>(partial + i);
    for (uint32_t s = 1; s < split; ++s) {
        float4 v = *reinterpret_cast<const float4*>(partial + s * total + i);
        sum.x += v.x;
        sum.y += v.y;
        sum.z += v.z;
        sum.w += v.w;
    }
    const uint32_t tok = (uint32_t)(i / n_rows), row = (uint32_t)(i % n_rows);
    float4* out = reinterpret_cast<float4*>(y + (uint64_t)tok * y_stride + row);
    if (store == BC_STORE_ACCUMULATE) {
        float4 o = *out;
        sum.x += o.x;
        sum.y += o.y;
        sum.z += o.z;
        sum.w += o.w;
    } else if (store == BC_STORE_SWIGLU) {
        float4 g = *out;
        sum.x = g.x / (1.f + expf(-g.x)) * sum.x;
        sum.y = g.y / (1.f + expf(-g.y)) * sum.y;
        sum.z = g.z / (1.f + expf(-g.z)) * sum.z;
        sum.w = g.w / (1.f + expf(-g.w)) * sum.w;
    }
    *out = sum;
}

// How a product is cut into CTAs: the token tile's width and the parts K is split into.
struct Tiling {
    uint32_t tile_tokens, split;
};

// Pick the tiling with the smallest modelled time. A CTA costs a fixed prologue and epilogue plus,
// per 64-column chunk, a handshake and MMA time in proportion to the tile width; the launch takes
// as many waves as its CTAs need on the device; a split adds its reduction launch. The constants
// are rough fits to measurements on this kernel; only the ranking matters. Narrower token tiles
// trade a little MMA efficiency for fuller waves (84 row tiles x 2 token tiles fill 1.14 waves;
// x 3 fill 1.7 waves of tiles two thirds the size).
Tiling choose_tiling(uint32_t n_rows, uint32_t n_cols, uint32_t n_tokens, uint32_t y_stride, int dual, bool may_split) {
    const uint32_t row_tiles = (n_rows + kRows - 1) / kRows, chunks = n_cols / kChunkK, sms = (uint32_t)sm_count();
    const bool can_split = may_split && dual == 1 && n_rows % 4 == 0 && y_stride % 4 == 0;
    const uint32_t widest = dual == 2 ? Shape<2>::kTileTokens : Shape<1>::kTileTokens;
    Tiling best{widest, 1};
    double best_cost = 1e30;
    const uint32_t min_tiles = (n_tokens + widest - 1) / widest;
    for (uint32_t token_tiles = min_tiles; token_tiles <= min_tiles + 6; ++token_tiles) {
        uint32_t width = (((n_tokens + token_tiles - 1) / token_tiles) + 15u) & ~15u;
        if (width < 64 && token_tiles > min_tiles) break;
        const uint32_t tiles_needed = (n_tokens + width - 1) / width;
        for (uint32_t split = 1; split <= (can_split ? kMaxSplit : 1u); ++split) {
            if (split > 1 && chunks / split < 8) break;
            const uint32_t ctas = row_tiles * tiles_needed * split;
            const double waves = (double)((ctas + sms - 1) / sms);
            const double per_chunk = 0.25 + 0.25 * dual * width / 256.0;  // microseconds
            double cost = waves * (5.0 + ((chunks + split - 1) / split) * per_chunk);
            if (split > 1) cost += 4.0 + 0.5 * split;
            if (cost < best_cost) {
                best_cost = cost;
                best = Tiling{width, split};
            }
        }
    }
    return best;
}

bool umma_disabled() {
    static const bool off = [] {
        const char* v = std::getenv("BOBCAT_NO_UMMA_MATMUL");
        return v && v[0] == '1';
    }();
    return off;
}

}  // namespace

uint64_t matmul_pack_bytes(uint32_t n_tokens, uint32_t n_cols) { return (uint64_t)((n_tokens + 15u) & ~15u) * n_cols * 2; }

uint64_t matmul_partial_bytes(const Mat& w, uint32_t n_tokens) {
    if (const uint32_t slices = matmul_few_slices(w, n_tokens)) return (uint64_t)slices * n_tokens * w.n_rows * 4;
    uint32_t split = choose_tiling(w.n_rows, w.n_cols, n_tokens, w.n_rows, 1, true).split;
    return split > 1 ? (uint64_t)split * n_tokens * w.n_rows * 4 : 0;
}

uint64_t matmul_scratch_bytes(const Mat& w, uint32_t n_tokens) {
    uint64_t pack = (matmul_pack_bytes(n_tokens, w.n_cols) + 255) & ~255ull;
    return pack + matmul_partial_bytes(w, n_tokens);
}

int matmul_umma_launches(const Mat& w, uint32_t n_tokens) {
    if (matmul_few_supported(w, n_tokens)) return 2;
    if (matmul_few_slices(w, n_tokens)) return 3;
    return choose_tiling(w.n_rows, w.n_cols, n_tokens, w.n_rows, 1, true).split > 1 ? 3 : 2;
}

bool matmul_umma_supported(const Mat& w, uint32_t n_tokens, uint32_t min_tokens) {
    return !umma_disabled() && w.format == BC_Q4_0 && w.n_cols % kChunkK == 0 && w.n_cols > 0 && n_tokens >= min_tokens && n_tokens > 0;
}

cudaError_t matmul_pack(cudaStream_t stream, const float* x, uint32_t n_tokens, uint32_t n_cols, void* packed) {
    uint32_t token_groups = ((n_tokens + 15u) & ~15u) / 8;
    uint64_t total = (uint64_t)(n_cols / kChunkK) * token_groups * (8 * kCores);
    if (total == 0) return cudaSuccess;
    return launch_dependent(pack_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, static_cast<__half*>(packed), n_tokens, n_cols,
                            token_groups, total);
}

cudaError_t matmul_pack_norm(cudaStream_t stream, float* x, Norm norm, uint32_t n_tokens, uint32_t n_cols, void* packed, const Deferred* add) {
    uint32_t token_groups = ((n_tokens + 15u) & ~15u) / 8;
    if (token_groups == 0 || n_cols == 0) return cudaSuccess;
    const bool adding = add && add->partial;
    if (adding && (add->n_tokens != n_tokens || add->n_rows != n_cols || n_cols % 4 != 0)) return cudaErrorInvalidValue;
    const uint32_t shares = token_groups >= 256 ? 1 : token_groups >= 64 ? 4 : 8;
    if (adding) {
        return launch_dependent(pack_norm_add_kernel, dim3(token_groups * 2), dim3(512), 0, stream, x, norm.weight, norm.eps, static_cast<__half*>(packed),
                                n_tokens, n_cols, token_groups, add->partial, add->split);
    }
    return launch_dependent(pack_norm_kernel, dim3(token_groups, shares), dim3(256), 0, stream, static_cast<const float*>(x), norm.weight, norm.eps,
                            static_cast<__half*>(packed), n_tokens, n_cols, token_groups);
}

cudaError_t matmul_reduce(cudaStream_t stream, const Deferred& d, float* y) {
    if (!d.partial || d.n_tokens == 0) return cudaSuccess;
    const uint64_t quads = (uint64_t)d.n_tokens * d.n_rows / 4;
    return launch_dependent(reduce_kernel, dim3((unsigned)((quads + 255) / 256)), dim3(256), 0, stream, d.partial, y, d.n_rows, d.n_tokens, d.n_rows, d.split,
                            (int)BC_STORE_ACCUMULATE);
}

cudaError_t matmul_umma(cudaStream_t stream, const Mat& w, const void* scratch, float* y, uint32_t n_tokens, uint32_t y_stride,
                        int32_t store, float* partial_at, Deferred* defer) {
    if (defer) *defer = Deferred{};
    if (n_tokens == 0 || w.n_rows == 0) return cudaSuccess;
    if (matmul_few_supported(w, n_tokens)) {
        const Mat* ws[1] = {&w};
        float* ys[1] = {y};
        const uint32_t strides[1] = {y_stride};
        return matmul_few(stream, ws, ys, strides, 1, scratch, n_tokens, store);
    }
    if (const uint32_t slices = matmul_few_slices(w, n_tokens)) {
        // A wide matrix against few tokens: slices of K on the few-token kernel, summed in order.
        float* partial = partial_at ? partial_at
                                    : reinterpret_cast<float*>(static_cast<char*>(const_cast<void*>(scratch)) +
                                                               ((matmul_pack_bytes(n_tokens, w.n_cols) + 255) & ~255ull));
        cudaError_t e = matmul_few_sliced(stream, w, scratch, partial, n_tokens);
        if (e != cudaSuccess) return e;
        if (defer && store == BC_STORE_ACCUMULATE && y_stride == w.n_rows) {
            *defer = Deferred{partial, slices, n_tokens, w.n_rows};
            return cudaSuccess;
        }
        const uint64_t quads = (uint64_t)n_tokens * w.n_rows / 4;
        return launch_dependent(reduce_kernel, dim3((unsigned)((quads + 255) / 256)), dim3(256), 0, stream, static_cast<const float*>(partial), y, w.n_rows,
                                n_tokens, y_stride, slices, (int)store);
    }
    cudaError_t err = ensure_dynamic_smem(reinterpret_cast<const void*>(&matmul_umma_kernel<1>), Shape<1>::kSmemBytes);
    if (err != cudaSuccess) return err;
    // The split must match matmul_scratch_bytes, which sized the scratch for a dense output.
    const Tiling tiling = choose_tiling(w.n_rows, w.n_cols, n_tokens, y_stride, 1, y_stride == w.n_rows);
    const uint32_t split = tiling.split;
    float* partial = partial_at ? partial_at
                                : reinterpret_cast<float*>(static_cast<char*>(const_cast<void*>(scratch)) +
                                                           ((matmul_pack_bytes(n_tokens, w.n_cols) + 255) & ~255ull));
    UmmaParams p{};
    p.quants[0] = static_cast<const uint4*>(w.data);
    p.scales[0] = w.scales;
    p.packed = static_cast<const __half*>(scratch);
    p.y = split > 1 ? partial : y;
    p.n_rows = w.n_rows;
    p.n_blocks = w.n_cols / 32;
    p.n_chunks = w.n_cols / kChunkK;  // matmul_umma_supported checked the width
    p.n_tokens = n_tokens;
    p.y_stride = split > 1 ? w.n_rows : y_stride;
    p.token_groups = ((n_tokens + 15u) & ~15u) / 8;
    p.split = split;
    p.tile_tokens = tiling.tile_tokens;
    p.store = split > 1 ? BC_STORE_OVERWRITE : store;
    dim3 grid((n_tokens + tiling.tile_tokens - 1) / tiling.tile_tokens, (w.n_rows + kRows - 1) / kRows, split);
    {
        void* args[] = {&p};
        cudaError_t launched = launch_kernel(reinterpret_cast<const void*>(&matmul_umma_kernel<1>), grid, dim3(Shape<1>::kThreads), Shape<1>::kSmemBytes, stream, args);
        if (launched != cudaSuccess) return launched;
    }
    err = cudaGetLastError();
    if (err != cudaSuccess || split == 1) return err;
    if (defer && store == BC_STORE_ACCUMULATE && y_stride == w.n_rows) {
        *defer = Deferred{partial, split, n_tokens, w.n_rows};
        return cudaSuccess;
    }
    const uint64_t quads = (uint64_t)n_tokens * w.n_rows / 4;
    return launch_dependent(reduce_kernel, dim3((unsigned)((quads + 255) / 256)), dim3(256), 0, stream, static_cast<const float*>(partial), y, w.n_rows,
                            n_tokens, y_stride, split, (int)store);
}

cudaError_t matmul_umma_several(cudaStream_t stream, const Mat* const* ws, float* const* ys, int n, const void* packed, uint32_t n_tokens) {
    if (n < 1 || n > 4) return cudaErrorInvalidValue;
    if (n_tokens == 0) return cudaSuccess;
    bool few = true;
    for (int i = 0; i < n; ++i) few = few && matmul_few_supported(*ws[i], n_tokens) && ws[i]->n_cols == ws[0]->n_cols;
    if (few) {
        uint32_t strides[4];
        for (int i = 0; i < n; ++i) strides[i] = ws[i]->n_rows;
        return matmul_few(stream, ws, ys, strides, n, packed, n_tokens, BC_STORE_OVERWRITE);
    }
    cudaError_t err = ensure_dynamic_smem(reinterpret_cast<const void*>(&matmul_umma_kernel<1>), Shape<1>::kSmemBytes);
    if (err != cudaSuccess) return err;
    uint32_t total_rows = 0, tiles = 0;
    for (int i = 0; i < n; ++i) {
        if (ws[i]->n_cols != ws[0]->n_cols || ws[i]->n_rows == 0) return cudaErrorInvalidValue;
        total_rows += ws[i]->n_rows;
    }
    UmmaParams p{};
    p.quants[0] = static_cast<const uint4*>(ws[0]->data);
    p.scales[0] = ws[0]->scales;
    p.packed = static_cast<const __half*>(packed);
    p.y = ys[0];
    p.n_rows = ws[0]->n_rows;
    p.y_stride = ws[0]->n_rows;
    tiles = (ws[0]->n_rows + kRows - 1) / kRows;
    p.n_more = (uint32_t)(n - 1);
    for (int i = 1; i < n; ++i) {
        p.more_first[i - 1] = tiles;
        p.more_rows[i - 1] = ws[i]->n_rows;
        p.more_quants[i - 1] = static_cast<const uint4*>(ws[i]->data);
        p.more_scales[i - 1] = ws[i]->scales;
        p.more_y[i - 1] = ys[i];
        tiles += (ws[i]->n_rows + kRows - 1) / kRows;
    }
    p.n_blocks = ws[0]->n_cols / 32;
    p.n_chunks = ws[0]->n_cols / kChunkK;
    p.n_tokens = n_tokens;
    p.token_groups = ((n_tokens + 15u) & ~15u) / 8;
    p.split = 1;
    p.tile_tokens = choose_tiling(total_rows, ws[0]->n_cols, n_tokens, total_rows, 1, false).tile_tokens;
    p.store = BC_STORE_OVERWRITE;
    dim3 grid((n_tokens + p.tile_tokens - 1) / p.tile_tokens, tiles, 1);
    {
        void* args[] = {&p};
        cudaError_t launched = launch_kernel(reinterpret_cast<const void*>(&matmul_umma_kernel<1>), grid, dim3(Shape<1>::kThreads), Shape<1>::kSmemBytes, stream, args);
        if (launched != cudaSuccess) return launched;
    }
    return cudaGetLastError();
}

bool matmul_umma_swiglu_supported(const Mat& gate, const Mat& up, uint32_t n_tokens, uint32_t min_tokens) {
    return matmul_umma_supported(gate, n_tokens, min_tokens) && matmul_umma_supported(up, n_tokens, min_tokens) && gate.n_rows == up.n_rows &&
           gate.n_cols == up.n_cols;
}

cudaError_t matmul_umma_swiglu(cudaStream_t stream, const Mat& gate, const Mat& up, const void* packed, float* y, uint32_t n_tokens,
                               uint32_t y_stride, void* packed_out) {
    if (packed_out && (gate.n_rows % kChunkK != 0)) return cudaErrorInvalidValue;
    if (n_tokens == 0 || gate.n_rows == 0) return cudaSuccess;
    if (matmul_few_supported(gate, n_tokens) && matmul_few_supported(up, n_tokens))
        return matmul_few_swiglu(stream, gate, up, packed, y, n_tokens, y_stride, packed_out);
    cudaError_t err = ensure_dynamic_smem(reinterpret_cast<const void*>(&matmul_umma_kernel<2>), Shape<2>::kSmemBytes);
    if (err != cudaSuccess) return err;
    UmmaParams p{};
    p.quants[0] = static_cast<const uint4*>(gate.data);
    p.scales[0] = gate.scales;
    p.quants[1] = static_cast<const uint4*>(up.data);
    p.scales[1] = up.scales;
    p.packed = static_cast<const __half*>(packed);
    p.y = y;
    p.n_rows = gate.n_rows;
    p.n_blocks = gate.n_cols / 32;
    p.n_chunks = gate.n_cols / kChunkK;
    p.n_tokens = n_tokens;
    p.y_stride = y_stride;
    p.token_groups = ((n_tokens + 15u) & ~15u) / 8;
    p.split = 1;
    p.tile_tokens = choose_tiling(gate.n_rows, gate.n_cols, n_tokens, y_stride, 2, false).tile_tokens;
    p.store = BC_STORE_OVERWRITE;
    p.packed_out = static_cast<__half*>(packed_out);
    dim3 grid((n_tokens + p.tile_tokens - 1) / p.tile_tokens, (gate.n_rows + kRows - 1) / kRows, 1);
    {
        void* args[] = {&p};
        cudaError_t launched = launch_kernel(reinterpret_cast<const void*>(&matmul_umma_kernel<2>), grid, dim3(Shape<2>::kThreads), Shape<2>::kSmemBytes, stream, args);
        if (launched != cudaSuccess) return launched;
    }
    return cudaGetLastError();
}

// ---- grouped products over experts (mixture-of-experts prefill)

bool matmul_experts_umma_supported(const Mat& w, const Mat* up, uint32_t n_tokens) {
    static const bool experts_off = [] { const char* v = std::getenv("BOBCAT_NO_UMMA_EXPERTS"); return v && v[0] == '1'; }();
    if (umma_disabled() || experts_off || w.format != BC_Q4_0 || w.n_cols % kChunkK != 0 || n_tokens < 16) return false;
    return !up || (up->format == BC_Q4_0 && up->n_cols == w.n_cols && up->n_rows == w.n_rows);
}

uint64_t matmul_experts_scratch_bytes(uint32_t n_experts, uint32_t n_tokens, uint32_t n_cols) {
    return (uint64_t)n_experts * ((n_tokens + 15u) & ~15u) * n_cols * 2;
}

cudaError_t matmul_experts_umma(cudaStream_t stream, const Mat& w, const Mat* up, uint32_t n_rows, uint32_t n_experts, const float* x, bool gather,
                                const uint32_t* offsets, const uint32_t* entries, uint32_t n_used, float* y, uint32_t n_tokens, void* scratch) {
    if (n_tokens == 0 || n_rows == 0) return cudaSuccess;
    const uint32_t cap_groups = ((n_tokens + 15u) & ~15u) / 8, total = n_tokens * n_used;
    const uint64_t outputs = (uint64_t)total * (w.n_cols / kChunkK) * kCores;
    cudaError_t err = launch_dependent(pack_grouped_kernel, dim3((unsigned)((outputs + 255) / 256)), dim3(256), 0, stream, x, static_cast<__half*>(scratch),
                                       offsets, entries, n_experts, n_used, gather ? 1 : 0, w.n_cols, cap_groups, total);
    if (err != cudaSuccess) return err;
    if (matmul_few_experts_supported(w, up, n_rows, n_experts, n_tokens))
        return matmul_few_experts(stream, w, up, n_rows, n_experts, scratch, offsets, entries, y, n_tokens, total);
    UmmaParams p{};
    p.quants[0] = static_cast<const uint4*>(w.data);
    p.scales[0] = w.scales;
    if (up) {
        p.quants[1] = static_cast<const uint4*>(up->data);
        p.scales[1] = up->scales;
    }
    p.packed = static_cast<const __half*>(scratch);
    p.y = y;
    p.n_rows = n_rows;
    p.n_blocks = w.n_cols / 32;
    p.n_chunks = w.n_cols / kChunkK;
    p.n_tokens = n_tokens;
    p.y_stride = n_rows;
    p.token_groups = n_experts * cap_groups;
    p.split = 1;
    p.tile_tokens = up ? Shape<2>::kTileTokens : Shape<1>::kTileTokens;
    p.store = BC_STORE_OVERWRITE;
    p.offsets = offsets;
    p.entries = entries;
    p.cap_groups = cap_groups;
    // Any one expert can receive up to n_tokens entries (a token picks an expert at most once).
    dim3 grid((n_tokens + p.tile_tokens - 1) / p.tile_tokens, (n_rows + kRows - 1) / kRows, n_experts);
    if (up) {
        if ((err = ensure_dynamic_smem(reinterpret_cast<const void*>(&matmul_umma_kernel<2>), Shape<2>::kSmemBytes)) != cudaSuccess) return err;
        {
        void* args[] = {&p};
        cudaError_t launched = launch_kernel(reinterpret_cast<const void*>(&matmul_umma_kernel<2>), grid, dim3(Shape<2>::kThreads), Shape<2>::kSmemBytes, stream, args);
        if (launched != cudaSuccess) return launched;
    }
    } else {
        if ((err = ensure_dynamic_smem(reinterpret_cast<const void*>(&matmul_umma_kernel<1>), Shape<1>::kSmemBytes)) != cudaSuccess) return err;
        {
        void* args[] = {&p};
        cudaError_t launched = launch_kernel(reinterpret_cast<const void*>(&matmul_umma_kernel<1>), grid, dim3(Shape<1>::kThreads), Shape<1>::kSmemBytes, stream, args);
        if (launched != cudaSuccess) return launched;
    }
    }
    return cudaGetLastError();
}

int matmul_error_flag() {
    int flag = 0;
    cudaMemcpyFromSymbol(&flag, g_matmul_error, sizeof flag);
    if (flag) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_matmul_error, &zero, sizeof zero);
    }
    return flag;
}

}  // namespace k
}  // namespace bc
