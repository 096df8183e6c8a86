// Q4_0 products against a handful of tokens (at most 32): the weight products of a pass over
// several sequences, of a short prefill chunk, of an expert's few entries.
//
// Why it exists. The tcgen05 prefill kernel turns every weight tile into fp16 in shared memory
// before the tensor cores see it, and that conversion, not the token count, sets its time: about
// 0.7 TB/s of weights however few tokens there are. With 32 tokens or fewer the multiply-adds are
// so few that the warp-level MMA has room for them (measured here: one mma.m16n8k16 per 8 cycles
// and scheduler, 20 cycles from operand to result), and then the weights never need to exist as
// fp16 in memory: a lane unpacks its own share of a 16-row weight tile in registers (13 ALU
// instructions per 8 weights) straight into the A operand, the tokens are the B operand, and the
// kernel is a weight stream like the decode kernel. Same arithmetic as the prefill kernel: fp16
// weights (q - 8) * d rounded once, fp16 inputs, f32 sums (the reference's batched Q4_0 product,
// crates/bobcat-metal/src/matmul.metal:519-521).
//
// Operands. The weights come from the decode kernel's tile layout (kernels_matvec_mma.cu): for
// each pair of blocks a lane (g, t) = (lane / 4, lane % 4) finds, in 16 contiguous bytes, word t of
// the quants of rows g and g + 8 of both blocks: dequant_word of the two words of a block is the
// A fragment of its two k-steps, in the registers the MMA wants. The tokens come from the prefill
// kernel's packed fp16 operand (packed_operand_index): its 16-byte piece for (token, block, t)
// holds the inputs that meet exactly those eight weights, in the order dequant_word emits them, so
// a piece IS the B fragment of both k-steps, for token g of a group of 8. (With the tokens as A
// and the weights as B the same loads need four register moves per MMA: that form issued twice
// the instructions.)
//
// Where the tokens are read from. Every tile meets all the tokens, so a CTA reads them many times
// over. When the whole operand fits (up to 128 KB: 2048 columns of 32 tokens) the warps copy it
// into shared memory once per launch, permuting the eight pieces of each core matrix (piece g of
// core c goes to g ^ 2 (c % 4)): the four t-lanes of a quarter warp read cores 128 bytes apart,
// which unpermuted is a four-way bank conflict on every read - it, not the weights or the MMAs,
// set the kernel's time at first (40 us for gate and up of the 2.6B shape, 30 us without it).
// A wider operand is cut into slices of K that fit: the CTAs are divided among the slices, each
// keeps its slice's tokens, and slice s leaves its sums in array s of a scratch the host adds up in
// order (matmul_few_sliced). Experts (each has its own few tokens) read the pieces through L1.
//
// Work. A job is a 16-row tile over all of K (for gate/up: the tile of both matrices). A CTA is 16
// warps on one SM; the CTAs take the jobs in turn, in rounds of as many jobs as the CTA has groups
// of warps; a group's warps split the job's block pairs (with two matrices, half the group each),
// their partial sums meet in shared memory and are added in warp order, so results do not depend
// on timing. The host picks the group size that makes rounds x pairs per warp smallest. A warp
// streams its weights through two slots of shared memory by bulk copies (4 or 8 pairs each), the
// first two requested before the wait for the preceding launch; every wait is bounded.

#include <cstdlib>

#include "async_utils.cuh"
#include "device_utils.cuh"
#include "kernels.h"
#include "../../include/bobcat_cuda.h"

namespace bc {
namespace k {

namespace {

constexpr int kWarps = 16, kThreads = kWarps * 32;
constexpr int kChunkBlocks = 32;                          // blocks per chunk of the tile layout
constexpr int kBlockBytes = 288;                          // 16 rows x 18 bytes
constexpr int kChunkBytes = kChunkBlocks * kBlockBytes;
constexpr uint32_t kMaxFewTokens = 32;
constexpr uint32_t kMaxExperts = 512;

struct FewParams {
    // Plain: up to four matrices that share the tokens, one job per tile of their concatenation.
    // Dual: tiles[0] = gate, tiles[1] = up, one job per tile pair.
    const uint8_t* tiles[4];
    float* y[4];
    uint32_t seg_tiles[4], seg_rows[4], seg_stride[4];
    int n_segments, dual;
    uint32_t n_jobs;      // plain / dual; with experts: tiles per expert
    uint32_t n_blocks;    // per row
    const uint4* packed;  // [pair][token group][8 cores][8 tokens] pieces
    uint32_t token_groups, n_tokens;
    uint32_t token_bytes;  // the whole packed operand, when the CTAs are to keep it in shared memory; else 0
    int store;
    __half* packed_out;   // dual: the result as the packed operand of the next product
    // Experts: expert e multiplies entries offsets[e] .. offsets[e + 1], packed from token group
    // e * cap_groups on; entry i's output row is entries[i].
    const uint32_t* offsets;
    const uint32_t* entries;
    uint32_t n_experts, cap_groups;
    // The CTA's warps: groups of `width` warps per matrix (twice that with two matrices) take a
    // tile each, every warp `share` pairs of it.
    uint32_t width, share;
    // Wide matrices (more tokens than a CTA can keep): K is cut into slices of slice_pairs pairs,
    // ctas_per_slice CTAs work on a slice (tiles c, c + ctas_per_slice, ...) and keep only its
    // tokens; slice s writes its sums to y[0] + s * n_tokens * seg_stride[0] for the host to add up.
    uint32_t slice_pairs, ctas_per_slice;
};

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void group_barrier(uint32_t id, uint32_t threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

// Where pair `pair` of a tile keeps this lane's quants and scales.
__device__ __forceinline__ const uint4* quants_of(const uint8_t* tile, uint32_t pair, uint32_t lane) {
    return reinterpret_cast<const uint4*>(tile + (uint64_t)(pair >> 4) * kChunkBytes + ((pair & 15) * 32 + lane) * 16);
}
__device__ __forceinline__ const uint2* scales_of(const uint8_t* tile, uint32_t pair, uint32_t lane, uint32_t n_blocks) {
    const uint32_t chunk = pair >> 4, left = n_blocks - chunk * kChunkBlocks, cb = left < (uint32_t)kChunkBlocks ? left : (uint32_t)kChunkBlocks;
    return reinterpret_cast<const uint2*>(tile + (uint64_t)chunk * kChunkBytes + cb * 256 + ((pair & 15) * 8 + (lane >> 2)) * 8);
}

constexpr int kSlotBytes = 8 * 576;                          // a warp's slot: up to 8 pairs of blocks, quants then scales
constexpr uint32_t kMaxTokenBytes = 128 * 1024;              // packed tokens a CTA keeps in shared memory
constexpr uint32_t kSpinLimit = 1u << 22;                    // bounded waits: give up rather than hang

__device__ int g_few_error;

// Pairs [first, last) of one tile against NT groups of 8 tokens. acc[j]: rows g and g + 8 x tokens
// 8j + 2t, + 1 in the m16n8 accumulator layout. The weights come through the warp's
// two slots of shared memory, up to kSlotPairs pairs per slot and per bulk copy (two: quants,
// scales): while one slot is multiplied the other is on its way, and the first two requests go
// out before the wait for the preceding launch. The tokens' pieces come through L1, one block's
// worth on its way while a block is multiplied.
template <int NT, bool XS>
struct Worker {
    // Pairs per slot: with the tokens in shared memory (XS) there is room for half as much.
    static constexpr uint32_t kSlotPairs = XS ? 4 : 8, kSlotScales = kSlotPairs * 512, kSlotStep = kSlotPairs * 576;
    uint32_t slot, bar;      // of slot 0; slot 1 follows kSlotStep (8 bytes) further
    uint32_t tokens;         // XS: where the packed tokens start in shared memory
    uint32_t issued, taken;  // pieces requested / consumed since the kernel began: slot and parity follow from them
    uint32_t next, last;     // pairs not yet requested

    // Request the next piece: up to the end of the half chunk `next` lies in.
    __device__ __forceinline__ uint32_t request(const uint8_t* tile, uint32_t lane, uint32_t n_blocks) {
        const uint32_t piece_end = (next / kSlotPairs + 1) * kSlotPairs, end = last < piece_end ? last : piece_end, n = end - next;
        if (n == 0) return 0;
        if (lane == 0) {
            const uint32_t to = slot + (issued & 1) * kSlotStep, on = bar + (issued & 1) * 8;
            async::fence_proxy_async();  // the slot held this warp's partial sums a moment ago
            async::mbar_arrive_expect(on, n * 576);
            async::bulk_load(to, quants_of(tile, next, 0), n * 512, on);
            async::bulk_load(to + kSlotScales, scales_of(tile, next, 0, n_blocks), n * 64, on);
        }
        ++issued;
        next = end;
        return n;
    }
    // Token g of every group of 8 tokens for block `blk` of a pair: the B fragments of both k-steps.
    static __device__ __forceinline__ void tokens_of(const uint4* __restrict__ chunk, int blk, uint32_t t, uint4 (&frag)[NT]) {
#pragma unroll
        for (int j = 0; j < NT; ++j) frag[j] = __ldg(chunk + (j * 8 + blk * 4 + t) * 8);
    }
    static __device__ __forceinline__ uint4 shared_piece(uint32_t at) {
        uint4 v;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(at));
        return v;
    }
    static __device__ __forceinline__ void tokens_of(uint32_t chunk, int blk, uint32_t t, uint4 (&frag)[NT]) {
#pragma unroll
        for (int j = 0; j < NT; ++j) frag[j] = shared_piece(chunk + ((j * 8 + blk * 4 + t) * 8) * 16);
    }
    // One block: rows g and g + 8 (a word of quants each, their scales in `both`) are the A fragment,
    // straight out of dequant_word; a token piece is the B fragment of both k-steps as loaded.
    static __device__ __forceinline__ void multiply(float (&acc)[NT][4], uint32_t row_lo, uint32_t row_hi, __half2 both, const uint4 (&frag)[NT]) {
        const uint4 lo = dequant_word(row_lo, __low2half2(both)), hi = dequant_word(row_hi, __high2half2(both));
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            mma_f16(acc[j], lo.x, hi.x, lo.y, hi.y, frag[j].x, frag[j].y);
            mma_f16(acc[j], lo.z, hi.z, lo.w, hi.w, frag[j].z, frag[j].w);
        }
    }
    // `sizes`: the pairs of the two pieces requested so far (the second may be empty).
    __device__ __forceinline__ void run(const uint8_t* tile, uint32_t first, uint32_t size0, uint32_t size1, uint32_t lane, uint32_t n_blocks,
                                        const uint4* __restrict__ pieces, uint32_t token_groups, float (&acc)[NT][4]) {
        if (size0 == 0) return;
        const uint32_t g = lane >> 2, t = lane & 3;
        // The packed chunk of 64 columns is the pair; its cores 0-3 are the first block.
        const uint64_t chunk_pieces = (uint64_t)token_groups * 64;
        const uint4* chunk = pieces + first * chunk_pieces + g;
        // In shared memory the eight pieces of a core matrix stand at g ^ 2 (core % 4): lanes t = 0 .. 3
        // of a quarter warp read from rows 128 bytes apart, and this spreads them over the banks.
        uint32_t chunk_at = tokens + (uint32_t)(first * chunk_pieces + (g ^ (2 * t))) * 16;
        uint4 first_block[NT], second_block[NT];
        if (!XS) tokens_of(chunk, 0, t, first_block);
        uint32_t pending = size0, after = size1;
        while (pending > 0) {
            const uint32_t from = slot + (taken & 1) * kSlotStep;
            if (!async::mbar_wait(bar + (taken & 1) * 8, (taken >> 1) & 1, kSpinLimit, &g_few_error)) g_few_error = 1;  // and carry on: the group's barriers still need this warp
            ++taken;
#pragma unroll 2
            for (uint32_t i = 0; i < pending; ++i) {
                uint4 words;
                uint2 scales;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(words.x), "=r"(words.y), "=r"(words.z), "=r"(words.w) : "r"(from + (i * 32 + lane) * 16));
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(scales.x), "=r"(scales.y) : "r"(from + kSlotScales + (i * 8 + g) * 8));
                if (XS) {
                    tokens_of(chunk_at, 0, t, first_block);
                    tokens_of(chunk_at, 1, t, second_block);
                    multiply(acc, words.x, words.y, *reinterpret_cast<const __half2*>(&scales.x), first_block);
                    multiply(acc, words.z, words.w, *reinterpret_cast<const __half2*>(&scales.y), second_block);
                    chunk_at += (uint32_t)chunk_pieces * 16;
                    continue;
                }
                tokens_of(chunk, 1, t, second_block);
                multiply(acc, words.x, words.y, *reinterpret_cast<const __half2*>(&scales.x), first_block);
                chunk += chunk_pieces;
                if (after > 0 || i + 1 < pending) tokens_of(chunk, 0, t, first_block);
                multiply(acc, words.z, words.w, *reinterpret_cast<const __half2*>(&scales.y), second_block);
            }
            __syncwarp();  // every lane has read the slot before the piece after next lands in it
            pending = after;
            after = request(tile, lane, n_blocks);
        }
    }
};

struct Job {
    const uint8_t* tile[2];
    float* y;
    uint32_t row0, rows, stride;       // first row of the tile, rows of its matrix, floats per output row
    uint32_t group0, n_tokens, first;  // first token group of its tokens, their number, first entry (experts)
};

__device__ __forceinline__ Job job_of(const FewParams& p, uint32_t job, const uint32_t* active) {
    Job j{};
    const uint64_t tile_bytes = (uint64_t)p.n_blocks * kBlockBytes;
    if (p.offsets) {
        const uint32_t e = active[job / p.n_jobs], tile = job % p.n_jobs;
        j.first = p.offsets[e];
        j.n_tokens = p.offsets[e + 1] - j.first;
        j.group0 = e * p.cap_groups;
        j.tile[0] = p.tiles[0] + ((uint64_t)e * p.n_jobs + tile) * tile_bytes;
        if (p.dual) j.tile[1] = p.tiles[1] + ((uint64_t)e * p.n_jobs + tile) * tile_bytes;
        j.y = p.y[0], j.row0 = tile * 16, j.rows = p.seg_rows[0], j.stride = p.seg_stride[0];
        return j;
    }
    int seg = 0;
    uint32_t local = job;
    while (seg + 1 < p.n_segments && local >= p.seg_tiles[seg]) {
        local -= p.seg_tiles[seg];
        ++seg;
    }
    j.tile[0] = p.tiles[seg] + (uint64_t)local * tile_bytes;
    if (p.dual) j.tile[1] = p.tiles[1] + (uint64_t)local * tile_bytes;
    j.y = p.y[seg], j.row0 = local * 16, j.rows = p.seg_rows[seg], j.stride = p.seg_stride[seg];
    j.n_tokens = p.n_tokens;
    return j;
}

// The leader warp of a group stores a finished tile; `up` is the second matrix's with p.dual.
// A lane holds rows g and g + 8 of the tile for tokens 8j + 2t and 8j + 2t + 1 of every group j.
template <int NT>
__device__ __forceinline__ void store_tile(const FewParams& p, const Job& j, uint32_t lane, float (&acc)[NT][4], float (&up)[NT][4]) {
    const uint32_t g = lane >> 2, t = lane & 3;
    if (p.dual) {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float v = acc[n][e];
                acc[n][e] = v / (1.f + expf(-v)) * up[n][e];
            }
    }
    if (p.dual && p.packed_out) {
        // The rows are columns of the next product, whose pieces want columns (0, 2), (1, 3) of a
        // group of four as pairs of halves: the lanes of rows 0 and 1 of a group fetch rows 2 and 3
        // from the lanes 8 further on and store a pair each.
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t token = n * 8 + 2 * t + (e & 1), row = j.row0 + g + (e >> 1) * 8;
                const float other = __shfl_down_sync(0xffffffffu, acc[n][e], 8);
                if ((g & 3) < 2) *reinterpret_cast<__half2*>(p.packed_out + packed_operand_index(token, row, p.token_groups)) = __floats2half2_rn(acc[n][e], other);
            }
        return;
    }
    // Old values first, all in flight at once, so a read-modify-write store costs one round trip.
    float* out[NT][2];
    bool live[NT][2];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint32_t token = n * 8 + 2 * t + e;
            live[n][e] = token < j.n_tokens;
            const uint32_t dest = live[n][e] ? (p.entries ? __ldg(p.entries + j.first + token) : token) : 0;
            out[n][e] = j.y + (uint64_t)dest * j.stride + j.row0 + g;
        }
    const bool reads = !p.dual && p.store != BC_STORE_OVERWRITE;
    const bool low = j.row0 + g < j.rows, high = j.row0 + g + 8 < j.rows;
    float old[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) old[n][e] = reads && live[n][e & 1] && ((e >> 1) ? high : low) ? __ldcg(out[n][e & 1] + (e >> 1) * 8) : 0.f;
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (!live[n][e & 1] || !((e >> 1) ? high : low)) continue;
            float v = acc[n][e];
            if (reads && p.store == BC_STORE_ACCUMULATE) v += old[n][e];
            else if (reads && p.store == BC_STORE_SWIGLU) v = old[n][e] / (1.f + expf(-old[n][e])) * v;
            out[n][e & 1][(e >> 1) * 8] = v;
        }
}

// One warp's share of a job. The group's `width` warps per matrix split the pairs; with two
// matrices the second half of the group works on the second one. A warp's partial sums go into
// its own slots, [register][lane], once it has read the weights there.
template <int NT, bool XS>
__device__ __forceinline__ void do_job(const FewParams& p, const Job& j, uint32_t rank, uint32_t width, uint32_t group_warps, uint32_t group,
                                       uint32_t lane, uint8_t* slots, uint32_t copiers, uint32_t lo, uint32_t hi, Worker<NT, XS>& worker, bool& waited) {
    // The CTA's pairs are [lo, hi): all of them, or its slice.
    const uint32_t stream = rank >= width ? 1 : 0, part = rank - stream * width;
    const uint32_t first = lo + part * p.share < hi ? lo + part * p.share : hi, last = first + p.share < hi ? first + p.share : hi;
    float acc[NT][4], up[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f, up[n][e] = 0.f;
    const uint8_t* tile = j.tile[stream];
    worker.next = first, worker.last = last;
    const uint32_t size0 = worker.request(tile, lane, p.n_blocks), size1 = worker.request(tile, lane, p.n_blocks);
    if (!waited) {
        pdl_wait();  // the weights are nobody's output; the tokens and the outputs are
        waited = true;
        if (XS) {
            // The launch's tokens, one contiguous run of the packed operand, into shared memory: the
            // warps that have a job in the first round copy them together, 16 bytes a thread at a
            // time, each core matrix's pieces permuted as the readers expect.
            const uint4* src = p.packed + (uint64_t)lo * p.token_groups * 64;
            const uint32_t n_pieces = (hi - lo) * p.token_groups * 64, to = worker.tokens + lo * p.token_groups * 64 * 16;  // where pair lo stands
            for (uint32_t q = threadIdx.x; q < n_pieces; q += 4 * copiers) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (q + u * copiers < n_pieces) v[u] = __ldg(src + q + u * copiers);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t at = q + u * copiers;
                    if (at < n_pieces)
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(to + ((at & ~7u) + ((at & 7u) ^ (2 * ((at >> 3) & 3u)))) * 16), "r"(v[u].x),
                                     "r"(v[u].y), "r"(v[u].z), "r"(v[u].w)
                                     : "memory");
                }
            }
            group_barrier(15, copiers);
        }
    }
    worker.run(tile, first, size0, size1, lane, p.n_blocks, p.packed + (uint64_t)j.group0 * 64, p.token_groups, acc);
    if (group_warps > 1) {
        constexpr uint32_t kArea = 2 * Worker<NT, XS>::kSlotStep;  // a warp's two slots: 4.5 KB at least, 2 KB of sums at most
        float* mine = reinterpret_cast<float*>(slots + (uint64_t)(group * group_warps + rank) * kArea) + lane;
        if (rank > 0) {
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) mine[(n * 4 + e) * 32] = acc[n][e];
        }
        group_barrier(1 + group, group_warps * 32);
        if (rank == 0) {
            // The others' sums in warp order: first the rest of this matrix, then the second one.
            for (uint32_t r = 1; r < group_warps; ++r) {
                const float* theirs = mine + (uint64_t)r * (kArea / 4);
                if (r < width) {
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int e = 0; e < 4; ++e) acc[n][e] += theirs[(n * 4 + e) * 32];
                } else {
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int e = 0; e < 4; ++e) up[n][e] += theirs[(n * 4 + e) * 32];
                }
            }
        }
        group_barrier(1 + group, group_warps * 32);  // the sums are read before the next round writes there
    }
    if (rank == 0) store_tile<NT>(p, j, lane, acc, up);
}

__global__ void __launch_bounds__(kThreads, 1) matmul_few_kernel(FewParams p) {
    extern __shared__ __align__(128) uint8_t few_smem[];  // two slots per warp, then the tokens when they fit
    __shared__ __align__(8) uint64_t bars[kWarps][2];
    __shared__ uint32_t active[kMaxExperts];
    __shared__ uint32_t n_active;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane < 2) async::mbar_init(async::smem_u32(&bars[warp][lane]), 1);
    async::mbar_init_fence();
    __syncthreads();
    pdl_launch_dependents();
    bool waited = false;
    uint32_t n_jobs = p.n_jobs;
    uint32_t issued = 0, taken = 0;
    if (p.offsets) {
        // Experts with entries, in any order: the order only decides which CTA takes which tile.
        pdl_wait();
        waited = true;
        if (threadIdx.x == 0) n_active = 0;
        __syncthreads();
        for (uint32_t e = threadIdx.x; e < p.n_experts; e += kThreads)
            if (p.offsets[e + 1] > p.offsets[e]) active[atomicAdd(&n_active, 1u)] = e;
        __syncthreads();
        n_jobs = n_active * p.n_jobs;
    }
    uint32_t job0 = blockIdx.x, job_step = gridDim.x, lo = 0, hi = p.n_blocks / 2;
    uint64_t slice_out = 0;
    if (p.slice_pairs) {
        const uint32_t slice = blockIdx.x / p.ctas_per_slice;
        job0 = blockIdx.x % p.ctas_per_slice, job_step = p.ctas_per_slice;
        lo = slice * p.slice_pairs;
        hi = lo + p.slice_pairs < hi ? lo + p.slice_pairs : hi;
        slice_out = (uint64_t)slice * p.n_tokens * p.seg_stride[0];
    }
    const uint32_t my_jobs = n_jobs > job0 ? (n_jobs - job0 + job_step - 1) / job_step : 0;
    if (my_jobs == 0) return;
    const uint32_t width = p.width, streams = p.dual ? 2 : 1;
    const uint32_t group_warps = width * streams, groups = kWarps / group_warps, group = warp / group_warps, rank = warp % group_warps;
    if (group >= groups) return;  // the warps left over when 16 is not a multiple of the group size
    for (uint32_t i = group; i < my_jobs; i += groups) {
        Job j = job_of(p, job0 + i * job_step, active);
        j.y += slice_out;
        const uint32_t slot = async::smem_u32(few_smem + warp * (2 * kSlotBytes)), bar = async::smem_u32(&bars[warp][0]);
        // The address pair 0's tokens would have: a slice's CTA keeps only pairs lo .. hi, from here on.
        const uint32_t tokens = async::smem_u32(few_smem + kWarps * kSlotBytes) - lo * p.token_groups * 64 * 16;
        const uint32_t copiers = (my_jobs < groups ? my_jobs : groups) * group_warps * 32;  // the threads with a job in the first round
        const uint32_t small = async::smem_u32(few_smem + warp * kSlotBytes);  // slots of half the size when the tokens follow them
#define BC_FEW_JOB(NT, XS)                                                                                            \
    {                                                                                                                 \
        Worker<NT, XS> worker{XS ? small : slot, bar, XS ? tokens : 0u, issued, taken, 0, 0};                          \
        do_job<NT, XS>(p, j, rank, width, group_warps, group, lane, few_smem, copiers, lo, hi, worker, waited);        \
        issued = worker.issued, taken = worker.taken;                                                                 \
    }
        if (p.token_bytes) {
            if (j.n_tokens > 16) BC_FEW_JOB(4, true)
            else if (j.n_tokens > 8) BC_FEW_JOB(2, true)
            else BC_FEW_JOB(1, true)
        } else {
            if (j.n_tokens > 16) BC_FEW_JOB(4, false)
            else if (j.n_tokens > 8) BC_FEW_JOB(2, false)
            else BC_FEW_JOB(1, false)
        }
#undef BC_FEW_JOB
    }
}

constexpr size_t kFewSlots = (size_t)kWarps * 2 * kSlotBytes;  // 144 KB; with the tokens in shared memory half of it plus up to 128 KB

bool few_disabled() {
    static const bool off = [] { const char* v = std::getenv("BOBCAT_NO_FEW_MATMUL"); return v && v[0] == '1'; }();
    return off;
}

// Bytes of the packed operand of n_tokens rows of n_cols: 1 KB per group of 8 tokens and 64 columns.
uint32_t few_token_bytes(uint32_t n_cols, uint32_t n_tokens) { return (n_cols / 64) * (((n_tokens + 15u) & ~15u) / 8) * 1024; }

// `likely_jobs`: the jobs the launch will probably have (all of them, unless experts stay idle).
cudaError_t launch_few(cudaStream_t stream, FewParams p, uint32_t most_jobs, uint32_t likely_jobs) {
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(&matmul_few_kernel), kFewSlots / 2 + kMaxTokenBytes);
    const size_t smem = p.token_bytes ? kFewSlots / 2 + p.token_bytes : kFewSlots;
    if (e != cudaSuccess) return e;
    const uint32_t sms = (uint32_t)sm_count();
    uint32_t ctas = most_jobs < sms ? most_jobs : sms;
    if (p.slice_pairs) {
        const uint32_t slices = (p.n_blocks / 2 + p.slice_pairs - 1) / p.slice_pairs;
        p.ctas_per_slice = sms / slices > most_jobs ? most_jobs : sms / slices;
        if (p.ctas_per_slice == 0) return cudaErrorInvalidValue;
        ctas = p.ctas_per_slice * slices;
        likely_jobs *= slices;  // jobs per CTA: the tiles over the CTAs of a slice
    }
    // Warps per job. A group of warps takes a job, `width` of them per matrix, each a share of the
    // pairs; a CTA's jobs go through its groups in rounds. The cost of a choice is rounds x (pairs
    // per warp + a round's fixed cost, about 3 pairs' worth); the narrowest group with the least
    // cost wins.
    const uint32_t pairs = p.slice_pairs ? p.slice_pairs : p.n_blocks / 2, streams = p.dual ? 2 : 1, my_jobs = (likely_jobs + ctas - 1) / ctas;
    uint32_t best = 0xffffffffu;
    p.width = 1;
    for (uint32_t w = 1; w * streams <= (uint32_t)kWarps && w <= pairs; ++w) {
        const uint32_t groups = kWarps / (w * streams), rounds = (my_jobs + groups - 1) / groups;
        const uint32_t cost = rounds * ((pairs + w - 1) / w + 3);
        if (cost < best) best = cost, p.width = w;
    }
    p.share = (pairs + p.width - 1) / p.width;
    return launch_dependent(matmul_few_kernel, dim3(ctas), dim3(kThreads), smem, stream, p);
}

}  // namespace

int matmul_few_error_flag() {
    int flag = 0;
    cudaMemcpyFromSymbol(&flag, g_few_error, sizeof flag);
    if (flag) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_few_error, &zero, sizeof zero);
    }
    return flag;
}

bool matmul_few_supported(const Mat& w, uint32_t n_tokens) {
    return !few_disabled() && w.format == BC_Q4_0 && w.tiles != nullptr && n_tokens > 0 && n_tokens <= kMaxFewTokens && w.n_cols % 64 == 0 && w.n_cols > 0 &&
           few_token_bytes(w.n_cols, n_tokens) <= kMaxTokenBytes;
}

cudaError_t matmul_few(cudaStream_t stream, const Mat* const* ws, float* const* ys, const uint32_t* strides, int n, const void* packed,
                       uint32_t n_tokens, int32_t store) {
    if (n < 1 || n > 4) return cudaErrorInvalidValue;
    FewParams p{};
    p.n_segments = n;
    for (int i = 0; i < n; ++i) {
        if (ws[i]->n_cols != ws[0]->n_cols) return cudaErrorInvalidValue;
        p.tiles[i] = static_cast<const uint8_t*>(ws[i]->tiles);
        p.y[i] = ys[i];
        p.seg_tiles[i] = (ws[i]->n_rows + 15) / 16;
        p.seg_rows[i] = ws[i]->n_rows;
        p.seg_stride[i] = strides[i];
        p.n_jobs += p.seg_tiles[i];
    }
    p.n_blocks = ws[0]->n_cols / 32;
    p.packed = static_cast<const uint4*>(packed);
    p.token_groups = ((n_tokens + 15u) & ~15u) / 8;
    p.n_tokens = n_tokens;
    p.token_bytes = few_token_bytes(ws[0]->n_cols, n_tokens);
    p.store = store;
    if (p.n_jobs == 0) return cudaSuccess;
    return launch_few(stream, p, p.n_jobs, p.n_jobs);
}

uint32_t matmul_few_slices(const Mat& w, uint32_t n_tokens) {
    if (few_disabled() || w.format != BC_Q4_0 || w.tiles == nullptr || n_tokens == 0 || n_tokens > kMaxFewTokens || w.n_cols % 64 != 0 || w.n_cols == 0 || w.n_rows % 4 != 0) return 0;
    const uint32_t bytes = few_token_bytes(w.n_cols, n_tokens);
    if (bytes <= kMaxTokenBytes) return 0;  // fits whole: matmul_few
    const uint32_t slices = (bytes + kMaxTokenBytes - 1) / kMaxTokenBytes;
    return slices <= 16 ? slices : 0;
}

cudaError_t matmul_few_sliced(cudaStream_t stream, const Mat& w, const void* packed, float* partial, uint32_t n_tokens) {
    const uint32_t slices = matmul_few_slices(w, n_tokens);
    if (slices == 0) return cudaErrorInvalidValue;
    FewParams p{};
    p.n_segments = 1;
    p.tiles[0] = static_cast<const uint8_t*>(w.tiles);
    p.y[0] = partial;
    p.seg_tiles[0] = (w.n_rows + 15) / 16;
    p.seg_rows[0] = w.n_rows;
    p.seg_stride[0] = w.n_rows;
    p.n_jobs = p.seg_tiles[0];
    p.n_blocks = w.n_cols / 32;
    p.packed = static_cast<const uint4*>(packed);
    p.token_groups = ((n_tokens + 15u) & ~15u) / 8;
    p.n_tokens = n_tokens;
    p.slice_pairs = (p.n_blocks / 2 + slices - 1) / slices;
    p.token_bytes = p.slice_pairs * p.token_groups * 1024;
    p.store = BC_STORE_OVERWRITE;
    if (p.n_jobs == 0) return cudaSuccess;
    return launch_few(stream, p, p.n_jobs, p.n_jobs);
}

cudaError_t matmul_few_swiglu(cudaStream_t stream, const Mat& gate, const Mat& up, const void* packed, float* y, uint32_t n_tokens, uint32_t y_stride,
                              void* packed_out) {
    if (gate.n_rows != up.n_rows || gate.n_cols != up.n_cols || (packed_out && gate.n_rows % 64 != 0)) return cudaErrorInvalidValue;
    FewParams p{};
    p.n_segments = 1;
    p.tiles[0] = static_cast<const uint8_t*>(gate.tiles);
    p.tiles[1] = static_cast<const uint8_t*>(up.tiles);
    p.y[0] = y;
    p.seg_tiles[0] = (gate.n_rows + 15) / 16;
    p.seg_rows[0] = gate.n_rows;
    p.seg_stride[0] = y_stride;
    p.n_jobs = p.seg_tiles[0];
    p.n_blocks = gate.n_cols / 32;
    p.packed = static_cast<const uint4*>(packed);
    p.token_groups = ((n_tokens + 15u) & ~15u) / 8;
    p.n_tokens = n_tokens;
    p.token_bytes = few_token_bytes(gate.n_cols, n_tokens);
    p.store = BC_STORE_OVERWRITE;
    p.packed_out = static_cast<__half*>(packed_out);
    p.dual = 1;
    if (p.n_jobs == 0) return cudaSuccess;
    return launch_few(stream, p, p.n_jobs, p.n_jobs);
}

bool matmul_few_experts_supported(const Mat& w, const Mat* up, uint32_t n_rows, uint32_t n_experts, uint32_t n_tokens) {
    return !few_disabled() && w.format == BC_Q4_0 && w.tiles != nullptr && n_tokens > 0 && n_tokens <= kMaxFewTokens && w.n_cols % 64 == 0 && w.n_cols > 0 &&
           (!up || up->tiles != nullptr) && n_rows % 16 == 0 && n_experts <= kMaxExperts;
}

cudaError_t matmul_few_experts(cudaStream_t stream, const Mat& w, const Mat* up, uint32_t n_rows, uint32_t n_experts, const void* packed,
                               const uint32_t* offsets, const uint32_t* entries, float* y, uint32_t n_tokens, uint32_t n_entries) {
    FewParams p{};
    p.n_segments = 1;
    p.tiles[0] = static_cast<const uint8_t*>(w.tiles);
    if (up) p.tiles[1] = static_cast<const uint8_t*>(up->tiles), p.dual = 1;
    p.y[0] = y;
    p.seg_tiles[0] = n_rows / 16;
    p.seg_rows[0] = n_rows;
    p.seg_stride[0] = n_rows;
    p.n_jobs = n_rows / 16;
    p.n_blocks = w.n_cols / 32;
    p.packed = static_cast<const uint4*>(packed);
    p.cap_groups = ((n_tokens + 15u) & ~15u) / 8;
    p.token_groups = n_experts * p.cap_groups;
    p.n_tokens = n_tokens;
    p.store = BC_STORE_OVERWRITE;
    p.offsets = offsets;
    p.entries = entries;
    p.n_experts = n_experts;
    if (p.n_jobs == 0 || n_experts == 0) return cudaSuccess;
    // Each entry makes at most one expert busy.
    const uint32_t most = p.n_jobs * n_experts, busy = n_entries < n_experts ? n_entries : n_experts;
    return launch_few(stream, p, most, p.n_jobs * (busy ? busy : 1));
}

}  // namespace k
}  // namespace bc
