// Device helpers shared by the kernels: warp/block reductions, the shared-memory layout of an
// input vector, and the register-level Q4_0 unpack.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace bc {
namespace k {

constexpr int kWarpSize = 32;

// Programmatic dependent launch. `pdl_launch_dependents` lets the next launch of the stream begin
// while this grid still runs; `pdl_wait` blocks until every launch before this one has finished
// and its writes are visible. Both do nothing in a launch made without the attribute. A kernel
// launched with the attribute must call pdl_wait before it touches anything an earlier launch
// wrote or will read, which is what keeps a chain of such launches ordered.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the whole CTA; every thread receives the result. `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = lane < n_warps ? scratch[lane] : 0.f;
    return warp_sum(total);
}

// An input vector lives in shared memory as float4 chunks. Chunk c (elements 4c..4c+3) of 32-element
// block b sits at slot (b * 8) + ((c + b) & 7): rotating the eight chunks of a block by the block
// index lets 8 lanes that each own a different block read the same chunk number without bank
// conflicts, and lanes that walk consecutive chunks stay conflict-free too.
__device__ __forceinline__ int x_slot(int block, int chunk) { return (block << 3) | ((chunk + block) & 7); }

// The eight 4-bit quants of one 32-bit word of a Q4_0 block, minus 8, as floats: lo[i] is the low
// nibble of byte i (element 4k+i of the block for word k), hi[i] the high nibble (element
// 16+4k+i). The nibbles are masked in place into fp16 mantissas (0x6400 is 1024.0), so two
// quants convert per logic op and the subtraction is exact.
__device__ __forceinline__ void unpack_q4_word(uint32_t w, float (&lo)[4], float (&hi)[4]) {
    const uint32_t magic = 0x64006400u;
    uint32_t lo02 = (w & 0x000f000fu) | magic;   // 1024 + n        for bytes 0 and 2
    uint32_t hi02 = (w & 0x00f000f0u) | magic;   // 1024 + 16 n     for bytes 0 and 2
    uint32_t w8 = w >> 8;
    uint32_t lo13 = (w8 & 0x000f000fu) | magic;  // bytes 1 and 3
    uint32_t hi13 = (w8 & 0x00f000f0u) | magic;
    const __half2 bias_lo = __floats2half2_rn(1032.f, 1032.f);
    const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
    const __half2 bias_hi = __floats2half2_rn(-72.f, -72.f);  // (1024 + 16 n) / 16 - 72 = n - 8
    float2 a = __half22float2(__hsub2(*reinterpret_cast<__half2*>(&lo02), bias_lo));
    float2 b = __half22float2(__hsub2(*reinterpret_cast<__half2*>(&lo13), bias_lo));
    float2 c = __half22float2(__hfma2(*reinterpret_cast<__half2*>(&hi02), sixteenth, bias_hi));
    float2 d = __half22float2(__hfma2(*reinterpret_cast<__half2*>(&hi13), sixteenth, bias_hi));
    lo[0] = a.x; lo[2] = a.y; lo[1] = b.x; lo[3] = b.y;
    hi[0] = c.x; hi[2] = c.y; hi[1] = d.x; hi[3] = d.y;
}

// ---- formats kept in their GGUF byte layout on the device (rows of whole blocks, 2-byte aligned).
// Element `col` of a row, with the reference's arithmetic so the value is bit-identical to
// scalar::dequantize (crates/bobcat/src/scalar.rs:108-113 for Q8_0, :175-202 for Q6_K).
constexpr int kQ8_0BlockBytes = 34, kQ6KBlockBytes = 210;

__device__ __forceinline__ float half_at(const uint8_t* p) {
    return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(p)));
}

// Q8_0: an fp16 scale, then 32 int8 quants; value = f32(q) * d.
__device__ __forceinline__ float q8_0_at(const uint8_t* row, uint32_t col) {
    const uint8_t* block = row + (uint64_t)(col >> 5) * kQ8_0BlockBytes;
    return (float)(int)(signed char)block[2 + (col & 31)] * half_at(block);
}

// Q6_K: per super-block of 256, 128 bytes of low nibbles, 64 bytes of high bit pairs, 16 int8
// scales of 16-element blocks, then an fp16 d. Each half spreads 128 elements over 64 low bytes
// and 32 high bytes: element l + 32 k of a half (k = 0..3) takes the low nibble (k < 2) or high
// nibble (k >= 2) of low[l + 32 (k & 1)], bits 2k.. of high[l], and scale l / 16 + 2 k.
// value = (d * f32(scale)) * f32(q - 32).
__device__ __forceinline__ float q6k_at(const uint8_t* row, uint32_t col) {
    const uint8_t* block = row + (uint64_t)(col >> 8) * kQ6KBlockBytes;
    const uint32_t in_block = col & 255, half_index = in_block >> 7, e = in_block & 127, l = e & 31, k = e >> 5;
    const uint8_t* low = block + half_index * 64;
    const uint8_t* high = block + 128 + half_index * 32;
    const signed char* scales = reinterpret_cast<const signed char*>(block + 192 + half_index * 8);
    const uint8_t byte = low[l + 32 * (k & 1)];
    const uint32_t nibble = k < 2 ? (byte & 0xfu) : (byte >> 4);
    const uint32_t top = (high[l] >> (2 * k)) & 3u;
    const float d = half_at(block + 208);
    return (d * (float)(int)scales[(l >> 4) + 2 * k]) * (float)((int)(nibble | (top << 4)) - 32);
}

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float4 ldg_stream(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}

// The eight weights of Q4_0 quant word `w` (bytes 4t .. 4t + 3 of a block: weights 4t + e in the low
// nibbles, 16 + 4t + e in the high ones) times the block scale, as fp16: (e = 0, 2), (1, 3) of the low
// nibbles, then of the high ones. (q - 8) is exact in fp16 and the product is rounded once.
__device__ __forceinline__ uint4 dequant_word(uint32_t w, __half2 scale) {
    const uint32_t magic = 0x64006400u;  // half2(1024, 1024)
    uint32_t lo02 = (w & 0x000f000fu) | magic;
    uint32_t hi02 = (w & 0x00f000f0u) | magic;
    uint32_t w8 = w >> 8;
    uint32_t lo13 = (w8 & 0x000f000fu) | magic;
    uint32_t hi13 = (w8 & 0x00f000f0u) | magic;
    const __half2 bias_lo = __floats2half2_rn(1032.f, 1032.f);
    const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
    const __half2 bias_hi = __floats2half2_rn(-72.f, -72.f);  // (1024 + 16 q) / 16 - 72 = q - 8
    __half2 a = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&lo02), bias_lo), scale);
    __half2 b = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&lo13), bias_lo), scale);
    __half2 c = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&hi02), sixteenth, bias_hi), scale);
    __half2 d = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&hi13), sixteenth, bias_hi), scale);
    return make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b), *reinterpret_cast<uint32_t*>(&c),
                      *reinterpret_cast<uint32_t*>(&d));
}

// Where element (token, col) of a batch lies in the packed fp16 operand layout of the tensor-core
// prefill kernel (kernels_matmul_umma.cu), counted in halves: chunks of 64 columns, inside a chunk
// groups of 8 tokens, inside a group 8 core matrices of 8 tokens x 8 columns (16 bytes per token),
// with the columns of each block of 32 in the order the kernel's weight tiles use.
__device__ __forceinline__ uint64_t packed_operand_index(uint32_t token, uint32_t col, uint32_t token_groups) {
    const uint32_t chunk = col >> 6, c = col & 63, w = c & 31, e = w & 3;
    const uint32_t core = (c >> 5) * 4 + ((w & 15) >> 2), at = (w >> 4) * 4 + (e & 1) * 2 + (e >> 1);
    return ((((uint64_t)chunk * token_groups + (token >> 3)) * 8 + core) * 8 + (token & 7)) * 8 + at;
}

}  // namespace k
}  // namespace bc
