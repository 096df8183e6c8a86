// One-shot all-reduce over NVLink peer memory, for the small vectors of a tensor-parallel decode
// step (an output projection's partial result, n_embd floats): y += sum over ranks of partial.
//
// Every rank owns a buffer that its peers have mapped (CUDA IPC): per parity, one slot of floats per
// writing rank and one flag per writing rank, plus the rank's epoch counter. A call on rank r
//   1. adds one to its own epoch (every rank runs the same sequence of calls, so epochs agree),
//   2. stores its partial vector into slot [parity][r] of every rank's buffer (its own included)
//      with plain peer stores, makes them visible system-wide, and stores the epoch into flag
//      [parity][r] of every rank's buffer,
//   3. waits until all flags [parity][*] of its OWN buffer show the epoch (bounded: after the limit
//      it records an error code and goes on, so a missing peer cannot hang the GPU),
//   4. adds the slots in rank order to y - the same order on every rank, so every rank computes
//      the same bits.
// Parity = epoch & 1: a rank can be at most one call ahead of a peer (it needs the peer's flag of
// call k to finish call k), so the slots of call k + 1 never overwrite slots a peer still reads.
// Loads in step 3 and 4 touch only this GPU's memory; only the stores of step 2 cross NVLink. No
// multicast, no tensor-memory copies: plain st.global to peer addresses.
//
// The reference is single-GPU; this replaces ncclAllReduce + an add for vectors of up to
// kPeerSlotFloats floats. One CTA: the vector is a few thousand floats and the cost is latency.

#include "device_utils.cuh"
#include "kernels.h"

namespace bc {
namespace k {

namespace {

constexpr int kPeerThreads = 1024;
constexpr uint32_t kPeerSpinLimit = 1u << 21;  // polls of a local flag, each followed by a short sleep

__device__ int g_peer_error;

__global__ void __launch_bounds__(kPeerThreads) peer_all_reduce_add_kernel(PeerBuffers peers, const float* __restrict__ partial,
                                                                            float* __restrict__ y, uint32_t count) {
    __shared__ uint32_t epoch_shared;
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const uint32_t world = peers.world, rank = peers.rank;
    char* mine = static_cast<char*>(peers.base[rank]);
    uint32_t* epoch_word = reinterpret_cast<uint32_t*>(mine + peers.epoch_offset);
    if (tid == 0) {
        epoch_shared = *epoch_word + 1;
        *epoch_word = epoch_shared;
    }
    __syncthreads();
    const uint32_t epoch = epoch_shared, parity = epoch & 1u;
    const uint64_t slot_bytes = (uint64_t)peers.slot_floats * 4;
    // Step 2: this rank's partial into slot [parity][rank] of every rank.
    const uint32_t count4 = count / 4;
    const float4* p4 = reinterpret_cast<const float4*>(partial);
    for (uint32_t peer = 0; peer < world; ++peer) {
        float4* dst = reinterpret_cast<float4*>(static_cast<char*>(peers.base[peer]) + ((uint64_t)parity * world + rank) * slot_bytes);
        for (uint32_t i = tid; i < count4; i += kPeerThreads) dst[i] = p4[i];
        float* tail = reinterpret_cast<float*>(dst);
        for (uint32_t i = 4 * count4 + tid; i < count; i += kPeerThreads) tail[i] = partial[i];
    }
    __threadfence_system();
    __syncthreads();
    if ((uint32_t)tid < world) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(static_cast<char*>(peers.base[tid]) + peers.flags_offset) + parity * world + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
    }
    // Step 3: every rank's flag in this GPU's own buffer.
    if ((uint32_t)tid < world) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + peers.flags_offset) + parity * world + tid;
        bool seen = false;
        for (uint32_t spin = 0; spin < kPeerSpinLimit; ++spin) {
            uint32_t value;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(flag) : "memory");
            // A flag can only be at this epoch or, from a peer one call ahead on the other parity, untouched here.
            if (value == epoch) {
                seen = true;
                break;
            }
            __nanosleep(40);
        }
        if (!seen) atomicExch(&g_peer_error, 1 + tid);
    }
    __syncthreads();
    // Step 4: the slots in rank order.
    const char* slots = mine + (uint64_t)parity * world * slot_bytes;
    for (uint32_t i = tid; i < count4; i += kPeerThreads) {
        float4 sum = __ldcg(reinterpret_cast<const float4*>(slots) + i);
        for (uint32_t r = 1; r < world; ++r) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(slots + r * slot_bytes) + i);
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        float4 out = reinterpret_cast<float4*>(y)[i];
        out.x += sum.x; out.y += sum.y; out.z += sum.z; out.w += sum.w;
        reinterpret_cast<float4*>(y)[i] = out;
    }
    for (uint32_t i = 4 * count4 + tid; i < count; i += kPeerThreads) {
        float sum = __ldcg(reinterpret_cast<const float*>(slots) + i);
        for (uint32_t r = 1; r < world; ++r) sum += __ldcg(reinterpret_cast<const float*>(slots + r * slot_bytes) + i);
        y[i] += sum;
    }
}

}  // namespace

cudaError_t peer_all_reduce_add(cudaStream_t stream, const PeerBuffers& peers, const float* partial, float* y, uint32_t count) {
    if (count == 0) return cudaSuccess;
    if (count > peers.slot_floats || (reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(y)) % 16 != 0) return cudaErrorInvalidValue;
    PeerBuffers p = peers;
    void* args[] = {&p, &partial, &y, &count};
    return launch_kernel((const void*)peer_all_reduce_add_kernel, dim3(1), dim3(kPeerThreads), 0, stream, args);
}

int peer_error_flag() {
    int flag = 0;
    cudaMemcpyFromSymbol(&flag, g_peer_error, sizeof flag);
    if (flag) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_peer_error, &zero, sizeof zero);
    }
    return flag;
}

}  // namespace k
}  // namespace bc
