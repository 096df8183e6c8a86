// The communicator handle behind bc_comm and the collectives the sharded passes record.
#pragma once

#include "backend.h"


// ncclUniqueId: 128 opaque bytes, passed by value.
struct NcclId {
    char bytes[BC_COMM_ID_BYTES];
};

struct bc_comm {
    bc_backend* backend = nullptr;
    void* nccl = nullptr;  // ncclComm_t; null in a world of one
    int rank = 0, world = 1;
    uint64_t collectives = 0;  // collectives recorded so far (NCCL calls and peer all-reduces)
    // Peer-memory all-reduce of the decode step: this rank's buffer, the peers' buffers mapped
    // through CUDA IPC, and the table the kernel receives. Absent (peer_ready false) when the
    // devices cannot map each other's memory or BOBCAT_NO_PEER_REDUCE=1; NCCL then serves alone.
    void* peer_local = nullptr;
    void* peer_mapped[bc::k::kMaxPeers] = {};
    bc::k::PeerBuffers peers{};
    bool peer_ready = false;
    uint64_t peer_reduces = 0;
};

namespace bc {

// In-place sum over ranks of `count` floats; every rank ends with the same bits.
bc_status comm_all_reduce_sum(bc_comm* c, float* data, size_t count);
// all[r * count_per_rank ...] = rank r's `mine`.
bc_status comm_all_gather(bc_comm* c, const float* mine, float* all, size_t count_per_rank);
bc_status comm_all_gather_words(bc_comm* c, const uint32_t* mine, uint32_t* all, size_t count_per_rank);
// y += sum over ranks of `partial` (count floats); `partial` may be overwritten. Small vectors go
// through the peer-memory kernel, larger ones through ncclAllReduce and an add.
bc_status comm_all_reduce_add(bc_comm* c, float* partial, float* y, size_t count);
// mine = sum over ranks of their all[rank * count_per_rank ...].
bc_status comm_reduce_scatter_sum(bc_comm* c, const float* all, float* mine, size_t count_per_rank);

}  // namespace bc
