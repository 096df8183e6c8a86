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
    uint64_t collectives = 0;  // collectives recorded so far
};

namespace bc {

// In-place sum over ranks of `count` floats; every rank ends with the same bits.
bc_status comm_all_reduce_sum(bc_comm* c, float* data, size_t count);
// all[r * count_per_rank ...] = rank r's `mine`.
bc_status comm_all_gather(bc_comm* c, const float* mine, float* all, size_t count_per_rank);
bc_status comm_all_gather_words(bc_comm* c, const uint32_t* mine, uint32_t* all, size_t count_per_rank);
// mine = sum over ranks of their all[rank * count_per_rank ...].
bc_status comm_reduce_scatter_sum(bc_comm* c, const float* all, float* mine, size_t count_per_rank);

}  // namespace bc
