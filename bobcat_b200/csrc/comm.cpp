// The communicator of the sharded configurations: one rank per GPU, NCCL over NVLink / NVSwitch.
//
// The reference is single-GPU (crates/bobcat-metal/src/lib.rs:5-8); the sharded configurations
// (expert-parallel mixture of experts, tensor-parallel attention / DeltaNet / FFN) are additions of
// this library. NCCL is bound at run time (dlopen of libnccl.so.2, the library a PyTorch process
// already has loaded), so the shared library itself has no link-time dependency on it and
// single-GPU users never load it. All collectives run on the backend's stream, in order with the
// kernels around them; all data they move lies in this GPU's own memory on both ends of every call
// (NCCL does the peer transfers), and nothing here waits on a flag of its own.

#include "comm.h"

#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

using namespace bc;

namespace {

struct Nccl {
    void* handle = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*ReduceScatter)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    std::string error;
};

// ncclDataType_t / ncclRedOp_t values of the NCCL 2.x ABI.
constexpr int kNcclFloat32 = 7, kNcclUint32 = 3, kNcclSum = 0, kNcclMax = 2;

Nccl* nccl() {
    static Nccl lib;
    static std::once_flag once;
    std::call_once(once, [] {
        for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
            lib.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (lib.handle) break;
        }
        if (!lib.handle) {
            lib.error = dlerror() ? dlerror() : "libnccl.so.2 not found";
            return;
        }
        auto bind = [&](const char* symbol) {
            void* p = dlsym(lib.handle, symbol);
            if (!p && lib.error.empty()) lib.error = std::string("libnccl lacks ") + symbol;
            return p;
        };
        lib.GetUniqueId = reinterpret_cast<decltype(lib.GetUniqueId)>(bind("ncclGetUniqueId"));
        lib.CommInitRank = reinterpret_cast<decltype(lib.CommInitRank)>(bind("ncclCommInitRank"));
        lib.CommDestroy = reinterpret_cast<decltype(lib.CommDestroy)>(bind("ncclCommDestroy"));
        lib.GetErrorString = reinterpret_cast<decltype(lib.GetErrorString)>(bind("ncclGetErrorString"));
        lib.AllReduce = reinterpret_cast<decltype(lib.AllReduce)>(bind("ncclAllReduce"));
        lib.AllGather = reinterpret_cast<decltype(lib.AllGather)>(bind("ncclAllGather"));
        lib.ReduceScatter = reinterpret_cast<decltype(lib.ReduceScatter)>(bind("ncclReduceScatter"));
    });
    return &lib;
}

bc_status nccl_ready(Nccl** out) {
    Nccl* lib = nccl();
    if (!lib->handle || !lib->error.empty()) return fail(BC_ERR_UNSUPPORTED, "NCCL is not available: %s", lib->error.c_str());
    *out = lib;
    return BC_OK;
}

bc_status nccl_check(Nccl* lib, int result, const char* what) {
    if (result == 0) return BC_OK;
    return fail(BC_ERR_EXECUTION, "NCCL error in %s: %s", what, lib->GetErrorString ? lib->GetErrorString(result) : "unknown");
}

// Every rank allocates a buffer, the ranks exchange its IPC handle (an all-gather of 128 bytes per
// rank over the new communicator) and map each other's buffers.
void setup_peer_buffers(bc_comm* c, Nccl* lib) {
    const char* off = getenv("BOBCAT_NO_PEER_REDUCE");
    if ((off && off[0] == '1') || c->world > k::kMaxPeers) return;
    cudaStream_t stream = c->backend->stream;
    const uint64_t bytes = k::peer_buffer_bytes((uint32_t)c->world);
    // Every rank takes part in the exchange below whatever happened here, so the collective completes.
    // The zeroed flags and epoch must be in memory before any peer's first store: the exchange
    // below orders every rank's first launch after every rank's synchronize here.
    bool ok = cudaMalloc(&c->peer_local, bytes) == cudaSuccess && cudaMemset(c->peer_local, 0, bytes) == cudaSuccess &&
              cudaDeviceSynchronize() == cudaSuccess;
    cudaIpcMemHandle_t handle;
    std::memset(&handle, 0, sizeof handle);
    if (ok) ok = cudaIpcGetMemHandle(&handle, c->peer_local) == cudaSuccess;
    struct Entry {
        cudaIpcMemHandle_t handle;
        uint32_t ok;
        uint32_t pad[15];
    };
    static_assert(sizeof(Entry) == 128, "handle entry");
    Entry mine;
    std::memset(&mine, 0, sizeof mine);
    mine.handle = handle;
    mine.ok = ok ? 1 : 0;
    Entry* exchange = nullptr;
    if (cudaMalloc(&exchange, sizeof(Entry) * c->world) != cudaSuccess) return;
    cudaMemcpyAsync(exchange + c->rank, &mine, sizeof mine, cudaMemcpyHostToDevice, stream);
    int rc = lib->AllGather(exchange + c->rank, exchange, sizeof(Entry), /*ncclUint8*/ 1, c->nccl, stream);
    std::vector<Entry> all(c->world);
    bool gathered = rc == 0 && cudaMemcpyAsync(all.data(), exchange, sizeof(Entry) * c->world, cudaMemcpyDeviceToHost, stream) == cudaSuccess &&
                    cudaStreamSynchronize(stream) == cudaSuccess;
    cudaFree(exchange);
    if (!gathered) return;
    for (int r = 0; r < c->world; ++r) ok = ok && all[r].ok;
    if (!ok) return;  // every rank sees the same entries, so every rank decides the same
    bool mapped = true;
    for (int r = 0; r < c->world && mapped; ++r) {
        if (r == c->rank) {
            c->peer_mapped[r] = c->peer_local;
            continue;
        }
        mapped = cudaIpcOpenMemHandle(&c->peer_mapped[r], all[r].handle, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
        if (!mapped) c->peer_mapped[r] = nullptr;
    }
    // The ranks agree on whether everyone mapped everyone: a sum of successes over ranks.
    float* votes = nullptr;
    if (cudaMalloc(&votes, 4) != cudaSuccess) return;
    const float vote = mapped ? 1.f : 0.f;
    cudaMemcpyAsync(votes, &vote, 4, cudaMemcpyHostToDevice, stream);
    float total = 0.f;
    const bool voted = lib->AllReduce(votes, votes, 1, kNcclFloat32, kNcclSum, c->nccl, stream) == 0 &&
                       cudaMemcpyAsync(&total, votes, 4, cudaMemcpyDeviceToHost, stream) == cudaSuccess && cudaStreamSynchronize(stream) == cudaSuccess;
    cudaFree(votes);
    cudaGetLastError();  // a failed mapping must not linger as the thread's last error
    if (!voted || (int)total != c->world) return;
    c->peers.world = (uint32_t)c->world;
    c->peers.rank = (uint32_t)c->rank;
    c->peers.slot_floats = k::kPeerSlotFloats;
    c->peers.flags_offset = (uint64_t)2 * c->world * k::kPeerSlotFloats * 4;
    c->peers.epoch_offset = c->peers.flags_offset + (uint64_t)2 * c->world * 4;
    for (int r = 0; r < c->world; ++r) c->peers.base[r] = c->peer_mapped[r];
    c->peer_ready = true;
}

}  // namespace

namespace bc {

bc_status comm_all_reduce_sum(bc_comm* c, float* data, size_t count) {
    if (!c || c->world == 1 || count == 0) return BC_OK;
    Nccl* lib = nullptr;
    BC_TRY(nccl_ready(&lib));
    c->collectives += 1;
    return nccl_check(lib, lib->AllReduce(data, data, count, kNcclFloat32, kNcclSum, c->nccl, c->backend->stream), "ncclAllReduce");
}

bc_status comm_all_reduce_add(bc_comm* c, float* partial, float* y, size_t count) {
    if (!c || c->world == 1 || count == 0) {
        if (count && c) BC_CUDA(k::add_floats(c->backend->stream, y, partial, count));
        return BC_OK;
    }
    if (c->peer_ready && count <= k::kPeerSlotFloats && (reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(y)) % 16 == 0) {
        c->collectives += 1;
        c->peer_reduces += 1;
        cudaError_t e = k::peer_all_reduce_add(c->backend->stream, c->peers, partial, y, (uint32_t)count);
        if (e != cudaSuccess) return cuda_fail(e, "peer_all_reduce_add");
        return BC_OK;
    }
    BC_TRY(comm_all_reduce_sum(c, partial, count));
    BC_CUDA(k::add_floats(c->backend->stream, y, partial, count));
    return BC_OK;
}

bc_status comm_all_gather(bc_comm* c, const float* mine, float* all, size_t count_per_rank) {
    if (!c || c->world == 1) {
        if (mine != all && count_per_rank) BC_CUDA(cudaMemcpyAsync(all, mine, count_per_rank * 4, cudaMemcpyDeviceToDevice, c ? c->backend->stream : nullptr));
        return BC_OK;
    }
    Nccl* lib = nullptr;
    BC_TRY(nccl_ready(&lib));
    c->collectives += 1;
    return nccl_check(lib, lib->AllGather(mine, all, count_per_rank, kNcclFloat32, c->nccl, c->backend->stream), "ncclAllGather");
}

bc_status comm_reduce_scatter_sum(bc_comm* c, const float* all, float* mine, size_t count_per_rank) {
    if (!c || c->world == 1) {
        if (mine != all && count_per_rank) BC_CUDA(cudaMemcpyAsync(mine, all, count_per_rank * 4, cudaMemcpyDeviceToDevice, c ? c->backend->stream : nullptr));
        return BC_OK;
    }
    Nccl* lib = nullptr;
    BC_TRY(nccl_ready(&lib));
    c->collectives += 1;
    return nccl_check(lib, lib->ReduceScatter(all, mine, count_per_rank, kNcclFloat32, kNcclSum, c->nccl, c->backend->stream), "ncclReduceScatter");
}

bc_status comm_all_gather_words(bc_comm* c, const uint32_t* mine, uint32_t* all, size_t count_per_rank) {
    if (!c || c->world == 1) {
        if (mine != all && count_per_rank) BC_CUDA(cudaMemcpyAsync(all, mine, count_per_rank * 4, cudaMemcpyDeviceToDevice, c ? c->backend->stream : nullptr));
        return BC_OK;
    }
    Nccl* lib = nullptr;
    BC_TRY(nccl_ready(&lib));
    c->collectives += 1;
    return nccl_check(lib, lib->AllGather(mine, all, count_per_rank, kNcclUint32, c->nccl, c->backend->stream), "ncclAllGather");
}

}  // namespace bc

extern "C" {

bc_status bc_comm_unique_id(uint8_t* out, size_t len) {
    if (!out || len != BC_COMM_ID_BYTES) return fail(BC_ERR_ARGUMENT, "out must hold %d bytes", BC_COMM_ID_BYTES);
    Nccl* lib = nullptr;
    BC_TRY(nccl_ready(&lib));
    NcclId id;
    BC_TRY(nccl_check(lib, lib->GetUniqueId(&id), "ncclGetUniqueId"));
    std::memcpy(out, id.bytes, BC_COMM_ID_BYTES);
    return BC_OK;
}

bc_status bc_comm_init(bc_backend* backend, const uint8_t* id, size_t id_len, int32_t rank, int32_t world, bc_comm** out) {
    if (!backend || !id || !out) return fail(BC_ERR_ARGUMENT, "backend, id and out must be non-null");
    if (id_len != BC_COMM_ID_BYTES) return fail(BC_ERR_ARGUMENT, "the id holds %d bytes", BC_COMM_ID_BYTES);
    if (world < 1 || rank < 0 || rank >= world) return fail(BC_ERR_ARGUMENT, "rank %d outside a world of %d", rank, world);
    BC_TRY(backend->activate());
    std::unique_ptr<bc_comm> c(new bc_comm());
    c->backend = backend;
    c->rank = rank;
    c->world = world;
    if (world > 1) {
        Nccl* lib = nullptr;
        BC_TRY(nccl_ready(&lib));
        NcclId nid;
        std::memcpy(nid.bytes, id, BC_COMM_ID_BYTES);
        BC_TRY(nccl_check(lib, lib->CommInitRank(&c->nccl, world, nid, rank), "ncclCommInitRank"));
        // Failing to set up the peer buffers is not an error: NCCL then carries every collective.
        setup_peer_buffers(c.get(), lib);
    }
    *out = c.release();
    return BC_OK;
}

void bc_comm_free(bc_comm* comm) {
    if (!comm) return;
    if (comm->nccl) {
        Nccl* lib = nccl();
        if (comm->backend) {
            cudaSetDevice(comm->backend->device);
            cudaStreamSynchronize(comm->backend->stream);
        }
        // No rank unmaps or frees a buffer a peer may still write: meet first (a one-word sum).
        if (comm->peer_ready && lib->AllReduce) {
            float* word = nullptr;
            if (cudaMalloc(&word, 4) == cudaSuccess) {
                cudaMemsetAsync(word, 0, 4, comm->backend->stream);
                lib->AllReduce(word, word, 1, kNcclFloat32, kNcclSum, comm->nccl, comm->backend->stream);
                cudaStreamSynchronize(comm->backend->stream);
                cudaFree(word);
            }
        }
        for (int r = 0; r < comm->world && r < k::kMaxPeers; ++r)
            if (r != comm->rank && comm->peer_mapped[r]) cudaIpcCloseMemHandle(comm->peer_mapped[r]);
        if (comm->peer_local) cudaFree(comm->peer_local);
        if (lib->CommDestroy) lib->CommDestroy(comm->nccl);
    }
    delete comm;
}

int32_t bc_comm_rank(const bc_comm* comm) { return comm ? comm->rank : 0; }
int32_t bc_comm_world(const bc_comm* comm) { return comm ? comm->world : 1; }
uint64_t bc_comm_collectives(const bc_comm* comm) { return comm ? comm->collectives : 0; }
uint64_t bc_comm_peer_reduces(const bc_comm* comm) { return comm ? comm->peer_reduces : 0; }

}  // extern "C"
