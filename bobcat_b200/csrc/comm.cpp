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

#include <cstring>
#include <mutex>

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

}  // namespace

namespace bc {

bc_status comm_all_reduce_sum(bc_comm* c, float* data, size_t count) {
    if (!c || c->world == 1 || count == 0) return BC_OK;
    Nccl* lib = nullptr;
    BC_TRY(nccl_ready(&lib));
    c->collectives += 1;
    return nccl_check(lib, lib->AllReduce(data, data, count, kNcclFloat32, kNcclSum, c->nccl, c->backend->stream), "ncclAllReduce");
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
        if (lib->CommDestroy) lib->CommDestroy(comm->nccl);
    }
    delete comm;
}

int32_t bc_comm_rank(const bc_comm* comm) { return comm ? comm->rank : 0; }
int32_t bc_comm_world(const bc_comm* comm) { return comm ? comm->world : 1; }
uint64_t bc_comm_collectives(const bc_comm* comm) { return comm ? comm->collectives : 0; }

}  // extern "C"
