// Paged KV cache on the CUDA virtual memory management API (cuMemCreate / cuMemAddressReserve /
// cuMemMap), reached through cudaGetDriverEntryPoint so that the library links against the
// runtime only. See kv_pages.h.

#include "kv_pages.h"

#include <mutex>

using namespace bc;

namespace {

struct Driver {
    CUresult (*GetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*AddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*AddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*Create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*Release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*Unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    bool ok = false;
};

Driver* driver() {
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
        auto bind = [](const char* name, void** fn) {
            cudaDriverEntryPointQueryResult status;
            return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &status) == cudaSuccess && status == cudaDriverEntryPointSuccess && *fn;
        };
        d.ok = bind("cuMemGetAllocationGranularity", reinterpret_cast<void**>(&d.GetAllocationGranularity)) &&
               bind("cuMemAddressReserve", reinterpret_cast<void**>(&d.AddressReserve)) && bind("cuMemAddressFree", reinterpret_cast<void**>(&d.AddressFree)) &&
               bind("cuMemCreate", reinterpret_cast<void**>(&d.Create)) && bind("cuMemRelease", reinterpret_cast<void**>(&d.Release)) &&
               bind("cuMemMap", reinterpret_cast<void**>(&d.Map)) && bind("cuMemUnmap", reinterpret_cast<void**>(&d.Unmap)) &&
               bind("cuMemSetAccess", reinterpret_cast<void**>(&d.SetAccess));
    });
    return &d;
}

CUmemAllocationProp device_memory(int device) {
    CUmemAllocationProp prop = {};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    return prop;
}

bc_status driver_fail(CUresult r, const char* what) { return fail(BC_ERR_ALLOCATION, "%s failed with driver error %d", what, (int)r); }

bc_status new_page(int device, uint64_t bytes, std::shared_ptr<PhysicalPage>* out) {
    Driver* d = driver();
    CUmemAllocationProp prop = device_memory(device);
    auto page = std::make_shared<PhysicalPage>();
    page->device = device;
    CUresult r = d->Create(&page->handle, bytes, &prop, 0);
    if (r != CUDA_SUCCESS) {
        page->handle = 0;
        return driver_fail(r, "cuMemCreate");
    }
    *out = page;
    return BC_OK;
}

}  // namespace

namespace bc {

PhysicalPage::~PhysicalPage() {
    if (handle && driver()->ok) driver()->Release(handle);
}

uint32_t page_positions_for(int device, uint32_t kv_dim, uint32_t element_bytes) {
    Driver* d = driver();
    if (!d->ok || kv_dim == 0) return 0;
    CUmemAllocationProp prop = device_memory(device);
    size_t granularity = 0;
    if (d->GetAllocationGranularity(&granularity, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM) != CUDA_SUCCESS || granularity == 0) return 0;
    const uint64_t row = (uint64_t)kv_dim * element_bytes;
    if (granularity % row != 0) return 0;
    return (uint32_t)(granularity / row);
}

bc_status PagedCache::create(int device, const PageGeometry& geometry) {
    Driver* d = driver();
    if (!d->ok) return fail(BC_ERR_UNSUPPORTED, "the CUDA virtual memory management API is not available");
    device_ = device;
    geometry_ = geometry;
    const uint32_t slots = geometry.n_layers * geometry.pages_per_layer();
    reserved_ = (uint64_t)slots * geometry.page_bytes();
    CUresult r = d->AddressReserve(&base_, reserved_, geometry.page_bytes(), 0, 0);
    if (r != CUDA_SUCCESS) {
        base_ = 0;
        return driver_fail(r, "cuMemAddressReserve");
    }
    pages_.assign(slots, nullptr);
    for (uint32_t slot = 0; slot < slots; ++slot) {
        std::shared_ptr<PhysicalPage> page;
        BC_TRY(new_page(device, geometry.page_bytes(), &page));
        BC_TRY(map(slot, page));
    }
    return BC_OK;
}

bc_status PagedCache::map(uint32_t slot, const std::shared_ptr<PhysicalPage>& page) {
    Driver* d = driver();
    const uint64_t bytes = geometry_.page_bytes();
    const CUdeviceptr at = base_ + (uint64_t)slot * bytes;
    if (pages_[slot]) {
        CUresult r = d->Unmap(at, bytes);
        if (r != CUDA_SUCCESS) return driver_fail(r, "cuMemUnmap");
        pages_[slot].reset();
    }
    CUresult r = d->Map(at, bytes, 0, page->handle, 0);
    if (r != CUDA_SUCCESS) return driver_fail(r, "cuMemMap");
    CUmemAccessDesc access = {};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device_;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = d->SetAccess(at, bytes, &access, 1);
    if (r != CUDA_SUCCESS) return driver_fail(r, "cuMemSetAccess");
    pages_[slot] = page;
    return BC_OK;
}

bc_status PagedCache::share(uint32_t slot, const std::shared_ptr<PhysicalPage>& page) {
    if (slot >= pages_.size() || !page) return fail(BC_ERR_ARGUMENT, "no page slot %u", slot);
    if (pages_[slot] == page) return BC_OK;
    return map(slot, page);
}

bc_status PagedCache::make_private(uint32_t slot) {
    if (slot >= pages_.size()) return fail(BC_ERR_ARGUMENT, "no page slot %u", slot);
    if (pages_[slot] && pages_[slot].use_count() == 1) return BC_OK;
    std::shared_ptr<PhysicalPage> page;
    BC_TRY(new_page(device_, geometry_.page_bytes(), &page));
    return map(slot, page);
}

uint32_t PagedCache::shared_pages() const {
    uint32_t n = 0;
    for (const auto& p : pages_)
        if (p && p.use_count() > 1) ++n;
    return n;
}

PagedCache::~PagedCache() {
    Driver* d = driver();
    if (!base_ || !d->ok) return;
    cudaSetDevice(device_);
    const uint64_t bytes = geometry_.page_bytes();
    for (uint32_t slot = 0; slot < pages_.size(); ++slot)
        if (pages_[slot]) d->Unmap(base_ + (uint64_t)slot * bytes, bytes);
    pages_.clear();
    d->AddressFree(base_, reserved_);
}

}  // namespace bc

extern "C" {

// The rule of the paged cache as arithmetic: the reference's flat index of (layer, pos, kv_head, d)
// and the (page, offset) that holds it. Declared in bobcat_cuda.h.
bc_status bc_kv_page_locate(uint32_t kv_dim, uint32_t head_dim, uint32_t page_positions, uint32_t stride, uint32_t layer, uint32_t pos,
                            uint32_t kv_head, uint32_t d, uint64_t* flat_index, uint32_t* page, uint64_t* offset) {
    if (!flat_index || !page || !offset) return fail(BC_ERR_ARGUMENT, "the outputs must be non-null");
    if (kv_dim == 0 || head_dim == 0 || kv_dim % head_dim != 0 || page_positions == 0 || stride == 0 || stride % page_positions != 0)
        return fail(BC_ERR_ARGUMENT, "rows of whole heads and a layer stride of whole pages");
    if (pos >= stride || kv_head >= kv_dim / head_dim || d >= head_dim) return fail(BC_ERR_OUT_OF_BOUNDS, "the position, head or element lies outside the cache");
    PageGeometry g;
    g.kv_dim = kv_dim;
    g.page_positions = page_positions;
    g.stride = stride;
    *flat_index = g.flat_index(layer, pos, kv_head, d, head_dim);
    g.locate(layer, pos, kv_head, d, head_dim, page, offset);
    return BC_OK;
}

}  // extern "C"
