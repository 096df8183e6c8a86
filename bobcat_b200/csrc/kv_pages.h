// Paged KV cache: physical pages of device memory mapped into one contiguous virtual range per
// cache, so that the kernels keep the reference's flat index
//     layer * stride * kv_dim + pos * kv_dim + kv_head * head_dim + d
// (crates/bobcat/src/lfm2_metal.rs:1064-1067, with `stride` the positions between two layers) while
// the memory behind it comes in pages that can be shared between sequences. A page holds
// `page_positions` consecutive positions of one layer of one cache (K or V). Sequences that start
// from the same cached prefix map the same physical pages for the prefix's full pages and own
// private pages from there on, so a prefix is stored once however many requests continue it.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <vector>

#include "common.h"

namespace bc {

// The logical-to-physical rule, as plain arithmetic (also exported for the tests).
struct PageGeometry {
    uint32_t kv_dim = 0;          // n_kv_heads * head_dim
    uint32_t element_bytes = 2;   // 2 (f16) or 4 (f32)
    uint32_t page_positions = 0;  // positions per page
    uint32_t stride = 0;          // positions between two layers: n_ctx rounded up to whole pages
    uint32_t n_layers = 0;
    uint32_t pages_per_layer() const { return stride / page_positions; }
    uint64_t page_bytes() const { return (uint64_t)page_positions * kv_dim * element_bytes; }
    // The reference's flat element index of (layer, pos, kv_head, d).
    uint64_t flat_index(uint32_t layer, uint32_t pos, uint32_t kv_head, uint32_t d, uint32_t head_dim) const {
        return (uint64_t)layer * stride * kv_dim + (uint64_t)pos * kv_dim + (uint64_t)kv_head * head_dim + d;
    }
    // The page that holds it (numbered layer-major) and the element offset inside the page.
    void locate(uint32_t layer, uint32_t pos, uint32_t kv_head, uint32_t d, uint32_t head_dim, uint32_t* page, uint64_t* offset) const {
        *page = layer * pages_per_layer() + pos / page_positions;
        *offset = (uint64_t)(pos % page_positions) * kv_dim + (uint64_t)kv_head * head_dim + d;
    }
};

// One physical page (a cuMemCreate allocation of the device's granularity), released with its last owner.
struct PhysicalPage {
    CUmemGenericAllocationHandle handle = 0;
    int device = 0;
    ~PhysicalPage();
};

// A cache: a reserved virtual range with a physical page mapped at every page slot.
class PagedCache {
public:
    PagedCache() = default;
    PagedCache(const PagedCache&) = delete;
    PagedCache& operator=(const PagedCache&) = delete;
    ~PagedCache();

    // Reserve the range and map a fresh private page at every slot.
    bc_status create(int device, const PageGeometry& geometry);
    void* base() const { return reinterpret_cast<void*>(base_); }
    const PageGeometry& geometry() const { return geometry_; }
    const std::shared_ptr<PhysicalPage>& page(uint32_t slot) const { return pages_[slot]; }
    // Map `page` (another cache's, typically a prefix's) at `slot` in place of what is there.
    bc_status share(uint32_t slot, const std::shared_ptr<PhysicalPage>& page);
    // Give `slot` a fresh private page if the one there is shared with anyone else.
    bc_status make_private(uint32_t slot);
    // Pages of this cache that other owners also hold.
    uint32_t shared_pages() const;

private:
    bc_status map(uint32_t slot, const std::shared_ptr<PhysicalPage>& page);
    int device_ = 0;
    PageGeometry geometry_;
    CUdeviceptr base_ = 0;
    uint64_t reserved_ = 0;
    std::vector<std::shared_ptr<PhysicalPage>> pages_;
};

// Positions per page for rows of kv_dim elements on `device`, or 0 when rows do not divide the
// device's allocation granularity evenly.
uint32_t page_positions_for(int device, uint32_t kv_dim, uint32_t element_bytes);

}  // namespace bc
