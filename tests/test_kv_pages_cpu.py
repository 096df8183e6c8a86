"""The page table of the paged KV cache as arithmetic, exhaustively on the host (no GPU): for
every element of a small cache, the flat index equals the reference's
layer * stride * kv_dim + pos * kv_dim + kv_head * head_dim + d
(crates/bobcat/src/lfm2_metal.rs:1064-1067), the (page, offset) pair names the same element of the
paged range, and no two elements share a place."""

import ctypes as C

import pytest

from bobcat_b200 import errors


def locate(lib, kv_dim, head_dim, page_positions, stride, layer, pos, kv_head, d):
    flat, page, offset = C.c_uint64(), C.c_uint32(), C.c_uint64()
    errors.check(lib.bc_kv_page_locate(kv_dim, head_dim, page_positions, stride, layer, pos, kv_head, d, C.byref(flat), C.byref(page), C.byref(offset)), lib)
    return int(flat.value), int(page.value), int(offset.value)


@pytest.mark.parametrize("shape", [(2, 4, 8, 24, 3), (1, 8, 4, 4, 2), (4, 2, 16, 64, 2)])
def test_every_element_has_the_reference_index_and_one_place(lib, shape):
    n_kv_heads, head_dim, page_positions, stride, n_layers = shape
    kv_dim = n_kv_heads * head_dim
    seen = set()
    for layer in range(n_layers):
        for pos in range(stride):
            for kv_head in range(n_kv_heads):
                for d in range(head_dim):
                    flat, page, offset = locate(lib, kv_dim, head_dim, page_positions, stride, layer, pos, kv_head, d)
                    assert flat == layer * stride * kv_dim + pos * kv_dim + kv_head * head_dim + d
                    # The paged range is the pages in order, so the place in it is the flat index.
                    assert page * page_positions * kv_dim + offset == flat
                    assert page == layer * (stride // page_positions) + pos // page_positions
                    assert 0 <= offset < page_positions * kv_dim
                    assert (page, offset) not in seen
                    seen.add((page, offset))
    assert len(seen) == n_layers * stride * kv_dim


def test_locate_rejects_what_lies_outside(lib):
    flat, page, offset = C.c_uint64(), C.c_uint32(), C.c_uint64()
    out = (C.byref(flat), C.byref(page), C.byref(offset))
    assert lib.bc_kv_page_locate(8, 4, 8, 24, 0, 24, 0, 0, *out) == errors.OutOfBounds.status   # position past the stride
    assert lib.bc_kv_page_locate(8, 4, 8, 24, 0, 0, 2, 0, *out) == errors.OutOfBounds.status    # no such head
    assert lib.bc_kv_page_locate(8, 4, 8, 24, 0, 0, 0, 4, *out) == errors.OutOfBounds.status    # no such element
    assert lib.bc_kv_page_locate(8, 4, 8, 20, 0, 0, 0, 0, *out) == errors.Argument.status       # stride not whole pages
    assert lib.bc_kv_page_locate(8, 3, 8, 24, 0, 0, 0, 0, *out) == errors.Argument.status       # rows not whole heads
