"""Which rank owns what in the sharded configurations, and the communicator handle.

Expert parallelism (``bc_batch_new_expert_parallel``): experts in contiguous ranges, sequences in
contiguous ranges; the gathered rows of a pass are ordered by rank, then by the rank's own
sequence order. Tensor parallelism (``bc_seq_new_tensor_parallel``): attention heads by KV head,
DeltaNet heads by key head (value head j reads key head j % n_k_heads,
crates/bobcat-metal/src/gdn.metal:244), feed-forward rows and vocabulary rows in contiguous ranges.
These functions are the host-side statement of the index rules the C++ side applies; the CPU tests
check them against a single-process computation over ``gloo``."""

from __future__ import annotations

import ctypes as C

from . import _lib, errors

COMM_ID_BYTES = 128


def expert_range(rank: int, world: int, n_experts: int) -> range:
    """The experts rank ``rank`` multiplies: ``n_experts / world`` consecutive ids."""
    if n_experts % world:
        raise ValueError("%d experts do not split over %d ranks" % (n_experts, world))
    per = n_experts // world
    return range(rank * per, (rank + 1) * per)


def expert_owner(expert: int, world: int, n_experts: int) -> int:
    return expert // (n_experts // world)


def gathered_row(rank: int, local_row: int, n_local: int) -> int:
    """Row of (rank, its sequence ``local_row``) among the rows every rank sees after the dispatch."""
    return rank * n_local + local_row


def row_owner(row: int, n_local: int) -> tuple[int, int]:
    """(rank, local row) of a gathered row: the rank whose combine receives its expert outputs."""
    return row // n_local, row % n_local


def split_range(rank: int, world: int, n: int, unit: int = 1) -> range:
    """Contiguous share of ``n`` items in multiples of ``unit`` (feed-forward rows in tiles of 16,
    vocabulary rows): the first ``n / unit % world`` ranks take one unit more."""
    units = n // unit
    base, extra = divmod(units, world)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return range(first * unit, (first + count) * unit)


def kv_heads_of(rank: int, world: int, n_kv_heads: int) -> list[int]:
    """KV heads of a rank. With more ranks than KV heads, ranks share a head (rank r reads head
    r * n_kv_heads // world) and split its query heads between them."""
    if world <= n_kv_heads:
        if n_kv_heads % world:
            raise ValueError("%d KV heads do not split over %d ranks" % (n_kv_heads, world))
        per = n_kv_heads // world
        return list(range(rank * per, (rank + 1) * per))
    if world % n_kv_heads:
        raise ValueError("%d ranks do not share %d KV heads evenly" % (world, n_kv_heads))
    return [rank * n_kv_heads // world]


def query_heads_of(rank: int, world: int, n_heads: int, n_kv_heads: int) -> list[int]:
    """Query heads of a rank: those of its KV heads (head h reads KV head h // group), or its share
    of one KV head's group when ranks share a head."""
    group = n_heads // n_kv_heads
    if world <= n_kv_heads:
        return [kv * group + g for kv in kv_heads_of(rank, world, n_kv_heads) for g in range(group)]
    sharers = world // n_kv_heads
    if group % sharers:
        raise ValueError("a group of %d query heads does not split over %d ranks" % (group, sharers))
    kv = kv_heads_of(rank, world, n_kv_heads)[0]
    per = group // sharers
    first = kv * group + (rank % sharers) * per
    return list(range(first, first + per))


def delta_heads_of(rank: int, world: int, n_k_heads: int, n_v_heads: int) -> tuple[list[int], list[int]]:
    """(key heads, value heads) of a rank: key heads in a contiguous range, and every value head
    that reads one of them, ordered so that local value head j reads local key head j % len(keys)."""
    if n_k_heads % world:
        raise ValueError("%d key heads do not split over %d ranks" % (n_k_heads, world))
    per = n_k_heads // world
    keys = list(range(rank * per, (rank + 1) * per))
    values = [k + rep * n_k_heads for rep in range(n_v_heads // n_k_heads) for k in keys]
    return keys, values


class Comm:
    """One rank of a NCCL communicator on a backend's device (``bc_comm``)."""

    def __init__(self, cuda, unique_id: bytes, rank: int, world: int):
        self._L = _lib.load()
        self.cuda, self.rank, self.world = cuda, rank, world
        if len(unique_id) != COMM_ID_BYTES:
            raise ValueError("the id holds %d bytes" % COMM_ID_BYTES)
        h = C.c_void_p()
        buf = (C.c_uint8 * COMM_ID_BYTES).from_buffer_copy(unique_id)
        errors.check(self._L.bc_comm_init(cuda._h, buf, COMM_ID_BYTES, rank, world, C.byref(h)), self._L)
        self._h = h

    @staticmethod
    def unique_id() -> bytes:
        L = _lib.load()
        buf = (C.c_uint8 * COMM_ID_BYTES)()
        errors.check(L.bc_comm_unique_id(buf, COMM_ID_BYTES), L)
        return bytes(buf)

    def collectives(self) -> int:
        return int(self._L.bc_comm_collectives(self._h))

    def peer_reduces(self) -> int:
        """Sums over ranks taken by the library's own NVLink peer-memory kernel rather than NCCL."""
        return int(self._L.bc_comm_peer_reduces(self._h))

    def close(self) -> None:
        if self._h:
            self._L.bc_comm_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
