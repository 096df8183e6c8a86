"""Request replicas: the one way this path shards across GPUs without a data-path collective.

Every rank holds a full copy of the weights and serves its own share of the requests (the
reference serves requests one at a time on one GPU, crates/bobcat-cli/src/serve.rs:4-7; replicas
are N such servers). Ranks only meet to agree on timing and to collect results, through
``torch.distributed`` (NCCL on GPUs, gloo in CPU tests)."""

from __future__ import annotations

import torch
import torch.distributed as dist


def requests_of(rank: int, world: int, n_requests: int) -> list[int]:
    """Round-robin: request i goes to rank i % world."""
    if not (0 <= rank < world):
        raise ValueError("rank %d outside world of %d" % (rank, world))
    return list(range(rank, n_requests, world))


def prompt_seed(request: int, base: int = 1) -> int:
    """Each request has its own prompt seed, the same whichever rank serves it."""
    return base + request


def max_over_ranks(values: list[float], device: str | torch.device = "cpu") -> list[float]:
    """Per-value maximum over all ranks (the slowest rank sets the job's time)."""
    t = torch.tensor(values, dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def sum_over_ranks(values: list[int], device: str | torch.device = "cpu") -> list[int]:
    t = torch.tensor(values, dtype=torch.int64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [int(v) for v in t.tolist()]


def gather_token_hashes(local: dict[int, int], n_requests: int, device: str | torch.device = "cpu") -> list[int]:
    """Collect the token hash of every request (``local`` maps request -> hash) on every rank.
    A request's hash must not depend on which rank served it."""
    t = torch.zeros(n_requests, dtype=torch.int64, device=device)
    for request, value in local.items():
        t[request] = value & 0x7FFFFFFFFFFFFFFF
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [int(v) for v in t.tolist()]


def token_hash(tokens) -> int:
    """The reference benchmark's token hash, h = h * 1000003 + token (bobcat_bench.rs:230-232)."""
    h = 0
    for tok in tokens:
        h = (h * 1000003 + int(tok)) & 0xFFFFFFFFFFFFFFFF
    return h
