"""The multi-rank host logic of request replicas on two gloo ranks (no GPU): every request is served
exactly once, timing reduces to the slowest rank, and per-request results meet on every rank."""

import os
import socket

import torch.distributed as dist
import torch.multiprocessing as mp

from bobcat_b200 import replicas


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, n_requests: int, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = replicas.requests_of(rank, world, n_requests)
    hashes = {r: replicas.token_hash([replicas.prompt_seed(r), r * 7, 3]) for r in mine}
    slowest = replicas.max_over_ranks([1.0 + rank, 5.0 - rank])
    served = replicas.sum_over_ranks([len(mine)])
    everyone = replicas.gather_token_hashes(hashes, n_requests)
    out.put((rank, mine, slowest, served, everyone))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_partition_requests_and_reduce():
    world, n_requests = 2, 7
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, n_requests, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    served = sorted(r for _, mine, _, _, _ in results for r in mine)
    assert served == list(range(n_requests))
    want = [replicas.token_hash([replicas.prompt_seed(r), r * 7, 3]) & 0x7FFFFFFFFFFFFFFF for r in range(n_requests)]
    for rank, mine, slowest, count, everyone in results:
        assert mine == list(range(rank, n_requests, world))
        assert slowest == [2.0, 5.0]
        assert count == [n_requests]
        assert everyone == want


def test_single_rank_needs_no_process_group():
    assert replicas.requests_of(0, 1, 3) == [0, 1, 2]
    assert replicas.max_over_ranks([3.0]) == [3.0]
    assert replicas.token_hash([1, 2]) == (1 * 1000003 + 2)
