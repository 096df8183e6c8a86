"""The index rules of the sharded configurations on two gloo ranks (no GPU): the expert-parallel
dispatch / combine reproduces the single-process mixture of experts bit for bit, and the
tensor-parallel head and row ranges cover every head and row exactly once with the DeltaNet
value-to-key-head rule intact."""

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bobcat_b200 import sharding


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


N_EXPERTS, N_USED, N_EMBD, N_LOCAL = 8, 2, 16, 3


def _expert(e: int, x: np.ndarray) -> np.ndarray:
    """A stand-in for an expert's SwiGLU block: any deterministic function of (expert, row)."""
    return np.tanh(x * np.float32(e + 1)) + np.float32(0.25 * e)


def _inputs(world: int):
    rng = np.random.default_rng(5)
    n = N_LOCAL * world
    rows = rng.standard_normal((n, N_EMBD)).astype(np.float32)
    ids = np.stack([rng.permutation(N_EXPERTS)[:N_USED] for _ in range(n)]).astype(np.int64)
    weights = rng.uniform(0.1, 1.0, (n, N_USED)).astype(np.float32)
    hidden = rng.standard_normal((n, N_EMBD)).astype(np.float32)
    return rows, ids, weights, hidden


def _single_process(world: int) -> np.ndarray:
    """crates/bobcat/src/lfm2.rs:426-439: block_out += w * expert(x), in picked order."""
    rows, ids, weights, hidden = _inputs(world)
    out = hidden.copy()
    for t in range(rows.shape[0]):
        block = np.zeros(N_EMBD, dtype=np.float32)
        for s in range(N_USED):
            block += weights[t, s] * _expert(int(ids[t, s]), rows[t])
        out[t] += block
    return out


def _rank_main(rank: int, world: int, port: int, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rows, ids, weights, hidden = _inputs(world)
    n = N_LOCAL * world
    # Dispatch: every rank contributes its own rows and ends with all of them, ordered by rank.
    mine = torch.from_numpy(rows[[sharding.gathered_row(rank, i, N_LOCAL) for i in range(N_LOCAL)]].copy())
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    everyone = torch.cat(gathered).numpy()
    assert np.array_equal(everyone, rows)
    # Each rank multiplies the entries of its own experts; the other output rows stay zero.
    local = sharding.expert_range(rank, world, N_EXPERTS)
    expert_out = np.zeros((n, N_USED, N_EMBD), dtype=np.float32)
    for t in range(n):
        for s in range(N_USED):
            if int(ids[t, s]) in local:
                assert sharding.expert_owner(int(ids[t, s]), world, N_EXPERTS) == rank
                expert_out[t, s] = _expert(int(ids[t, s]), everyone[t])
    # Combine: sum over ranks (one nonzero contributor per row), each rank keeps its own rows.
    total = torch.from_numpy(expert_out)
    dist.all_reduce(total)
    total = total.numpy()
    result = {}
    for i in range(N_LOCAL):
        t = sharding.gathered_row(rank, i, N_LOCAL)
        assert sharding.row_owner(t, N_LOCAL) == (rank, i)
        block = np.zeros(N_EMBD, dtype=np.float32)
        for s in range(N_USED):
            block += weights[t, s] * total[t, s]
        result[t] = hidden[t] + block
    out.put((rank, result))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_dispatch_and_combine_are_exact():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = _single_process(world)
    seen = set()
    for rank, rows in results.items():
        for t, value in rows.items():
            assert np.array_equal(value, want[t]), (rank, t)
            seen.add(t)
    assert seen == set(range(N_LOCAL * world))


def test_expert_ranges_partition_the_experts():
    for world in (1, 2, 4, 8):
        covered = [e for r in range(world) for e in sharding.expert_range(r, world, 32)]
        assert covered == list(range(32))
        assert all(sharding.expert_owner(e, world, 32) == r for r in range(world) for e in sharding.expert_range(r, world, 32))


def test_tensor_parallel_ranges():
    # Qwen3.5-9B: 16 query / 4 KV heads, 16 key / 32 value heads, FFN 12288, vocabulary 151936.
    for world in (1, 2, 4, 8):
        q = [h for r in range(world) for h in sharding.query_heads_of(r, world, 16, 4)]
        assert sorted(q) == list(range(16))
        for r in range(world):
            kv = sharding.kv_heads_of(r, world, 4)
            assert all(h // 4 in kv for h in sharding.query_heads_of(r, world, 16, 4))
        keys, values = [], []
        for r in range(world):
            k, v = sharding.delta_heads_of(r, world, 16, 32)
            keys += k
            values += v
            # Local value head j reads local key head j % len(k): that must be its global key head.
            assert all(k[j % len(k)] == v[j] % 16 for j in range(len(v)))
        assert sorted(keys) == list(range(16)) and sorted(values) == list(range(32))
        ff = [i for r in range(world) for i in sharding.split_range(r, world, 12288, 32)]
        assert ff == list(range(12288))
        vocab = [sharding.split_range(r, world, 151936, 16) for r in range(world)]
        assert sum(len(v) for v in vocab) == 151936 and all(len(v) % 16 == 0 for v in vocab)
