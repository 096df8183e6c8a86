"""Expert-parallel mixture of experts on two GPUs: every sequence must decode to the tokens the
one-GPU multi-sequence pass gives it. Each rank is a child process with its own GPU and a NCCL
communicator; the parent runs the one-GPU batch. Skipped with fewer than two GPUs."""

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

N_CTX, N_DECODE = 96, 20


def prompts_for(n_vocab, n_seqs):
    rng = np.random.default_rng(21)
    return [rng.integers(0, n_vocab, size=9 + (7 * i) % 30).astype(np.uint32) for i in range(n_seqs)]


def _rank_main(rank, world, unique_id, path, n_seqs, kv_half, out):
    import os
    # A rank that dies must not leave the others bound to an NVLink multicast object.
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from bobcat_b200 import BatchCuda, Cuda, Model
    from bobcat_b200.sharding import Comm, gathered_row

    torch.cuda.set_device(rank)
    model = Model.load(path)
    hp = model.hyperparameters()
    cuda = Cuda.open(rank)
    comm = Comm(cuda, unique_id, rank, world)
    n_local = n_seqs // world
    prompts = prompts_for(hp.n_vocab, n_seqs)
    batch = BatchCuda(model, cuda, n_local, N_CTX, kv_half, comm=comm)
    for i in range(n_local):
        batch.seq(i).prefill(prompts[gathered_row(rank, i, n_local)])
    tokens = batch.generate(N_DECODE)
    out.put((rank, tokens.tolist(), comm.collectives()))
    batch.close()
    comm.close()
    cuda.close()


@pytest.mark.parametrize("case", [("lfm2moe-tiny", 8, False), ("lfm2moe-tiny", 32, True)])
def test_two_ranks_decode_what_one_gpu_decodes(model_path, cuda, case):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from bobcat_b200 import BatchCuda, Model
    from bobcat_b200.sharding import Comm

    config, n_seqs, kv_half = case
    path = model_path(config)
    model = Model.load(path)
    hp = model.hyperparameters()
    prompts = prompts_for(hp.n_vocab, n_seqs)
    single = BatchCuda(model, cuda, n_seqs, N_CTX, kv_half)
    for i, prompt in enumerate(prompts):
        single.seq(i).prefill(prompt)
    want = single.generate(N_DECODE)
    single.close()

    world = 2
    unique_id = Comm.unique_id()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, unique_id, path, n_seqs, kv_half, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted((out.get(timeout=300) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    n_local = n_seqs // world
    moe_layers = sum(1 for _ in range(hp.n_layers)) - 1  # lfm2moe-tiny has one leading dense layer
    for rank, tokens, collectives in results:
        # Two collectives (dispatch, combine) per mixture-of-experts layer per pass.
        assert collectives == 2 * moe_layers * N_DECODE
        for i in range(n_local):
            assert tokens[i] == want[rank * n_local + i].tolist(), (rank, i)
