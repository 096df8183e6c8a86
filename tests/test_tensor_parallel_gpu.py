"""Tensor-parallel Qwen3.5 on two GPUs against the one-GPU sequence: same logits to the rounding
of a sum taken in another order, same greedy tokens. Each rank is a child process with its own GPU;
the parent runs the one-GPU sequence. Skipped with fewer than two GPUs."""

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import rel_error

pytestmark = pytest.mark.gpu


def _rank_main(rank, world, unique_id, path, prompt, n_ctx, n_decode, kv_half, peer, out):
    import os
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ["BOBCAT_NO_PEER_REDUCE"] = "0" if peer else "1"
    from bobcat_b200 import Cuda, Model, Qwen35Cuda
    from bobcat_b200.sharding import Comm

    torch.cuda.set_device(rank)
    model = Model.load(path)
    hp = model.hyperparameters()
    cuda = Cuda.open(rank)
    comm = Comm(cuda, unique_id, rank, world)
    seq = Qwen35Cuda(model, cuda, n_ctx, kv_half, comm=comm)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    split = len(prompt) // 2
    # Half the prompt batched, the other half token by token: both paths end in sums over ranks.
    seq.prefill(prompt[:split], logits)
    step_logits = np.zeros_like(logits)
    for tok in prompt[split:]:
        seq.step(int(tok), step_logits)
    ckpt = seq.checkpoint()
    tokens = seq.generate(n_decode).tolist()
    seq.restore(ckpt)
    again = seq.generate(n_decode).tolist()
    out.put((rank, logits, step_logits, tokens, again, comm.collectives(), comm.peer_reduces()))
    seq.close()
    comm.close()
    cuda.close()


# The sums over ranks of the decode step by the library's own NVLink peer-memory kernel (peer) and
# by NCCL alone.
@pytest.mark.parametrize("peer", [True, False], ids=["peer", "nccl"])
@pytest.mark.parametrize("case", [("qwen35-tiny", False, 30, 20), ("qwen35-tiny", True, 30, 20), ("qwen35-2b", True, 24, 24)])
def test_two_ranks_decode_what_one_gpu_decodes(model_path, cuda, case, peer):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from bobcat_b200 import Model, Qwen35Cuda
    from bobcat_b200.sharding import Comm

    config, kv_half, n_prompt, n_decode = case
    path = model_path(config)
    model = Model.load(path)
    hp = model.hyperparameters()
    n_ctx = 64
    prompt = np.random.default_rng(31).integers(0, hp.n_vocab, size=n_prompt).astype(np.uint32)
    split = n_prompt // 2
    single = Qwen35Cuda(model, cuda, n_ctx, kv_half)
    want_logits = np.zeros(hp.n_vocab, dtype=np.float32)
    want_step = np.zeros_like(want_logits)
    single.prefill(prompt[:split], want_logits)
    for tok in prompt[split:]:
        single.step(int(tok), want_step)
    # The one-GPU sequence decodes step by step here, so that the logits behind every token are at
    # hand: where the ranks' tokens part from it, the logits say whether that was a tie.
    want_tokens, want_each = [], [want_step.copy()]
    for _ in range(n_decode):
        want_tokens.append(int(np.argmax(want_each[-1])))
        nxt = np.zeros_like(want_logits)
        single.step(want_tokens[-1], nxt)
        want_each.append(nxt)
    single.close()

    world = 2
    unique_id = Comm.unique_id()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, unique_id, path, prompt, n_ctx, n_decode, kv_half, peer, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted((out.get(timeout=600) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, logits, step_logits, tokens, again, collectives, peer_reduces in results:
        assert collectives > 0
        # Two GPUs of one machine can map each other's memory, so the peer kernel must have run
        # when it was allowed to, and must not have when it was switched off.
        assert (peer_reduces > 0) == peer, (rank, peer_reduces)
        # The batched half runs with half-precision operands on both sides (5e-3 class between two
        # tilings); the stepped half with f32 operands (1e-4, the single-step tolerance).
        assert rel_error(logits, want_logits) < 5e-3, rank
        assert rel_error(step_logits, want_step) < (5e-3 if kv_half else 1e-4), rank
        if tokens != want_tokens:
            # Sums over ranks associate differently, so a token may differ where the one-GPU logits
            # themselves hold a tie: two candidates closer than the agreement this test asks of the
            # logits (1e-4 of the largest logit with an f32 cache, 5e-3 with an f16 one). Anything
            # wider is a failure.
            i = next(j for j, (a, b) in enumerate(zip(tokens, want_tokens)) if a != b)
            gap = float(want_each[i][want_tokens[i]] - want_each[i][tokens[i]])
            scale = float(np.abs(want_each[i]).max())
            assert 0.0 <= gap <= (5e-3 if kv_half else 1e-4) * scale, "rank %d: token %d differs (%d against %d), logits %.3g apart of %.3g" % (
                rank, i, tokens[i], want_tokens[i], gap, scale)
        assert again == tokens, rank
    # Every rank holds the same logits bit for bit (the gathered vocabulary rows).
    assert np.array_equal(results[0][2], results[1][2])
