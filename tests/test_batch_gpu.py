"""Multi-sequence decode: several sequences of one model advance together, one token each per
pass. Every sequence must get the tokens it gets when it decodes alone (the single-sequence path
is itself held to the CPU parity checker in the other test files), whatever the other rows hold and
wherever they stand in their contexts."""

import numpy as np
import pytest

from bobcat_b200 import BatchCuda, Lfm2Cuda, Model, errors
from oracle import oracle

pytestmark = pytest.mark.gpu


def prompts_for(n_vocab, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, n_vocab, size=n).astype(np.uint32) for n in lengths]


def alone(model, cuda, n_ctx, kv_half, prompt, n_decode):
    seq = Lfm2Cuda(model, cuda, n_ctx, kv_half)
    seq.prefill(prompt)
    tokens = seq.generate(n_decode).tolist()
    seq.close()
    return tokens


# (model, sequences, kv_half): fewer than 16 rows run the f32 tile products, 16 and more the
# tensor-core products; the mixture-of-experts model routes every row separately.
CASES = [("lfm2-small", 5, False), ("lfm2-small", 5, True), ("lfm2-medium", 32, True), ("lfm2moe-tiny", 6, False), ("lfm2moe-tiny", 20, True)]


@pytest.mark.parametrize("case", CASES)
def test_batch_rows_equal_sequences_alone(model_path, cuda, case):
    config, n_seqs, kv_half = case
    model = Model.load(model_path(config))
    hp = model.hyperparameters()
    n_ctx, n_decode = 96, 24
    lengths = [7 + (5 * i) % 40 for i in range(n_seqs)]  # the rows stand at different positions
    prompts = prompts_for(hp.n_vocab, lengths, seed=n_seqs)
    batch = BatchCuda(model, cuda, n_seqs, n_ctx, kv_half)
    for i, prompt in enumerate(prompts):
        batch.seq(i).prefill(prompt)
    got = batch.generate(n_decode)
    assert batch.launches() > 0 and batch.last_gpu_seconds() > 0
    for i, prompt in enumerate(prompts):
        assert batch.seq(i).n_past() == len(prompt) + n_decode
        assert got[i].tolist() == alone(model, cuda, n_ctx, kv_half, prompt, n_decode), "sequence %d" % i
    # A second call continues every sequence where the first one stopped.
    more = batch.generate(8)
    for i in (0, n_seqs - 1):
        assert np.concatenate([got[i], more[i]]).tolist() == alone(model, cuda, n_ctx, kv_half, prompts[i], n_decode + 8)
    batch.close()


def test_batch_against_the_checker(model_path, cuda):
    """Rows of a batch against the CPU parity checker directly, not only against the GPU's own
    single-sequence path."""
    path = model_path("lfm2-small")
    model, ref = Model.load(path), oracle.Model(path)
    hp = model.hyperparameters()
    prompts = prompts_for(hp.n_vocab, [12, 30, 21], seed=3)
    batch = BatchCuda(model, cuda, 3, 64, kv_half=False)
    for i, prompt in enumerate(prompts):
        batch.seq(i).prefill(prompt)
    got = batch.generate(20)
    for i, prompt in enumerate(prompts):
        want, _ = oracle.greedy(ref, prompt, 20, n_ctx=64)
        assert got[i].tolist() == want
    batch.close()


def test_batch_validates_before_it_runs(model_path, cuda):
    model = Model.load(model_path("lfm2-small"))
    hp = model.hyperparameters()
    with pytest.raises(errors.Argument):
        BatchCuda(model, cuda, 0, 64, True)
    with pytest.raises(errors.Argument):
        BatchCuda(model, cuda, 40, 32, True)  # fewer positions than sequences
    batch = BatchCuda(model, cuda, 2, 32, True)
    batch.seq(0).prefill(prompts_for(hp.n_vocab, [10], 1)[0])
    with pytest.raises(errors.Argument):
        batch.generate(4)  # sequence 1 has no prompt
    batch.seq(1).prefill(prompts_for(hp.n_vocab, [30], 2)[0])
    with pytest.raises(errors.ContextFull):
        batch.generate(4)  # sequence 1 has 2 positions left
    assert batch.seq(0).n_past() == 10 and batch.seq(1).n_past() == 30
    assert batch.generate(2).shape == (2, 2)
    qwen = Model.load(model_path("qwen35-tiny"))
    with pytest.raises(errors.Unsupported):
        BatchCuda(qwen, cuda, 2, 32, True)
    batch.close()


def test_batch_of_32_on_the_moe_benchmark_shape(model_path, cuda):
    """32 sequences of the 8B-A1B shape (32 experts, 4 used). With f32 operands every row decodes
    as the sequence does alone. With the default half-precision operands (the arithmetic of the
    reference's batched products) the 5e-3-class differences of the activations flip a 4th-against-
    5th expert choice of this random-init router now and then, after which a row's tokens part from
    its single-sequence decode (the reference cut its own batched mixture-of-experts check short for
    the same reason, crates/bobcat/tests/lfm2_reference.rs:57-71): counted and recorded, not hidden."""
    import json
    import os

    model = Model.load(model_path("lfm2moe-8b-a1b"))
    hp = model.hyperparameters()
    n_seqs, n_ctx, n_decode = 32, 64, 16
    prompts = prompts_for(hp.n_vocab, [16 + i % 9 for i in range(n_seqs)], seed=11)
    want = [alone(model, cuda, n_ctx, True, prompt, n_decode) for prompt in prompts]
    same = {}
    for exact in (True, False):
        batch = BatchCuda(model, cuda, n_seqs, n_ctx, kv_half=True)
        batch.set_exact(exact)
        for i, prompt in enumerate(prompts):
            batch.seq(i).prefill(prompt)
        got = batch.generate(n_decode)
        same[exact] = sum(got[i].tolist() == want[i] for i in range(n_seqs))
        # The first token comes from the prefill's logits, the same on every path.
        assert all(int(got[i][0]) == want[i][0] for i in range(n_seqs))
        batch.close()
    path = os.environ.get("BOBCAT_MEASUREMENTS")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"test": "lfm2moe-8b-a1b 32 sequences vs alone, 16 tokens", "identical_f32_operands": same[True],
                                "identical_half_operands": same[False], "of": n_seqs}) + "\n")
    assert same[True] == n_seqs, "%d of %d sequences decode as they do alone with f32 operands" % (same[True], n_seqs)
    assert same[False] >= n_seqs // 4, "%d of %d sequences decode as they do alone with half-precision operands" % (same[False], n_seqs)
