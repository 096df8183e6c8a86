"""The LFM2 sequence API on the GPU against the CPU parity checker, in the shape of the
reference's model tests (crates/bobcat/tests/lfm2_reference.rs)."""

import numpy as np
import pytest

from bobcat_b200 import Lfm2Cuda, Model, errors
from conftest import rel_error
from oracle import oracle

pytestmark = pytest.mark.gpu

# Tolerances of the reference's own GPU-vs-dump tests (lfm2_reference.rs:19-25): f32 cache and
# single steps 1e-4; half cache or batched prefill 5e-3.
STEP_TOLERANCE = 1e-4
HALF_TOLERANCE = 5e-3


def prompt_tokens(n_vocab, n, seed=1):
    return np.random.default_rng(seed).integers(0, n_vocab, size=n).astype(np.uint32)


@pytest.fixture(scope="module", params=["lfm2-tiny", "lfm2-small"])
def pair(request, model_path, cuda):
    path = model_path(request.param)
    return Model.load(path), oracle.Model(path)


def test_steps_match_layer_by_layer(pair, cuda):
    model, ref = pair
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 70)  # crosses the 64-position attention chunk
    seq = Lfm2Cuda(model, cuda, 96, kv_half=False)
    st = ref.state(96)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    for tok in tokens:
        trace = model.trace(1)
        seq.step(int(tok), logits, trace)
        want = st.step(int(tok), want_trace=True)
        assert np.array_equal(trace.embedding[0], want["embedding"])
        for il in range(hp.n_layers):
            assert rel_error(trace.layers[il, 0], want["layers"][il]) < STEP_TOLERANCE, il
        assert rel_error(trace.final_norm[0], want["final_norm"]) < STEP_TOLERANCE
        assert rel_error(logits, want["logits"]) < STEP_TOLERANCE
    assert seq.n_past() == len(tokens)
    # Sequence state: conv history and KV cache rows equal the checker's.
    assert rel_error(seq.read_state(0), st.conv_state()) < STEP_TOLERANCE
    n = len(tokens) * hp.n_kv_heads * hp.head_dim
    for layer in range(hp.n_attention_layers):
        for which in (0, 1):
            assert rel_error(seq.read_state(1 + which, layer)[:n], st.kv(layer, which)[:n]) < STEP_TOLERANCE


@pytest.mark.parametrize("kv_half", [False, True])
def test_prefill_matches_steps_and_oracle(pair, cuda, kv_half):
    model, ref = pair
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 150, seed=2)
    seq = Lfm2Cuda(model, cuda, 256, kv_half)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    trace = model.trace(len(tokens))
    seq.prefill(tokens, logits, trace=trace)
    st = ref.state(256)
    tolerance = HALF_TOLERANCE
    for i, tok in enumerate(tokens):
        want = st.step(int(tok), want_logits=(i == len(tokens) - 1), want_trace=True)
        assert np.array_equal(trace.embedding[i], want["embedding"])
        assert rel_error(trace.layers[:, i], want["layers"]) < tolerance, i
        assert rel_error(trace.final_norm[i], want["final_norm"]) < tolerance
    assert rel_error(logits, want["logits"]) < tolerance
    # The same tokens one step at a time give the same logits (long_prefill_matches_steps).
    steps = Lfm2Cuda(model, cuda, 256, kv_half)
    step_logits = np.zeros_like(logits)
    for tok in tokens:
        steps.step(int(tok), step_logits)
    assert rel_error(logits, step_logits) < tolerance


def test_long_prefill_matches_steps(model_path, cuda):
    """512 tokens in two batched calls against 512 single steps, on a model wide enough that the
    prefill kernels' stage rings wrap many times (crates/bobcat/tests/lfm2_reference.rs:118-151),
    then the oracle on the last token's logits and a greedy continuation."""
    path = model_path("lfm2-medium")
    model = Model.load(path)
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 512, seed=5)
    seq = Lfm2Cuda(model, cuda, 640, kv_half=True)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    seq.prefill(tokens[:300])
    seq.prefill(tokens[300:], logits)
    steps = Lfm2Cuda(model, cuda, 640, kv_half=True)
    step_logits = np.zeros_like(logits)
    for tok in tokens:
        steps.step(int(tok), step_logits)
    assert rel_error(logits, step_logits) < HALF_TOLERANCE
    assert seq.generate(16).tolist() == steps.generate(16).tolist()
    # A second pass over the same prompt gives the same bits: nothing in the batched path depends on scheduling.
    again = np.zeros_like(logits)
    seq.reset()
    seq.prefill(tokens[:300])
    seq.prefill(tokens[300:], again)
    assert np.array_equal(logits, again)
    ref = oracle.Model(path, threads=8)
    st = ref.state(64)
    short = tokens[:40]
    for i, tok in enumerate(short):
        want = st.step(int(tok), want_logits=(i == len(short) - 1))
    check = Lfm2Cuda(model, cuda, 64, kv_half=False)
    got = np.zeros_like(logits)
    check.prefill(short, got)
    assert rel_error(got, want["logits"]) < HALF_TOLERANCE


def test_greedy_tokens_match(pair, cuda):
    model, ref = pair
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 40, seed=3)
    want, _ = oracle.greedy(ref, tokens, 64, n_ctx=128)
    seq = Lfm2Cuda(model, cuda, 128, kv_half=False)
    seq.prefill(tokens)
    assert seq.generate(64).tolist() == want
    assert seq.n_past() == 104


def test_quantised_embedding_matrix(model_path, cuda):
    """A file whose embedding / output matrix is Q8_0 (quantised checkpoints keep it quantised,
    lfm2_reference.rs:39) loads and decodes as the checker does."""
    path = model_path("lfm2-tiny-q8")
    model, ref = Model.load(path), oracle.Model(path)
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 30, seed=8)
    want, want_logits = oracle.greedy(ref, tokens, 24, n_ctx=64)
    seq = Lfm2Cuda(model, cuda, 64, kv_half=False)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    seq.prefill(tokens, logits)
    assert rel_error(logits, want_logits) < HALF_TOLERANCE
    assert seq.generate(24).tolist() == want
    steps = Lfm2Cuda(model, cuda, 64, kv_half=False)
    for tok in tokens:
        steps.step(int(tok), logits)
    assert rel_error(logits, want_logits) < STEP_TOLERANCE


def test_reset_matches_a_fresh_state(pair, cuda):
    model, _ = pair
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 20, seed=4)
    seq = Lfm2Cuda(model, cuda, 64, kv_half=True)
    first = np.zeros(hp.n_vocab, dtype=np.float32)
    seq.prefill(tokens, first)
    seq.generate(5)
    seq.reset()
    assert seq.n_past() == 0
    again = np.zeros_like(first)
    seq.prefill(tokens, again)
    assert np.array_equal(first, again)


def test_restore_continues_from_the_checkpoint(pair, cuda):
    model, _ = pair
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 30, seed=5)
    seq = Lfm2Cuda(model, cuda, 128, kv_half=True)
    seq.prefill(tokens)
    ckpt = seq.checkpoint()
    a = seq.generate(12)
    seq.restore(ckpt)
    assert seq.n_past() == 30
    b = seq.generate(12)
    assert a.tolist() == b.tolist()
    seq.restore(ckpt)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    seq.step(int(a[0]), logits)
    seq.reset()
    with pytest.raises(errors.Argument):
        seq.restore(ckpt)


def test_restore_rejects_another_sequences_checkpoint(pair, cuda):
    """A checkpoint carries the recurrent state only; the KV rows of its prefix stay in the cache
    of the sequence that took it (lfm2_metal.rs:250-288), so a second sequence of the same model
    must refuse it instead of decoding over rows it never wrote."""
    model, _ = pair
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 12, seed=6)
    a = Lfm2Cuda(model, cuda, 64, kv_half=True)
    b = Lfm2Cuda(model, cuda, 64, kv_half=True)
    a.prefill(tokens)
    b.prefill(tokens)
    ckpt = a.checkpoint()
    with pytest.raises(errors.Argument):
        b.restore(ckpt)
    assert b.n_past() == 12
    a.restore(ckpt)


def test_streaming_matches_generate(pair, cuda):
    model, _ = pair
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 16, seed=6)
    a = Lfm2Cuda(model, cuda, 64, kv_half=True)
    a.prefill(tokens)
    want = a.generate(10).tolist()
    b = Lfm2Cuda(model, cuda, 64, kv_half=True)
    b.prefill(tokens)
    emitted = []
    gained = b.generate_stream(10, lambda t: emitted.append(t) or True)
    assert emitted == want
    assert gained.tolist() == want[:9] and b.n_past() == 16 + 9
    # An early stop: the steps already submitted still run and are reported.
    c = Lfm2Cuda(model, cuda, 64, kv_half=True)
    c.prefill(tokens)
    seen = []
    gained = c.generate_stream(10, lambda t: seen.append(t) or len(seen) < 3)
    assert seen == want[:3]
    assert 2 <= len(gained) <= 2 + 3 and gained.tolist() == want[:len(gained)]
    assert c.n_past() == 16 + len(gained)


def test_greedy_selection_preserves_sequence_state(pair, cuda):
    model, _ = pair
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 8, seed=7)
    seq = Lfm2Cuda(model, cuda, 12, kv_half=False)
    with pytest.raises(errors.Argument):
        seq.greedy_token()
    seq.prefill(tokens)
    first = seq.greedy_token()
    assert seq.greedy_token() == first and seq.n_past() == 8
    rest = seq.generate_next(3)
    full = Lfm2Cuda(model, cuda, 12, kv_half=False)
    full.prefill(tokens)
    assert full.generate(4).tolist() == [first] + rest.tolist()
    assert seq.n_past() == 11
    # Context capacity.
    with pytest.raises(errors.ContextFull):
        seq.generate(2)
    seq.generate(1)
    with pytest.raises(errors.ContextFull):
        seq.step(0)


def test_argument_errors_come_before_device_work(pair, cuda):
    model, _ = pair
    hp = model.hyperparameters()
    seq = Lfm2Cuda(model, cuda, 8, kv_half=False)
    with pytest.raises(errors.Token):
        seq.step(hp.n_vocab)
    with pytest.raises(errors.Argument):
        seq.step(0, np.zeros(3, dtype=np.float32))
    with pytest.raises(errors.Argument):
        seq.prefill(np.zeros(0, dtype=np.uint32))
    with pytest.raises(errors.ContextFull):
        seq.prefill(np.zeros(9, dtype=np.uint32))
    with pytest.raises(errors.Token):
        seq.prefill(np.array([0, hp.n_vocab], dtype=np.uint32))
    with pytest.raises(errors.Argument):
        seq.prefill(np.zeros(2, dtype=np.uint32), trace=model.trace(3))
    with pytest.raises(errors.Argument):
        seq.generate(1)
    assert seq.n_past() == 0
    with pytest.raises(errors.Argument):
        Lfm2Cuda(model, cuda, 0, kv_half=False)


def test_full_size_properties(model_path, cuda):
    """The benchmark's own model (LFM2.5-2.6B shape, 1.9 GB of weights), where the CPU checker would
    take minutes per token: properties that do not need it. A 512-token batched prefill gives the
    logits of 512 single steps (lfm2_reference.rs:118-151); the greedy continuations agree; a reset
    and a second pass reproduce the first bit for bit; a checkpoint restores to the same
    continuation; a short prompt still matches the checker's logits."""
    path = model_path("lfm2-2.6b")
    model = Model.load(path)
    hp = model.hyperparameters()
    tokens = prompt_tokens(hp.n_vocab, 512, seed=9)
    seq = Lfm2Cuda(model, cuda, 640, kv_half=True)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    seq.prefill(tokens, logits)
    ckpt = seq.checkpoint()
    batched = seq.generate(32).tolist()
    steps = Lfm2Cuda(model, cuda, 640, kv_half=True)
    step_logits = np.zeros_like(logits)
    for tok in tokens[:-1]:
        steps.step(int(tok))
    steps.step(int(tokens[-1]), step_logits)
    assert rel_error(logits, step_logits) < HALF_TOLERANCE
    # The batched pick is the stepped pick, or ties with it inside the tolerance.
    scale = float(np.abs(step_logits).max())
    assert step_logits[int(np.argmax(logits))] >= step_logits.max() - HALF_TOLERANCE * scale
    seq.restore(ckpt)
    assert seq.generate(32).tolist() == batched
    seq.reset()
    again = np.zeros_like(logits)
    seq.prefill(tokens, again)
    assert np.array_equal(logits, again)
    assert seq.generate(32).tolist() == batched
    ref = oracle.Model(path, threads=16)
    st = ref.state(8)
    short = tokens[:3]
    for i, tok in enumerate(short):
        want = st.step(int(tok), want_logits=(i == len(short) - 1))
    check = Lfm2Cuda(model, cuda, 8, kv_half=False)
    got = np.zeros_like(logits)
    for tok in short:
        check.step(int(tok), got)
    assert rel_error(got, want["logits"]) < STEP_TOLERANCE
