"""The token-level engine (crates/bobcat-cli/src/engine.rs:372-446, :510-647): requests reuse what
earlier requests left on the device without changing a single token, and score() gives the
log-probabilities a prompt-by-prompt computation gives."""

import numpy as np
import pytest

from bobcat_b200 import Engine, Lfm2Cuda, Model, _lib, errors
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small(model_path):
    path = model_path("lfm2-small")
    return Model.load(path), path


def fresh_reply(model, cuda, tokens, n):
    seq = Lfm2Cuda(model, cuda, 256, True)
    seq.prefill(np.asarray(tokens, dtype=np.uint32))
    out = seq.generate(n).tolist()
    seq.close()
    return out


def test_requests_reuse_the_device_state(small, cuda):
    model, _ = small
    hp = model.hyperparameters()
    rng = np.random.default_rng(1)
    first = rng.integers(0, hp.n_vocab, 40).tolist()
    engine = Engine(model, cuda, 256, True)
    # Request 1: nothing cached; the prompt up to its turn (token 30) becomes the history.
    reply1, cached = engine.generate(first, 12, turn=30)
    assert cached == 0 and reply1 == fresh_reply(model, cuda, first, 12)
    assert engine.consumed() == 40 + 11  # the last emitted token has not been stepped
    # Request 2 extends everything consumed so far (the usual next turn of a conversation).
    second = first + reply1[:11] + rng.integers(0, hp.n_vocab, 9).tolist()
    reply2, cached = engine.generate(second, 10, turn=len(second) - 4)
    assert cached == 51 and reply2 == fresh_reply(model, cuda, second, 10)
    # Request 3 regenerates the last reply: it shares only the history up to request 2's turn.
    third = second[: len(second) - 4] + rng.integers(0, hp.n_vocab, 6).tolist()
    reply3, cached = engine.generate(third, 10, turn=len(second) - 4)
    assert cached == len(second) - 4 and reply3 == fresh_reply(model, cuda, third, 10)
    # Request 4 shares nothing.
    other = rng.integers(0, hp.n_vocab, 25).tolist()
    reply4, cached = engine.generate(other, 8)
    assert cached == 0 and reply4 == fresh_reply(model, cuda, other, 8)
    # A caller that stops early still leaves a consistent state behind.
    seen = []
    reply5, _ = engine.generate(other + reply4[:7] + [5, 6], 20, emit=lambda t: (seen.append(t), len(seen) < 3)[1])
    assert reply5[:3] == seen[:3] and 3 <= len(reply5) <= 3 + 3  # steps already in flight still ran
    with pytest.raises(errors.ContextFull):
        engine.generate(list(range(256)), 4)
    engine.close()


def test_sampled_requests_pick_on_the_device(small, cuda):
    model, _ = small
    hp = model.hyperparameters()
    prompt = np.random.default_rng(2).integers(0, hp.n_vocab, 30).tolist()
    sampling = _lib.Sampling(0.8, 40, 0.95, 0.0, 1.1)
    a = Engine(model, cuda, 128, True, seed=7)
    b = Engine(model, cuda, 128, True, seed=7)
    c = Engine(model, cuda, 128, True, seed=8)
    ra, _ = a.generate(prompt, 16, sampling=sampling)
    rb, _ = b.generate(prompt, 16, sampling=sampling)
    rc, _ = c.generate(prompt, 16, sampling=sampling)
    assert ra == rb and len(ra) == 16 and all(0 <= t < hp.n_vocab for t in ra)
    assert ra != rc  # another stream of draws
    # A temperature of zero with a penalty is the penalised greedy pick.
    greedy, _ = a.generate(prompt, 6, sampling=_lib.Sampling(0.0, 0, 1.0, 0.0, 1.0))
    assert greedy == fresh_reply(model, cuda, prompt, 6)
    for e in (a, b, c):
        e.close()


def test_score_shares_the_common_prefix(small, cuda):
    model, path = small
    hp = model.hyperparameters()
    rng = np.random.default_rng(3)
    common = rng.integers(0, hp.n_vocab, 33).tolist()
    prompts = [common + rng.integers(0, hp.n_vocab, n).tolist() for n in (1, 5, 9)]
    labels = [rng.integers(0, hp.n_vocab, 3).tolist() for _ in prompts]
    engine = Engine(model, cuda, 128, False)
    got = engine.score(prompts, labels)
    ref = oracle.Model(path)
    for prompt, label, row in zip(prompts, labels, got):
        _, logits = oracle.greedy(ref, np.asarray(prompt, dtype=np.uint32), 0, n_ctx=128)
        logits = logits.astype(np.float64)
        log_sum = logits.max() + np.log(np.exp(logits - logits.max()).sum())
        assert np.allclose(row, logits[label] - log_sum, atol=5e-3)
    # Prompts with nothing in common still score, one by one.
    loose = engine.score([prompts[0], prompts[1][::-1]], [labels[0], labels[1]])
    assert np.allclose(loose[0], got[0], atol=5e-3)
    with pytest.raises(errors.Argument):
        engine.score([[]], [[1]])
    with pytest.raises(errors.Token):
        engine.score([[hp.n_vocab]], [[1]])
    engine.close()
