"""Device-side sampling against a restatement of the reference's sampler
(crates/bobcat-cli/src/sampler.rs:45-112) with the same uniform draw. The random stream itself
is the host's; what is compared is the mapping (logits, settings, draw) -> token: exact for the
greedy pick, and for sampled picks at every draw that does not fall within rounding of a boundary
between two candidates, which also pins the distribution (a fine grid of draws covers the CDF)."""

import numpy as np
import pytest

from bobcat_b200 import Lfm2Cuda, Model, _lib, errors
from oracle import sampler as ref

pytestmark = pytest.mark.gpu


def settings(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0):
    return _lib.Sampling(temperature, top_k, top_p, min_p, repeat_penalty)


def gpu_sample(cuda, logits, recent, s, uniform):
    lb = cuda.buffer_from(logits)
    rb = cuda.buffer_from(np.asarray(recent, dtype=np.uint32)) if len(recent) else None
    ob = cuda.new_buffer(4)
    cuda.begin(); cuda.sample(lb, logits.size, rb, len(recent), s, uniform, ob); cuda.end()
    token = int(cuda.read(ob, np.zeros(1, dtype=np.uint32))[0])
    changed = cuda.read(lb, np.zeros_like(logits))
    return token, changed


def test_greedy_and_penalty_are_exact(cuda):
    rng = np.random.default_rng(1)
    logits = rng.standard_normal(70001).astype(np.float32)
    logits[[40000, 123]] = 9.0  # a tie: the lowest index wins
    token, changed = gpu_sample(cuda, logits, [], settings(), 0.3)
    assert token == 123 and np.array_equal(changed, logits)
    recent = [123, 5, 123, 40000, 7] + list(range(1000, 1100))  # only the last 64 count
    s = settings(repeat_penalty=1.3)
    token, changed = gpu_sample(cuda, logits, recent, s, 0.3)
    want = ref.penalised(logits, recent, 1.3)
    assert np.array_equal(changed, want)
    assert token == ref.sample(logits, recent, 0.3, 0.0, 0, 1.0, 0.0, 1.3)
    assert np.array_equal(want[[123, 40000]], logits[[123, 40000]])  # they fell out of the 64-token window


CASES = [
    dict(temperature=1.0),
    dict(temperature=0.7, top_k=40),
    dict(temperature=1.0, top_p=0.9),
    dict(temperature=0.8, top_k=50, top_p=0.95, min_p=0.05),
    dict(temperature=1.5, min_p=0.1),
    dict(temperature=0.6, top_k=5, repeat_penalty=1.2),
]


@pytest.mark.parametrize("case", CASES)
def test_sampled_tokens_follow_the_reference_cdf(cuda, case):
    rng = np.random.default_rng(7)
    n_vocab = 3000
    logits = (rng.standard_normal(n_vocab) * 2.5).astype(np.float32)
    recent = rng.integers(0, n_vocab, 30).tolist() + [int(np.argmax(logits))]
    full = dict(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0)
    full.update(case)
    order, probs = ref.candidates(logits, recent, **full)
    edges = np.cumsum(probs.astype(np.float64))
    s = settings(**full)
    checked = 0
    for uniform in np.linspace(0.0005, 0.9995, 160):
        if np.min(np.abs(edges - uniform)) < 2e-5:
            continue  # within rounding of a boundary: either neighbour is right
        token, _ = gpu_sample(cuda, logits, recent, s, float(uniform))
        assert token == ref.sample(logits, recent, float(uniform), **full), uniform
        assert token in set(order.tolist())
        checked += 1
    assert checked > 140


def test_equal_logits_are_told_apart_by_index(cuda):
    logits = np.full(1000, -3.0, dtype=np.float32)
    logits[[10, 500, 900]] = 2.0  # three equally likely candidates, nothing else survives min-p
    s = settings(temperature=1.0, min_p=0.5)
    picks = [gpu_sample(cuda, logits, [], s, u)[0] for u in (0.05, 0.3, 0.4, 0.6, 0.7, 0.95)]
    assert picks == [10, 10, 500, 500, 900, 900]


def test_sampling_arguments(cuda):
    b = cuda.new_buffer(4096)
    cuda.begin()
    with pytest.raises(errors.Argument):
        cuda.sample(b, 100, None, 0, settings(temperature=1.0), 1.0, b)   # the draw lies in [0, 1)
    with pytest.raises(errors.Argument):
        cuda.sample(b, 100, None, 0, settings(temperature=1.0, top_p=0.0), 0.5, b)
    with pytest.raises(errors.OutOfBounds):
        cuda.sample(b, 5000, None, 0, settings(), 0.5, b)
    cuda.discard()


def test_sequence_sampling_loop(model_path, cuda):
    """The engine's loop with the pick on the device: sample, step, sample ... A temperature of
    zero reproduces generate(); a sampled run stays inside the vocabulary and is a function of its draws."""
    model = Model.load(model_path("lfm2-small"))
    hp = model.hyperparameters()
    prompt = np.random.default_rng(3).integers(0, hp.n_vocab, 20).astype(np.uint32)
    seq = Lfm2Cuda(model, cuda, 64, True)
    seq.prefill(prompt)
    want = seq.generate(10).tolist()

    def run(s, draws):
        seq.reset()
        seq.prefill(prompt)
        out, logits = [], np.zeros(hp.n_vocab, dtype=np.float32)
        for u in draws:
            tok = seq.sample(s, float(u), recent=list(prompt) + out)
            out.append(tok)
            seq.step(tok, logits)
        return out

    assert run(settings(), [0.5] * 10) == want
    draws = np.random.default_rng(4).uniform(0, 1, 10)
    s = settings(temperature=1.0, top_k=20, top_p=0.9, repeat_penalty=1.1)
    a, b = run(s, draws), run(s, draws)
    assert a == b and all(0 <= t < hp.n_vocab for t in a)
