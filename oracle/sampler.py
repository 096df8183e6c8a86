"""TEST INFRASTRUCTURE - NOT PRODUCT CODE.

A numpy restatement of the reference's token sampler, ``Sampler::sample``
(crates/bobcat-cli/src/sampler.rs:45-112), with the random draw passed in: repetition penalty,
top-k, top-p, min-p, temperature, then the walk over the sorted candidates. f32 arithmetic in the
reference's order; the sort is stable (the reference's is unstable, which only matters for equal
logits). Only the tests import this module."""

from __future__ import annotations

import numpy as np

REPEAT_LAST_N = 64  # sampler.rs:9-10


def _softmax(values: np.ndarray, temperature: float) -> np.ndarray:
    """sampler.rs:116-130: exp((v - max) / t), a running f32 sum, then the division."""
    e = np.exp((values - values.max()) / np.float32(temperature)).astype(np.float32)
    total = np.float32(0)
    for v in e:
        total = np.float32(total + v)
    return (e / total).astype(np.float32)


def penalised(logits: np.ndarray, recent, repeat_penalty: float) -> np.ndarray:
    out = np.array(logits, dtype=np.float32)
    if abs(repeat_penalty - 1.0) > np.finfo(np.float32).eps:
        for token in sorted(set(int(t) for t in list(recent)[-REPEAT_LAST_N:])):
            if token < out.size:
                out[token] = out[token] / np.float32(repeat_penalty) if out[token] > 0 else out[token] * np.float32(repeat_penalty)
    return out


def candidates(logits: np.ndarray, recent, temperature, top_k, top_p, min_p, repeat_penalty):
    """The (token ids, probabilities) the draw walks, in order; for temperature <= 0 the one pick."""
    logits = penalised(logits, recent, repeat_penalty)
    if temperature <= 0:
        return np.array([int(np.argmax(logits))]), np.array([1.0], dtype=np.float32)
    order = np.argsort(-logits, kind="stable")
    if 0 < top_k < logits.size:
        order = order[:top_k]
    probs = _softmax(logits[order], 1.0)
    cumulative, keep = np.float32(0), len(order)
    for i, p in enumerate(probs):
        cumulative = np.float32(cumulative + p)
        if cumulative >= np.float32(top_p):
            keep = i + 1
            break
    order, probs = order[:keep], probs[:keep]
    floor = probs[0] * np.float32(min_p)
    mask = probs >= floor
    order, probs = order[mask], probs[mask]
    return order, _softmax(np.log(probs).astype(np.float32), temperature)


def sample(logits, recent, uniform: float, temperature, top_k, top_p, min_p, repeat_penalty) -> int:
    order, probs = candidates(logits, recent, temperature, top_k, top_p, min_p, repeat_penalty)
    draw = np.float32(uniform)
    for token, p in zip(order, probs):
        if draw < p:
            return int(token)
        draw = np.float32(draw - p)
    return int(order[-1])
