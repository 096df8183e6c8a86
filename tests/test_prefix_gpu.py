"""Paged KV caches and cached prefixes on the GPU. A paged sequence must give the bits a
contiguous one gives (the kernels index both the same way); a sequence that loads a cached prefix
must continue exactly as one that computed the prefix itself (reuse == no reuse, bit for bit), with
the prefix's full pages stored once however many sequences continue it."""

import numpy as np
import pytest

from bobcat_b200 import Lfm2Cuda, Model, Qwen35Cuda, errors

pytestmark = pytest.mark.gpu


def tokens_for(n_vocab, n, seed):
    return np.random.default_rng(seed).integers(0, n_vocab, size=n).astype(np.uint32)


@pytest.mark.parametrize("config", ["lfm2-small", "qwen35-tiny", "lfm2moe-tiny"])
@pytest.mark.parametrize("kv_half", [False, True])
def test_paged_equals_contiguous(model_path, cuda, config, kv_half):
    model = Model.load(model_path(config))
    hp = model.hyperparameters()
    prompt = tokens_for(hp.n_vocab, 70, 1)
    outs = []
    for paged in (False, True):
        seq = Lfm2Cuda(model, cuda, 128, kv_half, paged=paged)
        logits = np.zeros(hp.n_vocab, dtype=np.float32)
        seq.prefill(prompt[:50], logits)
        for tok in prompt[50:]:
            seq.step(int(tok), logits)
        outs.append((logits.copy(), seq.generate(24).tolist(), seq.kv_pages()))
        seq.close()
    assert np.array_equal(outs[0][0], outs[1][0]) and outs[0][1] == outs[1][1]
    assert outs[0][2] == (0, 0, 0)
    page_positions, pages, shared = outs[1][2]
    assert page_positions > 0 and pages == 2 * hp.n_attention_layers * -(-128 // page_positions) and shared == 0


@pytest.mark.parametrize("case", [("lfm2-tiny", False, False), ("lfm2-tiny", False, True), ("qwen35-tiny", True, True), ("qwen35-tiny", True, False)])
def test_prefix_reuse_equals_no_reuse(model_path, cuda, case):
    """One shared prefix prefilled in chunks and cached, then 8 requests that each append their own
    suffix and decode: every request equals the same request computed from scratch."""
    config, kv_half, paged = case
    model = Model.load(model_path(config))
    hp = model.hyperparameters()
    Seq = Qwen35Cuda if config.startswith("qwen") else Lfm2Cuda
    kv_dim = hp.n_kv_heads * hp.head_dim
    # Long enough to fill one whole page of every layer when paged (pages are the device's 2 MiB granules).
    page_positions = (2 << 20) // (kv_dim * (2 if kv_half else 4))
    n_prefix = page_positions + 37 if paged else 300
    n_suffix, n_decode, chunk = 23, 12, 512
    n_ctx = n_prefix + n_suffix + n_decode + 8
    prefix_tokens = tokens_for(hp.n_vocab, n_prefix, 2)
    suffixes = [tokens_for(hp.n_vocab, n_suffix, 10 + i) for i in range(8)]

    def prefill_in_chunks(seq, tokens, logits=None):
        for first in range(0, len(tokens), chunk):
            seq.prefill(tokens[first:first + chunk], logits if first + chunk >= len(tokens) else None)

    source = Seq(model, cuda, n_ctx, kv_half, paged=paged)
    prefill_in_chunks(source, prefix_tokens)
    prefix = source.save_prefix()
    assert prefix.n_past() == n_prefix
    source.close()  # the prefix outlives the sequence that computed it

    reused = []
    seqs = [Seq(model, cuda, n_ctx, kv_half, paged=paged) for _ in range(2)]
    for i, suffix in enumerate(suffixes):
        seq = seqs[i % 2]
        seq.load_prefix(prefix)
        assert seq.n_past() == n_prefix
        if paged:
            _, pages, shared = seq.kv_pages()
            assert shared == 2 * hp.n_attention_layers  # one full page per layer of K and of V, mapped not copied
        logits = np.zeros(hp.n_vocab, dtype=np.float32)
        seq.prefill(suffix, logits)
        reused.append((logits, seq.generate(n_decode).tolist()))
    # The same requests from scratch (same chunking, so the batched products see the same tiles).
    fresh = Seq(model, cuda, n_ctx, kv_half, paged=False)
    for i in (0, 3, 7):
        fresh.reset()
        prefill_in_chunks(fresh, prefix_tokens)
        logits = np.zeros(hp.n_vocab, dtype=np.float32)
        fresh.prefill(suffixes[i], logits)
        assert np.array_equal(logits, reused[i][0]), i
        assert fresh.generate(n_decode).tolist() == reused[i][1], i
    # A reset gives a sequence pages of its own again, and it still computes the same.
    seq = seqs[0]
    seq.reset()
    if paged:
        assert seq.kv_pages()[2] == 0
    prefill_in_chunks(seq, prefix_tokens)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    seq.prefill(suffixes[0], logits)
    assert np.array_equal(logits, reused[0][0])
    for s in seqs:
        s.close()
    fresh.close()
    prefix.close()


def test_prefix_checks(model_path, cuda):
    model = Model.load(model_path("lfm2-tiny"))
    other = Model.load(model_path("lfm2-small"))
    hp = model.hyperparameters()
    seq = Lfm2Cuda(model, cuda, 64, True)
    with pytest.raises(errors.Argument):
        seq.save_prefix()  # nothing to save yet
    seq.prefill(tokens_for(hp.n_vocab, 40, 3))
    prefix = seq.save_prefix()
    with pytest.raises(errors.Argument):
        Lfm2Cuda(other, cuda, 64, True).load_prefix(prefix)   # another model
    with pytest.raises(errors.Argument):
        Lfm2Cuda(model, cuda, 64, False).load_prefix(prefix)  # another cache type
    with pytest.raises(errors.ContextFull):
        Lfm2Cuda(model, cuda, 32, True).load_prefix(prefix)   # too short a context
    target = Lfm2Cuda(model, cuda, 64, True)
    target.load_prefix(prefix)
    assert target.generate(8).tolist() == seq.generate(8).tolist()
