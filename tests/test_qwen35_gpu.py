"""Qwen3.5 kernels against f64 arithmetic, in the shape of the reference's kernel tests
(crates/bobcat/tests/metal_gdn.rs:70-392), and the Qwen3.5 sequence path against the CPU parity
checker (crates/bobcat/tests/qwen35_reference.rs)."""

import numpy as np
import pytest

from bobcat_b200 import Model, Qwen35Cuda, errors
from conftest import rel_error
from oracle import oracle

pytestmark = pytest.mark.gpu
# metal_gdn.rs compares its kernels with f64 formulas at 1e-5.
GDN_TOLERANCE = 1e-5


def silu(v):
    return v / (1 + np.exp(-v))


def test_gdn_conv_carries_history_across_batches(cuda):
    rng = np.random.default_rng(1)
    conv_dim, kernel = 160, 4
    taps = rng.uniform(-1, 1, (conv_dim, kernel)).astype(np.float32)
    tb, hb = cuda.buffer_from(taps), cuda.buffer_from(np.zeros((conv_dim, kernel - 1), dtype=np.float32))
    past = np.zeros((conv_dim, kernel - 1))
    for n in (1, 2, 7, 1, 64, 3):
        x = rng.uniform(-1, 1, (n, conv_dim)).astype(np.float32)
        xb, ob = cuda.buffer_from(x), cuda.new_buffer(x.nbytes)
        cuda.begin(); cuda.gdn_conv(xb, tb, hb, ob, conv_dim, kernel, n); cuda.end()
        got = cuda.read(ob, np.zeros_like(x))
        want = np.zeros_like(x, dtype=np.float64)
        for t in range(n):
            s = taps[:, kernel - 1] * x[t].astype(np.float64) + (taps[:, :kernel - 1] * past).sum(axis=1)
            want[t] = silu(s)
            past = np.concatenate([past[:, 1:], x[t][:, None].astype(np.float64)], axis=1)
        assert np.abs(got - want).max() < GDN_TOLERANCE
        assert np.abs(cuda.read(hb, np.zeros((conv_dim, kernel - 1), dtype=np.float32)) - past).max() < 1e-6
    cuda.begin()
    with pytest.raises(errors.DeltaNetLimits):
        cuda.gdn_conv(xb, tb, hb, ob, conv_dim, 9, 1)
    cuda.discard()


def test_gdn_gates_including_the_linear_branch(cuda):
    n_v, n_tokens = 4, 3
    beta = np.array([[-2, 0, 1, 5]] * n_tokens, dtype=np.float32)
    alpha = np.array([[-3, 0.5, 19.5, 25.0], [30, -30, 1, 2], [0, 0, 0, 0]], dtype=np.float32)  # softplus switches at 20
    a = np.array([-0.5, -1.0, -0.01, -0.02], dtype=np.float32)
    dt = np.array([0.1, -0.1, 0.6, 0.0], dtype=np.float32)
    bb, ab, a_b, dt_b = cuda.buffer_from(beta), cuda.buffer_from(alpha), cuda.buffer_from(a), cuda.buffer_from(dt)
    cuda.begin(); cuda.gdn_gates(bb, ab, a_b, dt_b, n_v, n_tokens); cuda.end()
    v = alpha.astype(np.float64) + dt
    sp = np.where(v > 20, v, np.log1p(np.exp(np.minimum(v, 50))))
    assert np.abs(cuda.read(bb, np.zeros_like(beta)) - 1 / (1 + np.exp(-beta.astype(np.float64)))).max() < 1e-6
    assert np.abs(cuda.read(ab, np.zeros_like(alpha)) - np.exp(a * sp)).max() < 1e-6


def delta_rule_f64(qkv, beta, decay, state, n_k, n_v, kd, vd, normalize):
    """metal_gdn.rs:206-243 in f64: value head h reads key head h % n_k."""
    n = qkv.shape[0]
    key_dim = n_k * kd
    out = np.zeros((n, n_v * vd))
    for t in range(n):
        q, k, v = qkv[t, :key_dim].astype(np.float64), qkv[t, key_dim:2 * key_dim].astype(np.float64), qkv[t, 2 * key_dim:].astype(np.float64)
        for h in range(n_v):
            kh = h % n_k
            qh, kk = q[kh * kd:(kh + 1) * kd], k[kh * kd:(kh + 1) * kd]
            if normalize:
                qh = qh / np.sqrt((qh ** 2).sum() + 1e-6) / np.sqrt(kd)
                kk = kk / np.sqrt((kk ** 2).sum() + 1e-6)
            S = state[h] * decay[t, h]
            delta = (v[h * vd:(h + 1) * vd] - S.T @ kk) * beta[t, h]
            S = S + np.outer(kk, delta)
            state[h] = S
            out[t, h * vd:(h + 1) * vd] = S.T @ qh
    return out


@pytest.mark.parametrize("kd,vd", [(32, 32), (128, 128), (64, 96)])
def test_recurrence_carries_state(cuda, kd, vd):
    rng = np.random.default_rng(kd + vd)
    n_k, n_v = 2, 4
    conv_dim = 2 * n_k * kd + n_v * vd
    state = np.zeros((n_v, kd, vd))
    sb = cuda.buffer_from(state.astype(np.float32))
    for n in (1, 5, 1):
        qkv = rng.uniform(-1, 1, (n, conv_dim)).astype(np.float32)
        beta = rng.uniform(0.1, 0.9, (n, n_v)).astype(np.float32)
        decay = rng.uniform(0.8, 1.0, (n, n_v)).astype(np.float32)
        ob = cuda.new_buffer(n * n_v * vd * 4)
        qb, bb, db = cuda.buffer_from(qkv), cuda.buffer_from(beta), cuda.buffer_from(decay)
        cuda.begin()
        cuda.gdn_recurrence(qb, bb, db, sb, ob, n_k, n_v, kd, vd, n, normalize=True)
        cuda.end()
        want = delta_rule_f64(qkv, beta.astype(np.float64), decay.astype(np.float64), state, n_k, n_v, kd, vd, True)
        assert np.abs(cuda.read(ob, np.zeros((n, n_v * vd), dtype=np.float32)) - want).max() < GDN_TOLERANCE
        assert np.abs(cuda.read(sb, np.zeros((n_v, kd, vd), dtype=np.float32)) - state).max() < GDN_TOLERANCE
    cuda.begin()
    with pytest.raises(errors.DeltaNetLimits):
        cuda.gdn_recurrence(sb, sb, sb, sb, sb, 2, 3, 32, 32, 1)
    with pytest.raises(errors.DeltaNetLimits):
        cuda.gdn_recurrence(sb, sb, sb, sb, sb, 2, 4, 160, 32, 1)
    cuda.discard()


def test_gated_norm_and_attention_gate(cuda):
    rng = np.random.default_rng(3)
    rows, vd = 9, 128
    x = rng.standard_normal((rows, vd)).astype(np.float32)
    z = rng.standard_normal((rows, vd)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, vd).astype(np.float32)
    xb, zb, wb = cuda.buffer_from(x), cuda.buffer_from(z), cuda.buffer_from(w)
    cuda.begin(); cuda.gdn_gated_norm(xb, zb, wb, vd, rows, 1e-6); cuda.end()
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + 1e-6) * w * silu(z.astype(np.float64))
    assert np.abs(cuda.read(xb, np.zeros_like(x)) - want).max() < GDN_TOLERANCE
    n_tokens, n_heads, hd = 3, 4, 64
    out = rng.standard_normal((n_tokens, n_heads, hd)).astype(np.float32)
    q_gate = rng.standard_normal((n_tokens, n_heads, 2 * hd)).astype(np.float32)
    ob, gb = cuda.buffer_from(out), cuda.buffer_from(q_gate)
    cuda.begin(); cuda.attention_gate(ob, gb, n_heads, hd, n_tokens); cuda.end()
    want = out / (1 + np.exp(-q_gate[:, :, hd:].astype(np.float64)))
    assert np.abs(cuda.read(ob, np.zeros_like(out)) - want).max() < 1e-6


@pytest.fixture(scope="module")
def qwen_pair(model_path, cuda):
    path = model_path("qwen35-tiny")
    return Model.load(path), oracle.Model(path)


def test_qwen_steps_match_layer_by_layer(qwen_pair, cuda):
    model, ref = qwen_pair
    hp = model.hyperparameters()
    tokens = np.random.default_rng(1).integers(0, hp.n_vocab, size=70).astype(np.uint32)
    seq = Qwen35Cuda(model, cuda, 96, kv_half=False)
    st = ref.state(96)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    for tok in tokens:
        trace = model.trace(1)
        seq.step(int(tok), logits, trace)
        want = st.step(int(tok), want_trace=True)
        assert np.array_equal(trace.embedding[0], want["embedding"])
        for il in range(hp.n_layers):
            assert rel_error(trace.layers[il, 0], want["layers"][il]) < 1e-4, il
        assert rel_error(trace.final_norm[0], want["final_norm"]) < 1e-4
        assert rel_error(logits, want["logits"]) < 1e-4
    for layer in range(hp.n_delta_layers):
        assert rel_error(seq.read_state(3, layer), st.delta_state(layer)) < 1e-4
    conv = seq.read_state(0)
    want_conv = np.concatenate([st.conv_state(layer) for layer in range(hp.n_delta_layers)])
    assert rel_error(conv, want_conv) < 1e-4


@pytest.mark.parametrize("kv_half", [False, True])
def test_qwen_prefill_batches_match_steps_and_oracle(qwen_pair, cuda, kv_half):
    model, ref = qwen_pair
    hp = model.hyperparameters()
    tokens = np.random.default_rng(2).integers(0, hp.n_vocab, size=150).astype(np.uint32)
    want_tokens, want_logits = oracle.greedy(ref, tokens, 24, n_ctx=256)
    seq = Qwen35Cuda(model, cuda, 256, kv_half)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    final_norm = np.zeros(hp.n_embd, dtype=np.float32)
    # Two calls, so the second batch starts from carried conv history, DeltaNet state and KV rows.
    seq.prefill(tokens[:67])
    seq.prefill(tokens[67:], logits, final_norm=final_norm)
    assert rel_error(logits, want_logits) < 5e-3
    if not kv_half:
        assert seq.generate(24).tolist() == want_tokens
    steps = Qwen35Cuda(model, cuda, 256, kv_half)
    step_logits = np.zeros_like(logits)
    trace = model.trace(1)
    for tok in tokens:
        steps.step(int(tok), step_logits, trace)
    assert rel_error(logits, step_logits) < 5e-3
    assert rel_error(final_norm, trace.final_norm[0]) < 5e-3


def test_qwen_reset_and_restore(qwen_pair, cuda):
    model, _ = qwen_pair
    hp = model.hyperparameters()
    tokens = np.random.default_rng(4).integers(0, hp.n_vocab, size=20).astype(np.uint32)
    seq = Qwen35Cuda(model, cuda, 64, kv_half=True)
    first = np.zeros(hp.n_vocab, dtype=np.float32)
    seq.prefill(tokens, first)
    ckpt = seq.checkpoint()
    a = seq.generate(8)
    seq.restore(ckpt)
    assert seq.n_past() == 20 and seq.generate(8).tolist() == a.tolist()
    seq.reset()
    again = np.zeros_like(first)
    seq.prefill(tokens, again)
    assert np.array_equal(first, again)
    with pytest.raises(errors.Argument):
        seq.restore(ckpt)


def test_qwen_full_size_properties(model_path, cuda):
    """The Qwen3.5-2B shape (18 gated DeltaNet layers, 6 gated attention layers of 256-element
    heads, vocabulary 151936), without the CPU checker: batched prefill in two calls against single
    steps, a bit-identical second pass, a checkpoint that restores the DeltaNet state."""
    path = model_path("qwen35-2b")
    model = Model.load(path)
    hp = model.hyperparameters()
    tokens = np.random.default_rng(9).integers(0, hp.n_vocab, size=256).astype(np.uint32)
    seq = Qwen35Cuda(model, cuda, 320, kv_half=True)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    seq.prefill(tokens[:100])
    seq.prefill(tokens[100:], logits)
    ckpt = seq.checkpoint()
    batched = seq.generate(16).tolist()
    steps = Qwen35Cuda(model, cuda, 320, kv_half=True)
    step_logits = np.zeros_like(logits)
    for tok in tokens[:-1]:
        steps.step(int(tok))
    steps.step(int(tokens[-1]), step_logits)
    assert rel_error(logits, step_logits) < 5e-3
    seq.restore(ckpt)
    assert seq.generate(16).tolist() == batched
    seq.reset()
    again = np.zeros_like(logits)
    seq.prefill(tokens[:100])
    seq.prefill(tokens[100:], again)
    assert np.array_equal(logits, again)
