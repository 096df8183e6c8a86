"""Mixture-of-experts kernels and the LFM2-MoE sequence path against the CPU parity checker. The
reference pins these ops only through whole-model dumps (crates/bobcat/tests/lfm2_reference.rs:
57-71); here each op is checked on its own as well."""

import numpy as np
import pytest

from bobcat_b200 import F32, Q4_0, Lfm2Cuda, Model, Norm, errors
from conftest import random_q4_0, rel_error
from oracle import oracle

pytestmark = pytest.mark.gpu


def silu(v):
    return v / (1 + np.exp(-v.astype(np.float64)))


@pytest.mark.parametrize("n_tokens,fused_norm", [(1, True), (1, False), (37, True), (130, False)])
def test_route_ids_are_bit_exact(cuda, n_tokens, fused_norm):
    """Expert ids must equal the reference's route() on the same input; weights to float rounding."""
    rng = np.random.default_rng(n_tokens)
    n_cols, n_experts, n_used = 256, 32, 4
    x = rng.standard_normal((n_tokens, n_cols)).astype(np.float32)
    nw = rng.uniform(0.5, 1.5, n_cols).astype(np.float32)
    router = (rng.standard_normal((n_experts, n_cols)) * 0.05).astype(np.float32)
    bias = (rng.standard_normal(n_experts) * 0.1).astype(np.float32)
    xb, nb, rb, bb = cuda.buffer_from(x), cuda.buffer_from(nw), cuda.buffer_from(router), cuda.buffer_from(bias)
    normed_b = cuda.new_buffer(x.nbytes)
    route_b = cuda.new_buffer(cuda.route_bytes(n_used, n_tokens))
    cuda.begin()
    cuda.moe_route(xb, (Norm(nb.at(0), 1e-5), normed_b.at(0)) if fused_norm else None, rb, bb, route_b, n_cols, n_experts, n_used, n_tokens)
    cuda.end()
    route = cuda.read(route_b, np.zeros((n_tokens, 2 * n_used), dtype=np.uint32))
    for t in range(n_tokens):
        xin = oracle.rms_norm(x[t], nw, 1e-5) if fused_norm else x[t]
        logits = oracle.matvec(0, router, xin, n_experts, threads=1)
        experts, scores = oracle.lfm2_route(logits, bias, n_used)
        assert route[t, :n_used].tolist() == experts[:n_used].tolist(), t
        weights = route[t, n_used:].view(np.float32)
        assert np.abs(weights - scores[experts[:n_used]]).max() < 1e-6
    if fused_norm:
        normed = cuda.read(normed_b, np.zeros_like(x))
        want = np.stack([oracle.rms_norm(r, nw, 1e-5) for r in x])
        assert rel_error(normed, want) < 1e-6


def test_route_ties_go_to_the_lower_expert_and_limits(cuda):
    n_cols, n_experts, n_used = 32, 8, 3
    x = np.ones((1, n_cols), dtype=np.float32)
    router = np.zeros((n_experts, n_cols), dtype=np.float32)
    router[[2, 5, 6]] = 0.25  # three equal best scores, then the rest tie at zero
    bias = np.zeros(n_experts, dtype=np.float32)
    xb, rb, bb = cuda.buffer_from(x), cuda.buffer_from(router), cuda.buffer_from(bias)
    route_b = cuda.new_buffer(cuda.route_bytes(n_used, 1))
    cuda.begin(); cuda.moe_route(xb, None, rb, bb, route_b, n_cols, n_experts, n_used, 1); cuda.end()
    assert cuda.read(route_b, np.zeros(2 * n_used, dtype=np.uint32))[:n_used].tolist() == [2, 5, 6]
    cuda.begin()
    with pytest.raises(errors.ExpertLimits):
        cuda.moe_route(xb, None, rb, bb, route_b, n_cols, n_experts, 9, 1)
    with pytest.raises(errors.ExpertLimits):
        cuda.moe_route(xb, None, rb, bb, route_b, n_cols, 200, 2, 1)
    cuda.discard()


def make_routes(rng, n_tokens, n_experts, n_used):
    route = np.zeros((n_tokens, 2 * n_used), dtype=np.uint32)
    for t in range(n_tokens):
        route[t, :n_used] = rng.choice(n_experts, size=n_used, replace=False)
        w = rng.uniform(0.1, 1.0, n_used).astype(np.float32)
        route[t, n_used:] = (w / w.sum()).astype(np.float32).view(np.uint32)
    return route


def test_group_is_a_stable_counting_sort(cuda):
    rng = np.random.default_rng(5)
    n_tokens, n_experts, n_used = 77, 16, 4
    route = make_routes(rng, n_tokens, n_experts, n_used)
    rb = cuda.buffer_from(route)
    ob, eb = cuda.new_buffer((n_experts + 1) * 4), cuda.new_buffer(n_tokens * n_used * 4)
    cuda.begin(); cuda.moe_group(rb, ob, eb, n_experts, n_used, n_tokens); cuda.end()
    offsets = cuda.read(ob, np.zeros(n_experts + 1, dtype=np.uint32))
    entries = cuda.read(eb, np.zeros(n_tokens * n_used, dtype=np.uint32))
    flat = route[:, :n_used].reshape(-1)
    want_entries = np.argsort(flat, kind="stable").astype(np.uint32)
    want_offsets = np.concatenate([[0], np.cumsum(np.bincount(flat, minlength=n_experts))]).astype(np.uint32)
    assert np.array_equal(offsets, want_offsets) and np.array_equal(entries, want_entries)


# (n_tokens, n_ff): widths that are multiples of 64 with at least 16 tokens send the grouped product to the
# tensor-core kernel (fp16 operands, like the reference's Q4_0 prefill kernel); the rest stay on the f32 tile kernel.
@pytest.mark.parametrize("n_tokens,n_ff,n_embd", [(1, 96, 128), (5, 96, 128), (70, 96, 128), (70, 128, 128), (300, 192, 128), (300, 256, 1024),
                                                     (16, 128, 128), (24, 192, 256), (32, 128, 1024), (32, 1792, 2048)])
def test_expert_paths_match_the_scalar_block(cuda, n_tokens, n_ff, n_embd):
    """Decode (per-token expert matvecs) and prefill (group, grouped matmul, combine) both equal
    lfm2.rs:413-440 computed with the checker's f64 matvec."""
    rng = np.random.default_rng(n_tokens + 11)
    n_experts, n_used = 8, 2
    prefill_tolerance = 5e-3 if n_tokens >= 16 else 1e-5
    gate_raw, up_raw = random_q4_0(rng, n_experts * n_ff, n_embd), random_q4_0(rng, n_experts * n_ff, n_embd)
    down_raw = random_q4_0(rng, n_experts * n_embd, n_ff)
    x = rng.uniform(-1, 1, (n_tokens, n_embd)).astype(np.float32)
    y0 = rng.uniform(-1, 1, (n_tokens, n_embd)).astype(np.float32)
    route = make_routes(rng, n_tokens, n_experts, n_used)
    gate = oracle.dequantize(2, gate_raw, gate_raw.shape[0] * n_embd).reshape(-1, n_embd).astype(np.float64)
    up = oracle.dequantize(2, up_raw, up_raw.shape[0] * n_embd).reshape(-1, n_embd).astype(np.float64)
    down = oracle.dequantize(2, down_raw, down_raw.shape[0] * n_ff).reshape(-1, n_ff).astype(np.float64)
    want = y0.astype(np.float64).copy()
    for t in range(n_tokens):
        for s in range(n_used):
            e, w = int(route[t, s]), float(route[t, n_used + s:n_used + s + 1].view(np.float32)[0])
            g, u = gate[e * n_ff:(e + 1) * n_ff] @ x[t], up[e * n_ff:(e + 1) * n_ff] @ x[t]
            want[t] += w * (down[e * n_embd:(e + 1) * n_embd] @ (silu(g.astype(np.float32)) * u).astype(np.float32))
    gb = cuda.upload_matrix(Q4_0, gate_raw, n_experts * n_ff, n_embd)
    ub = cuda.upload_matrix(Q4_0, up_raw, n_experts * n_ff, n_embd)
    db = cuda.upload_matrix(Q4_0, down_raw, n_experts * n_embd, n_ff)
    xb, rb = cuda.buffer_from(x), cuda.buffer_from(route)
    ffn = cuda.new_buffer(n_tokens * n_used * n_ff * 4)
    # Decode path.
    yb = cuda.buffer_from(y0)
    cuda.begin()
    cuda.matvec_experts_swiglu(Q4_0, gb, ub, n_ff, n_embd, n_experts, xb, rb, n_used, ffn, n_tokens)
    cuda.matvec_experts_down(Q4_0, db, n_embd, n_ff, n_experts, ffn, rb, n_used, yb, n_tokens)
    cuda.end()
    decode = cuda.read(yb, np.zeros_like(y0))
    assert rel_error(decode, want) < 1e-5
    # Prefill path.
    yb2 = cuda.buffer_from(y0)
    ob, eb = cuda.new_buffer((n_experts + 1) * 4), cuda.new_buffer(n_tokens * n_used * 4)
    eo = cuda.new_buffer(n_tokens * n_used * n_embd * 4)
    cuda.begin()
    cuda.moe_group(rb, ob, eb, n_experts, n_used, n_tokens)
    cuda.matmul_experts(Q4_0, gb, ub, n_ff, n_embd, n_experts, xb, True, ob, eb, n_used, ffn, n_tokens)
    cuda.matmul_experts(Q4_0, db, None, n_embd, n_ff, n_experts, ffn, False, ob, eb, n_used, eo, n_tokens)
    cuda.moe_combine(eo, rb, yb2, n_embd, n_used, n_tokens)
    cuda.end()
    prefill = cuda.read(yb2, np.zeros_like(y0))
    assert rel_error(prefill, want) < prefill_tolerance


@pytest.fixture(scope="module")
def moe_pair(model_path, cuda):
    path = model_path("lfm2moe-tiny")
    return Model.load(path), oracle.Model(path)


def test_moe_steps_match_layer_by_layer(moe_pair, cuda):
    model, ref = moe_pair
    hp = model.hyperparameters()
    tokens = np.random.default_rng(1).integers(0, hp.n_vocab, size=40).astype(np.uint32)
    seq = Lfm2Cuda(model, cuda, 64, kv_half=False)
    st = ref.state(64)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    for tok in tokens:
        trace = model.trace(1)
        seq.step(int(tok), logits, trace)
        want = st.step(int(tok), want_trace=True)
        for il in range(hp.n_layers):
            assert rel_error(trace.layers[il, 0], want["layers"][il]) < 1e-4, il
        assert rel_error(logits, want["logits"]) < 1e-4


def test_moe_prefill_and_greedy_match(moe_pair, cuda):
    model, ref = moe_pair
    hp = model.hyperparameters()
    tokens = np.random.default_rng(2).integers(0, hp.n_vocab, size=90).astype(np.uint32)
    want_tokens, want_logits = oracle.greedy(ref, tokens, 32, n_ctx=128)
    seq = Lfm2Cuda(model, cuda, 128, kv_half=False)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    seq.prefill(tokens, logits)
    assert rel_error(logits, want_logits) < 5e-3
    assert seq.generate(32).tolist() == want_tokens
    steps = Lfm2Cuda(model, cuda, 128, kv_half=False)
    step_logits = np.zeros_like(logits)
    for tok in tokens:
        steps.step(int(tok), step_logits)
    assert rel_error(logits, step_logits) < 5e-3


def test_moe_full_size_properties(model_path, cuda):
    """The 8B-A1B shape (32 experts, 4 used, 4.6 GB of weights), without the CPU checker: a batched
    prefill tracks single steps (loosely: a router near-tie that falls the other way for one token is a
    legitimate difference between the two paths, lfm2_reference.rs:57-71), a second pass reproduces
    the first bit for bit, and a checkpoint restores to the same continuation."""
    path = model_path("lfm2moe-8b-a1b")
    model = Model.load(path)
    hp = model.hyperparameters()
    tokens = np.random.default_rng(9).integers(0, hp.n_vocab, size=192).astype(np.uint32)
    seq = Lfm2Cuda(model, cuda, 256, kv_half=True)
    logits = np.zeros(hp.n_vocab, dtype=np.float32)
    seq.prefill(tokens, logits)
    ckpt = seq.checkpoint()
    batched = seq.generate(16).tolist()
    steps = Lfm2Cuda(model, cuda, 256, kv_half=True)
    step_logits = np.zeros_like(logits)
    for tok in tokens[:-1]:
        steps.step(int(tok))
    steps.step(int(tokens[-1]), step_logits)
    # Batched rows reach the router with fp16-class differences from the stepped rows, and of the
    # 4224 top-4-of-32 choices behind these logits a few percent are near-ties on random weights,
    # so the two paths legitimately part ways for some tokens; the check is loose on purpose. The
    # grouped products themselves are held to the scalar block in test_expert_paths_match_the_scalar_block.
    assert rel_error(logits, step_logits) < 0.5
    cosine = float(np.dot(logits, step_logits) / (np.linalg.norm(logits) * np.linalg.norm(step_logits)))
    assert cosine > 0.97
    seq.restore(ckpt)
    assert seq.generate(16).tolist() == batched
    seq.reset()
    again = np.zeros_like(logits)
    seq.prefill(tokens, again)
    assert np.array_equal(logits, again)
