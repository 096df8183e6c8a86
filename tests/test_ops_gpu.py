"""Every kernel against the CPU parity checker on the same seeded inputs, through the C ABI.
Shapes, generators and tolerances follow the reference's kernel tests
(crates/bobcat/tests/metal_matvec.rs, metal_matmul.rs, metal_attention.rs)."""

import numpy as np
import pytest

from bobcat_b200 import ACCUMULATE, F16, F32, OVERWRITE, Q4_0, SWIGLU, Norm, errors
from conftest import random_q4_0, rel_error
from oracle import oracle

pytestmark = pytest.mark.gpu

# (n_rows, n_cols): the reference's list (metal_matvec.rs:26-36) plus the decode shapes of the
# benchmark models.
MATVEC_SHAPES = [(1, 32), (7, 64), (2, 1024), (33, 96), (1000, 1024), (65536, 1024), (6144, 2048), (512, 2048), (2048, 10752), (10752, 2048)]
# Error allowed per unit of sum |w x| (metal_matvec.rs:19).
MATVEC_TOLERANCE = 1e-5


def make_matrix(rng, fmt, n_rows, n_cols):
    """Random matrix as (GGUF bytes, dequantised f32 values)."""
    if fmt == Q4_0:
        raw = random_q4_0(rng, n_rows, n_cols)
        return raw, oracle.dequantize(2, raw, n_rows * n_cols).reshape(n_rows, n_cols)
    scale = 2.0 ** -7
    values = (rng.standard_normal((n_rows, n_cols)) * scale).astype(np.float32)
    if fmt == F16:
        half = values.astype(np.float16)
        return half.view(np.uint8).reshape(n_rows, -1), half.astype(np.float32)
    return values.view(np.uint8).reshape(n_rows, -1), values


def scaled_error(got, want, w, x):
    budget = np.abs(w.astype(np.float64)) @ np.abs(x.astype(np.float64))
    return float((np.abs(got.astype(np.float64) - want.astype(np.float64)) / np.maximum(budget, 1e-30)).max())


@pytest.mark.parametrize("fmt", [Q4_0, F32, F16])
@pytest.mark.parametrize("shape", MATVEC_SHAPES)
def test_matvec_modes(cuda, fmt, shape):
    n_rows, n_cols = shape
    if fmt != Q4_0 and n_rows * n_cols > 2 ** 25:
        pytest.skip("large float matrices add nothing over Q4_0 here")
    rng = np.random.default_rng(n_rows * 131 + n_cols + fmt)
    raw, w = make_matrix(rng, fmt, n_rows, n_cols)
    x = rng.uniform(-1, 1, n_cols).astype(np.float32)
    nw = rng.uniform(0.5, 1.5, n_cols).astype(np.float32)
    y0 = rng.uniform(-1, 1, n_rows).astype(np.float32)
    type_id = {Q4_0: 2, F32: 0, F16: 1}[fmt]
    wb = cuda.upload_matrix(fmt, raw, n_rows, n_cols)
    xb, nb, yb = cuda.buffer_from(x), cuda.buffer_from(nw), cuda.buffer_from(y0)
    plain = oracle.matvec(type_id, raw, x, n_rows)
    normed_x = oracle.rms_norm(x, nw, 1e-5)
    normed = oracle.matvec(type_id, raw, normed_x, n_rows)
    out = np.zeros(n_rows, dtype=np.float32)

    cuda.begin(); cuda.matvec(fmt, wb, n_rows, n_cols, xb, yb); cuda.end()
    assert scaled_error(cuda.read(yb, out), plain, w, x) < MATVEC_TOLERANCE
    cuda.begin(); cuda.matvec(fmt, wb, n_rows, n_cols, xb, yb, norm=Norm(nb.at(0), 1e-5)); cuda.end()
    assert scaled_error(cuda.read(yb, out), normed, w, normed_x) < MATVEC_TOLERANCE
    cuda.write(yb, y0)
    cuda.begin(); cuda.matvec(fmt, wb, n_rows, n_cols, xb, yb, accumulate=True); cuda.end()
    assert scaled_error(cuda.read(yb, out), y0 + plain, w, x) < MATVEC_TOLERANCE

    if n_rows % 2 == 0:
        half = n_rows // 2
        row_bytes = raw.shape[1]
        cuda.begin()
        cuda.matvec_swiglu(fmt, wb.at(0), wb.at(half * row_bytes), half, n_cols, xb, Norm(nb.at(0), 1e-5), yb)
        cuda.end()
        got = cuda.read(yb, np.zeros(half, dtype=np.float32))
        gate, up = normed[:half], normed[half:]
        want = np.array([oracle.silu(float(g)) for g in gate], dtype=np.float32) * up
        # silu is 1-Lipschitz-ish, so the product's error scales with both budgets.
        budget = np.abs(w.astype(np.float64)) @ np.abs(normed_x.astype(np.float64))
        err = np.abs(got.astype(np.float64) - want) / np.maximum(budget[:half] * (np.abs(up) + 1) + budget[half:] * (np.abs(gate) + 1), 1e-30)
        assert float(err.max()) < MATVEC_TOLERANCE
    for b in (wb, xb, nb, yb):
        b.free()


def test_matvec_rejects_bad_ranges(cuda):
    rng = np.random.default_rng(0)
    raw, _ = make_matrix(rng, Q4_0, 8, 64)
    wb = cuda.upload_matrix(Q4_0, raw, 8, 64)
    xb, yb = cuda.new_buffer(64 * 4), cuda.new_buffer(8 * 4)
    with pytest.raises(errors.NotRecording):
        cuda.matvec(Q4_0, wb, 8, 64, xb, yb)
    cuda.begin()
    with pytest.raises(errors.OutOfBounds):
        cuda.matvec(Q4_0, wb, 9, 64, xb, yb)
    with pytest.raises(errors.OutOfBounds):
        cuda.matvec(Q4_0, wb, 8, 64, xb.at(4), yb)
    with pytest.raises(errors.AlreadyRecording):
        cuda.begin()
    with pytest.raises(errors.Busy):
        cuda.read(yb, np.zeros(8, dtype=np.float32))
    cuda.discard()
    from bobcat_b200 import Cuda
    other = Cuda.open(0)
    foreign = other.new_buffer(64 * 4)
    cuda.begin()
    with pytest.raises(errors.ForeignBuffer):
        cuda.matvec(Q4_0, wb, 8, 64, foreign, yb)
    cuda.discard()
    foreign.free()
    other.close()


@pytest.mark.parametrize("shape", [(1, 32), (7, 64), (1000, 1024), (4096, 2048)])
def test_expand_is_bit_exact(cuda, shape):
    """Dequantisation must equal scalar::dequantize bit for bit (f32), and round once to half."""
    n_rows, n_cols = shape
    rng = np.random.default_rng(n_rows + n_cols)
    raw = random_q4_0(rng, n_rows, n_cols)
    want = oracle.dequantize(2, raw, n_rows * n_cols)
    wb = cuda.upload_matrix(Q4_0, raw, n_rows, n_cols)
    out = cuda.new_buffer(n_rows * n_cols * 4)
    cuda.begin(); cuda.expand(Q4_0, wb, out, n_rows, n_cols, out_half=False); cuda.end()
    got = cuda.read(out, np.zeros(n_rows * n_cols, dtype=np.float32))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    cuda.begin(); cuda.expand(Q4_0, wb, out, n_rows, n_cols, out_half=True); cuda.end()
    half = cuda.read(out, np.zeros(n_rows * n_cols, dtype=np.float16))
    assert np.array_equal(half.view(np.uint16), want.astype(np.float16).view(np.uint16))
    wb.free(); out.free()


@pytest.mark.parametrize("fmt", [Q4_0, F32])
def test_embed_rows_are_bit_exact(cuda, fmt):
    rng = np.random.default_rng(9)
    n_vocab, n_embd = 300, 96
    raw, w = make_matrix(rng, fmt, n_vocab, n_embd)
    tokens = np.array([0, 299, 17, 17, 123], dtype=np.uint32)
    wb = cuda.upload_matrix(fmt, raw, n_vocab, n_embd)
    tb, out = cuda.buffer_from(tokens), cuda.new_buffer(len(tokens) * n_embd * 4)
    cuda.begin(); cuda.embed(fmt, wb, n_vocab, tb, out, n_embd, len(tokens)); cuda.end()
    got = cuda.read(out, np.zeros((len(tokens), n_embd), dtype=np.float32))
    assert np.array_equal(got.view(np.uint32), w[tokens].view(np.uint32))


def test_rms_norm_rows(cuda):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((5, 1024)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, 1024).astype(np.float32)
    xb, wb, ob = cuda.buffer_from(x), cuda.buffer_from(w), cuda.new_buffer(x.nbytes)
    cuda.begin(); cuda.rms_norm(xb, wb, ob, 1024, 5, 1e-5); cuda.end()
    got = cuda.read(ob, np.zeros_like(x))
    want = np.stack([oracle.rms_norm(r, w, 1e-5) for r in x])
    assert rel_error(got, want) < 1e-6


@pytest.mark.parametrize("head_dim,n_rot,dst_half", [(64, 64, False), (64, 64, True), (256, 64, False), (128, 128, True), (32, 16, False)])
def test_norm_rope_matches_scalar(cuda, head_dim, n_rot, dst_half):
    rng = np.random.default_rng(head_dim + n_rot)
    n_heads, n_tokens, first_pos, theta, eps = 3, 5, 1021, 1e6, 1e-5
    src = rng.standard_normal((n_tokens, n_heads, head_dim)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, head_dim).astype(np.float32)
    sb, wb = cuda.buffer_from(src), cuda.buffer_from(w)
    db = cuda.new_buffer(src.size * (2 if dst_half else 4))
    stride = n_heads * head_dim
    cuda.begin()
    cuda.norm_rope(sb, db, dst_half, wb, n_heads, head_dim, head_dim, n_rot, first_pos, n_tokens, stride, stride, theta, eps)
    cuda.end()
    got = cuda.read(db, np.zeros(src.shape, dtype=np.float16 if dst_half else np.float32)).astype(np.float32)
    want = np.zeros_like(src)
    for t in range(n_tokens):
        for h in range(n_heads):
            v = oracle.rms_norm(src[t, h], w, eps)
            v[:n_rot] = oracle.rope_neox(v[:n_rot], first_pos + t, theta)
            want[t, h] = v
    if dst_half:
        want = want.astype(np.float16).astype(np.float32)
        assert rel_error(got, want) < 2e-3
    else:
        assert rel_error(got, want) < 2e-6


# (first_pos, n_queries, n_heads, n_kv_heads, head_dim): crates/bobcat/tests/metal_attention.rs:19-27
ATTENTION_CASES = [(0, 1, 4, 2, 64), (5, 1, 4, 2, 64), (63, 3, 8, 2, 64), (100, 70, 4, 4, 32), (0, 130, 4, 1, 64), (37, 2, 2, 1, 256), (700, 1, 32, 8, 64),
                   (0, 512, 8, 2, 64), (100, 70, 8, 2, 64), (3, 33, 4, 2, 64), (61, 200, 4, 4, 64), (45, 1, 8, 1, 128), (130, 4, 16, 4, 128),
                   (15, 2, 6, 2, 64), (300, 1, 4, 4, 256),
                   # Batches of wide heads on the tensor-core prefill kernel (Qwen3.5's attention layers: 256 elements).
                   (50, 96, 8, 2, 256), (0, 64, 4, 1, 128), (300, 40, 16, 4, 256), (1000, 33, 2, 1, 256)]


def on_flash_kernel(kv_half, n_q, hd):
    """The shapes attention sends to its tensor-core prefill kernel (the reference's rule for its flash kernel, which
    knows heads of 64, extended to heads of 128 and 256)."""
    return kv_half and hd in (64, 128, 256) and n_q >= 32


def attention_f64(q, k, v, first_pos, n_heads, n_kv_heads):
    n_q, hd = q.shape[0], q.shape[2]
    group = n_heads // n_kv_heads
    out = np.zeros((n_q, n_heads, hd))
    for i in range(n_q):
        n_keys = first_pos + i + 1
        for h in range(n_heads):
            kh = k[:n_keys, h // group].astype(np.float64)
            s = kh @ q[i, h].astype(np.float64) / np.sqrt(hd)
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, h] = p @ v[:n_keys, h // group].astype(np.float64)
    return out


@pytest.mark.parametrize("kv_half", [False, True])
@pytest.mark.parametrize("case", ATTENTION_CASES)
def test_attention_against_f64(cuda, case, kv_half):
    first_pos, n_q, n_heads, n_kv, hd = case
    n_ctx = first_pos + n_q + 3
    rng = np.random.default_rng(sum(case))
    q = rng.uniform(-1, 1, (n_q, n_heads, hd)).astype(np.float32)
    k = rng.uniform(-1, 1, (n_ctx, n_kv, hd)).astype(np.float32)
    v = rng.uniform(-1, 1, (n_ctx, n_kv, hd)).astype(np.float32)
    if kv_half:
        k, v = k.astype(np.float16), v.astype(np.float16)
    qb, kb, vb = cuda.buffer_from(q), cuda.buffer_from(k), cuda.buffer_from(v)
    sb = cuda.new_buffer(cuda.attention_scratch_floats(n_heads, hd, n_ctx, n_q) * 4)
    ob = cuda.new_buffer(q.nbytes)
    cuda.begin(); cuda.attention(qb, kb, vb, kv_half, sb, ob, n_heads, n_kv, hd, first_pos, n_q, n_ctx); cuda.end()
    got = cuda.read(ob, np.zeros_like(q))
    want = attention_f64(q, k.astype(np.float32), v.astype(np.float32), first_pos, n_heads, n_kv)
    # The reference's kernel test allows 1e-6 absolute on inputs of this size (metal_attention.rs).
    flash = on_flash_kernel(kv_half, n_q, hd)
    # The tensor-core kernel carries queries and probabilities as two fp16 halves (about 22 bits).
    assert np.abs(got - want).max() < (4e-6 if flash else 2e-6)
    if n_q > 1:
        # Batched equals one query at a time, to rounding: a single query splits its keys into smaller chunks than a
        # batch does (and a batch may run on tensor cores), so the sums are taken in another order.
        one = np.zeros_like(q)
        tmp = cuda.new_buffer(n_heads * hd * 4)
        for i in range(0, n_q, 7 if n_q > 100 else 1):
            cuda.begin(); cuda.attention(qb.at(i * n_heads * hd * 4), kb, vb, kv_half, sb, tmp, n_heads, n_kv, hd, first_pos + i, 1, n_ctx); cuda.end()
            cuda.read(tmp, one[i])
            assert np.abs(one[i] - got[i]).max() < (4e-6 if flash else 2e-6)


def test_attention_limits(cuda):
    b = cuda.new_buffer(1 << 16)
    cuda.begin()
    with pytest.raises(errors.AttentionLimits):
        cuda.attention(b, b, b, False, b, b, 4, 2, 48, 0, 1, 8)
    with pytest.raises(errors.AttentionLimits):
        cuda.attention(b, b, b, False, b, b, 4, 2, 64, 7, 2, 8)
    cuda.discard()


@pytest.mark.parametrize("kernel", [2, 3, 4, 9])
def test_short_conv_batches_carry_history(cuda, kernel):
    """Batches of 1, 2, 7, 1, 64, 3 tokens with the history carried, against lfm2.rs:456-475 in f64."""
    rng = np.random.default_rng(kernel)
    n_embd = 96
    taps = rng.uniform(-1, 1, (n_embd, kernel)).astype(np.float32)
    hist = np.zeros((kernel - 1, n_embd), dtype=np.float32)
    tb, hb = cuda.buffer_from(taps), cuda.buffer_from(hist)
    ref_hist = np.zeros((kernel - 1, n_embd))
    for n in (1, 2, 7, 1, 64, 3):
        bcx = rng.uniform(-1, 1, (n, 3, n_embd)).astype(np.float32)
        bb, ob = cuda.buffer_from(bcx), cuda.new_buffer(n * n_embd * 4)
        cuda.begin(); cuda.short_conv(bb, tb, hb, ob, n_embd, kernel, n); cuda.end()
        got = cuda.read(ob, np.zeros((n, n_embd), dtype=np.float32))
        want = np.zeros((n, n_embd))
        for t in range(n):
            bx = (bcx[t, 0] * bcx[t, 2]).astype(np.float64)
            s = taps[:, kernel - 1] * bx + sum(taps[:, kk] * ref_hist[kk] for kk in range(kernel - 1))
            ref_hist = np.concatenate([ref_hist[1:], bx[None]])
            want[t] = bcx[t, 1] * s.astype(np.float32)
        assert np.abs(got - want).max() < 1e-5
        assert np.abs(cuda.read(hb, np.zeros_like(hist)) - ref_hist).max() < 1e-6


def test_matvec_conv_equals_projection_then_conv(cuda):
    rng = np.random.default_rng(4)
    n_embd, kernel = 128, 3
    raw, w = make_matrix(rng, Q4_0, 3 * n_embd, n_embd)
    x = rng.uniform(-1, 1, n_embd).astype(np.float32)
    nw = rng.uniform(0.5, 1.5, n_embd).astype(np.float32)
    taps = rng.uniform(-1, 1, (n_embd, kernel)).astype(np.float32)
    hist = rng.uniform(-1, 1, (kernel - 1, n_embd)).astype(np.float32)
    wb = cuda.upload_matrix(Q4_0, raw, 3 * n_embd, n_embd)
    xb, nb, tb, hb, ob = cuda.buffer_from(x), cuda.buffer_from(nw), cuda.buffer_from(taps), cuda.buffer_from(hist), cuda.new_buffer(n_embd * 4)
    cuda.begin(); cuda.matvec_conv(Q4_0, wb, n_embd, xb, Norm(nb.at(0), 1e-5), tb, hb, ob, n_embd, kernel); cuda.end()
    got = cuda.read(ob, np.zeros(n_embd, dtype=np.float32))
    bcx = oracle.matvec(2, raw, oracle.rms_norm(x, nw, 1e-5), 3 * n_embd)
    b, c, xx = bcx[:n_embd], bcx[n_embd:2 * n_embd], bcx[2 * n_embd:]
    bx = b * xx
    s = taps[:, 2].astype(np.float64) * bx + taps[:, 0].astype(np.float64) * hist[0] + taps[:, 1].astype(np.float64) * hist[1]
    assert np.abs(got - c * s.astype(np.float32)).max() < 1e-5
    new_hist = cuda.read(hb, np.zeros_like(hist))
    assert np.array_equal(new_hist[0], hist[1]) and np.abs(new_hist[1] - bx).max() < 1e-5


def test_argmax_ties_go_to_the_lowest_index(cuda):
    x = np.zeros(70001, dtype=np.float32)
    x[[69999, 1234, 40000]] = 3.5
    xb, ob = cuda.buffer_from(x), cuda.new_buffer(4)
    cuda.begin(); cuda.argmax(xb, ob, x.size); cuda.end()
    assert int(cuda.read(ob, np.zeros(1, dtype=np.uint32))[0]) == 1234
    x = -np.arange(1, 50, dtype=np.float32)
    cuda.write(xb, x)
    cuda.begin(); cuda.argmax(xb, ob, x.size); cuda.end()
    assert int(cuda.read(ob, np.zeros(1, dtype=np.uint32))[0]) == 0


# Full and partial tiles (crates/bobcat/tests/metal_matmul.rs:226-294): (n_rows, n_cols, n_tokens)
MATMUL_SHAPES = [(64, 64, 32), (128, 256, 64), (70, 96, 33), (1, 32, 1), (6144, 2048, 128), (2048, 10752, 65), (513, 2048, 512),
                 (128, 64, 16), (256, 128, 272), (300, 192, 100), (128, 4096, 257),
                 # at most 32 tokens: the warp-level kernel over the decode tiles (groups of 16, 3, 2 and 1 warps per tile)
                 (2048, 10752, 32), (6144, 2048, 20), (100, 64, 24), (16, 64, 16), (10752, 2048, 32), (4100, 1088, 17)]
# Tolerance of the reference's matmul test (metal_matmul.rs), per unit of sum |w x|.
MATMUL_TOLERANCE = 1e-4
# The tensor-core kernel rounds weights and inputs to fp16 like the reference's Q4_0 prefill kernel
# (matmul.metal:519-521): each product carries up to 2 * 2^-11 of relative error, so against exact
# operands the bound per unit of sum |w x| is 1e-3; against operands rounded the same way only the
# f32 accumulation is left.
HALF_OPERAND_TOLERANCE = 1e-3
ROUNDED_OPERAND_TOLERANCE = 2e-5


def on_tensor_cores(fmt, n_cols, n_tokens):
    """The shapes the batched multiply sends to its tcgen05 kernel."""
    return fmt == Q4_0 and n_cols % 64 == 0 and n_tokens >= 16


@pytest.mark.parametrize("fmt", [Q4_0, F32])
@pytest.mark.parametrize("shape", MATMUL_SHAPES)
def test_matmul_stores(cuda, fmt, shape):
    n_rows, n_cols, n_tokens = shape
    if fmt == F32 and n_rows * n_cols > 2 ** 22:
        pytest.skip("large float matrices add nothing over Q4_0 here")
    rng = np.random.default_rng(sum(shape) + fmt)
    raw, w = make_matrix(rng, fmt, n_rows, n_cols)
    x = rng.uniform(-1, 1, (n_tokens, n_cols)).astype(np.float32)
    y0 = rng.uniform(-1, 1, (n_tokens, n_rows)).astype(np.float32)
    wb = cuda.upload_matrix(fmt, raw, n_rows, n_cols)
    xb, yb = cuda.buffer_from(x), cuda.buffer_from(y0)
    exact = x.astype(np.float64) @ w.astype(np.float64).T
    tolerance, product = MATMUL_TOLERANCE, exact
    if on_tensor_cores(fmt, n_cols, n_tokens):
        tolerance = ROUNDED_OPERAND_TOLERANCE
        product = x.astype(np.float16).astype(np.float64) @ w.astype(np.float16).astype(np.float64).T
    budget = np.abs(x.astype(np.float64)) @ np.abs(w.astype(np.float64)).T
    out = np.zeros_like(y0)

    def check(want, extra=1.0):
        err = np.abs(cuda.read(yb, out).astype(np.float64) - want) / np.maximum(budget * extra, 1e-30)
        assert float(err.max()) < tolerance
        if product is not exact and want is product:
            loose = np.abs(cuda.read(yb, out).astype(np.float64) - exact) / np.maximum(budget, 1e-30)
            assert float(loose.max()) < HALF_OPERAND_TOLERANCE

    cuda.begin(); cuda.matmul(fmt, wb, n_rows, n_cols, xb, yb, n_tokens, OVERWRITE); cuda.end()
    check(product)
    cuda.write(yb, y0)
    cuda.begin(); cuda.matmul(fmt, wb, n_rows, n_cols, xb, yb, n_tokens, ACCUMULATE); cuda.end()
    check(y0 + product)
    cuda.write(yb, y0)
    cuda.begin(); cuda.matmul(fmt, wb, n_rows, n_cols, xb, yb, n_tokens, SWIGLU); cuda.end()
    silu = y0 / (1 + np.exp(-y0.astype(np.float64)))
    check(silu * product)
    for b in (wb, xb, yb):
        b.free()


@pytest.mark.parametrize("shape", [(100, 64, 5), (64, 2048, 32), (1000, 96, 17), (129, 32, 1), (4096, 1024, 32)])
def test_matmul_f32_few_tokens(cuda, shape):
    """An f32 matrix against at most 32 tokens (the logits of a pass over several sequences) runs on
    a kernel of its own: ragged row counts, fewer than 32 tokens, and nothing written past the
    tokens asked for."""
    n_rows, n_cols, n_tokens = shape
    rng = np.random.default_rng(sum(shape))
    raw, w = make_matrix(rng, F32, n_rows, n_cols)
    x = rng.uniform(-1, 1, (n_tokens, n_cols)).astype(np.float32)
    y0 = np.full((n_tokens + 1, n_rows), 7.5, dtype=np.float32)
    wb = cuda.upload_matrix(F32, raw, n_rows, n_cols)
    xb, yb = cuda.buffer_from(x), cuda.buffer_from(y0)
    cuda.begin(); cuda.matmul(F32, wb, n_rows, n_cols, xb, yb, n_tokens, OVERWRITE); cuda.end()
    out = cuda.read(yb, np.zeros_like(y0))
    exact = x.astype(np.float64) @ w.astype(np.float64).T
    budget = np.abs(x.astype(np.float64)) @ np.abs(w.astype(np.float64)).T
    err = np.abs(out[:n_tokens, :n_rows].astype(np.float64) - exact) / np.maximum(budget, 1e-30)
    assert float(err.max()) < ROUNDED_OPERAND_TOLERANCE
    assert (out[n_tokens] == 7.5).all()


def test_matmul_row_equals_matvec(cuda):
    """One token through the batched multiply equals the decode multiply, the self-consistency the
    reference checks between its prefill and step paths."""
    rng = np.random.default_rng(1)
    raw, w = make_matrix(rng, Q4_0, 256, 512)
    x = rng.uniform(-1, 1, 512).astype(np.float32)
    wb = cuda.upload_matrix(Q4_0, raw, 256, 512)
    xb, ya, yb = cuda.buffer_from(x), cuda.new_buffer(1024), cuda.new_buffer(1024)
    cuda.begin(); cuda.matvec(Q4_0, wb, 256, 512, xb, ya); cuda.matmul(Q4_0, wb, 256, 512, xb, yb, 1, OVERWRITE); cuda.end()
    a = cuda.read(ya, np.zeros(256, dtype=np.float32))
    b = cuda.read(yb, np.zeros(256, dtype=np.float32))
    assert scaled_error(a, b, w, x) < MATMUL_TOLERANCE


def test_profile_table(cuda):
    rng = np.random.default_rng(1)
    raw, _ = make_matrix(rng, Q4_0, 64, 64)
    wb = cuda.upload_matrix(Q4_0, raw, 64, 64)
    xb, yb = cuda.new_buffer(256), cuda.new_buffer(256)
    cuda.set_profiling(True)
    cuda.begin()
    for _ in range(3):
        cuda.matvec(Q4_0, wb, 64, 64, xb, yb)
    cuda.end()
    cuda.set_profiling(False)
    entries = cuda.profile()
    entry = [e for e in entries if e["name"] == "matvec" and e["n_rows"] == 64][0]
    assert entry["calls"] == 3 and entry["seconds"] > 0 and entry["bytes"] == 3 * 64 * 64 // 32 * 18


def test_unaligned_attention_views_take_the_scalar_kernels(cuda):
    """A view may start at any float (the reference's View allows any element-aligned offset). The
    tensor-core and the 16-byte-load kernels need aligned rows, so a q that starts 4 bytes into its
    buffer must run on the scalar chunk kernels and give what the aligned call gives."""
    rng = np.random.default_rng(5)
    first_pos, n_q, n_heads, n_kv, hd = 40, 40, 8, 2, 64  # a shape the tensor-core prefill kernel takes
    n_ctx = first_pos + n_q
    q = rng.uniform(-1, 1, (n_q, n_heads, hd)).astype(np.float32)
    k = rng.uniform(-1, 1, (n_ctx, n_kv, hd)).astype(np.float16)
    v = rng.uniform(-1, 1, (n_ctx, n_kv, hd)).astype(np.float16)
    shifted = np.concatenate([np.zeros(1, dtype=np.float32), q.ravel()])
    qb, qs, kb, vb = cuda.buffer_from(q), cuda.buffer_from(shifted), cuda.buffer_from(k), cuda.buffer_from(v)
    sb = cuda.new_buffer(cuda.attention_scratch_floats(n_heads, hd, n_ctx, n_q) * 4)
    a, b = cuda.new_buffer(q.nbytes), cuda.new_buffer(q.nbytes + 4)
    cuda.begin()
    cuda.attention(qb, kb, vb, True, sb, a, n_heads, n_kv, hd, first_pos, n_q, n_ctx)
    cuda.end()
    cuda.begin()
    cuda.attention(qs.at(4), kb, vb, True, sb, b.at(4), n_heads, n_kv, hd, first_pos, n_q, n_ctx)
    cuda.end()
    aligned = cuda.read(a, np.zeros_like(q))
    unaligned = cuda.read(b.at(4), np.zeros_like(q))
    assert np.abs(aligned - unaligned).max() < 4e-6
    # One query, where the aligned call takes the 16-byte-load decode kernel.
    cuda.begin()
    cuda.attention(qb, kb, vb, True, sb, a, n_heads, n_kv, hd, first_pos, 1, n_ctx)
    cuda.attention(qs.at(4), kb, vb, True, sb, b.at(4), n_heads, n_kv, hd, first_pos, 1, n_ctx)
    cuda.end()
    one_a = cuda.read(a, np.zeros((n_heads, hd), dtype=np.float32))
    one_b = cuda.read(b.at(4), np.zeros((n_heads, hd), dtype=np.float32))
    assert np.abs(one_a - one_b).max() < 2e-6


def test_unaligned_activation_offsets_are_rejected_before_launch(cuda):
    """The matrix-vector and batched products read their vectors 16 bytes at a time and have no
    scalar variant, so an offset off that boundary is an argument error, never a launch."""
    rng = np.random.default_rng(6)
    raw, _ = make_matrix(rng, Q4_0, 64, 64)
    wb = cuda.upload_matrix(Q4_0, raw, 64, 64)
    xb, yb, nb = cuda.new_buffer(1024), cuda.new_buffer(1024), cuda.new_buffer(1024)
    cuda.begin()
    with pytest.raises(errors.Argument):
        cuda.matvec(Q4_0, wb, 64, 64, xb.at(4), yb)
    with pytest.raises(errors.Argument):
        cuda.matvec(Q4_0, wb, 64, 64, xb, yb.at(8))
    with pytest.raises(errors.Argument):
        cuda.matvec(Q4_0, wb, 64, 64, xb, yb, Norm(nb.at(12), 1e-5))
    with pytest.raises(errors.Argument):
        cuda.matvec_swiglu(Q4_0, wb, wb, 64, 64, xb.at(4), Norm(nb.at(0), 1e-5), yb)
    with pytest.raises(errors.Argument):
        cuda.matmul(Q4_0, wb, 64, 64, xb.at(4), yb, 2, OVERWRITE)
    cuda.matvec(Q4_0, wb, 64, 64, xb.at(16), yb.at(32))  # aligned offsets still launch
    cuda.end()


def test_argmax_readback_slots(cuda):
    """Metal::argmax_readback / read_readback (backend.rs:2619-2663): the slot holds the token once
    the recording that wrote it has finished; an unwritten slot is out of bounds; a slot whose
    writer is still open is busy."""
    x = np.zeros(5000, dtype=np.float32)
    x[777] = 2.0
    xb, ob = cuda.buffer_from(x), cuda.new_buffer(4)
    rb = cuda.new_readback(3)
    with pytest.raises(errors.OutOfBounds):
        cuda.read_readback(rb, 1)
    cuda.begin()
    cuda.argmax_readback(xb, ob, rb, 1, x.size)
    with pytest.raises(errors.Busy):
        cuda.read_readback(rb, 1)
    with pytest.raises(errors.OutOfBounds):
        cuda.argmax_readback(xb, ob, rb, 3, x.size)
    ticket = cuda.commit()
    cuda.wait(ticket)
    assert cuda.read_readback(rb, 1) == 777
    assert int(cuda.read(ob, np.zeros(1, dtype=np.uint32))[0]) == 777
    with pytest.raises(errors.OutOfBounds):
        cuda.read_readback(rb, 0)
    rb.close()


@pytest.mark.parametrize("fmt", ["Q8_0", "Q6_K"])
def test_byte_layout_formats(cuda, fmt):
    """Q8_0 and Q6_K (the embedding type of the published Q4_0 files, lfm2_reference.rs:39) through
    every op that takes a matrix: dequantisation and embedding rows bit for bit
    (scalar.rs:108-113, :175-202), the decode products in their three forms and the batched product
    at the matvec tolerance."""
    from bobcat_b200 import Q6_K, Q8_0
    from conftest import random_q6k, random_q8_0
    rng = np.random.default_rng(17)
    fid, make, type_id = (Q8_0, random_q8_0, 8) if fmt == "Q8_0" else (Q6_K, random_q6k, 14)
    n_rows, n_cols = 200, 512
    raw = make(rng, n_rows, n_cols)
    w = oracle.dequantize(type_id, raw, n_rows * n_cols).reshape(n_rows, n_cols)
    wb = cuda.upload_matrix(fid, raw, n_rows, n_cols)
    out = cuda.new_buffer(n_rows * n_cols * 4)
    cuda.begin(); cuda.expand(fid, wb, out, n_rows, n_cols, out_half=False); cuda.end()
    got = cuda.read(out, np.zeros((n_rows, n_cols), dtype=np.float32))
    assert np.array_equal(got.view(np.uint32), w.view(np.uint32))
    tokens = np.array([0, 199, 17, 17, 123], dtype=np.uint32)
    tb, eb = cuda.buffer_from(tokens), cuda.new_buffer(tokens.size * n_cols * 4)
    cuda.begin(); cuda.embed(fid, wb, n_rows, tb, eb, n_cols, tokens.size); cuda.end()
    assert np.array_equal(cuda.read(eb, np.zeros((tokens.size, n_cols), dtype=np.float32)), w[tokens])
    # matvec: plain, with a fused norm, accumulating
    x = rng.uniform(-1, 1, n_cols).astype(np.float32)
    nw = rng.uniform(0.5, 1.5, n_cols).astype(np.float32)
    xb, nb, yb = cuda.buffer_from(x), cuda.buffer_from(nw), cuda.new_buffer(n_rows * 4)
    cuda.begin(); cuda.matvec(fid, wb, n_rows, n_cols, xb, yb); cuda.end()
    y = cuda.read(yb, np.zeros(n_rows, dtype=np.float32))
    assert scaled_error(y, oracle.matvec(type_id, raw, x, n_rows), w, x) < 1e-5
    cuda.begin(); cuda.matvec(fid, wb, n_rows, n_cols, xb, yb, Norm(nb.at(0), 1e-5), accumulate=True); cuda.end()
    xn = oracle.rms_norm(x, nw, 1e-5)
    y2 = cuda.read(yb, np.zeros(n_rows, dtype=np.float32))
    assert scaled_error(y2 - y, oracle.matvec(type_id, raw, xn, n_rows), w, xn) < 1e-5
    # SwiGLU of a gate / up pair
    raw_up = make(rng, n_rows, n_cols)
    ub = cuda.upload_matrix(fid, raw_up, n_rows, n_cols)
    cuda.begin(); cuda.matvec_swiglu(fid, wb, ub, n_rows, n_cols, xb, Norm(nb.at(0), 1e-5), yb); cuda.end()
    g, u = oracle.matvec(type_id, raw, xn, n_rows), oracle.matvec(type_id, raw_up, xn, n_rows)
    want = g / (1 + np.exp(-g.astype(np.float64))) * u
    assert np.abs(cuda.read(yb, np.zeros(n_rows, dtype=np.float32)) - want).max() < 1e-4 * max(1.0, float(np.abs(want).max()))
    # batched product
    xt = rng.uniform(-1, 1, (9, n_cols)).astype(np.float32)
    xtb, ytb = cuda.buffer_from(xt), cuda.new_buffer(9 * n_rows * 4)
    cuda.begin(); cuda.matmul(fid, wb, n_rows, n_cols, xtb, ytb, 9, OVERWRITE); cuda.end()
    yt = cuda.read(ytb, np.zeros((9, n_rows), dtype=np.float32))
    exact = xt.astype(np.float64) @ w.astype(np.float64).T
    budget = np.abs(xt.astype(np.float64)) @ np.abs(w.astype(np.float64)).T
    assert float((np.abs(yt - exact) / np.maximum(budget, 1e-30)).max()) < MATMUL_TOLERANCE
