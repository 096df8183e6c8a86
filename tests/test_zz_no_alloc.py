"""bc_attention_static, the attention entry point for callers that cannot allocate device memory
(an engine that owns one pre-planned device pool, or a decode loop that cannot take cudaMalloc's
device-wide synchronisation): its chunk partials live in an array built into the library instead of
a caller-provided scratch buffer. It must give exactly what bc_op_attention gives, call after call,
whatever the previous call left in the shared array. Collected last on purpose."""

import ctypes as C

import numpy as np
import pytest

from bobcat_b200 import Cuda, errors

pytestmark = pytest.mark.gpu


def run_both(cuda, rng, first_pos, n_q, n_heads, n_kv, hd, kv_half):
    n_ctx = first_pos + n_q + 5
    q = rng.uniform(-1, 1, (n_q, n_heads, hd)).astype(np.float32)
    kv_type = np.float16 if kv_half else np.float32
    k = rng.uniform(-1, 1, (n_ctx, n_kv, hd)).astype(kv_type)
    v = rng.uniform(-1, 1, (n_ctx, n_kv, hd)).astype(kv_type)
    qb, kb, vb = cuda.buffer_from(q), cuda.buffer_from(k), cuda.buffer_from(v)
    scratch = cuda.new_buffer(cuda.attention_scratch_floats(n_heads, hd, n_ctx, n_q) * 4)
    want_b, got_b = cuda.new_buffer(q.nbytes), cuda.new_buffer(q.nbytes)
    cuda.begin(); cuda.attention(qb, kb, vb, kv_half, scratch, want_b, n_heads, n_kv, hd, first_pos, n_q, n_ctx); cuda.end()
    L = cuda._L
    status = L.bc_attention_static(cuda.stream, qb.device_ptr, kb.device_ptr, vb.device_ptr, int(kv_half), got_b.device_ptr,
                                   n_heads, n_kv, hd, first_pos, n_q, n_ctx)
    errors.check(status, L)
    want = cuda.read(want_b, np.zeros_like(q))
    got = cuda.read(got_b, np.zeros_like(q))
    return got, want


def test_static_scratch_attention_matches_twice_in_a_row():
    cuda = Cuda.open(0)
    rng = np.random.default_rng(42)
    # Two different shapes back to back, so the second call runs over the first call's leftovers.
    for case in [(700, 1, 32, 8, 64, True), (37, 70, 8, 2, 128, False), (700, 1, 32, 8, 64, True)]:
        got, want = run_both(cuda, rng, *case)
        # Same kernels on the same inputs: the tolerance of the attention tests (1e-6 absolute)
        # is generous, the results are expected to be identical.
        assert np.abs(got - want).max() <= 1e-6
        assert np.array_equal(got, want)
    cuda.close()


def test_static_scratch_attention_allocates_nothing():
    """The property the entry point exists for: after a warm-up call (which looks up the array's
    address once), further calls on all three dispatch paths (16-position chunks, 64-position
    chunks, the tensor-core prefill kernel) leave the device's free memory unchanged."""
    import torch

    cuda = Cuda.open(0)
    rng = np.random.default_rng(7)
    L = cuda._L
    cases = [(300, 1, 32, 8, 64, True), (20, 40, 8, 2, 128, False), (64, 64, 16, 4, 64, True)]
    prepared = []
    for first_pos, n_q, n_heads, n_kv, hd, kv_half in cases:
        n_ctx = first_pos + n_q
        kv_type = np.float16 if kv_half else np.float32
        q = cuda.buffer_from(rng.uniform(-1, 1, (n_q, n_heads, hd)).astype(np.float32))
        k = cuda.buffer_from(rng.uniform(-1, 1, (n_ctx, n_kv, hd)).astype(kv_type))
        v = cuda.buffer_from(rng.uniform(-1, 1, (n_ctx, n_kv, hd)).astype(kv_type))
        out = cuda.new_buffer(n_q * n_heads * hd * 4)
        prepared.append((q, k, v, out, int(kv_half), n_heads, n_kv, hd, first_pos, n_q, n_ctx))

    def call(c):
        q, k, v, out, half, n_heads, n_kv, hd, first_pos, n_q, n_ctx = c
        errors.check(L.bc_attention_static(cuda.stream, q.device_ptr, k.device_ptr, v.device_ptr, half, out.device_ptr, n_heads, n_kv, hd,
                                           first_pos, n_q, n_ctx), L)

    for c in prepared:  # warm-up: kernels loaded, shared-memory limits raised, address looked up
        call(c)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        for c in prepared:
            call(c)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    cuda.close()


def test_static_scratch_attention_at_its_capacity():
    """One query over 32 heads of 64 elements fits up to 15 872 positions (992 chunks of 16); the
    largest accepted shape matches bc_op_attention and one chunk more is rejected. The capacity
    follows the positions in use, not the cache's size."""
    cuda = Cuda.open(0)
    rng = np.random.default_rng(3)
    got, want = run_both(cuda, rng, 15871, 1, 32, 8, 64, True)
    assert np.array_equal(got, want)
    L = cuda._L
    b = cuda.new_buffer(1 << 12)
    p = b.device_ptr
    status = L.bc_attention_static(cuda.stream, p, p, p, 1, p, 32, 8, 64, 15872, 1, 1 << 18)
    assert status == errors.Argument.status and b"built-in scratch" in L.bc_last_error()
    cuda.close()


def test_static_scratch_attention_rejects_what_does_not_fit():
    cuda = Cuda.open(0)
    L = cuda._L
    b = cuda.new_buffer(1 << 12)
    p = b.device_ptr
    # 64 queries x 32 heads x 4096 chunks x 66 floats is far beyond the built-in 2 Mi floats.
    status = L.bc_attention_static(cuda.stream, p, p, p, 0, p, 32, 8, 64, (1 << 18) - 64, 64, 1 << 18)
    assert status == errors.Argument.status and b"built-in scratch" in L.bc_last_error()
    assert L.bc_attention_static(cuda.stream, None, p, p, 0, p, 32, 8, 64, 0, 1, 64) == errors.Argument.status
    assert L.bc_attention_static(cuda.stream, p, p, p, 0, p, 32, 8, 48, 0, 1, 64) == errors.AttentionLimits.status
    cuda.close()
