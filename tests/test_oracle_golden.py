"""The CPU parity checker against its pins: float32 `transformers` runs of random-init models
(tests/golden/*.npz, made by tests/golden/make_transformers_golden.py), the `gguf` package's
dequantiser, and closed-form f64 arithmetic."""

import hashlib

import numpy as np
import pytest

from conftest import random_q4_0, rel_error
from oracle import oracle

GOLDEN = ["lfm2-tiny", "lfm2moe-tiny", "qwen35-tiny"]
# The reference's own scalar-vs-transformers tolerance (crates/bobcat/tests/lfm2_reference.rs:19).
TOLERANCE = 1e-4


@pytest.mark.parametrize("config", GOLDEN)
def test_step_matches_transformers(config, model_path):
    g = np.load("tests/golden/%s.npz" % config)
    path = model_path(config)
    assert hashlib.sha256(open(path, "rb").read()).hexdigest() == str(g["gguf_sha256"]), "the synthetic writer's bytes changed"
    m = oracle.Model(path)
    st = m.state(64)
    out = None
    for i, tok in enumerate(g["tokens"]):
        out = st.step(int(tok), want_trace=True)
        assert np.array_equal(out["embedding"], g["embedding"][i])
        for il in range(m.n_layers):
            assert rel_error(out["layers"][il], g["layers"][il][i]) < TOLERANCE, (i, il)
        assert rel_error(out["final_norm"], g["final_norm"][i]) < TOLERANCE
        assert rel_error(out["logits"], g["logits"][i]) < TOLERANCE
    logits, generated = out["logits"], []
    for _ in range(len(g["generated"])):
        tok = int(np.argmax(logits))
        generated.append(tok)
        logits = st.step(tok)["logits"]
    assert generated == g["generated"].tolist()


def test_q4_0_dequant_matches_gguf_package():
    import gguf
    rng = np.random.default_rng(7)
    raw = random_q4_0(rng, 64, 256)
    want = gguf.quants.dequantize(raw, gguf.GGMLQuantizationType.Q4_0).astype(np.float32)
    got = oracle.dequantize(oracle.TYPE_IDS["Q4_0"], raw, 64 * 256).reshape(64, 256)
    assert np.array_equal(got, want)


def test_f16_conversion_is_exact():
    bits = np.arange(0, 65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.lib().orc_f16_to_f32(int(b)) for b in bits[::7]], dtype=np.float32)
    w = want[::7]
    assert np.array_equal(got[~np.isnan(w)], w[~np.isnan(w)])


def test_matvec_is_an_f64_dot_of_dequantised_rows():
    rng = np.random.default_rng(3)
    raw = random_q4_0(rng, 7, 64)
    x = rng.standard_normal(64).astype(np.float32)
    w = oracle.dequantize(2, raw, 7 * 64).reshape(7, 64)
    want = (w.astype(np.float64) @ x.astype(np.float64)).astype(np.float32)
    for threads in (1, 4):
        assert np.array_equal(oracle.matvec(2, raw, x, 7, threads=threads), want)


def test_rms_norm_rope_softmax_against_f64():
    rng = np.random.default_rng(5)
    x = rng.standard_normal(96).astype(np.float32)
    w = rng.standard_normal(96).astype(np.float32)
    scale = np.float32(1.0 / np.sqrt(np.mean(x.astype(np.float64) ** 2) + np.float64(np.float32(1e-5))))
    assert np.array_equal(oracle.rms_norm(x, w, 1e-5), w * (x * scale))
    v = rng.standard_normal(64).astype(np.float32)
    got = oracle.rope_neox(v, 37, 1e6)
    i = np.arange(32)
    ang = 37.0 / (1e6 ** (2 * i / 64.0))
    want = np.concatenate([v[:32] * np.cos(ang) - v[32:] * np.sin(ang), v[32:] * np.cos(ang) + v[:32] * np.sin(ang)])
    assert np.abs(got - want).max() < 1e-5
    s = oracle.softmax(x)
    e = np.exp(x.astype(np.float64) - x.max())
    assert np.abs(s - e / e.sum()).max() < 1e-7 and abs(float(s.sum()) - 1) < 1e-6


def test_route_picks_top_experts_with_ties_to_lower_ids():
    logits = np.array([0.5, 2.0, 2.0, -1.0, 0.0, 2.0, 0.1, 0.2], dtype=np.float32)
    bias = np.zeros(8, dtype=np.float32)
    experts, scores = oracle.lfm2_route(logits, bias, 2)
    assert experts[:2].tolist() == [1, 2]
    s = 1 / (1 + np.exp(-np.float32(2.0)))
    assert abs(scores[1] - s / (2 * s + 1e-6)) < 1e-6
    # The bias steers the pick and leaves the weights to the unbiased scores.
    bias[3] = 10.0
    experts, scores = oracle.lfm2_route(logits, bias, 2)
    assert experts[:2].tolist() == [3, 1]
    s3, s1 = 1 / (1 + np.exp(1.0)), 1 / (1 + np.exp(-2.0))
    assert abs(scores[3] - s3 / (s3 + s1 + 1e-6)) < 1e-6


def test_byte_layout_formats_match_the_gguf_package():
    """Q8_0 and Q6_K dequantisation of the checker against the `gguf` package on random blocks, bit for bit."""
    import gguf
    from conftest import random_q6k, random_q8_0
    rng = np.random.default_rng(5)
    for name, make, qtype, cols in (("Q8_0", random_q8_0, gguf.GGMLQuantizationType.Q8_0, 256), ("Q6_K", random_q6k, gguf.GGMLQuantizationType.Q6_K, 512)):
        raw = make(rng, 64, cols)
        want = gguf.quants.dequantize(raw, qtype).astype(np.float32)
        got = oracle.dequantize(oracle.TYPE_IDS[name], raw, 64 * cols).reshape(64, cols)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name
