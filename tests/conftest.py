import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def lib():
    from bobcat_b200 import _lib
    return _lib.load()


@pytest.fixture(scope="session")
def synth_dir(tmp_path_factory):
    return str(tmp_path_factory.mktemp("synth"))


@pytest.fixture(scope="session")
def model_path(synth_dir):
    """Return a function that writes (once) and returns the path of a synthetic model."""
    from bobcat_b200 import synth
    made = {}

    def get(config: str, seed: int = 0) -> str:
        key = (config, seed)
        if key not in made:
            made[key] = synth.write_model(os.path.join(synth_dir, "%s-%d.gguf" % key), config, seed)
        return made[key]

    return get


@pytest.fixture(scope="session")
def cuda():
    from bobcat_b200 import Cuda
    backend = Cuda.open(0)
    yield backend
    backend.close()


def rel_error(got: np.ndarray, want: np.ndarray) -> float:
    """Largest absolute difference relative to the largest reference magnitude, the measure of
    the reference's model tests (crates/bobcat/tests/lfm2_reference.rs `compare`)."""
    scale = float(np.abs(want).max())
    return float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max()) / (scale if scale > 0 else 1.0)


class XorShift:
    """The generator of the reference's kernel tests (crates/bobcat/tests/metal_matvec.rs:57-92):
    xorshift64, `unit()` floats in [-1, 1), fp16 scale bits in [2^-10, 2^-6)."""

    def __init__(self, seed: int = 0x9E3779B97F4A7C15):
        self.state = seed

    def next(self) -> int:
        x = self.state
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        self.state = x
        return x

    def unit(self) -> float:
        return (self.next() >> 40) / float(1 << 23) - 1.0

    def units(self, n: int) -> np.ndarray:
        return np.array([self.unit() for _ in range(n)], dtype=np.float32)


def random_q4_0(rng: np.random.Generator, n_rows: int, n_cols: int) -> np.ndarray:
    """Random Q4_0 rows: random nibbles and fp16 scales in [2^-10, 2^-6), as bytes [n_rows, n_cols/32*18]."""
    nb = n_cols // 32
    blocks = np.zeros((n_rows, nb, 18), dtype=np.uint8)
    # fp16 with exponent field 5..8 (2^-10 .. 2^-7) and random mantissa, random sign.
    bits = (rng.integers(5, 9, size=(n_rows, nb)) << 10) | rng.integers(0, 1024, size=(n_rows, nb)) | (rng.integers(0, 2, size=(n_rows, nb)) << 15)
    blocks[:, :, 0] = bits & 0xFF
    blocks[:, :, 1] = bits >> 8
    blocks[:, :, 2:] = rng.integers(0, 256, size=(n_rows, nb, 16), dtype=np.uint8)
    return blocks.reshape(n_rows, nb * 18)


def random_q8_0(rng: np.random.Generator, n_rows: int, n_cols: int) -> np.ndarray:
    """Random Q8_0 rows: fp16 scales in [2^-10, 2^-6), random int8 quants, as bytes [n_rows, n_cols/32*34]."""
    nb = n_cols // 32
    blocks = np.zeros((n_rows, nb, 34), dtype=np.uint8)
    bits = (rng.integers(5, 9, size=(n_rows, nb)) << 10) | rng.integers(0, 1024, size=(n_rows, nb)) | (rng.integers(0, 2, size=(n_rows, nb)) << 15)
    blocks[:, :, 0] = bits & 0xFF
    blocks[:, :, 1] = bits >> 8
    blocks[:, :, 2:] = rng.integers(0, 256, size=(n_rows, nb, 32), dtype=np.uint8)
    return blocks.reshape(n_rows, nb * 34)


def random_q6k(rng: np.random.Generator, n_rows: int, n_cols: int) -> np.ndarray:
    """Random Q6_K rows: random quant bits and int8 scales, fp16 d in [2^-14, 2^-10), as bytes [n_rows, n_cols/256*210]."""
    nb = n_cols // 256
    blocks = rng.integers(0, 256, size=(n_rows, nb, 210), dtype=np.uint8)
    bits = (rng.integers(1, 5, size=(n_rows, nb)) << 10) | rng.integers(0, 1024, size=(n_rows, nb)) | (rng.integers(0, 2, size=(n_rows, nb)) << 15)
    blocks[:, :, 208] = bits & 0xFF
    blocks[:, :, 209] = bits >> 8
    return blocks.reshape(n_rows, nb * 210)
